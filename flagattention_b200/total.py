"""total_attention: column sums of the attention matrix recomputed from the
log-normaliser (src/flag_attn/total.py:9-47)."""
import math

import torch

from . import _C
from .flash import _total_attention


def total_attention(q, k, l, causal=False, sm_scale=None):
    Dq, Dk = q.shape[-1], k.shape[-1]
    assert Dq == Dk
    assert Dk in {16, 32, 64, 128}
    B, H, M, D = q.shape
    Hk = k.shape[1]
    assert H % Hk == 0, "number of heads in q must be a multiple of that in k"
    if sm_scale is None:
        sm_scale = 1. / math.sqrt(D)
    q, k = _C.kernel_ready(q), _C.kernel_ready(k)
    with torch.cuda.device(q.device):
        return _total_attention(q, k, l.contiguous(), causal, sm_scale)
