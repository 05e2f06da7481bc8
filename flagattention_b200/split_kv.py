"""Split-KV ("flash decoding") forward for decode-shaped queries.

Mirrors src/flag_attn/split_kv.py:229-330: `attention` is the standalone
forward-only operator, `num_splits_herustic` the split-count rule that
flash_attention's forward also consults.
"""
import math

import torch

from . import _C

__all__ = ["attention"]

_SPLIT_BLOCK_N = 64  # keys per tile of the stage-1 kernel; split sizes are multiples of it


def get_fwd_config(B, H, M, N, D, causal):
    """(BLOCK_M, BLOCK_N, stages, warps) fed to the split heuristic, the values
    of the reference (src/flag_attn/split_kv.py:229-231) so the same calls split."""
    return (16, 128, 1, 4)


def num_splits_herustic(B, H, M, N, BLOCK_M, BLOCK_N, num_sms, max_splits):
    """Split count, computed by the library's restatement of
    src/flag_attn/split_kv.py:234-262 (name kept as spelled there)."""
    return int(_C.load().fa_num_splits_heuristic(B, H, M, N, BLOCK_M, BLOCK_N, num_sms, max_splits))


def _splitkv_forward(q, k, v, causal, sm_scale, S):
    B, H, M, D = q.shape
    N, Hk = k.shape[2], k.shape[1]
    lib = _C.load()
    n_blocks = (N + _SPLIT_BLOCK_N - 1) // _SPLIT_BLOCK_N
    n_split_size = ((n_blocks + S - 1) // S) * _SPLIT_BLOCK_N
    S = (N + n_split_size - 1) // n_split_size  # drop splits that would be empty
    o_part = torch.empty((B, H, S, M, D), dtype=torch.float32, device=q.device)
    l_part = torch.empty((B, H, S, M), dtype=torch.float32, device=q.device)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    L = torch.empty((B, H, M), dtype=torch.float32, device=q.device)
    shape = _C.flash_shape(q.dtype, B, H, Hk, M, N, D, causal, sm_scale)
    tq, tk, tv, to = _C.tensor4(q), _C.tensor4(k), _C.tensor4(v), _C.tensor4(o)
    stream = _C.stream_ptr(q.device)
    st = lib.fa_splitkv_fwd(_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.byref(tv), S,
                            n_split_size, _C.fptr(o_part), _C.fptr(l_part), stream)
    _C.check(st, "fa_splitkv_fwd")
    st = lib.fa_splitkv_combine(_C.byref(shape), S, _C.fptr(o_part), _C.fptr(l_part),
                                _C.byref(to), _C.fptr(L), stream)
    _C.check(st, "fa_splitkv_combine")
    return o, L


def attention(q, k, v, causal=False, sm_scale=None):
    """Forward-only flash attention that always takes the split-KV path
    (src/flag_attn/split_kv.py:266-330). Returns the output in q's dtype."""
    Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Dq == Dk == Dv
    assert Dk in {16, 32, 64, 128}
    B, H, M, D = q.shape
    N = k.shape[2]
    Hk, Hv = k.shape[1], v.shape[1]
    assert Hk == Hv, "num of heads in k and v should be equal"
    assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"
    if sm_scale is None:
        sm_scale = 1. / math.sqrt(D)
    q, k, v = _C.kernel_ready(q), _C.kernel_ready(k), _C.kernel_ready(v)
    with torch.cuda.device(q.device):
        num_sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        cfg = get_fwd_config(B, H, M, N, D, causal)
        S = num_splits_herustic(B, H, M, N, cfg[0], cfg[1], num_sms, 128)
        o, _ = _splitkv_forward(q, k, v, causal, sm_scale, S)
    return o
