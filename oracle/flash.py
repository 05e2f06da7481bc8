"""Oracle for flash_attention (test infrastructure, see oracle/__init__.py).

Follows src/flag_attn/testing/flash.py:5-70 of the reference step by step:
optional fp32 upcast (:16-17), GQA by repeating kv heads (:28-30), scaled
scores (:39), bottom-right causal fill with -inf (:33,:40-41), scores to fp32
(:43), logsumexp (:44-45), fp32 softmax (:48), re-masking so rows without a
visible key become zero (:49-50), column sums (:52-53), P cast to v's dtype
before P@V (:60), output cast back to the input dtype (:61).
Dropout follows :55-60 there: the keep-mask is an input, dropped probabilities are zeroed after the
column sums and before P@V, and the result is scaled by 1 / (1 - dropout_p).
"""
import math

import torch


def flash_attention(q, k, v, causal, sm_scale=None, return_log_normalizer=False,
                    return_total_attention=False, upcast=False, dropout_p=0.0, dropout_mask=None):
    in_dtype = q.dtype
    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    head_dim = q.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    hq, hk = q.shape[1], k.shape[1]
    assert hq % hk == 0
    if hq != hk:
        k = k.repeat_interleave(hq // hk, dim=1)
        v = v.repeat_interleave(hq // hk, dim=1)
    len_q, len_k = q.shape[-2], k.shape[-2]
    shift = len_k - len_q
    rows = torch.arange(len_q, device=q.device)[:, None]
    cols = torch.arange(len_k, device=q.device)[None, :]
    visible = (rows + shift) >= cols

    scores = (q @ k.transpose(-1, -2)) * sm_scale
    if causal:
        scores = torch.where(visible, scores, float("-inf"))
    scores = scores.to(torch.float32)
    lse = torch.logsumexp(scores, dim=-1) if return_log_normalizer else None
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32)
    if causal:
        probs = torch.where(visible, probs, 0.0)
    total = probs.sum(dim=-2) if return_total_attention else None
    if dropout_mask is not None:
        probs = probs.masked_fill(~dropout_mask, 0.0)
    out = ((probs.to(v.dtype) @ v) * (1.0 / (1 - dropout_p))).to(in_dtype)
    if return_log_normalizer or return_total_attention:
        return out, lse, total
    return out
