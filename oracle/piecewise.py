"""Oracle for piecewise_attention (test infrastructure, see oracle/__init__.py).

Follows src/flag_attn/testing/piecewise.py:5-34 (forward) and :36-78 (the
closed-form gradients) of the reference: both score products are formed, the
far one is selected where (m + N - M) - n >= dist_threshold (:21-24), causal
positions are filled with the dtype's most negative finite value, not -inf
(:26-27), the fp32 softmax is cast to v's dtype before the re-mask and P@V
(:30-33).
"""
import math

import torch


def _masks(len_q, len_k, dist_threshold, device):
    rows = torch.arange(len_q, device=device)[:, None]
    cols = torch.arange(len_k, device=device)[None, :]
    shift = len_k - len_q
    far = (rows + shift - cols) >= dist_threshold
    visible = (rows + shift) >= cols
    return far, visible


def piecewise_attention(q1, k1, q2, k2, v, dist_threshold, causal, sm_scale=None, upcast=False):
    in_dtype = q1.dtype
    if upcast:
        q1, k1, q2, k2, v = (t.float() for t in (q1, k1, q2, k2, v))
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q1.shape[-1])
    far, visible = _masks(q1.shape[-2], k1.shape[-2], dist_threshold, q1.device)
    near_scores = q1 @ k1.transpose(-1, -2)
    far_scores = q2 @ k2.transpose(-1, -2)
    scores = torch.where(far, far_scores, near_scores) * sm_scale
    if causal:
        scores = torch.where(visible, scores, torch.finfo(scores.dtype).min)
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(v.dtype)
    if causal:
        probs = torch.where(visible, probs, 0.0)
    return (probs @ v).to(in_dtype)


def piecewise_attention_grad(q1, k1, q2, k2, v, dist_threshold, causal, sm_scale, o, do,
                             upcast=False):
    """Closed-form (dq1, dk1, dq2, dk2, dv), as src/flag_attn/testing/piecewise.py:36-78."""
    in_dtype = q1.dtype
    if upcast:
        q1, k1, q2, k2, v, o, do = (t.float() for t in (q1, k1, q2, k2, v, o, do))
    far, visible = _masks(q1.shape[-2], k1.shape[-2], dist_threshold, q1.device)
    scores = torch.where(far, q2 @ k2.transpose(-1, -2), q1 @ k1.transpose(-1, -2)) * sm_scale
    if causal:
        scores = torch.where(visible, scores, torch.finfo(scores.dtype).min)
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(v.dtype)
    dv = probs.transpose(-1, -2) @ do
    dprobs = do @ v.transpose(-1, -2)
    delta = (do * o).sum(-1, keepdim=True)
    dscores = probs * (dprobs - delta) * sm_scale
    d_far = torch.where(far, dscores, 0.0)
    d_near = torch.where(far, 0.0, dscores)
    dq1, dk1 = d_near @ k1, d_near.transpose(-1, -2) @ q1
    dq2, dk2 = d_far @ k2, d_far.transpose(-1, -2) @ q2
    return tuple(t.to(in_dtype) for t in (dq1, dk1, dq2, dk2, dv))
