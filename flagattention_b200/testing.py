"""Plain-PyTorch reference implementations shipped with the package, the
counterpart of `flag_attn.testing` (src/flag_attn/testing/__init__.py:1-4).

They run on any device torch supports and exist so that users can check the
kernels the way the reference's README describes: compare against
`upcast=True` (fp32 math) and require the kernel's error to be at most twice
that of the same-precision PyTorch path.  They materialise the full score
matrix, so memory grows with seqlen_q * seqlen_k.
"""
import math

import torch

from .dropout import recompute_mask  # noqa: F401

__all__ = ["flash_attention", "piecewise_attention", "paged_attention", "recompute_mask", "rotary_pair"]


def _causal_mask(m, n, device):
    return (torch.arange(m, device=device)[:, None] + (n - m)) >= torch.arange(n, device=device)


def flash_attention(q, k, v, causal, dropout_p=0.0, dropout_mask=None, sm_scale=None,
                    return_log_normalizer=False, return_total_attention=False, upcast=False):
    dtype = q.dtype
    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    scale = sm_scale if sm_scale is not None else q.shape[-1] ** -0.5
    groups = q.shape[1] // k.shape[1]
    if groups > 1:
        k, v = k.repeat_interleave(groups, 1), v.repeat_interleave(groups, 1)
    s = torch.matmul(q, k.transpose(2, 3)) * scale
    keep = _causal_mask(q.shape[2], k.shape[2], q.device) if causal else None
    if causal:
        s = s.masked_fill(~keep, float("-inf"))
    s = s.float()
    p = torch.softmax(s, dim=-1, dtype=torch.float32)
    if causal:
        p = p.masked_fill(~keep, 0.0)
    tot = p.sum(dim=-2) if return_total_attention else None
    if dropout_mask is not None:
        p = p.masked_fill(~dropout_mask, 0.0)
    o = (torch.matmul(p.to(v.dtype), v) * (1.0 / (1 - dropout_p))).to(dtype)
    if return_log_normalizer or return_total_attention:
        return (o, torch.logsumexp(s, dim=-1) if return_log_normalizer else None, tot)
    return o


def piecewise_attention(q1, k1, q2, k2, v, dist_threshold, causal, sm_scale=None, upcast=False):
    dtype = q1.dtype
    if upcast:
        q1, k1, q2, k2, v = q1.float(), k1.float(), q2.float(), k2.float(), v.float()
    scale = sm_scale if sm_scale is not None else q1.shape[-1] ** -0.5
    m, n = q1.shape[2], k1.shape[2]
    dist = (torch.arange(m, device=q1.device)[:, None] + (n - m)) - torch.arange(n, device=q1.device)
    s = torch.where(dist >= dist_threshold, torch.matmul(q2, k2.transpose(2, 3)),
                    torch.matmul(q1, k1.transpose(2, 3))) * scale
    if causal:
        s = s.masked_fill(dist < 0, torch.finfo(s.dtype).min)
    p = torch.softmax(s, dim=-1, dtype=torch.float32).to(v.dtype)
    if causal:
        p = p.masked_fill(dist < 0, 0.0)
    return torch.matmul(p, v).to(dtype)


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, scale):
    """Note the argument order: block_tables comes before context_lens here."""
    out = torch.empty_like(query)
    kv_heads, block, head = value_cache.shape[1:]
    groups = query.shape[1] // kv_heads
    for i, ctx in enumerate(context_lens.tolist()):
        ids = block_tables[i, : (ctx + block - 1) // block].long()
        kk = key_cache[ids].transpose(0, 1).reshape(kv_heads, -1, head)[:, :ctx].float()
        vv = value_cache[ids].transpose(0, 1).reshape(kv_heads, -1, head)[:, :ctx].float()
        qq = query[i].float().view(kv_heads, groups, head)
        p = torch.softmax(torch.bmm(qq, kk.transpose(1, 2)) * scale, dim=-1)
        out[i] = torch.bmm(p, vv).reshape(-1, head).to(out.dtype)
    return out


def rotary_pair(x, cos1, sin1, cos2, sin2, positions=None, interleaved=False, upcast=True):
    """PyTorch reference of flagattention_b200.rotary_pair, differentiable through autograd.
    upcast=False does the arithmetic in x's own dtype (the same-precision comparison)."""
    half = x.shape[-1] // 2
    if positions is None:
        positions = torch.arange(x.shape[2], device=x.device)
    positions = positions.to(device=x.device, dtype=torch.int64)
    if positions.dim() == 1:
        positions = positions[None]
    work = x.float() if upcast else x
    lo, hi = (work[..., 0::2], work[..., 1::2]) if interleaved else (work[..., :half], work[..., half:])

    def one(cos, sin):
        rows = positions.clamp(0, cos.shape[0] - 1)
        c = cos.to(work.device)[rows][:, None, :, :half].to(work.dtype)
        s = sin.to(work.device)[rows][:, None, :, :half].to(work.dtype)
        ylo, yhi = lo * c - hi * s, hi * c + lo * s
        y = torch.stack((ylo, yhi), dim=-1).flatten(-2) if interleaved else torch.cat((ylo, yhi), dim=-1)
        return y.to(x.dtype)

    return one(cos1, sin1), one(cos2, sin2)
