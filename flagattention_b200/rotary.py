"""Producer of piecewise_attention's operands: two rotary position embeddings in one pass.

The reference's README describes the step in prose only (two position embeddings applied to q
and k depending on the distance regime, giving q1, q2 and k1, k2: README.md:136-138); its
operator takes the four results (src/flag_attn/piecewise.py:169-191).  Here the step is one
HBM-bound kernel per tensor: x is read once and both rotated copies are written, and the
backward folds the two gradients into one.  Any position scheme fits, since the caller supplies
the cos / sin tables (and optionally the position of every token).
"""
import ctypes

import torch

from . import _C

__all__ = ["rotary_pair", "rotary_tables"]


def rotary_tables(num_positions, head_dim, base=10000.0, position_scale=1.0, device=None):
    """fp32 (cos, sin) tables of shape (num_positions, head_dim // 2):
    angle[p, i] = p * position_scale * base ** (-2 i / head_dim)."""
    assert head_dim % 2 == 0
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    pos = torch.arange(num_positions, dtype=torch.float32) * position_scale
    ang = torch.outer(pos, inv_freq)
    return ang.cos().to(device), ang.sin().to(device)


def _tables_ready(tables, half, device):
    for t in tables:
        assert t.device == device, \
            f"cos / sin tables are on {t.device}, x on {device} (rotary_tables(..., device=x.device))"
    rows, stride = tables[0].shape[0], tables[0].stride(0)
    ok = True
    for t in tables:
        assert t.dtype == torch.float32 and t.dim() == 2, "cos / sin tables are fp32 (positions, D/2)"
        assert t.shape[0] == rows and t.shape[1] >= half, "cos / sin tables must share their shape"
        ok = ok and t.stride(1) == 1 and t.stride(0) == stride and stride % 4 == 0 \
            and t.data_ptr() % 16 == 0
    if not ok:
        tables = [t[:, :half].contiguous() for t in tables]
        stride = half
    return tables, rows, stride


def _positions_ready(positions, B, L, device):
    if positions is None:
        return None, ctypes.c_void_p(0), 0
    assert not positions.is_floating_point(), "positions are integers"
    if positions.dim() == 1:
        positions = positions[None]
    assert positions.shape[-1] == L and positions.shape[0] in (1, B)
    pos = positions.to(device=device, dtype=torch.int64).contiguous()
    return pos, _C.fptr(pos), (L if pos.shape[0] > 1 else 0)


class RotaryPair(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos1, sin1, cos2, sin2, positions, interleaved):
        assert x.dim() == 4, "x is (batch, heads, length, head_dim)"
        B, H, L, D = x.shape
        assert D % 16 == 0 and D <= 512, "head_dim must be a multiple of 16, at most 512"
        assert x.is_cuda, "x must be a CUDA tensor"
        x = _C.kernel_ready(x)
        tables, rows, stride = _tables_ready([cos1, sin1, cos2, sin2], D // 2, x.device)
        pos, pos_ptr, pos_stride = _positions_ready(positions, B, L, x.device)
        out1, out2 = torch.empty_like(x), torch.empty_like(x)
        lib = _C.load()
        with torch.cuda.device(x.device):
            st = lib.fa_rotary_pair_fwd(
                _C.dtype_code(x.dtype), B, H, L, D, 1 if interleaved else 0,
                _C.byref(_C.tensor4(x)), *[_C.fptr(t) for t in tables], ctypes.c_int64(stride), rows,
                pos_ptr, ctypes.c_int64(pos_stride), _C.byref(_C.tensor4(out1)),
                _C.byref(_C.tensor4(out2)), _C.stream_ptr(x.device))
        _C.check(st, "fa_rotary_pair_fwd")
        ctx.save_for_backward(*tables, *([pos] if pos is not None else []))
        ctx.args = (stride, rows, pos_stride, bool(interleaved), pos is not None)
        return out1, out2

    @staticmethod
    def backward(ctx, g1, g2):
        stride, rows, pos_stride, interleaved, has_pos = ctx.args
        saved = ctx.saved_tensors
        tables = saved[:4]
        pos_ptr = _C.fptr(saved[4]) if has_pos else ctypes.c_void_p(0)
        assert g1.device == g2.device == tables[0].device, "gradients must be on the tables' device"
        g1, g2 = _C.kernel_ready(g1), _C.kernel_ready(g2)
        B, H, L, D = g1.shape
        dx = torch.empty_like(g1)
        lib = _C.load()
        with torch.cuda.device(g1.device):
            st = lib.fa_rotary_pair_bwd(
                _C.dtype_code(g1.dtype), B, H, L, D, 1 if interleaved else 0,
                _C.byref(_C.tensor4(g1)), _C.byref(_C.tensor4(g2)), *[_C.fptr(t) for t in tables],
                ctypes.c_int64(stride), rows, pos_ptr, ctypes.c_int64(pos_stride),
                _C.byref(_C.tensor4(dx)), _C.stream_ptr(g1.device))
        _C.check(st, "fa_rotary_pair_bwd")
        return dx, None, None, None, None, None, None


def rotary_pair(x, cos1, sin1, cos2, sin2, positions=None, interleaved=False):
    """Returns (x1, x2): x under two rotary embeddings, e.g. q -> (q1, q2) and k -> (k1, k2) of
    piecewise_attention.

    x: (batch, heads, length, head_dim) fp16 / bf16.  cos_e, sin_e: fp32 (num_positions, head_dim / 2).
    positions: None (token l sits at position l) or integers of shape (length,) or (batch, length);
    values outside the tables are clamped.  interleaved: pairs are (2i, 2i + 1) instead of
    (i, i + head_dim / 2).  Differentiable with respect to x."""
    return RotaryPair.apply(x, cos1, sin1, cos2, sin2, positions, interleaved)
