"""piecewise_attention: host side of the B200 kernels.

Mirrors src/flag_attn/piecewise.py:25-191: score(m, n) = q2.k2 when the
bottom-right-aligned distance (m + N - M) - n is at least `dist_threshold`,
else q1.k1; returns the output only; gradients for the five tensors.
"""
import ctypes
import math

import torch

from . import _C
from .flash import use_one_pass_backward

__all__ = ["attention"]


class PiecewiseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q1, k1, q2, k2, v, w, causal, sm_scale):
        Dq1, Dk1, Dq2, Dk2, Dv = q1.shape[-1], k1.shape[-1], q2.shape[-1], k2.shape[-1], v.shape[-1]
        assert Dq1 == Dk1 == Dq2 == Dk2 == Dv
        assert Dk1 in {16, 32, 64, 128}
        assert q1.shape == q2.shape and k1.shape == k2.shape == v.shape
        assert q1.shape[1] == k1.shape[1], "piecewise attention has no grouped-query mode"
        assert q1.is_cuda, "inputs must be CUDA tensors"
        assert all(x.device == q1.device for x in (k1, q2, k2, v)), "inputs must share a device"
        assert q1.dtype == k1.dtype == q2.dtype == k2.dtype == v.dtype

        B, H, M, D = q1.shape
        N = k1.shape[2]
        if sm_scale is None:
            sm_scale = 1. / math.sqrt(D)
        q1, k1, q2, k2, v = (_C.kernel_ready(x) for x in (q1, k1, q2, k2, v))
        lib = _C.load()

        with torch.cuda.device(q1.device):
            o = torch.empty(q1.shape, dtype=q1.dtype, device=q1.device)
            L = torch.empty((B, H, M), device=q1.device, dtype=torch.float32)
            shape = _C.flash_shape(q1.dtype, B, H, H, M, N, D, causal, sm_scale)
            ts = [_C.tensor4(x) for x in (q1, k1, q2, k2, v, o)]
            st = lib.fa_piecewise_fwd(_C.byref(shape), int(w), *[_C.byref(t) for t in ts],
                                      _C.fptr(L), _C.stream_ptr(q1.device))
            _C.check(st, "fa_piecewise_fwd")

        ctx.save_for_backward(q1, k1, q2, k2, v, o, L)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.w = int(w)
        return o

    @staticmethod
    def backward(ctx, do):
        q1, k1, q2, k2, v, o, L = ctx.saved_tensors
        w, causal, sm_scale = ctx.w, ctx.causal, ctx.sm_scale
        B, H, M, D = q1.shape
        N = k1.shape[2]
        lib = _C.load()
        do = _C.kernel_ready(do)

        with torch.cuda.device(q1.device):
            stream = _C.stream_ptr(q1.device)
            shape = _C.flash_shape(q1.dtype, B, H, H, M, N, D, causal, sm_scale)
            delta = torch.empty_like(L)
            to, tdo = _C.tensor4(o), _C.tensor4(do)
            st = lib.fa_flash_bwd_delta(_C.byref(shape), _C.byref(to), _C.byref(tdo),
                                        _C.fptr(delta), stream)
            _C.check(st, "fa_flash_bwd_delta")

            ins = [_C.tensor4(x) for x in (q1, k1, q2, k2, v)]
            dk1 = torch.empty(k1.shape, dtype=k1.dtype, device=k1.device)
            dk2 = torch.empty(k2.shape, dtype=k2.dtype, device=k2.device)
            dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
            ws_bytes = (lib.fa_piecewise_bwd_fused_workspace_bytes(_C.byref(shape))
                        if use_one_pass_backward() else 0)
            if ws_bytes > 0:
                # one launch: every key block walks its near tiles, then its far tiles; dq1 / dq2
                # accumulate in two fp32 workspaces, dV in TMEM across both walks
                dq1 = torch.empty(q1.shape, dtype=q1.dtype, device=q1.device)
                dq2 = torch.empty(q2.shape, dtype=q2.dtype, device=q2.device)
                ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q1.device)
                outs = [_C.tensor4(x) for x in (dq1, dq2, dk1, dk2, dv)]
                st = lib.fa_piecewise_bwd_fused(_C.byref(shape), w, *[_C.byref(t) for t in ins],
                                                _C.byref(tdo), _C.fptr(L), _C.fptr(delta),
                                                *[_C.byref(t) for t in outs], _C.fptr(ws),
                                                ctypes.c_int64(ws_bytes), stream)
                # a layout the one-pass kernel cannot map (a broadcast stride) goes to the pair below
                if st != _C.FA_ERR_UNSUPPORTED:
                    _C.check(st, "fa_piecewise_bwd_fused")
                    return dq1, dk1, dq2, dk2, dv, None, None, None
            outs = [_C.tensor4(x) for x in (dk1, dk2, dv)]
            st = lib.fa_piecewise_bwd_dkdv(_C.byref(shape), w, *[_C.byref(t) for t in ins],
                                           _C.byref(tdo), _C.fptr(L), _C.fptr(delta),
                                           *[_C.byref(t) for t in outs], stream)
            _C.check(st, "fa_piecewise_bwd_dkdv")

            dq1 = torch.empty(q1.shape, dtype=q1.dtype, device=q1.device)
            dq2 = torch.empty(q2.shape, dtype=q2.dtype, device=q2.device)
            outs = [_C.tensor4(x) for x in (dq1, dq2)]
            st = lib.fa_piecewise_bwd_dq(_C.byref(shape), w, *[_C.byref(t) for t in ins],
                                         _C.byref(tdo), _C.fptr(L), _C.fptr(delta),
                                         *[_C.byref(t) for t in outs], stream)
            _C.check(st, "fa_piecewise_bwd_dq")
        return dq1, dk1, dq2, dk2, dv, None, None, None


def attention(q1, k1, q2, k2, v, dist_threshold, causal=False, sm_scale=None):
    """Piecewise attention (for NLPE): the attention score of (q_i, k_j) is
    q1_i.k1_j when their distance is below `dist_threshold` and q2_i.k2_j
    otherwise.  All tensors are (batch, heads, seqlen, headdim); returns the
    output, shaped like q1."""
    return PiecewiseAttention.apply(q1, k1, q2, k2, v, dist_threshold, causal, sm_scale)
