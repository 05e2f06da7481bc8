"""GPU parity of piecewise_attention against the oracle over the reference's shape matrix
(tests/flag_attn/test_piecewise_attention.py there) and the golden fixtures."""
import os

import pytest
import torch

import flagattention_b200 as fa
import oracle
from flagattention_b200 import _C
from helpers import GOLDEN, assert_within_2x

pytestmark = pytest.mark.gpu

SHAPES = [(2, 4, 512, 612, 128), (2, 4, 1024, 1034, 64), (2, 4, 2048, 2048, 32),
          (2, 4, 4096, 4096, 16), (2, 4, 4096, 4001, 16), (1, 2, 8192, 8192, 16),
          (1, 2, 8192, 8192, 32), (1, 2, 8192, 3867, 32), (1, 3, 700, 700, 128), (1, 2, 1500, 1300, 64)]


def _inputs(B, H, M, N, D, dtype, layout, std, seed):
    gen = torch.Generator().manual_seed(seed)

    def mk(l):
        if layout == "BHTD":
            return (torch.randn((B, H, l, D), generator=gen) * std).to(dtype).cuda()
        return (torch.randn((B, l, H, D), generator=gen) * std).to(dtype).cuda().transpose(1, 2)

    return mk(M), mk(N), mk(M), mk(N), mk(N), mk(M)   # q1 k1 q2 k2 v do


def _params():
    out = []
    for i, shp in enumerate(SHAPES):
        for causal in (True, False):
            for dtype in (torch.float16, torch.bfloat16):
                layout = "BHTD" if (i + int(causal) + (dtype == torch.float16)) % 2 else "BTHD"
                std = 1.0 + (i + int(causal)) % 4
                out.append(pytest.param(*shp, causal, dtype, layout, std,
                                        id=f"{'x'.join(map(str, shp))}-{'c' if causal else 'f'}-"
                                           f"{str(dtype)[6:]}-{layout}-s{std:g}"))
    return out


@pytest.mark.parametrize("B,H,M,N,D,causal,dtype,layout,std", _params())
def test_forward_backward(B, H, M, N, D, causal, dtype, layout, std):
    q1, k1, q2, k2, v, do = _inputs(B, H, M, N, D, dtype, layout, std, seed=M + N + D)
    w = (M // 2) if M < N else (M - N // 2)
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]
    o_ref = oracle.piecewise_attention(*ins, w, causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, ins, do)
    o_torch = oracle.piecewise_attention(*ins, w, causal, upcast=False)
    g_torch = torch.autograd.grad(o_torch, ins, do)
    o_hyp = fa.piecewise_attention(*ins, w, causal=causal)
    g_hyp = torch.autograd.grad(o_hyp, ins, do)
    assert_within_2x(o_hyp, o_ref, o_torch, "o")
    for name, h, r, t in zip(("dq1", "dk1", "dq2", "dk2", "dv"), g_hyp, g_ref, g_torch):
        assert h.shape == r.shape and h.dtype == dtype
        assert_within_2x(h, r, t, name)


@pytest.mark.parametrize("w", [-5, 0, 1, 63, 64, 65, 200, 10 ** 6])
def test_threshold_edges(w):
    """Thresholds on, next to and far outside the tile boundaries; with the causal mask, w <= 0 means every visible pair is far,
    a huge w means every pair is near (then the result equals flash_attention on q1, k1)."""
    q1, k1, q2, k2, v, do = _inputs(1, 2, 200, 264, 64, torch.bfloat16, "BHTD", 1.0, seed=w + 17)
    for causal in (True, False):
        o_ref = oracle.piecewise_attention(q1, k1, q2, k2, v, w, causal, upcast=True)
        o_torch = oracle.piecewise_attention(q1, k1, q2, k2, v, w, causal, upcast=False)
        o_hyp = fa.piecewise_attention(q1, k1, q2, k2, v, w, causal=causal)
        assert_within_2x(o_hyp, o_ref, o_torch, f"o w={w}")
        # degenerate thresholds reduce to flash_attention on one of the two branches
        if w == 10 ** 6:
            assert_within_2x(fa.flash_attention(q1, k1, v, causal), o_ref, o_torch, "flash(q1,k1)")
        if w <= -5 and causal:   # under the causal mask every visible pair has distance >= 0 > w
            assert_within_2x(fa.flash_attention(q2, k2, v, causal), o_ref, o_torch, "flash(q2,k2)")


def test_golden_fixtures_on_gpu():
    cases = torch.load(os.path.join(GOLDEN, "piecewise.pt"))["cases"]
    for c in cases:
        ins = [c[n].cuda().requires_grad_() for n in ("q1", "k1", "q2", "k2", "v")]
        o = fa.piecewise_attention(*ins, c["w"], causal=c["causal"])
        grads = torch.autograd.grad(o, ins, c["do"].cuda())
        assert_within_2x(o.cpu(), c["ref"]["o"], c["torch"]["o"], "o")
        for h, r, t in zip(grads, c["ref"]["grads"], c["torch"]["grads"]):
            assert_within_2x(h.cpu(), r, t, "grad")


@pytest.mark.parametrize("B,H,M,N,D", [(2, 4, 512, 612, 128), (2, 4, 1024, 1034, 64), (1, 3, 700, 700, 128),
                                       (1, 2, 1500, 1300, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_generic_kernels_at_tensor_core_head_dims(B, H, M, N, D, causal):
    """head_dim 64/128 normally run on the tcgen05 kernels; the kernel-family switch routes them to the
    shape-generic kernels, which must meet the same bar."""
    dtype = torch.bfloat16 if causal else torch.float16
    q1, k1, q2, k2, v, do = _inputs(B, H, M, N, D, dtype, "BHTD", 1.0, seed=M + D)
    w = (M // 2) if M < N else (M - N // 2)
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]
    o_ref = oracle.piecewise_attention(*ins, w, causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, ins, do)
    o_tor = oracle.piecewise_attention(*ins, w, causal, upcast=False)
    g_tor = torch.autograd.grad(o_tor, ins, do)
    for mode in ("1", "0"):
        with _C.kernel_family("generic" if mode == "1" else "auto"):
            o = fa.piecewise_attention(*ins, w, causal=causal)
            g = torch.autograd.grad(o, ins, do)
        assert_within_2x(o, o_ref, o_tor, f"o generic={mode}")
        for name, h, r, t in zip(("dq1", "dk1", "dq2", "dk2", "dv"), g, g_ref, g_tor):
            assert_within_2x(h, r, t, f"{name} generic={mode}")


def test_dv_of_the_one_pass_backward_is_rounded_once():
    """The one-pass backward walks every key block twice in one launch (near tiles, then far tiles)
    and keeps dV in fp32 across both walks, so dV sees one rounding to 16 bits; the two-kernel mode
    launches per branch and adds the far branch's dV to the near branch's 16-bit result.  Against
    the fp32 oracle the one-pass dV must therefore be at least as close on average."""
    from flagattention_b200 import flash as fl
    B, H, L, D, w = 1, 4, 1024, 128, 300
    q1, k1, q2, k2, v, do = _inputs(B, H, L, L, D, torch.bfloat16, "BHTD", 1.0, seed=77)
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]
    o_ref = oracle.piecewise_attention(*ins, w, True, upcast=True)
    dv_ref = torch.autograd.grad(o_ref, ins, do)[4].float()
    err = {}
    for mode in ("one_pass", "two_kernel"):
        with fl.backward_mode(mode):
            o = fa.piecewise_attention(*ins, w, causal=True)
            dv = torch.autograd.grad(o, ins, do)[4].float()
        err[mode] = (dv - dv_ref).abs().mean().item()
    assert err["one_pass"] <= err["two_kernel"] * 1.02, err
