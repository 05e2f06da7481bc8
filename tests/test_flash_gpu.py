"""GPU parity of flash_attention against the oracle, over the reference's own shape matrix
(tests/flag_attn/test_flash_attention.py there) and the golden fixtures."""
import ctypes
import os

import pytest
import torch

import flagattention_b200 as fa
import oracle
from flagattention_b200 import _C
from flagattention_b200 import flash as fl
from helpers import GOLDEN, assert_within_2x, make_qkv, max_diff

pytestmark = pytest.mark.gpu

FWD_SHAPES = [
    (2, 4, 4, 512, 612, 128), (2, 4, 4, 1024, 1034, 64), (2, 4, 4, 2048, 2048, 32),
    (2, 4, 4, 4096, 4096, 16), (2, 4, 4, 4001, 4001, 32), (2, 4, 4, 4001, 4096, 64),
    (2, 4, 4, 4096, 4000, 128), (1, 2, 2, 8192, 8202, 16), (1, 2, 2, 8192, 8192, 32),
    (2, 4, 2, 512, 612, 128), (2, 4, 1, 1024, 1034, 64), (2, 4, 2, 2048, 2048, 32),
    (2, 4, 1, 4096, 4096, 16), (2, 4, 2, 4001, 4001, 32), (2, 4, 1, 4001, 4096, 64),
    (2, 4, 2, 4096, 4000, 128), (1, 2, 1, 8192, 8202, 16), (1, 2, 1, 8192, 8192, 32),
]
BWD_EXTRA = [(2, 4, 4, 10006, 10, 128), (2, 4, 2, 10006, 10, 128)]
SPLIT_SHAPES = [
    (2, 4, 4, 1, 612, 128), (2, 4, 4, 1, 1034, 64), (2, 4, 4, 1, 2048, 32), (2, 4, 4, 1, 4096, 16),
    (2, 4, 4, 1, 4001, 32), (2, 4, 4, 1, 4096, 64), (2, 4, 4, 2, 4000, 128), (1, 2, 2, 4, 8202, 16),
    (1, 2, 2, 1, 8192, 32), (2, 4, 2, 1, 612, 128), (2, 4, 1, 1, 1034, 64), (2, 4, 2, 1, 2048, 32),
    (2, 4, 1, 1, 4096, 16), (2, 4, 2, 1, 4001, 32), (2, 4, 1, 1, 4096, 64), (2, 4, 2, 2, 4000, 128),
    (1, 2, 1, 4, 8202, 16), (1, 2, 1, 1, 8192, 32),
]


def _case_params(shapes):
    out = []
    for i, shp in enumerate(shapes):
        for causal in (True, False):
            for dtype in (torch.float16, torch.bfloat16):
                layout = "BHTD" if (i + int(causal) + (dtype == torch.float16)) % 2 else "BTHD"
                std = 1.0 + (i + 2 * int(causal)) % 4
                out.append(pytest.param(*shp, causal, dtype, layout, std,
                                        id=f"{'x'.join(map(str, shp))}-{'c' if causal else 'f'}-"
                                           f"{str(dtype)[6:]}-{layout}-s{std:g}"))
    return out


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,layout,std", _case_params(FWD_SHAPES))
def test_forward(B, Hq, Hk, M, N, D, causal, dtype, layout, std):
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", std, layout, seed=M + N + D)
    o_ref = oracle.flash_attention(q, k, v, causal, upcast=True)
    o_torch = oracle.flash_attention(q, k, v, causal, upcast=False)
    o_hyp = fa.flash_attention(q, k, v, causal)
    assert o_hyp.shape == q.shape and o_hyp.dtype == dtype
    assert_within_2x(o_hyp, o_ref, o_torch, "o")


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,layout,std", _case_params(SPLIT_SHAPES))
def test_forward_split_kv_dispatch(B, Hq, Hk, M, N, D, causal, dtype, layout, std):
    """Decode-shaped M makes flash_attention take the split-KV path (std 10 as in the reference)."""
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 10.0, layout, seed=M + N + D)
    from flagattention_b200 import split_kv
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert split_kv.num_splits_herustic(B, Hq, M, N, 16, 128, sms, 128) > 1
    o_ref, l_ref, _ = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True, upcast=True)
    o_torch, l_torch, _ = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True, upcast=False)
    o_hyp, l_hyp, *_ = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)
    assert_within_2x(o_hyp, o_ref, o_torch, "o")
    assert_within_2x(l_hyp, l_ref, l_torch, "log_normalizer")
    o2 = fa.flash_attention_split_kv(q, k, v, causal)
    assert_within_2x(o2, o_ref, o_torch, "o (standalone split-kv)")


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,layout,std",
                         _case_params([s for s in FWD_SHAPES if s[4] != 4000] +
                                      [(2, 4, 4, 4096, 4001, 128), (2, 4, 2, 4096, 4001, 128)] + BWD_EXTRA))
def test_backward(B, Hq, Hk, M, N, D, causal, dtype, layout, std):
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", std, layout, seed=M + N + D + 1)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o_ref = oracle.flash_attention(q, k, v, causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_torch = oracle.flash_attention(q, k, v, causal, upcast=False)
    g_torch = torch.autograd.grad(o_torch, (q, k, v), do)
    del o_ref, o_torch
    o_hyp = fa.flash_attention(q, k, v, causal)
    g_hyp = torch.autograd.grad(o_hyp, (q, k, v), do)
    for name, h, r, t in zip(("dq", "dk", "dv"), g_hyp, g_ref, g_torch):
        assert h.shape == r.shape and h.dtype == dtype
        assert_within_2x(h, r, t, name)


@pytest.mark.parametrize("B,H,M,N,D", [s[:2] + s[3:] for s in FWD_SHAPES[:6]] +
                         [(2, 4, 4096, 4001, 128), (1, 2, 8192, 8202, 16), (1, 2, 8192, 8192, 32)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_aux_outputs(B, H, M, N, D, dtype, causal):
    layout = "BTHD" if (M + D) % 3 == 0 else "BHTD"
    q, k, v, _ = make_qkv(B, H, H, M, N, D, dtype, "cuda", 1.0 + D % 3, layout, seed=D)
    ref = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                 return_total_attention=True, upcast=True)
    tor = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                 return_total_attention=True, upcast=False)
    hyp = fa.flash_attention(q, k, v, causal, return_log_normalizer=True, return_total_attention=True)
    assert len(hyp) == 5 and hyp[3] is None and hyp[4] is None
    for name, h, r, t in zip(("o", "log_normalizer", "total_attention"), hyp[:3], ref, tor):
        assert_within_2x(h, r, t, name)
    only_l = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)
    assert only_l[2] is None and torch.equal(only_l[1], hyp[1])


def test_total_attention_gqa_and_standalone():
    from flagattention_b200.total import total_attention
    q, k, v, _ = make_qkv(2, 4, 2, 300, 333, 64, torch.bfloat16, "cuda", 1.0, "BHTD", seed=5)
    ref = oracle.flash_attention(q, k, v, True, return_log_normalizer=True,
                                 return_total_attention=True, upcast=True)
    tor = oracle.flash_attention(q, k, v, True, return_log_normalizer=True,
                                 return_total_attention=True, upcast=False)
    o, L, tot, *_ = fa.flash_attention(q, k, v, True, return_log_normalizer=True,
                                       return_total_attention=True)
    assert tot.shape == (2, 4, 333)
    assert_within_2x(tot, ref[2], tor[2], "total_attention")
    tot2 = total_attention(q, k, L, causal=True)
    assert torch.equal(tot, tot2)


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal", [(2, 4, 2, 700, 900, 128, True), (1, 6, 6, 1300, 1300, 64, True),
                                                  (2, 4, 1, 513, 257, 128, False), (1, 2, 2, 100, 1030, 64, True),
                                                  (1, 2, 2, 1030, 100, 128, True), (1, 3, 3, 4224, 4224, 128, True)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_total_attention_on_both_kernel_families(B, Hq, Hk, M, N, D, causal, dtype):
    """total_attention at head_dim 64 / 128 runs on a tcgen05 kernel (S^T tiles in TMEM, column sums
    in the element-wise warps); the shape-generic kernel serves the other head sizes.  Both are held
    to the oracle here: ragged sizes, GQA, M > N (rows without keys), N > M (keys past every query
    under the causal mask), BTHD strides, and a length with many query tiles per key block."""
    layout = "BTHD" if (M + N) % 2 else "BHTD"
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 1.0, layout, seed=M + N)
    ref = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                 return_total_attention=True, upcast=True)
    tor = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                 return_total_attention=True, upcast=False)
    got = {}
    for family in ("auto", "generic"):
        with _C.kernel_family(family):
            _, L, tot, *_ = fa.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                               return_total_attention=True)
        assert tot.shape == (B, Hq, N) and tot.dtype == torch.float32
        assert_within_2x(tot, ref[2], tor[2], f"total_attention ({family})")
        got[family] = tot
    assert max_diff(got["auto"], got["generic"]) <= 1e-3 * max(1.0, ref[2].abs().max().item())


def test_empty_rows_give_zero_output_and_neg_inf_lse():
    q, k, v, do = make_qkv(1, 2, 2, 100, 10, 64, torch.float16, "cuda", seed=3)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o, L, *_ = fa.flash_attention(q, k, v, True, return_log_normalizer=True)
    assert torch.all(o[:, :, :90] == 0)
    assert torch.all(torch.isinf(L[:, :, :90]) & (L[:, :, :90] < 0))
    assert torch.isfinite(L[:, :, 90:]).all()
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    assert torch.all(dq[:, :, :90] == 0)
    assert torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()


def _three_runs(mode):
    q, k, v, do = make_qkv(2, 4, 2, 777, 901, 128, torch.bfloat16, "cuda", seed=11)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    outs = []
    for use_side in (False, False, True):
        stream = torch.cuda.Stream() if use_side else torch.cuda.current_stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), fl.backward_mode(mode):
            o = fa.flash_attention(q, k, v, True)
            g = torch.autograd.grad(o, (q, k, v), do)
        stream.synchronize()
        outs.append((o, *g))
    return outs


def test_deterministic_and_stream_safe():
    """Two runs, and a run on a side stream, give the same bits for o, dk, dv.  dq of the one-pass
    backward is a sum of fp32 reductions in arbitrary order: equal to within a 16-bit rounding step."""
    outs = _three_runs("one_pass")
    for other in outs[1:]:
        for i, (a, b) in enumerate(zip(outs[0], other)):
            if i == 1:   # dq
                assert (a.float() - b.float()).abs().max().item() <= 2 ** -7 * a.float().abs().max().item()
            else:
                assert torch.equal(a, b)


def test_two_kernel_backward_is_bitwise_deterministic():
    """The dK/dV + dQ kernel pair uses no atomics: every output is bitwise reproducible."""
    outs = _three_runs("two_kernel")
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


def test_torch_determinism_switch_selects_the_atomics_free_backward():
    """Under torch.use_deterministic_algorithms(True) the default ("auto") backward is the
    dK/dV + dQ pair: the same bits as the explicit "two_kernel" mode, run after run."""
    q, k, v, do = make_qkv(1, 4, 2, 600, 600, 128, torch.bfloat16, "cuda", seed=21)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = fa.flash_attention(q, k, v, True)
    with fl.backward_mode("two_kernel"):
        want = torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    before = torch.are_deterministic_algorithms_enabled()
    try:
        torch.use_deterministic_algorithms(True)
        for _ in range(2):
            got = torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
            for a, b in zip(got, want):
                assert torch.equal(a, b)
    finally:
        torch.use_deterministic_algorithms(before)


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal", [(1, 4, 4, 1024, 1024, 128, True), (2, 4, 2, 500, 700, 64, True),
                                                  (1, 2, 2, 333, 1111, 128, False), (1, 2, 1, 1500, 300, 64, True)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_one_pass_backward_matches_two_kernel_backward(B, Hq, Hk, M, N, D, causal, dtype):
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", seed=5 + M)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = fa.flash_attention(q, k, v, causal)
    with fl.backward_mode("one_pass"):
        g1 = torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    with fl.backward_mode("two_kernel"):
        g2 = torch.autograd.grad(o, (q, k, v), do)
    for a, b in zip(g1, g2):
        scale = b.float().abs().max().item()
        assert (a.float() - b.float()).abs().max().item() <= 2 ** -6 * scale + 1e-6


def test_golden_fixtures_on_gpu():
    """Kernel vs the stored outputs of the reference's fp32 oracle (tests/golden/flash.pt)."""
    cases = torch.load(os.path.join(GOLDEN, "flash.pt"))["cases"]
    for c in cases:
        q, k, v = (c[n].cuda().requires_grad_() for n in ("q", "k", "v"))
        do = c["do"].cuda()
        o, L, tot, *_ = fa.flash_attention(q, k, v, c["causal"], return_log_normalizer=True,
                                           return_total_attention=True)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
        ref, tor = c["ref"], c["torch"]
        for name, h in (("o", o), ("lse", L), ("tot", tot), ("dq", dq), ("dk", dk), ("dv", dv)):
            assert_within_2x(h.cpu(), ref[name], tor[name], name)


def test_cfg1_shape_fp16_against_fp32_golden():
    """The CPU benchmark configuration run through the kernels in 16-bit: same inputs (rounded),
    compared with the stored fp32 results at 16-bit resolution."""
    c = torch.load(os.path.join(GOLDEN, "flash.pt"))["cfg1"]
    gen = torch.Generator().manual_seed(c["seed"])
    q, k, v, do = (torch.randn(c["shape"], generator=gen, dtype=torch.float32) for _ in range(4))
    qh, kh, vh, doh = (t.half().cuda() for t in (q, k, v, do))
    qh.requires_grad_(), kh.requires_grad_(), vh.requires_grad_()
    o, L, tot, *_ = fa.flash_attention(qh, kh, vh, True, sm_scale=c["sm_scale"],
                                       return_log_normalizer=True, return_total_attention=True)
    dq, dk, dv = torch.autograd.grad(o, (qh, kh, vh), doh)
    assert max_diff(L.cpu(), c["lse"]) < 2e-2
    assert max_diff(tot.cpu(), c["tot"]) < 2e-2
    h = c["head"]
    for got, name in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_diff(got[h].cpu(), c[name]) < 3e-2, name


@pytest.mark.parametrize("B,Hq,Hk,M,N,D", [(2, 4, 2, 512, 612, 128), (2, 4, 1, 1024, 1034, 64),
                                           (2, 4, 4, 4001, 4096, 64), (2, 4, 2, 4096, 4001, 128),
                                           (2, 4, 2, 10006, 10, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_generic_kernels_at_tensor_core_head_dims(B, Hq, Hk, M, N, D, causal):
    """head_dim 64/128 normally run on the tcgen05 kernels; the kernel-family switch routes them to
    the shape-generic kernels, which must meet the same bar (and agree with the tcgen05 ones)."""
    dtype = torch.bfloat16 if causal else torch.float16
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 1.0, "BHTD", seed=M + D)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o_ref, l_ref, _ = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_tor, l_tor, _ = oracle.flash_attention(q, k, v, causal, return_log_normalizer=True, upcast=False)
    g_tor = torch.autograd.grad(o_tor, (q, k, v), do)
    results = {}
    for mode in ("1", "0"):
        with _C.kernel_family("generic" if mode == "1" else "auto"):
            o, L, *_ = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)
            g = torch.autograd.grad(o, (q, k, v), do)
        assert_within_2x(o, o_ref, o_tor, f"o generic={mode}")
        assert_within_2x(L, l_ref, l_tor, f"lse generic={mode}")
        for name, h, r, t in zip(("dq", "dk", "dv"), g, g_ref, g_tor):
            assert_within_2x(h, r, t, f"{name} generic={mode}")
        results[mode] = (o, L, *g)
    for a, b_ in zip(results["0"], results["1"]):
        fin = torch.isfinite(a.float())
        assert max_diff(a[fin], b_[fin]) <= 4 * 2 ** -8 * max(1.0, a[fin].float().abs().max().item())


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("how", ["heads", "batch", "both"])
@pytest.mark.parametrize("mode", ["one_pass", "two_kernel"])
def test_broadcast_strides_of_k_and_v(D, how, mode):
    """K and V given as broadcast views (stride 0 on a dimension longer than one: one KV head
    expanded over the query heads, a prefix shared by the batch).  A tensor map cannot express
    that, so these calls must leave the tcgen05 path and still give the oracle's result, forward
    and backward (the gradient of an expanded view sums over the broadcast dimension)."""
    B, H, M, N = 2, 4, 200, 264
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(5 + D)
    q = torch.randn((B, H, M, D), generator=gen).to(dtype).cuda().requires_grad_()
    do = torch.randn((B, H, M, D), generator=gen).to(dtype).cuda()
    base_shape = {"heads": (B, 1, N, D), "batch": (1, H, N, D), "both": (1, 1, N, D)}[how]
    kb = torch.randn(base_shape, generator=gen).to(dtype).cuda().requires_grad_()
    vb = torch.randn(base_shape, generator=gen).to(dtype).cuda().requires_grad_()
    k, v = kb.expand(B, H, N, D), vb.expand(B, H, N, D)
    assert 0 in k.stride()
    with fl.backward_mode(mode):
        o, L, *_ = fa.flash_attention(q, k, v, True, return_log_normalizer=True)
        g = torch.autograd.grad(o, (q, kb, vb), do)
    o_ref, l_ref, _ = oracle.flash_attention(q, k, v, True, return_log_normalizer=True, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, kb, vb), do)
    o_tor, l_tor, _ = oracle.flash_attention(q, k, v, True, return_log_normalizer=True, upcast=False)
    g_tor = torch.autograd.grad(o_tor, (q, kb, vb), do)
    assert_within_2x(o, o_ref, o_tor, "o")
    assert_within_2x(L, l_ref, l_tor, "lse")
    for name, h, r, t in zip(("dq", "dk", "dv"), g, g_ref, g_tor):
        assert_within_2x(h, r, t, name)
    # and the same numbers as with K and V materialised (which do run on tcgen05)
    o2 = fa.flash_attention(q, k.contiguous(), v.contiguous(), True)
    assert max_diff(o, o2) <= 4 * 2 ** -8 * max(1.0, o2.float().abs().max().item())


def test_a_wait_that_runs_out_poisons_the_status_word_and_the_context_survives():
    """Every wait in the tensor-core kernels has a time limit.  fa_debug_wait_probe makes one run
    out on purpose (an mbarrier nobody arrives at, limit about a millisecond): the kernel must
    return normally, leave its code in the device status word, later tensor-core launches must do
    nothing until the word is cleared, and after clearing everything works again."""
    import ctypes
    lib = _C.load()
    out = ctypes.c_int32(-1)
    assert lib.fa_device_status(ctypes.byref(out), 1) == 0 and out.value == 0
    q, k, v, _ = make_qkv(1, 2, 2, 256, 256, 128, torch.bfloat16, "cuda", seed=31)
    o_good = fa.flash_attention(q, k, v, True)
    left = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        st = lib.fa_debug_wait_probe(2_000_000, ctypes.c_void_p(left.data_ptr()),
                                     _C.stream_ptr(q.device))
        assert st == 0
        torch.cuda.synchronize()                      # the kernel came back by itself
        assert left.item() == 1                       # ... because the wait was abandoned
        assert lib.fa_device_status(ctypes.byref(out), 0) == 0 and out.value == 990
        # a poisoned word: the forward kernel returns at once and leaves its output untouched
        shape = _C.flash_shape(q.dtype, 1, 2, 2, 256, 256, 128, True, 128 ** -0.5)
        o = torch.full_like(q, 7.0)
        lse = torch.full((1, 2, 256), 7.0, device="cuda")
        ts = [_C.tensor4(x) for x in (q, k, v, o)]
        st = lib.fa_flash_fwd(_C.byref(shape), *[_C.byref(t) for t in ts], _C.fptr(lse),
                              _C.stream_ptr(q.device))
        assert st == 0
        torch.cuda.synchronize()
        assert torch.all(o == 7.0) and torch.all(lse == 7.0)
    finally:
        assert lib.fa_device_status(ctypes.byref(out), 1) == 0
    assert lib.fa_device_status(ctypes.byref(out), 0) == 0 and out.value == 0
    assert torch.equal(fa.flash_attention(q, k, v, True), o_good)


@pytest.mark.parametrize("B,Hq,Hk,M,N,D", [(2, 8, 8, 2, 4096, 128), (1, 8, 2, 4, 2048, 64), (2, 4, 4, 16, 8192, 128),
                                            (1, 16, 2, 8, 1040 * 16, 128), (1, 4, 4, 3, 4112, 32), (3, 2, 1, 5, 1024, 64)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_few_queries_per_head_through_the_gather_kernel(B, Hq, Hk, M, N, D, causal, dtype):
    """Inference calls with a handful of queries per head (2 .. 16: speculative decoding, chunked
    prefill tails), where the reference splits the keys (src/flag_attn/flash.py:59-61), run on the
    paged-decode kernel with K and V in place: the M queries of a head ride as M rows of its kv
    head's query tile, each with its own causal limit.  Checked against the oracle, and the
    dispatch itself is checked (the call must not have gone to the tile kernels)."""
    from flagattention_b200 import flash as fl_mod
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 1.0, "BHTD", seed=M + N)
    taken = []
    real = fl_mod._decode_forward

    def spy(*args, **kw):
        taken.append(True)
        return real(*args, **kw)
    fl_mod._decode_forward = spy
    try:
        with torch.no_grad():
            o = fa.flash_attention(q, k, v, causal)
    finally:
        fl_mod._decode_forward = real
    assert taken, "expected the decode path"
    o_ref = oracle.flash_attention(q, k, v, causal, upcast=True)
    o_tor = oracle.flash_attention(q, k, v, causal, upcast=False)
    assert_within_2x(o, o_ref, o_tor, "o")
    # the tile kernels (what a call that needs gradients or the log-normaliser gets) agree
    o2, _lse, *_ = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)
    assert max_diff(o, o2) <= 4 * 2 ** -8 * max(1.0, o2.float().abs().max().item())


def test_device_status_word_is_clean():
    """Every wait in the tcgen05 kernels is bounded; none of them may have run out in this process."""
    import ctypes
    from flagattention_b200 import _C
    out = ctypes.c_int32(-1)
    assert _C.load().fa_device_status(ctypes.byref(out), 0) == 0
    assert out.value == 0


@pytest.mark.parametrize("B,Hq,Hk,N,D", [(2, 16, 16, 4096, 128), (1, 8, 2, 1040, 64), (3, 4, 1, 16, 32),
                                         (2, 32, 32, 65536, 64), (1, 4, 4, 8208, 16)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("layout", ["BHTD", "BTHD"])
def test_single_query_forward_streams_kv_in_place(B, Hq, Hk, N, D, dtype, layout):
    """M == 1 without gradients or extra outputs runs on the paged-decode kernels, K and V read in
    place through an identity block table (reference dispatch: src/flag_attn/flash.py:59-61 sends
    these shapes to split-KV)."""
    q, k, v, _ = make_qkv(B, Hq, Hk, 1, N, D, dtype, "cuda", 1.0, layout, seed=N + D)
    from flagattention_b200 import flash as fl
    assert fl._decode_covered(q, k, v)
    o = fa.flash_attention(q, k, v, causal=True)
    o_ref = oracle.flash_attention(q, k, v, True, upcast=True)
    o_tor = oracle.flash_attention(q, k, v, True, upcast=False)
    assert_within_2x(o, o_ref, o_tor, "o")
    # the same call with an extra output takes the split-KV kernels: both paths agree
    o2, lse, *_ = fa.flash_attention(q, k, v, causal=True, return_log_normalizer=True)
    assert_within_2x(o2, o_ref, o_tor, "o (split-KV)")


def test_single_query_forward_fallbacks():
    """Ragged N, mismatched K/V strides or a gradient request keep the split-KV / tile kernels."""
    from flagattention_b200 import flash as fl
    q, k, v, _ = make_qkv(2, 4, 4, 1, 1000, 64, torch.float16, "cuda", seed=3)
    assert not fl._decode_covered(q, k, v)          # 1000 % 16 != 0
    o = fa.flash_attention(q, k, v)
    assert_within_2x(o, oracle.flash_attention(q, k, v, False, upcast=True),
                     oracle.flash_attention(q, k, v, False, upcast=False), "o")
    q, k, v, do = make_qkv(2, 4, 4, 1, 1024, 64, torch.float16, "cuda", seed=4)
    assert not fl._decode_covered(q, k, v.transpose(1, 2).contiguous().transpose(1, 2))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = fa.flash_attention(q, k, v)
    g = torch.autograd.grad(o, (q, k, v), do)
    o_ref = oracle.flash_attention(q, k, v, False, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_tor = oracle.flash_attention(q, k, v, False, upcast=False)
    g_tor = torch.autograd.grad(o_tor, (q, k, v), do)
    for name, h, r, t in zip(("dq", "dk", "dv"), g, g_ref, g_tor):
        assert_within_2x(h, r, t, name)


@pytest.mark.parametrize("generic", ["1", "0"])
def test_rows_without_visible_keys_are_exact_zeros_every_time(generic):
    """M > N causal: CTAs whose rows see no key run no main-loop iteration.  Their output rows must
    be exact zeros (lse = -inf) on every run, whatever the freed memory they reuse holds (the
    shape-generic forward once let a late asynchronous copy of Q land in its staged output)."""
    B, Hq, Hk, M, N, D = 2, 4, 2, 10006, 10, 128
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, torch.bfloat16, "cuda", 1.0, "BHTD", seed=M + D)
    for rep in range(12):
        junk = torch.full((48 << 20,), float("nan") if rep % 2 else 3.0, device="cuda", dtype=torch.bfloat16)
        del junk
        with _C.kernel_family("generic" if generic == "1" else "auto"):
            o, L, *_ = fa.flash_attention(q, k, v, True, return_log_normalizer=True)
        assert torch.count_nonzero(o[:, :, :M - N]).item() == 0
        assert torch.isinf(L[:, :, :M - N]).all() and (L[:, :, :M - N] < 0).all()
        assert torch.isfinite(o).all() and torch.isfinite(L[:, :, M - N:]).all()


@pytest.mark.parametrize("B,Hq,Hk,M,N,D", [(1, 33, 33, 300, 300, 64),      # 33 pairs: groups of 32 + 1
                                           (3, 22, 11, 260, 390, 128),     # 33 kv pairs, 66 query pairs
                                           (1, 3, 3, 12288, 12288, 128)])  # backward: groups of 2 + 1
@pytest.mark.parametrize("causal", [True, False])
def test_ragged_last_group_of_the_launch_order(B, Hq, Hk, M, N, D, causal):
    """The tensor-core kernels number their CTAs over groups of (batch, head) pairs; the last group
    may hold fewer pairs than the others.  Checked head by head (the long case would not fit the
    oracle's score matrices otherwise), forward and both backward paths."""
    dtype = torch.bfloat16
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 1.0, "BHTD", seed=B + Hq + M)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = fa.flash_attention(q, k, v, causal)
    with fl.backward_mode("one_pass"):
        grads = torch.autograd.grad(o, (q, k, v), do)
    o2 = fa.flash_attention(q, k, v, causal)
    with fl.backward_mode("two_kernel"):
        grads2 = torch.autograd.grad(o2, (q, k, v), do)
    G = Hq // Hk
    for b in range(B):
        for hk in range(Hk):
            hs = slice(hk * G, (hk + 1) * G)
            qs, ks, vs = (t.detach()[b:b + 1, s].clone().requires_grad_()
                          for t, s in ((q, hs), (k, slice(hk, hk + 1)), (v, slice(hk, hk + 1))))
            dos = do[b:b + 1, hs]
            o_ref = oracle.flash_attention(qs, ks, vs, causal, upcast=True)
            g_ref = torch.autograd.grad(o_ref, (qs, ks, vs), dos)
            o_t = oracle.flash_attention(qs, ks, vs, causal, upcast=False)
            g_t = torch.autograd.grad(o_t, (qs, ks, vs), dos)
            assert_within_2x(o[b:b + 1, hs], o_ref, o_t, f"o[{b},{hk}]")
            for name, g, g2, r, t, s in zip(("dq", "dk", "dv"), grads, grads2, g_ref, g_t,
                                            (hs, slice(hk, hk + 1), slice(hk, hk + 1))):
                assert_within_2x(g[b:b + 1, s], r, t, f"{name}[{b},{hk}]")
                assert_within_2x(g2[b:b + 1, s], r, t, f"{name}[{b},{hk}] (two kernels)")
            del o_ref, g_ref, o_t, g_t


def test_ring_attention_of_one_rank_is_flash_attention(tmp_path):
    """The context-parallel forward with its default operator (this package's flash_attention), on a
    process group of one rank: no exchange, the same result as the direct call."""
    import torch.distributed as dist
    from flagattention_b200 import dist as fdist
    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/pg", rank=0, world_size=1)
    try:
        q, k, v, _ = make_qkv(2, 4, 2, 300, 300, 64, torch.float16, "cuda", seed=77)
        for causal in (True, False):
            o, lse = fdist.ring_flash_attention(q, k, v, causal)
            o_ref, lse_ref, *_ = fa.flash_attention(q, k, v, causal=causal, return_log_normalizer=True)
            assert torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
        # and its backward is the operator's backward (dq of the one-pass kernel: fp32 rounding only)
        q, k, v, do = make_qkv(1, 4, 2, 260, 260, 128, torch.bfloat16, "cuda", seed=78)
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        o, _ = fdist.ring_flash_attention(q, k, v, True)
        g = torch.autograd.grad(o, (q, k, v), do)
        g_ref = torch.autograd.grad(fa.flash_attention(q, k, v, causal=True), (q, k, v), do)
        assert torch.equal(g[1], g_ref[1]) and torch.equal(g[2], g_ref[2])
        assert max_diff(g[0], g_ref[0]) <= 2 ** -7 * g_ref[0].float().abs().max().item()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H,Hk,M,N,D,causal,dtype", [
    (4, 32, 32, 4096, 4096, 128, True, torch.bfloat16),     # the benchmark shape
    (64, 16, 16, 512, 512, 128, True, torch.bfloat16),      # many short query tiles
    (8, 16, 4, 1000, 1300, 64, True, torch.float16),        # ragged, GQA, M < N
    (8, 16, 16, 1300, 1000, 128, True, torch.float16),      # M > N: the first query rows see no key
    (6, 12, 12, 777, 901, 128, False, torch.bfloat16),
])
def test_persistent_forward_equals_one_cta_per_tile(B, H, Hk, M, N, D, causal, dtype):
    """With more query tiles than two per SM the forward runs as a persistent kernel (two CTAs per
    SM working through the tiles); it computes every tile exactly as the one-CTA-per-tile kernel
    does, so o and the log-normaliser must agree bit for bit, call after call and whatever earlier
    launches left in the library's table of work-item counters."""
    gen = torch.Generator().manual_seed(M * 7 + N)
    q = torch.randn((B, H, M, D), generator=gen).to(dtype).cuda()
    k, v = (torch.randn((B, Hk, N, D), generator=gen).to(dtype).cuda() for _ in range(2))
    with _C.kernel_family("one_cta_per_tile"):
        o_ref, lse_ref = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)[:2]
    for _ in range(3):
        # the outputs come from torch.empty: seed the allocator's cache with NaN blocks of their
        # sizes, so that a tile the kernel skipped cannot hide behind an earlier call's result
        junk = [torch.full((B, H, M, D), float("nan"), dtype=dtype, device="cuda"),
                torch.full((B, H, M), float("nan"), dtype=torch.float32, device="cuda")]
        del junk
        o, lse = fa.flash_attention(q, k, v, causal, return_log_normalizer=True)[:2]
        assert torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
    out = ctypes.c_int32(-1)
    assert _C.load().fa_device_status(ctypes.byref(out), 0) == 0 and out.value == 0
