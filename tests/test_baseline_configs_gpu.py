"""Parity at the full sizes of the benchmark configurations (flash bf16 L=4096 D=128 causal; flash fp16
L=8192 D=64 non-causal with log-normaliser; piecewise bf16 L=16384 D=128 w=4096; paged decode with 64
sequences up to 32768 tokens).  The oracle materialises the score matrix, so it is evaluated on a few
(batch, head) slices of the same inputs; every slice must meet the usual 2x rule."""
import pytest
import torch

import flagattention_b200 as fa
import oracle
from helpers import assert_within_2x, max_diff

pytestmark = pytest.mark.gpu


def _randn(gen, shape, dtype, scale=1.0):
    return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _check_flash_slices(q, k, v, do, causal, outs, grads, slices, lse=None):
    for (b, h) in slices:
        qs, ks, vs = (t[b:b + 1, h:h + 1].detach().clone().requires_grad_() for t in (q, k, v))
        ref = oracle.flash_attention(qs, ks, vs, causal, return_log_normalizer=True, upcast=True)
        g_ref = torch.autograd.grad(ref[0], (qs, ks, vs), do[b:b + 1, h:h + 1])
        tor = oracle.flash_attention(qs, ks, vs, causal, return_log_normalizer=True, upcast=False)
        g_tor = torch.autograd.grad(tor[0], (qs, ks, vs), do[b:b + 1, h:h + 1])
        assert_within_2x(outs[b:b + 1, h:h + 1], ref[0], tor[0], f"o[{b},{h}]")
        if lse is not None:
            assert_within_2x(lse[b:b + 1, h:h + 1], ref[1], tor[1], f"lse[{b},{h}]")
        for name, g, r, t in zip(("dq", "dk", "dv"), grads, g_ref, g_tor):
            assert_within_2x(g[b:b + 1, h:h + 1], r, t, f"{name}[{b},{h}]")


def test_config2_flash_bf16_hd128_causal_full_size():
    gen = torch.Generator(device="cuda").manual_seed(10086 + 2)
    B, H, L, D = 4, 32, 4096, 128
    q, k, v, do = (_randn(gen, (B, H, L, D), torch.bfloat16) for _ in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = fa.flash_attention(q, k, v, causal=True)
    grads = torch.autograd.grad(o, (q, k, v), do)
    _check_flash_slices(q, k, v, do, True, o, grads, [(0, 0), (1, 13), (3, 31)])
    # the whole tensor is finite and a second run is bitwise identical for o, dk, dv; dq of the
    # one-pass backward sums fp32 reductions in arbitrary order: equal to a 16-bit rounding step
    o2 = fa.flash_attention(q, k, v, causal=True)
    g2 = torch.autograd.grad(o2, (q, k, v), do)
    assert torch.equal(o, o2) and torch.equal(grads[1], g2[1]) and torch.equal(grads[2], g2[2])
    dq_gap = (grads[0].float() - g2[0].float()).abs().max().item()
    assert dq_gap <= 2 ** -7 * grads[0].float().abs().max().item()
    assert all(torch.isfinite(t.float()).all() for t in (o, *grads))


def test_config3_flash_fp16_hd64_noncausal_with_log_normalizer_full_size():
    gen = torch.Generator(device="cuda").manual_seed(10086 + 3)
    B, H, L, D = 2, 16, 8192, 64
    q, k, v = (_randn(gen, (B, H, L, D), torch.float16, 0.5) for _ in range(3))
    do = _randn(gen, (B, H, L, D), torch.float16)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o, lse, *_ = fa.flash_attention(q, k, v, causal=False, return_log_normalizer=True)
    grads = torch.autograd.grad(o, (q, k, v), do)
    _check_flash_slices(q, k, v, do, False, o, grads, [(0, 0), (1, 15)], lse=lse)
    assert all(torch.isfinite(t.float()).all() for t in (o, lse, *grads))


def test_config4_piecewise_bf16_aquila_shape_full_length():
    gen = torch.Generator(device="cuda").manual_seed(10086 + 4)
    B, H, L, D, w = 1, 48, 16384, 128, 4096
    q1, k1, q2, k2, v, do = (_randn(gen, (B, H, L, D), torch.bfloat16) for _ in range(6))
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]
    o = fa.piecewise_attention(*ins, w, causal=True)
    grads = torch.autograd.grad(o, ins, do)
    for h in (0, 47):
        sl = [t[:, h:h + 1].detach().clone().requires_grad_() for t in ins]
        o_ref = oracle.piecewise_attention(*sl, w, True, upcast=True)
        g_ref = torch.autograd.grad(o_ref, sl, do[:, h:h + 1])
        o_ref = o_ref.detach()
        o_tor = oracle.piecewise_attention(*sl, w, True, upcast=False)
        g_tor = torch.autograd.grad(o_tor, sl, do[:, h:h + 1])
        assert_within_2x(o[:, h:h + 1], o_ref, o_tor.detach(), f"o[{h}]")
        for name, g, r, t in zip(("dq1", "dk1", "dq2", "dk2", "dv"), grads, g_ref, g_tor):
            assert_within_2x(g[:, h:h + 1], r, t, f"{name}[{h}]")
        del sl, o_ref, g_ref, o_tor, g_tor
        torch.cuda.empty_cache()


def test_config5_paged_decode_full_size():
    gen = torch.Generator().manual_seed(10086 + 5)
    S, Hq, Hk, D, BS = 64, 32, 8, 128, 16
    lens = torch.randint(1024, 32769, (S,), generator=gen, dtype=torch.int32)
    lens[0] = 32768
    blocks = (lens.long() + BS - 1) // BS
    nb = int(blocks.sum())
    perm = torch.randperm(nb, generator=gen)
    bt = torch.zeros((S, 2048), dtype=torch.int32)
    off = 0
    for i, n in enumerate(blocks.tolist()):
        bt[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    dgen = torch.Generator(device="cuda").manual_seed(7)
    kc = torch.randn((nb, Hk, BS, D), generator=dgen, device="cuda", dtype=torch.float16)
    vc = torch.randn((nb, Hk, BS, D), generator=dgen, device="cuda", dtype=torch.float16)
    q = torch.randn((S, Hq, D), generator=gen).half().cuda()
    lens_d, scale = lens.cuda(), D ** -0.5
    ref = oracle.paged_attention_gathered(q, kc, vc, bt.cuda(), lens_d, scale)
    for tables in (bt.cuda(), bt.long().cuda()):                    # int32 and int64 block tables
        for num_splits in (64, 0, 1):                              # 512-token partitions, automatic, one pass
            out = fa.paged_attention(q, kc, vc, lens_d, tables, scale, 32768, num_splits)
            assert torch.allclose(out, ref, atol=2e-3, rtol=1e-5), (num_splits, max_diff(out, ref))
