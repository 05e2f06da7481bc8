"""Two rotary embeddings in one pass (flagattention_b200.rotary_pair): bit-exact against the CPU
statement in oracle/rotary.py, forward and backward, and end to end as the producer of
piecewise_attention's operands."""
import pytest
import torch

import flagattention_b200 as fa
import oracle
from flagattention_b200 import testing

pytestmark = pytest.mark.gpu


def _tables(rows, D, gen):
    """Two unrelated position schemes: plain angles and angles of compressed positions."""
    c1, s1 = fa.rotary_tables(rows, D)
    c2, s2 = fa.rotary_tables(rows, D, base=50000.0, position_scale=0.25)
    return c1, s1, c2, s2


@pytest.mark.parametrize("B,H,L,D", [(1, 1, 1, 16), (2, 3, 77, 64), (1, 5, 300, 128), (2, 2, 129, 48),
                                     (1, 2, 33, 256), (3, 1, 1000, 32), (1, 48, 64, 128), (1, 1, 40, 512)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_forward_and_backward_are_bit_exact(B, H, L, D, dtype, interleaved):
    gen = torch.Generator().manual_seed(B * 1000 + L + D)
    x = torch.randn((B, H, L, D), generator=gen).to(dtype)
    g1 = torch.randn((B, H, L, D), generator=gen).to(dtype)
    g2 = torch.randn((B, H, L, D), generator=gen).to(dtype)
    tabs = _tables(L + 5, D, gen)
    ref1, ref2 = oracle.rotary_pair(x, *tabs, None, interleaved)
    ref_dx = oracle.rotary_pair_backward(g1, g2, *tabs, None, interleaved)
    xd = x.cuda().requires_grad_()
    dev_tabs = [t.cuda() for t in tabs]
    o1, o2 = fa.rotary_pair(xd, *dev_tabs, interleaved=interleaved)
    (dx,) = torch.autograd.grad((o1, o2), (xd,), (g1.cuda(), g2.cuda()))
    assert torch.equal(o1.cpu(), ref1) and torch.equal(o2.cpu(), ref2)
    assert torch.equal(dx.cpu(), ref_dx)


@pytest.mark.parametrize("per_batch", [False, True])
def test_positions_are_looked_up_and_clamped(per_batch):
    gen = torch.Generator().manual_seed(3)
    B, H, L, D, rows = 2, 4, 150, 64, 97
    x = torch.randn((B, H, L, D), generator=gen).to(torch.bfloat16)
    tabs = _tables(rows, D, gen)
    shape = (B, L) if per_batch else (L,)
    pos = torch.randint(-4, rows + 4, shape, generator=gen)         # some fall outside the tables
    ref1, ref2 = oracle.rotary_pair(x, *tabs, pos, False)
    for p in (pos, pos.to(torch.int32)):
        o1, o2 = fa.rotary_pair(x.cuda(), *[t.cuda() for t in tabs], positions=p.cuda())
        assert torch.equal(o1.cpu(), ref1) and torch.equal(o2.cpu(), ref2)
    g = torch.randn((B, H, L, D), generator=gen).to(torch.bfloat16)
    xd = x.cuda().requires_grad_()
    o1, o2 = fa.rotary_pair(xd, *[t.cuda() for t in tabs], positions=pos.cuda())
    (dx,) = torch.autograd.grad((o1, o2), (xd,), (g.cuda(), g.cuda()))
    assert torch.equal(dx.cpu(), oracle.rotary_pair_backward(g, g, *tabs, pos, False))


def test_strided_input_and_padded_tables():
    """x as the (B, L, H, D) output of a projection viewed as (B, H, L, D); tables wider than D / 2
    (a table built once for the largest head) and tables with an odd row stride."""
    gen = torch.Generator().manual_seed(4)
    B, H, L, D = 2, 6, 90, 64
    x = torch.randn((B, L, H, D), generator=gen).to(torch.float16).cuda().permute(0, 2, 1, 3)
    wide = [t.cuda() for t in _tables(L, 128, gen)]                 # 64 columns, 32 used
    o1, o2 = fa.rotary_pair(x, *wide)
    ref1, ref2 = oracle.rotary_pair(x.cpu(), *[t.cpu() for t in wide])
    assert torch.equal(o1.cpu(), ref1) and torch.equal(o2.cpu(), ref2)
    odd = [torch.randn((L, 35), generator=gen).cuda()[:, :32] for _ in range(4)]   # row stride 35
    o1, o2 = fa.rotary_pair(x, *odd)
    ref1, ref2 = oracle.rotary_pair(x.cpu(), *[t.cpu() for t in odd])
    assert torch.equal(o1.cpu(), ref1) and torch.equal(o2.cpu(), ref2)
    empty = fa.rotary_pair(x[:, :, :0], *wide)
    assert empty[0].shape == (B, H, 0, D)


def test_matches_the_pytorch_reference_of_the_package():
    gen = torch.Generator().manual_seed(6)
    x = torch.randn((2, 4, 200, 128), generator=gen).to(torch.bfloat16).cuda()
    tabs = [t.cuda() for t in _tables(200, 128, gen)]
    for il in (False, True):
        o = fa.rotary_pair(x, *tabs, interleaved=il)
        r = testing.rotary_pair(x, *tabs, interleaved=il)
        assert torch.equal(o[0], r[0]) and torch.equal(o[1], r[1])


def test_feeds_piecewise_attention_end_to_end():
    """q, k -> (q1, q2), (k1, k2) -> piecewise_attention, gradients back to q and k: against the same
    chain of PyTorch references in fp32, by the reference's rule (kernel error at most twice the
    error of the same-precision PyTorch chain)."""
    gen = torch.Generator().manual_seed(7)
    B, H, L, D, w = 1, 4, 512, 128, 128
    dtype = torch.bfloat16
    q = torch.randn((B, H, L, D), generator=gen).to(dtype).cuda().requires_grad_()
    k = torch.randn((B, H, L, D), generator=gen).to(dtype).cuda().requires_grad_()
    v = torch.randn((B, H, L, D), generator=gen).to(dtype).cuda().requires_grad_()
    do = torch.randn((B, H, L, D), generator=gen).to(dtype).cuda()
    tabs = [t.cuda() for t in _tables(L, D, gen)]

    def chain(rot, attn, **kw):
        q1, q2 = rot(q, *tabs)
        k1, k2 = rot(k, *tabs)
        o = attn(q1, k1, q2, k2, v, w, causal=True, **kw)
        return (o,) + torch.autograd.grad(o, (q, k, v), do)

    hyp = chain(fa.rotary_pair, fa.piecewise_attention)

    def up(x, *t, **kw):
        a, b = testing.rotary_pair(x.float(), *t, **kw)
        return a, b
    ref = chain(up, lambda *a, **kw: testing.piecewise_attention(*a, upcast=True, **kw).to(dtype))
    low = chain(lambda x, *t: testing.rotary_pair(x, *t, upcast=False),
                lambda *a, **kw: testing.piecewise_attention(*a, upcast=False, **kw))
    for name, h, r, t in zip(("o", "dq", "dk", "dv"), hyp, ref, low):
        err_h = (h.float() - r.float()).abs().max().item()
        err_t = (t.float() - r.float()).abs().max().item()
        assert err_h <= 2 * err_t + 1e-5, (name, err_h, err_t)
