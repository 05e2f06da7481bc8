"""Dropout of flash_attention on the GPU (the reference's tests/flag_attn/test_flash_attention.py:225-320
and tests/flag_attn/test_dropout.py there): the keep-mask is regenerated from the returned (seed, offset)
and handed to the oracle."""
import pytest
import torch

import flagattention_b200 as fa
import oracle
from helpers import assert_within_2x, make_qkv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Hq,Hk,M,N,D", [(2, 4, 4, 512, 612, 128), (2, 4, 2, 1024, 1034, 64),
                                           (2, 4, 4, 2048, 2048, 32), (1, 2, 1, 1000, 1300, 16),
                                           (2, 4, 4, 4096, 4001, 128)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dropout_p", [0.5, 0.8])
def test_dropout_forward_backward(B, Hq, Hk, M, N, D, causal, dtype, dropout_p):
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, "cuda", 1.0, "BHTD", seed=M + N + D)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o, _, _, seed, offset = fa.flash_attention(q, k, v, causal, dropout_p=dropout_p, return_seed_offset=True)
    g = torch.autograd.grad(o, (q, k, v), do)
    mask = fa.testing.recompute_mask(B, Hq, M, N, dropout_p, seed, offset, "cuda")
    o_ref = oracle.flash_attention(q, k, v, causal, dropout_p=dropout_p, dropout_mask=mask, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_tor = oracle.flash_attention(q, k, v, causal, dropout_p=dropout_p, dropout_mask=mask, upcast=False)
    g_tor = torch.autograd.grad(o_tor, (q, k, v), do)
    assert_within_2x(o, o_ref, o_tor, "o")
    for name, h, r, t in zip(("dq", "dk", "dv"), g, g_ref, g_tor):
        assert_within_2x(h, r, t, name)


@pytest.mark.parametrize("dropout_p", [0.1, 0.5, 0.8])
def test_mask_statistics_and_generator_advance(dropout_p):
    B, H, M, N = 2, 4, 1000, 1100
    q, k, v, _ = make_qkv(B, H, H, M, N, 64, torch.float16, "cuda", seed=1)
    _, _, _, s1, o1 = fa.flash_attention(q, k, v, dropout_p=dropout_p, return_seed_offset=True)
    _, _, _, s2, o2 = fa.flash_attention(q, k, v, dropout_p=dropout_p, return_seed_offset=True)
    assert s1 == s2 and o2 - o1 == (B * H * M * N + 3) // 4 * 4      # counters never overlap
    m1 = fa.testing.recompute_mask(B, H, M, N, dropout_p, s1, o1, "cuda")
    m2 = fa.testing.recompute_mask(B, H, M, N, dropout_p, s2, o2, "cuda")
    dropped = 1.0 - m1.float().mean().item()
    assert abs(dropped - dropout_p) <= 0.01 * dropout_p + 1e-3
    assert not torch.equal(m1, m2)
    # neighbouring elements are uncorrelated
    a, b = m1[..., :-1].float(), m1[..., 1:].float()
    corr = ((a - a.mean()) * (b - b.mean())).mean() / (a.std() * b.std())
    assert abs(corr.item()) < 5e-3


def test_no_dropout_returns_none_seed_offset():
    q, k, v, _ = make_qkv(1, 2, 2, 300, 300, 64, torch.bfloat16, "cuda", seed=2)
    out = fa.flash_attention(q, k, v, return_seed_offset=True)
    assert len(out) == 5 and out[3] is None and out[4] is None


@pytest.mark.parametrize("B,H,M,N,p,seed,offset", [
    (1, 2, 5, 37, 0.5, 0, 0), (2, 3, 70, 400, 0.2, 12345, 8),
    (1, 1, 3, 1100, 0.8, 2 ** 40 + 17, 2 ** 32 - 64), (1, 2, 64, 160, 0.1, 2 ** 63 + 5, 10 ** 12)])
def test_mask_is_bit_exact_with_oracle(B, H, M, N, p, seed, offset):
    """The device Philox stream equals the CPU restatement, which the golden fixture pins to the
    reference's mask kernel."""
    from oracle.dropout import dropout_mask
    got = fa.testing.recompute_mask(B, H, M, N, p, seed, offset, "cuda").cpu()
    want = torch.from_numpy(dropout_mask(B, H, M, N, p, seed, offset))
    assert torch.equal(got, want)


def test_mask_matches_golden_fixture():
    import os
    from helpers import GOLDEN
    for c in torch.load(os.path.join(GOLDEN, "philox.pt"))["masks"]:
        got = fa.testing.recompute_mask(c["B"], c["H"], c["M"], c["N"], c["p"], c["seed"],
                                        c["offset"], "cuda").cpu()
        assert torch.equal(got, c["mask"])


def test_kernel_mask_equals_recomputed_mask():
    """With v = identity-like rows and one key per query block, the forward output exposes which
    weights were dropped: out[m] = sum_n keep[m, n] * p[m, n] * v[n] / (1 - p)."""
    B, H, M, N, D, p = 1, 2, 64, 64, 64, 0.5
    q = torch.zeros(B, H, M, D, device="cuda", dtype=torch.float16)
    k = torch.zeros(B, H, N, D, device="cuda", dtype=torch.float16)
    v = torch.eye(N, D, device="cuda", dtype=torch.float16).expand(B, H, N, D).contiguous()
    o, _, _, seed, offset = fa.flash_attention(q, k, v, dropout_p=p, return_seed_offset=True)
    mask = fa.testing.recompute_mask(B, H, M, N, p, seed, offset, "cuda")
    # uniform weights 1/N, so out[m, n] = keep[m, n] / (N * (1 - p))
    assert torch.equal(o > 0.5 / (N * (1 - p)), mask)
