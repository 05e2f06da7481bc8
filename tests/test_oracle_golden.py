"""Pins oracle/ (and the package's own torch references) against outputs of the
reference's PyTorch oracles, stored under tests/golden/ by make_golden.py. CPU only."""
import os

import pytest
import torch

import oracle
from flagattention_b200 import testing as pkg_testing
from helpers import GOLDEN, max_diff


def _tol(dtype_tag):
    # fp32 path: reduction-order noise only.  Same-precision path: the 16-bit matmul results may
    # differ in the last bit between batched and per-call evaluation.
    return 2e-5 if dtype_tag == "ref" else 2e-2


FLASH = torch.load(os.path.join(GOLDEN, "flash.pt"))
PIECE = torch.load(os.path.join(GOLDEN, "piecewise.pt"))
PAGED = torch.load(os.path.join(GOLDEN, "paged.pt"))


@pytest.mark.parametrize("impl", [oracle.flash_attention, pkg_testing.flash_attention])
@pytest.mark.parametrize("idx", range(len(FLASH["cases"])))
def test_flash_oracle_matches_reference(idx, impl):
    c = FLASH["cases"][idx]
    for tag, upcast in (("ref", True), ("torch", False)):
        q, k, v = (c[n].clone().requires_grad_() for n in ("q", "k", "v"))
        o, lse, tot = impl(q, k, v, c["causal"], return_log_normalizer=True,
                           return_total_attention=True, upcast=upcast)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), c["do"])
        g = c[tag]
        scale = max(1.0, g["o"].float().abs().max().item())
        assert max_diff(o, g["o"]) <= _tol(tag) * scale
        assert torch.equal(torch.isinf(lse), torch.isinf(g["lse"]))
        fin = ~torch.isinf(g["lse"])
        assert max_diff(lse[fin], g["lse"][fin]) <= _tol(tag) * 4
        assert max_diff(tot, g["tot"]) <= _tol(tag) * max(1.0, g["tot"].abs().max().item())
        for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
            gs = max(1.0, g[name].float().abs().max().item())
            assert max_diff(got, g[name]) <= _tol(tag) * gs, name


def test_flash_oracle_cfg1():
    """The CPU benchmark configuration (fp32, B=2, H=4, L=256, D=64, causal)."""
    c = FLASH["cfg1"]
    gen = torch.Generator().manual_seed(c["seed"])
    q, k, v, do = (torch.randn(c["shape"], generator=gen, dtype=torch.float32) for _ in range(4))
    chk = float(q.double().sum() + k.double().sum() + v.double().sum() + do.double().sum())
    assert abs(chk - c["input_checksum"]) < 1e-6, "torch RNG stream differs from the fixture's"
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    o, lse, tot = oracle.flash_attention(q, k, v, True, sm_scale=c["sm_scale"],
                                         return_log_normalizer=True, return_total_attention=True,
                                         upcast=True)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    assert max_diff(lse, c["lse"]) < 1e-5
    assert max_diff(tot, c["tot"]) < 1e-5
    h = c["head"]
    for got, name in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert max_diff(got[h], c[name]) < 2e-5, name


@pytest.mark.parametrize("impl", [oracle.piecewise_attention, pkg_testing.piecewise_attention])
@pytest.mark.parametrize("idx", range(len(PIECE["cases"])))
def test_piecewise_oracle_matches_reference(idx, impl):
    c = PIECE["cases"][idx]
    for tag, upcast in (("ref", True), ("torch", False)):
        ins = [c[n].clone().requires_grad_() for n in ("q1", "k1", "q2", "k2", "v")]
        o = impl(*ins, c["w"], c["causal"], upcast=upcast)
        grads = torch.autograd.grad(o, ins, c["do"])
        g = c[tag]
        assert max_diff(o, g["o"]) <= _tol(tag) * max(1.0, g["o"].float().abs().max().item())
        for got, want in zip(grads, g["grads"]):
            assert max_diff(got, want) <= _tol(tag) * max(1.0, want.float().abs().max().item())


@pytest.mark.parametrize("idx", range(len(PIECE["cases"])))
def test_piecewise_closed_form_grad(idx):
    c = PIECE["cases"][idx]
    D = c["q1"].shape[-1]
    got = oracle.piecewise_attention_grad(c["q1"], c["k1"], c["q2"], c["k2"], c["v"], c["w"],
                                          c["causal"], D ** -0.5, c["ref"]["o"], c["do"], upcast=True)
    for a, b in zip(got, c["closed_form"]):
        assert max_diff(a, b) <= 2e-5 * max(1.0, b.float().abs().max().item())
    # and the closed form agrees with autograd through the forward, as the reference checks
    # (src/flag_attn/testing/piecewise.py:80-101 there, atol 1e-2).  The closed form does not
    # re-mask P, so it only holds when every query row sees a key (M <= N).
    if c["q1"].shape[-2] > c["k1"].shape[-2]:
        return
    for a, b in zip(got, c["ref"]["grads"]):
        assert max_diff(a, b) <= 1e-2 * max(1.0, b.float().abs().max().item())


@pytest.mark.parametrize("impl", [oracle.paged_attention, oracle.paged_attention_gathered,
                                  pkg_testing.paged_attention])
@pytest.mark.parametrize("idx", range(len(PAGED["cases"])))
def test_paged_oracle_matches_reference(idx, impl):
    c = PAGED["cases"][idx]
    o = impl(c["q"], c["key_cache"], c["value_cache"], c["block_tables"], c["context_lens"], c["scale"])
    assert o.dtype == c["out"].dtype
    assert max_diff(o, c["out"]) <= 1e-6 + 2 ** -11 * c["out"].float().abs().max().item()


@pytest.mark.parametrize("idx", range(len(PAGED["cases"])))
def test_paged_same_precision_path_against_reference(idx):
    """The same-precision PyTorch path of paged decode (the flash oracle with upcast=False on
    gathered keys / values): on fp32 copies of a fixture it IS the fp32 computation, so it must
    reproduce the reference's stored output; in the cache dtype it stays within 16-bit rounding."""
    c = PAGED["cases"][idx]
    args32 = (c["q"].float(), c["key_cache"].float(), c["value_cache"].float(), c["block_tables"],
              c["context_lens"], c["scale"])
    o32 = oracle.paged_attention_same_precision(*args32)
    scale = c["out"].float().abs().max().item()
    assert max_diff(o32, c["out"]) <= 1e-6 + 2 ** -11 * scale
    unrounded = oracle.paged_attention_gathered(*args32, out_dtype=torch.float32)
    assert unrounded.dtype == torch.float32 and max_diff(unrounded, o32) <= 1e-6
    if c["q"].dtype == torch.bfloat16 or torch.cuda.is_available():
        return   # fp16 matmuls on CPU are not available in every torch build
    try:
        o16 = oracle.paged_attention_same_precision(c["q"], c["key_cache"], c["value_cache"],
                                                    c["block_tables"], c["context_lens"], c["scale"])
    except RuntimeError:
        return
    assert max_diff(o16, c["out"]) <= 2 ** -7 * scale + 1e-4


# ---- dropout random stream: oracle/dropout.py against the reference's mask kernel ----------------
def _philox_golden():
    return torch.load(os.path.join(GOLDEN, "philox.pt"))


def test_philox_uniform_matches_triton_rand():
    import numpy as np
    from oracle.dropout import philox_uniform
    for r in _philox_golden()["rands"]:
        ctr = np.arange(r["values"].numel(), dtype=np.uint64) + np.uint64(r["offset"])
        assert np.array_equal(philox_uniform(r["seed"], ctr), r["values"].numpy())   # bit-exact


def test_dropout_mask_matches_reference_kernel():
    import numpy as np
    from oracle.dropout import dropout_mask
    for c in _philox_golden()["masks"]:
        mine = dropout_mask(c["B"], c["H"], c["M"], c["N"], c["p"], c["seed"], c["offset"])
        assert np.array_equal(mine, c["mask"].numpy())


def test_rotary_oracle_matches_the_transformers_package():
    """The reference has no code for the rotary step that produces piecewise_attention's operands, so
    the oracle's formula is held to an independent implementation instead: llama's
    apply_rotary_pos_emb of the `transformers` package (half-split pairs), when importable."""
    llama = pytest.importorskip("transformers.models.llama.modeling_llama")
    import flagattention_b200 as fa
    gen = torch.Generator().manual_seed(11)
    q = torch.randn((2, 3, 40, 64), generator=gen)
    k = torch.randn((2, 3, 40, 64), generator=gen)
    cos, sin = fa.rotary_tables(100, 64)
    pos = torch.randint(0, 100, (2, 40), generator=gen)
    qe, ke = llama.apply_rotary_pos_emb(q, k, torch.cat((cos, cos), -1)[pos], torch.cat((sin, sin), -1)[pos])
    assert torch.equal(oracle.rotary(q, cos, sin, pos), qe)
    assert torch.equal(oracle.rotary(k, cos, sin, pos), ke)
    # the interleaved layout is the same rotation on a permuted head dimension
    perm = torch.stack((torch.arange(32), torch.arange(32) + 32), -1).flatten()
    assert torch.equal(oracle.rotary(q[..., perm], cos, sin, pos, interleaved=True), qe[..., perm])
    # the backward is the transpose: <R x, g> == <x, R^T g>
    g = torch.randn((2, 3, 40, 64), generator=gen)
    dx = oracle.rotary_pair_backward(g, g, cos, sin, cos, sin, pos)
    lhs = (oracle.rotary(q, cos, sin, pos) * g).sum() * 2
    assert abs(lhs.item() - (q * dx).sum().item()) < 1e-2
