"""Shared pieces of the parity tests."""
import os

import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def max_diff(a, b):
    return (a.float() - b.float()).abs().max().item()


def assert_within_2x(hyp, ref, same_precision, what=""):
    """The reference's tolerance rule (tests/flag_attn/test_flash_attention.py:61-65 there):
    the kernel's max error against the fp32 oracle may be at most twice the error of the
    same-precision PyTorch path, plus 1e-5."""
    assert torch.isfinite(hyp.float()).all() or not torch.isfinite(ref.float()).all(), \
        f"{what}: non-finite values in kernel output"
    # -inf entries (log-normaliser of rows that see no key) must match exactly
    inf_ref = torch.isinf(ref.float())
    if inf_ref.any():
        assert torch.equal(torch.isinf(hyp.float()), inf_ref), f"{what}: -inf pattern differs"
        hyp = torch.where(inf_ref, torch.zeros_like(hyp), hyp)
        same_precision = torch.where(inf_ref, torch.zeros_like(same_precision), same_precision)
        ref = torch.where(inf_ref, torch.zeros_like(ref), ref)
    e_hyp = max_diff(hyp, ref)
    e_torch = max_diff(same_precision, ref)
    assert e_hyp <= 2 * e_torch + 1e-5, f"{what}: kernel err {e_hyp:.3e} > 2 * torch err {e_torch:.3e}"
    return e_hyp, e_torch


def make_qkv(B, Hq, Hk, M, N, D, dtype, device, std=1.0, layout="BHTD", seed=0):
    """Seeded inputs generated on the CPU in fp32, cast, then moved (same bits on any box)."""
    gen = torch.Generator().manual_seed(seed)

    def mk(h, l):
        if layout == "BHTD":
            t = (torch.randn((B, h, l, D), generator=gen) * std).to(dtype).to(device)
            return t
        t = (torch.randn((B, l, h, D), generator=gen) * std).to(dtype).to(device)
        return t.transpose(1, 2)

    return mk(Hq, M), mk(Hk, N), mk(Hk, N), mk(Hq, M)
