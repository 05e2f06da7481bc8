"""TEST INFRASTRUCTURE ONLY: CPU statement of the two-embedding rotary step.

Parity unpinned against the reference: FlagAttention has no code for this step, only the prose
of README.md:136-138; the formula below is the standard rotary embedding, and
tests/test_oracle_golden.py checks it against the `transformers` package's llama implementation
when that package is importable.  Plain fp32 torch expressions on the CPU: every product and
sum is rounded on its own, which is what the CUDA kernel reproduces bit for bit.
"""
import torch


def _split(x, interleaved):
    if interleaved:
        return x[..., 0::2], x[..., 1::2]
    half = x.shape[-1] // 2
    return x[..., :half], x[..., half:]


def _join(lo, hi, interleaved):
    if interleaved:
        return torch.stack((lo, hi), dim=-1).flatten(-2)
    return torch.cat((lo, hi), dim=-1)


def _rows(table, positions, L, half):
    """(B or 1, 1, L, D/2) table rows of every token, positions clamped into the table."""
    if positions is None:
        positions = torch.arange(L)
    positions = positions.to(torch.int64).cpu()
    if positions.dim() == 1:
        positions = positions[None]
    positions = positions.clamp(0, table.shape[0] - 1)
    return table.float().cpu()[positions][:, None, :, :half]


def rotary(x, cos, sin, positions=None, interleaved=False):
    """x (B, H, L, D) of any float dtype -> the rotated tensor in x's dtype."""
    half = x.shape[-1] // 2
    lo, hi = _split(x.float().cpu(), interleaved)
    c, s = _rows(cos, positions, x.shape[2], half), _rows(sin, positions, x.shape[2], half)
    return _join(lo * c - hi * s, hi * c + lo * s, interleaved).to(x.dtype)


def rotary_pair(x, cos1, sin1, cos2, sin2, positions=None, interleaved=False):
    return (rotary(x, cos1, sin1, positions, interleaved),
            rotary(x, cos2, sin2, positions, interleaved))


def rotary_pair_backward(g1, g2, cos1, sin1, cos2, sin2, positions=None, interleaved=False):
    """dx = R1^T g1 + R2^T g2, one rounding to the 16-bit type at the end."""
    half = g1.shape[-1] // 2
    L = g1.shape[2]
    lo1, hi1 = _split(g1.float().cpu(), interleaved)
    lo2, hi2 = _split(g2.float().cpu(), interleaved)
    c1, s1 = _rows(cos1, positions, L, half), _rows(sin1, positions, L, half)
    c2, s2 = _rows(cos2, positions, L, half), _rows(sin2, positions, L, half)
    lo = (lo1 * c1 + hi1 * s1) + (lo2 * c2 + hi2 * s2)
    hi = (hi1 * c1 - lo1 * s1) + (hi2 * c2 - lo2 * s2)
    return _join(lo, hi, interleaved).to(g1.dtype)
