"""PyTorch references under the reference's module names (src/flag_attn/testing/__init__.py:1-4):
`flag_attn.testing.flash_attention`, `.piecewise_attention`, `.paged_attention`,
`.recompute_mask`, and the submodules `flash`, `piecewise`, `paged`, `dropout`, each with the
function under the name the reference gives it there."""
from flagattention_b200.testing import (flash_attention, paged_attention,  # noqa: F401
                                        piecewise_attention, recompute_mask, rotary_pair)

from . import dropout, flash, paged, piecewise  # noqa: F401,E402
