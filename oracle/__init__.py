"""CPU/torch restatement of the reference's attention math.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py, and only as the checker or as the
timed CPU baseline.

Each function restates one of the reference's PyTorch oracles
(src/flag_attn/testing/{flash,piecewise,paged}.py of FlagOpen/FlagAttention)
and is pinned against outputs of those very functions: tests/golden/*.pt
holds input seeds and outputs produced by importing the reference
(tests/golden/make_golden.py), and tests/test_oracle_golden.py compares.
"""
from .flash import flash_attention  # noqa: F401
from .piecewise import piecewise_attention, piecewise_attention_grad  # noqa: F401
from .paged import (paged_attention, paged_attention_gathered,  # noqa: F401
                    paged_attention_same_precision, cache_append)  # noqa: F401
from .dropout import dropout_mask, philox_uniform  # noqa: F401
from .rotary import rotary, rotary_pair, rotary_pair_backward  # noqa: F401
