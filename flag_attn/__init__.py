"""`import flag_attn`: the FlagAttention package name, served by the B200 implementation.

Code written against FlagOpen/FlagAttention (`flag_attn.flash_attention`, `flag_attn.flash.*`,
`flag_attn.testing.*`: src/flag_attn/__init__.py:9-14, src/flag_attn/testing/__init__.py:1-4) runs
unchanged with this directory on the import path.  Every name here IS the object of the same name
in `flagattention_b200` (the submodules are the very same module objects, so overriding
`flag_attn.flash.get_fwd_config` reaches the one the operator reads).
"""
from flagattention_b200 import __version__  # noqa: F401
from flagattention_b200 import (flash_attention, flash_attention_split_kv,  # noqa: F401
                                paged_attention, piecewise_attention)

from . import dropout, flash, paged, piecewise, split_kv, total  # noqa: F401,E402
from . import testing  # noqa: F401,E402

version_tuple = tuple(int(x) for x in __version__.split("."))
