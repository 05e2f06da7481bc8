"""B200-native implementation of the FlagAttention operators.

Drop-in for the `flag_attn` package: `import flagattention_b200 as flag_attn`.
Everything computes in hand-written sm_100a CUDA kernels behind the C ABI of
libflagattn_b200.so; importing the package does not need a GPU, calling an
operator does.
"""
__version__ = "0.1.0"

from .piecewise import attention as piecewise_attention  # noqa: F401
from .flash import attention as flash_attention  # noqa: F401
from .split_kv import attention as flash_attention_split_kv  # noqa: F401
from .paged import attention as paged_attention  # noqa: F401
from .paged import reshape_and_cache  # noqa: F401  (writer of the paged caches; no reference counterpart)
from .rotary import rotary_pair, rotary_tables  # noqa: F401  (producer of piecewise_attention's operands)
from . import dist  # noqa: F401  (shard helpers, ring attention over a process group)
from . import testing  # noqa: F401
