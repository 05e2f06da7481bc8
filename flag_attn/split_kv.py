"""Alias: this module is `flagattention_b200.split_kv` itself."""
import sys

from flagattention_b200 import split_kv as _impl

sys.modules[__name__] = _impl
