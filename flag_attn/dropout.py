"""Alias: this module is `flagattention_b200.dropout` itself."""
import sys

from flagattention_b200 import dropout as _impl

sys.modules[__name__] = _impl
