"""Alias: this module is `flagattention_b200.total` itself."""
import sys

from flagattention_b200 import total as _impl

sys.modules[__name__] = _impl
