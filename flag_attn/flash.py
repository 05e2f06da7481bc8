"""Alias: this module is `flagattention_b200.flash` itself."""
import sys

from flagattention_b200 import flash as _impl

sys.modules[__name__] = _impl
