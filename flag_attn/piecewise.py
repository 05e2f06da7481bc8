"""Alias: this module is `flagattention_b200.piecewise` itself."""
import sys

from flagattention_b200 import piecewise as _impl

sys.modules[__name__] = _impl
