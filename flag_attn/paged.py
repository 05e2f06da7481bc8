"""Alias: this module is `flagattention_b200.paged` itself."""
import sys

from flagattention_b200 import paged as _impl

sys.modules[__name__] = _impl
