from flagattention_b200.testing import piecewise_attention as attention  # noqa: F401
