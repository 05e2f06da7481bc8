from flagattention_b200.testing import paged_attention as attention  # noqa: F401
