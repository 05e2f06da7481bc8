from flagattention_b200.testing import flash_attention as attention  # noqa: F401
