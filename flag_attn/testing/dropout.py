from flagattention_b200.dropout import recompute_mask  # noqa: F401
