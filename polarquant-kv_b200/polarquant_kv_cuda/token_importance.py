"""token_importance.py of the reference's GPU package (the plan and its accounting; a cache that follows a plan is
polarquant_kv.policy.mixed_precision_compress / mixed_precision_attention, whose arguments differ from the
reference's dict-returning function)."""
from polarquant_kv.policy import compute_token_bitwidths, estimate_mixed_compression_ratio  # noqa: F401
