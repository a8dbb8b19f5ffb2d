"""adaptive_bitwidth.py of the reference's GPU package."""
from polarquant_kv.policy import compute_layer_bitwidths, estimate_adaptive_compression_ratio  # noqa: F401
