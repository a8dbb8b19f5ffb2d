"""inference/attention.py of the reference's GPU package."""
from polarquant_kv.inference.reference_layers import CompressedMultiHeadAttention  # noqa: F401
