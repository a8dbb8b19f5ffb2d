"""inference/transformer.py of the reference's GPU package."""
from polarquant_kv.inference.reference_layers import SimpleTransformer, SimpleTransformerLayer  # noqa: F401
