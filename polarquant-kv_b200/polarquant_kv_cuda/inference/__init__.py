"""inference/ of the reference's GPU package."""
from polarquant_kv.inference import (CompressedMultiHeadAttention, KVCacheManager, PolarQuantConfig,  # noqa: F401
                                     SimpleTransformer, SimpleTransformerLayer)
