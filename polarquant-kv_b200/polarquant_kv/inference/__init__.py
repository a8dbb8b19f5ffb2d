"""Inference-side users of the compressed cache (the reference's src/polarquant_kv_cuda/inference/
package): configuration, the per-layer cache manager, and a decoder that attends through it."""

from .config import PolarQuantConfig
from .kv_cache import KVCacheManager
from .model import CompressedAttention, DecoderConfig, DecoderLM
from .reference_layers import CompressedMultiHeadAttention, SimpleTransformer, SimpleTransformerLayer

__all__ = ["PolarQuantConfig", "KVCacheManager", "CompressedAttention", "DecoderConfig", "DecoderLM",
           "CompressedMultiHeadAttention", "SimpleTransformer", "SimpleTransformerLayer"]
