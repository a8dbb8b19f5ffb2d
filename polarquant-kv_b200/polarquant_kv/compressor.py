"""High-level facade with the names of src/polarquant_kv_cuda/compressor.py:11-38."""

from __future__ import annotations

from .attention import compressed_attention as _attention
from .quantizer import compress as _compress
from .quantizer import decompress as _decompress
from .types import CompressedKV


def compress(kv, rotation_matrix, n_bits=4, group_size=32, jl_matrix=None):
    return _compress(kv, rotation_matrix, n_bits, group_size, jl_matrix)


def decompress(cache, rotation_matrix, dtype=None):
    import torch
    return _decompress(cache, rotation_matrix, dtype or torch.float16)


def compressed_attention(query, compressed_keys, compressed_values, rotation_matrix, jl_matrix=None,
                         enable_qjl=True, num_kv_heads=None, return_scores=False):
    return _attention(query, compressed_keys, compressed_values, rotation_matrix, jl_matrix,
                      enable_qjl, num_kv_heads, return_scores=return_scores)


def get_memory_bytes(cache: CompressedKV) -> int:
    """Exact device bytes of a compressed cache (compressor.py:28-38)."""
    return cache.memory_bytes()
