"""Small helpers: similarity, compression-ratio formulas, memory estimates.

Mirrors python/polarquant_kv/utils.py of the reference; the block_pq4 variants count the
bits that layout actually stores (one fp16 radius per 32 elements, no group min/scale).
"""

from __future__ import annotations

import math

import numpy as np
import torch


def cosine_similarity(a, b) -> float:
    """Cosine of the angle between two tensors/arrays, 0.0 if either is (near) zero
    (utils.py:9-15 of the reference)."""
    if isinstance(a, torch.Tensor):
        a = a.detach().double().flatten().cpu().numpy()
    if isinstance(b, torch.Tensor):
        b = b.detach().double().flatten().cpu().numpy()
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na < 1e-30 or nb < 1e-30:
        return 0.0
    return float(np.dot(a, b) / (na * nb))


def compute_compression_ratio(d: int, n_bits: int, group_size: int, jl_dim: int) -> float:
    """The reference's formula for its group-min/max layout (utils.py:18-31):
    16 d / (16 + n_bits d + 32 ceil(d/group) + jl_dim)."""
    num_groups = math.ceil(d / group_size)
    return (d * 16) / (16 + n_bits * d + num_groups * 32 + jl_dim)


def block_pq4_bits_per_vector(d: int, n_bits: int, jl_dim: int = 0) -> int:
    """Bits block_pq4 stores per vector: (16 + 32 n_bits) per block [+ jl_dim + 16]."""
    bits = (d // 32) * (16 + 32 * n_bits)
    if jl_dim:
        bits += jl_dim + 16
    return bits


def block_pq4_compression_ratio(d: int, n_bits: int, jl_dim: int = 0) -> float:
    return (d * 16) / block_pq4_bits_per_vector(d, n_bits, jl_dim)


def estimate_memory_bytes(batch: int, num_heads: int, seq_len: int, head_dim: int, n_bits: int,
                          group_size: int = 32, jl_dim: int = 0) -> int:
    """Bytes of a block_pq4 cache tensor of this shape (cf. utils.py:39-53)."""
    return math.ceil(batch * num_heads * seq_len * block_pq4_bits_per_vector(head_dim, n_bits, jl_dim) / 8)


def check_memory_warning(estimated_bytes: int, device=None) -> bool:
    """True when ``estimated_bytes`` exceeds 80 % of the free memory (utils.py:56-59 of the
    reference, which asks psutil for host RAM).  With ``device`` (a CUDA device) the free HBM of
    that GPU is the yardstick, which is what matters for a cache that lives on the GPU."""
    if device is not None:
        free, _total = torch.cuda.mem_get_info(device)
        return estimated_bytes > free * 0.8
    import psutil
    return estimated_bytes > psutil.virtual_memory().available * 0.8


def attention_score_mse(a, b) -> float:
    a = a.detach().double().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a, dtype=np.float64)
    b = b.detach().double().cpu().numpy() if isinstance(b, torch.Tensor) else np.asarray(b, dtype=np.float64)
    return float(np.mean((a - b) ** 2))
