"""Seeded synthetic K/V/q tensors with the value distribution the benchmark configs
name (TEST INFRASTRUCTURE; stands in for real KV-cache traces, which are not available
offline).

Distribution: every tensor is N(0,1) times a per-channel lognormal(0,1) scale, with two
of the head_dim channels scaled by a further x10 ("outlier channels"), rounded to
float16.  The query is plain N(0,1) float16.  Draw order is fixed so a seed always
reproduces the same bytes:

    rng = default_rng(seed)
    k_scale = lognormal(0,1,D); k_hot = choice(D,2,replace=False); k_scale[k_hot] *= 10
    K = float16(standard_normal(kv_shape) * k_scale)
    v_scale, v_hot, V likewise
    q = float16(standard_normal(q_shape))
"""

from __future__ import annotations

import hashlib

import numpy as np


def channel_scale(rng: np.random.Generator, D: int) -> np.ndarray:
    scale = rng.lognormal(0.0, 1.0, D)
    hot = rng.choice(D, 2, replace=False)
    scale[hot] *= 10.0
    return scale


def make_kvq(batch: int, kv_heads: int, q_heads: int, seq: int, head_dim: int, seed: int = 0,
             q_len: int = 1):
    """Returns (K, V, q): K/V float16 [B, Hkv, S, D], q float16 [B, Hq, q_len, D]."""
    rng = np.random.default_rng(seed)
    shape = (batch, kv_heads, seq, head_dim)
    with np.errstate(over="ignore"):
        K = (rng.standard_normal(shape) * channel_scale(rng, head_dim)).astype(np.float16)
        V = (rng.standard_normal(shape) * channel_scale(rng, head_dim)).astype(np.float16)
        q = rng.standard_normal((batch, q_heads, q_len, head_dim)).astype(np.float16)
    return K, V, q


def make_vectors(n: int, head_dim: int, seed: int = 0) -> np.ndarray:
    """n float16 vectors [n, D] from the same distribution (bulk-compress workload)."""
    rng = np.random.default_rng(seed)
    scale = channel_scale(rng, head_dim)
    with np.errstate(over="ignore"):
        return (rng.standard_normal((n, head_dim)) * scale).astype(np.float16)


def digest(*arrays: np.ndarray) -> str:
    """sha256 over the raw bytes of the arrays, to detect generator drift."""
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


# The CPU-runnable reference configuration: single layer, batch 1, 2 KV heads,
# 14 query heads (GQA 7:1), 512 tokens, head_dim 64, seed 0.
C0 = dict(batch=1, kv_heads=2, q_heads=14, seq=512, head_dim=64, seed=0)
