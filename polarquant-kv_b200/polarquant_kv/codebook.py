"""Lloyd-Max codebooks for block_pq4 and the exact decision thresholds the kernels use.

``build_lloyd_max_codebook`` keeps the reference's signature and algorithm
(src/polarquant_kv_cuda/lloyd_max.py:12-79): centroids of the coordinate density of a
random unit vector in R^dim, Beta((dim-1)/2, (dim-1)/2) on [-1, 1], sampled on a grid over
+-6/sqrt(dim), 300 Lloyd iterations from a uniform start, returned as float32.  block_pq4
quantises 32-element blocks, so the kernels always use dim = 32.

The per-iteration interval means are taken from prefix sums over the grid (one pass per
iteration) rather than one masked reduction per level.
"""

from __future__ import annotations

from functools import lru_cache

import numpy as np
from scipy.stats import beta as _beta

BLOCK = 32


def build_lloyd_max_codebook(dim: int, n_bits: int, n_iterations: int = 300,
                             grid_size: int = 50000) -> tuple[np.ndarray, np.ndarray]:
    """Returns (centroids float32 [2^n_bits], boundaries float32 [2^n_bits + 1])."""
    n_levels = 1 << n_bits
    a = (dim - 1) / 2.0
    span = 6.0 / np.sqrt(dim)
    grid = np.linspace(-span, span, grid_size)
    t = np.clip((grid + 1) / 2, 1e-10, 1 - 1e-10)
    pdf = _beta.pdf(t, a, a) / 2
    pdf = pdf / (pdf.sum() * (grid[1] - grid[0]))

    centroids = np.linspace(-span, span, n_levels)
    edges = np.empty(n_levels + 1)
    for _ in range(n_iterations):
        edges[0], edges[-1] = -2 * span, 2 * span
        edges[1:-1] = (centroids[:-1] + centroids[1:]) / 2
        cut = np.searchsorted(grid, edges, side="left")     # grid[cut[i]:cut[i+1]] lies in [e_i, e_{i+1})
        new = centroids.copy()
        for i in range(n_levels):
            lo, hi = cut[i], cut[i + 1]
            if hi > lo:
                w = pdf[lo:hi]
                wsum = w.sum()
                if wsum > 0:
                    new[i] = (grid[lo:hi] * w).sum() / wsum
        centroids = new
    return centroids.astype(np.float32), edges.astype(np.float32)


@lru_cache(maxsize=16)
def block_codebook(n_bits: int) -> np.ndarray:
    """The dim-32 codebook block_pq4 uses (cached; ~0.5 s to build)."""
    c, _ = build_lloyd_max_codebook(BLOCK, n_bits)
    c.setflags(write=False)
    return c


def quantize_with_codebook(values: np.ndarray, centroids: np.ndarray) -> np.ndarray:
    """Host utility: nearest centroid, first index on ties (lloyd_max.py:82-90)."""
    diffs = np.abs(np.asarray(values)[..., np.newaxis] - centroids)
    return diffs.argmin(axis=-1).astype(np.uint8)


def dequantize_with_codebook(indices: np.ndarray, centroids: np.ndarray) -> np.ndarray:
    """Host utility: table lookup (lloyd_max.py:93-98)."""
    return centroids[indices]


def decision_thresholds(centroids: np.ndarray) -> np.ndarray:
    """float32 thresholds t[0..n-2] with  index(v) = #{i : v > t[i]}  reproducing
    argmin_i |v - c_i| evaluated in float32 with first-index ties, bit for bit.

    For v between two adjacent centroids the winner is the lower one iff
    fl(v - c_i) <= fl(c_{i+1} - v); both sides are monotone in v, so there is a largest
    float32 v for which it holds.  That value is found by bisection over the ordered
    float32 numbers between the two centroids (around zero the tie region spans many
    subnormals, so stepping from the midpoint is not enough).
    """
    c = np.asarray(centroids, dtype=np.float32)
    out = np.empty(c.shape[0] - 1, dtype=np.float32)

    def to_key(x: np.float32) -> int:
        """Order-preserving integer image of a float32."""
        b = int(np.float32(x).view(np.int32))
        return b if b >= 0 else -(b & 0x7FFFFFFF)

    def from_key(k: int) -> np.float32:
        b = k if k >= 0 else ((-k) | 0x80000000)
        return np.uint32(b).view(np.float32)

    for i in range(c.shape[0] - 1):
        def lower_wins(v: np.float32) -> bool:
            return bool(np.float32(v - c[i]) <= np.float32(c[i + 1] - v))

        lo, hi = to_key(c[i]), to_key(c[i + 1])      # wins at c[i], loses at c[i+1]
        while hi - lo > 1:                            # bisection on the float32 number line
            mid = (lo + hi) // 2
            if lower_wins(from_key(mid)):
                lo = mid
            else:
                hi = mid
        out[i] = from_key(lo)
    return out
