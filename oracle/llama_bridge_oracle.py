"""CPU restatement (numpy) of the kernels behind the reference's llama.cpp bridge.

TEST INFRASTRUCTURE ONLY: imported by tests/; the product never imports it.

Source followed: integration/polarquant-kv.patch of hilllief/polarquant-kv (decoded as UTF-8;
line numbers are those of the decoded patch).  PARITY UNPINNED for this file: the patch ships
no fixtures or tests for these kernels and its CUDA source only builds inside a llama.cpp tree,
so nothing here has been checked against an execution of the reference.

Arithmetic is float64 where the reference's is float32; the tests allow for that with an
explained-mismatch window on the indices and a tolerance on the floats.
"""

from __future__ import annotations

import numpy as np


def rotate(x: np.ndarray, R: np.ndarray) -> np.ndarray:
    """x · Rᵀ (patch 395-411, polarquant_rotate_kernel: out[t] = sum_j in[j] R[t][j])."""
    return np.asarray(x, np.float64) @ np.asarray(R, np.float64).T


def inverse_rotate(y: np.ndarray, R: np.ndarray) -> np.ndarray:
    """y · R (patch 418-435, polarquant_inv_rotate_kernel: out[t] = sum_j in[j] R[j][t])."""
    return np.asarray(y, np.float64) @ np.asarray(R, np.float64)


def nearest_level(direction: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    """Linear scan with a strict `<`, so the first of equally near centroids wins (patch 254-262)."""
    dist = np.abs(direction[..., None] - np.asarray(codebook, np.float64))
    return np.argmin(dist, axis=-1).astype(np.uint8)      # argmin returns the first minimum


def compress(x: np.ndarray, R: np.ndarray, codebook: np.ndarray):
    """patch 193-270 (polarquant_compress_kernel): rotate, radius = ||rotated||, direction =
    rotated / radius (0 when radius <= 1e-30), nearest centroid, byte k = idx[2k] | idx[2k+1] << 4.
    Returns (radius f64 [N], packed u8 [N, D/2], direction f64 [N, D])."""
    rot = rotate(x, R)
    radius = np.sqrt((rot * rot).sum(-1))
    safe = np.where(radius > 1e-30, radius, 1.0)
    direction = np.where(radius[:, None] > 1e-30, rot / safe[:, None], 0.0)
    idx = nearest_level(direction, codebook)
    packed = (idx[:, 0::2] | (idx[:, 1::2] << 4)).astype(np.uint8)
    return radius, packed, direction


def unpack(packed: np.ndarray, n_levels: int) -> np.ndarray:
    """Nibbles back to indices, masked with n_levels - 1 as the attention kernel does (patch 329, 380)."""
    lo = packed & (n_levels - 1)
    hi = (packed >> 4) & (n_levels - 1)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def fused_attention(q_rot, packed_k, k_radius, packed_v, v_radius, codebook, n_levels, scale):
    """patch 276-390 (polarquant_attention_kernel).  q_rot [Hq, D]; packed_* [Hkv, S, D/2];
    *_radius [Hkv, S].  score = dot(q, cb[k idx]) * k_radius * scale; softmax; out = sum_s w_s *
    cb[v idx] * v_radius; q head h uses kv head h // (Hq // Hkv).  Output stays in rotated space."""
    q_rot = np.asarray(q_rot, np.float64)
    cb = np.asarray(codebook, np.float64)
    hq, hkv = q_rot.shape[0], packed_k.shape[0]
    ratio = hq // hkv
    k = cb[unpack(packed_k, n_levels)]
    v = cb[unpack(packed_v, n_levels)] * np.asarray(v_radius, np.float64)[..., None]
    out = np.empty_like(q_rot)
    for h in range(hq):
        g = h // ratio
        s = (k[g] @ q_rot[h]) * np.asarray(k_radius[g], np.float64) * scale
        w = np.exp(s - s.max())
        out[h] = (w / w.sum()) @ v[g]
    return out
