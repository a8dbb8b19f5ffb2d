"""CPU oracle for the block_pq4 hot path (TEST INFRASTRUCTURE, not product code).

This module restates, in plain numpy, the algorithm of hilllief/polarquant-kv for the
path  rotate -> per-32 block radius -> Lloyd-Max nearest centroid -> nibble pack ->
(dequantise -> inverse rotate) -> attention [+ QJL score correction].

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import it; the shipped package never does.

Parity status: PINNED.  Every function here is checked (``tests/test_oracle_golden.py``) against the
committed fixtures in ``tests/golden/``, which were produced by calling the reference's own Python
functions (``tests/golden/make_golden.py`` imports the reference and calls nothing else).

No single reference function emits block_pq4 (the layout exists only as prose in the
reference's README.md:73-78); the oracle is the composition

    rotation.rotate                      python/polarquant_kv/rotation.py:38-48
    quantizer.compress polar split       python/polarquant_kv/quantizer.py:99-121
    lloyd_max.quantize_with_codebook     src/polarquant_kv_cuda/lloyd_max.py:82-90
    compress_kernel._bit_pack_quantized  src/polarquant_kv_cuda/compress_kernel.py:17-63
    lloyd_max.dequantize_with_codebook   src/polarquant_kv_cuda/lloyd_max.py:93-98
    quantizer.decompress                 python/polarquant_kv/quantizer.py:137-158
    qjl.compute_signatures/_correction   python/polarquant_kv/qjl.py:25-57
    attention.compressed_attention       python/polarquant_kv/attention.py:83-191

applied per 32-element block with one fp16 radius per block.
"""

from __future__ import annotations

import math

import numpy as np

BLOCK = 32  # elements per block_pq4 block (README.md:73-78 of the reference)


def block_bytes(n_bits: int) -> int:
    """Bytes of one stored block: fp16 radius + 32 packed indices."""
    if n_bits not in (2, 4):
        raise ValueError(f"block_pq4 stores 2- or 4-bit indices, got {n_bits}")
    return 2 + BLOCK * n_bits // 8


# --------------------------------------------------------------------------- rotation
def rotation_matrix(d: int, seed: int | None = None) -> np.ndarray:
    """Seeded Haar-orthogonal d x d matrix, float64.

    Follows python/polarquant_kv/rotation.py:7-35.  The reference draws from
    scipy.stats.ortho_group (scipy 1.17/1.18), whose published algorithm (Mezzadri 2006)
    is: Gaussian matrix from the generator, Householder QR, then scale column j of Q by
    sign(R[j, j]).  d == 1 is the reference's special case (rotation.py:27-31).
    """
    if not isinstance(d, (int, np.integer)):
        raise ValueError(f"d must be an integer, got {type(d).__name__}")
    if d <= 0:
        raise ValueError(f"d must be positive, got {d}")
    if d == 1:
        rng = np.random.Generator(np.random.PCG64(seed))
        return np.array([[rng.choice([-1.0, 1.0])]], dtype=np.float64)
    rng = np.random.default_rng(seed)
    z = rng.normal(size=(d, d))
    q, r = np.linalg.qr(z)
    diag = np.diagonal(r)
    return (q * (diag / np.abs(diag))[np.newaxis, :]).astype(np.float64)


def rotate(v: np.ndarray, R: np.ndarray) -> np.ndarray:
    """v @ R.T evaluated in float64, cast back to v.dtype (rotation.py:38-48)."""
    return (v.astype(np.float64) @ R.T).astype(v.dtype)


def inverse_rotate(v: np.ndarray, R: np.ndarray) -> np.ndarray:
    """v @ R evaluated in float64, cast back to v.dtype (rotation.py:51-61)."""
    return (v.astype(np.float64) @ R).astype(v.dtype)


# --------------------------------------------------------------------------- codebook
def lloyd_max_codebook(dim: int, n_bits: int, n_iterations: int = 300,
                       grid_size: int = 50000) -> tuple[np.ndarray, np.ndarray]:
    """Lloyd-Max centroids for one coordinate of a random unit vector in R^dim.

    Follows src/polarquant_kv_cuda/lloyd_max.py:12-79: the coordinate density is
    Beta((dim-1)/2, (dim-1)/2) mapped to [-1, 1]; it is sampled on ``grid_size`` points
    over +-6/sqrt(dim); centroids start uniformly spaced and each iteration moves every
    centroid to the density-weighted mean of the grid points in
    [boundary_i, boundary_{i+1}); outer boundaries are +-12/sqrt(dim).  Returned as
    float32 (centroids [2^b], boundaries [2^b + 1] of the last iteration).
    block_pq4 uses dim = 32.
    """
    from scipy.stats import beta as beta_dist  # same density routine as the reference

    n_levels = 1 << n_bits
    a = (dim - 1) / 2.0
    half_width = 6.0 / np.sqrt(dim)
    grid = np.linspace(-half_width, half_width, grid_size)
    t = np.clip((grid + 1) / 2, 1e-10, 1 - 1e-10)
    pdf = beta_dist.pdf(t, a, a) / 2
    pdf = pdf / (pdf.sum() * (grid[1] - grid[0]))

    centroids = np.linspace(-half_width, half_width, n_levels)
    boundaries = np.zeros(n_levels + 1)
    for _ in range(n_iterations):
        boundaries = np.zeros(n_levels + 1)
        boundaries[0] = -2 * half_width
        boundaries[-1] = 2 * half_width
        for i in range(1, n_levels):
            boundaries[i] = (centroids[i - 1] + centroids[i]) / 2
        updated = np.zeros(n_levels)
        for i in range(n_levels):
            inside = (grid >= boundaries[i]) & (grid < boundaries[i + 1])
            if inside.sum() > 0 and pdf[inside].sum() > 0:
                w = pdf[inside]
                updated[i] = (grid[inside] * w).sum() / w.sum()
            else:
                updated[i] = centroids[i]
        centroids = updated
    return centroids.astype(np.float32), boundaries.astype(np.float32)


def nearest_centroid(values: np.ndarray, centroids: np.ndarray) -> np.ndarray:
    """argmin_i |v - c_i| in the dtype of the operands, first index on ties -> uint8.

    Follows lloyd_max.py:82-90.  Chunked so the [..., n_levels] temporary stays small.
    """
    flat = np.ascontiguousarray(values).reshape(-1)
    out = np.empty(flat.shape[0], dtype=np.uint8)
    step = 1 << 18
    for lo in range(0, flat.shape[0], step):
        chunk = flat[lo:lo + step]
        out[lo:lo + step] = np.abs(chunk[:, np.newaxis] - centroids).argmin(axis=-1)
    return out.reshape(values.shape)


# --------------------------------------------------------------------------- packing
def pack_indices(idx: np.ndarray, n_bits: int) -> np.ndarray:
    """[..., n] uint8 indices -> [..., n*n_bits/8] bytes.

    4-bit: byte = idx[2k] | idx[2k+1] << 4; 2-bit: v0 | v1<<2 | v2<<4 | v3<<6
    (src/polarquant_kv_cuda/compress_kernel.py:34-50; known answer 0xA5 -> low 5, high 10,
    scripts/debug_kernel2.py:58-82).
    """
    idx = idx.astype(np.uint8)
    if n_bits == 4:
        return (idx[..., 0::2] | (idx[..., 1::2] << 4)).astype(np.uint8)
    if n_bits == 2:
        return (idx[..., 0::4] | (idx[..., 1::4] << 2) | (idx[..., 2::4] << 4)
                | (idx[..., 3::4] << 6)).astype(np.uint8)
    raise ValueError(f"unsupported n_bits {n_bits}")


def unpack_indices(packed: np.ndarray, n_bits: int) -> np.ndarray:
    """Inverse of pack_indices (compress_kernel.py:66-97)."""
    packed = packed.astype(np.uint8)
    if n_bits == 4:
        out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
        out[..., 0::2] = packed & 0x0F
        out[..., 1::2] = packed >> 4
        return out
    if n_bits == 2:
        out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 4,), dtype=np.uint8)
        for k in range(4):
            out[..., k::4] = (packed >> (2 * k)) & 0x03
        return out
    raise ValueError(f"unsupported n_bits {n_bits}")


def blocks_from_parts(d16: np.ndarray, idx: np.ndarray, n_bits: int) -> np.ndarray:
    """Assemble stored blocks: uint8 [..., D/32, 2 + 32*n_bits/8] = {fp16 d, qs[]}."""
    nblk = d16.shape[-1]
    qs = pack_indices(idx.reshape(idx.shape[:-1] + (nblk, BLOCK)), n_bits)
    out = np.empty(d16.shape + (block_bytes(n_bits),), dtype=np.uint8)
    out[..., 0:2] = np.ascontiguousarray(d16.astype("<f2")).view(np.uint8).reshape(d16.shape + (2,))
    out[..., 2:] = qs
    return out


def parts_from_blocks(blocks: np.ndarray, n_bits: int) -> tuple[np.ndarray, np.ndarray]:
    """Split stored blocks into (d16 [..., nblk] float16, idx [..., nblk*32] uint8)."""
    d16 = np.ascontiguousarray(blocks[..., 0:2]).view("<f2").reshape(blocks.shape[:-1])
    idx = unpack_indices(blocks[..., 2:], n_bits)
    return d16.astype(np.float16), idx.reshape(blocks.shape[:-2] + (-1,))


# --------------------------------------------------------------------------- compress
def block_norm(blk: np.ndarray) -> np.ndarray:
    """float32 Euclidean norm of the last axis (32 elements), with the summation order
    written out so the value does not depend on the numpy build or a BLAS.

    The reference takes np.float32(np.linalg.norm(v)) of a float32 vector
    (quantizer.py:105); numpy evaluates that in float32, and the order of the 32
    additions depends on the code path (1-D input: BLAS sdot; axis reduction: pairwise
    sum) - they differ by up to 2 ulp on 16 % of random inputs.  The oracle fixes the
    order to numpy's axis-reduction one: squares rounded to float32; eight partial sums
    r[j] = ((a[j] + a[8+j]) + a[16+j]) + a[24+j]; then
    ((r0+r1)+(r2+r3)) + ((r4+r5)+(r6+r7)); correctly rounded square root.
    """
    a = blk.astype(np.float32)
    sq = (a * a).astype(np.float32)
    r = [sq[..., j] for j in range(8)]
    for base in (8, 16, 24):
        r = [(r[j] + sq[..., base + j]).astype(np.float32) for j in range(8)]
    total = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]))
    return np.sqrt(total.astype(np.float32)).astype(np.float32)


def compress_parts(x: np.ndarray, R: np.ndarray, codebook: np.ndarray) -> dict:
    """block_pq4 compress of x [..., D] (any float dtype) -> intermediate parts.

    Steps and their sources: float32 cast (quantizer.py:99); rotate (quantizer.py:102);
    per block: radius = float32(norm) (quantizer.py:105), radius < 1e-30 -> radius 0 and
    all-zero indices (quantizer.py:107-119), direction = block / radius in float32
    (quantizer.py:121), nearest centroid (lloyd_max.py:82-90).  The stored radius is the
    float16 rounding of the float32 radius (README.md:73-78 of the reference: "FP16 d"),
    clamped to 65504 first (src/polarquant_kv_cuda/compress_kernel.py:178).

    Returns dict(xr, d32, d16, direction, idx) with block axes flattened back to D where
    it applies.
    """
    D = x.shape[-1]
    if D % BLOCK:
        raise ValueError(f"head_dim {D} is not a multiple of {BLOCK}")
    nblk = D // BLOCK
    xr = rotate(x.astype(np.float32), R)
    blk = xr.reshape(xr.shape[:-1] + (nblk, BLOCK))
    d32 = block_norm(blk)
    zero = d32 < 1e-30
    safe = np.where(zero, np.float32(1.0), d32).astype(np.float32)
    direction = (blk / safe[..., np.newaxis]).astype(np.float32)
    idx = nearest_centroid(direction, codebook.astype(np.float32))
    idx[zero] = 0
    d32 = np.where(zero, np.float32(0.0), d32).astype(np.float32)
    # clamp to the float16 range before rounding (compress_kernel.py:178 of the reference)
    d16 = np.minimum(d32, np.float32(65504.0)).astype(np.float16)
    return {
        "xr": xr, "d32": d32, "d16": d16,
        "direction": direction.reshape(xr.shape), "idx": idx.reshape(xr.shape),
    }


def compress(x: np.ndarray, R: np.ndarray, codebook: np.ndarray, n_bits: int) -> np.ndarray:
    """x [..., D] -> stored blocks uint8 [..., D/32, 18 | 10]."""
    p = compress_parts(x, R, codebook)
    return blocks_from_parts(p["d16"], p["idx"], n_bits)


def dequant_rotated(blocks: np.ndarray, codebook: np.ndarray, n_bits: int) -> np.ndarray:
    """Stored blocks -> float32 values in rotated space: centroid[idx] * float32(d).

    lloyd_max.py:93-98 then quantizer.py:151; the radius used is the stored float16 one.
    """
    d16, idx = parts_from_blocks(blocks, n_bits)
    c = codebook.astype(np.float32)[idx]
    nblk = d16.shape[-1]
    c = c.reshape(c.shape[:-1] + (nblk, BLOCK)) * d16.astype(np.float32)[..., np.newaxis]
    return c.reshape(c.shape[:-2] + (nblk * BLOCK,)).astype(np.float32)


def decompress(blocks: np.ndarray, R: np.ndarray, codebook: np.ndarray, n_bits: int) -> np.ndarray:
    """Stored blocks -> float32 [..., D] in the original space (quantizer.py:137-158)."""
    return inverse_rotate(dequant_rotated(blocks, codebook, n_bits), R).astype(np.float32)


def boundary_distance(direction: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    """Distance of every direction coordinate to the nearest decision boundary
    (midpoint of adjacent float32 centroids), used to classify index mismatches."""
    c = codebook.astype(np.float64)
    mid = (c[:-1] + c[1:]) / 2
    flat = direction.astype(np.float64).reshape(-1)
    out = np.empty(flat.shape[0])
    step = 1 << 18
    for lo in range(0, flat.shape[0], step):
        out[lo:lo + step] = np.abs(flat[lo:lo + step, np.newaxis] - mid).min(axis=-1)
    return out.reshape(direction.shape)


# --------------------------------------------------------------------------- QJL
def jl_matrix(jl_dim: int, d: int, seed: int | None = None) -> np.ndarray:
    """P [jl_dim, d] ~ N(0, 1/jl_dim), PCG64(seed), float64 (qjl.py:8-22)."""
    if jl_dim <= 0:
        raise ValueError(f"jl_dim must be positive, got {jl_dim}")
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((jl_dim, d)).astype(np.float64) / np.sqrt(jl_dim)


def qjl_signatures(residual: np.ndarray, P: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """signs = (P @ e >= 0) in float64 and ||e|| (qjl.py:25-35), vectorised over [..., d]."""
    e = residual.astype(np.float64)
    proj = e @ P.T
    return proj >= 0, np.linalg.norm(e, axis=-1)


def pack_sign_bits(signs: np.ndarray) -> np.ndarray:
    """bool [..., m] -> uint8 [..., ceil(m/8)], bit k of byte j = sign[8j + k]
    (src/polarquant_kv_cuda/qjl_kernel.py:72-92, 110-123)."""
    return np.packbits(signs.astype(np.uint8), axis=-1, bitorder="little")


def unpack_sign_bits(packed: np.ndarray, m: int) -> np.ndarray:
    return np.unpackbits(packed, axis=-1, bitorder="little")[..., :m].astype(bool)


def qjl_correction(q: np.ndarray, signs: np.ndarray, norms: np.ndarray, P: np.ndarray) -> np.ndarray:
    """corr[qi, s] = dot(2*signs[s]-1, P @ q[qi]) / m, 0 where ||e|| < 1e-30 (qjl.py:38-57)."""
    m = P.shape[0]
    qp = q.astype(np.float64) @ P.T
    sv = 2.0 * signs.astype(np.float64) - 1.0
    corr = qp @ sv.T / m
    return np.where(norms[np.newaxis, :] < 1e-30, 0.0, corr)


# --------------------------------------------------------------------------- attention
def _softmax(x: np.ndarray) -> np.ndarray:
    z = np.exp(x - np.max(x, axis=-1, keepdims=True))
    return z / np.sum(z, axis=-1, keepdims=True)


def standard_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """softmax(q k^T / sqrt(d)) v for q [n_q, d], k/v [S, d]; non-causal (attention.py:40-53)."""
    d = q.shape[-1]
    if k.shape[0] == 0:
        return np.zeros((q.shape[0], d), dtype=np.float32)
    scores = q @ k.T / np.sqrt(d)
    return (_softmax(scores) @ v).astype(np.float32)


def compressed_attention_2d(q, key, value, R, codebook_k, codebook_v, bits_k=4, bits_v=4,
                            P=None, enable_qjl=True, return_scores=False):
    """attention.py:111-163 with block_pq4 as the codec, vectorised over the sequence.

    q [n_q, d]; key/value [S, d].  K and V are compressed and decompressed token by
    token (attention.py:138-144); scores = q @ K_hat^T / sqrt(d) (:147); with QJL the
    residual is key - K_hat in the original space (:141) and scores += corr / sqrt(d)
    (:150-155); softmax; weights @ V_hat cast to float32 (:162-163).  An empty sequence
    gives zeros (:127-131).
    """
    S, d = key.shape[0], q.shape[-1]
    n_q = q.shape[0]
    if S == 0:
        out = np.zeros((n_q, d), dtype=np.float32)
        if return_scores:
            return {"output": out, "scores": np.empty((n_q, 0), dtype=np.float32)}
        return out
    k_hat = decompress(compress(key, R, codebook_k, bits_k), R, codebook_k, bits_k)
    v_hat = decompress(compress(value, R, codebook_v, bits_v), R, codebook_v, bits_v)
    scores = q @ k_hat.T / np.sqrt(d)
    if enable_qjl and P is not None:
        signs, norms = qjl_signatures(key - k_hat, P)
        scores = scores + qjl_correction(q, signs, norms, P) / np.sqrt(d)
    out = (_softmax(scores) @ v_hat).astype(np.float32)
    if return_scores:
        return {"output": out, "scores": scores}
    return out


def compressed_attention(q, key, value, R, codebook_k, codebook_v, bits_k=4, bits_v=4,
                         P=None, enable_qjl=True):
    """GQA form (attention.py:166-191): q [Hq, Sq, d], key/value [Hkv, S, d];
    q head h reads kv head h // (Hq / Hkv) (np.repeat on axis 0, attention.py:10-17)."""
    Hq, Hkv = q.shape[0], key.shape[0]
    rep = Hq // Hkv
    out = np.zeros(q.shape, dtype=np.float32)
    for h in range(Hq):
        out[h] = compressed_attention_2d(q[h], key[h // rep], value[h // rep], R,
                                         codebook_k, codebook_v, bits_k, bits_v, P, enable_qjl)
    return out


def attention_from_blocks(q, k_blocks, v_blocks, R, codebook_k, codebook_v, bits_k=4, bits_v=4,
                          P=None, qjl_bits=None, qjl_norms=None, scale=None):
    """Same attention evaluated from already-stored blocks (what a decode kernel sees).

    q [Hq, Sq, d]; k_blocks/v_blocks uint8 [Hkv, S, d/32, bytes]; optional QJL side band
    qjl_bits uint8 [Hkv, S, m/8], qjl_norms [Hkv, S].  Float64 arithmetic throughout.
    """
    Hq, Sq, d = q.shape
    Hkv = k_blocks.shape[0]
    rep = Hq // Hkv
    sc = 1.0 / math.sqrt(d) if scale is None else scale
    out = np.zeros((Hq, Sq, d), dtype=np.float64)
    cache = {}
    for h in range(Hq):
        g = h // rep
        if g not in cache:
            cache = {g: (decompress(k_blocks[g], R, codebook_k, bits_k).astype(np.float64),
                         decompress(v_blocks[g], R, codebook_v, bits_v).astype(np.float64))}
        k_hat, v_hat = cache[g]
        if k_hat.shape[0] == 0:
            continue
        s = q[h].astype(np.float64) @ k_hat.T * sc
        if P is not None and qjl_bits is not None:
            signs = unpack_sign_bits(qjl_bits[g], P.shape[0])
            s = s + qjl_correction(q[h], signs, qjl_norms[g].astype(np.float64), P) * sc
        out[h] = _softmax(s) @ v_hat
    return out.astype(np.float32)
