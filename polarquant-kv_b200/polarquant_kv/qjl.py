"""QJL residual sketch helpers (python/polarquant_kv/qjl.py, src/polarquant_kv_cuda/qjl_kernel.py).

The sketch itself (signs of P e and ||e||) is produced inside pq_compress and consumed
inside pq_decode_attn; this module holds the matrix generator and the bit-layout helpers.
"""

from __future__ import annotations

import numpy as np
import torch


def generate_jl_matrix(jl_dim: int, d: int, seed: int | None = None) -> np.ndarray:
    """P [jl_dim, d] with N(0, 1/jl_dim) entries from PCG64(seed), float64 (qjl.py:8-22)."""
    if jl_dim <= 0:
        raise ValueError(f"jl_dim must be a positive integer, got {jl_dim}")
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((jl_dim, d)).astype(np.float64) / np.sqrt(jl_dim)


def compute_signatures(residual: torch.Tensor, jl_matrix):
    """signs = (P e >= 0) and ||e|| of residual vectors [..., d] on the GPU, in float64 like the
    reference (qjl.py:25-35) -> QJLSignatures(signs bool [..., jl_dim], jl_dim, residual_norm).
    ``residual_norm`` is a Python float for a single vector (as in the reference), a float32 tensor
    [...] for a batch.  (pq_compress sketches its own residual in-kernel; this serves residuals a
    caller computed itself.)"""
    import ctypes

    from . import _ext
    from .types import QJLSignatures
    if not isinstance(residual, torch.Tensor) or not residual.is_cuda:
        raise TypeError("residual must be a CUDA tensor: this package has no CPU path")
    P = torch.as_tensor(np.asarray(jl_matrix, dtype=np.float64) if not isinstance(jl_matrix, torch.Tensor)
                        else jl_matrix).to(device=residual.device, dtype=torch.float64).contiguous()
    m, d = P.shape
    if residual.shape[-1] != d:
        raise ValueError(f"residual has {residual.shape[-1]} dims, the JL matrix {d}")
    e = residual.reshape(-1, d).to(torch.float32).contiguous()
    n = e.shape[0]
    bits = torch.empty((n, (m + 7) // 8), dtype=torch.uint8, device=e.device)
    norms = torch.empty((n,), dtype=torch.float32, device=e.device)
    st = _ext.lib().pq_qjl_sketch(e.data_ptr(), P.data_ptr(), n, d, m, bits.data_ptr(), norms.data_ptr(),
                                  ctypes.c_void_p(torch.cuda.current_stream(e.device).cuda_stream))
    _ext.check(st, "pq_qjl_sketch")
    signs = bit_unpack(bits, m).reshape(*residual.shape[:-1], m)
    if residual.dim() == 1:
        return QJLSignatures(signs=signs, jl_dim=m, residual_norm=float(norms[0].item()))
    return QJLSignatures(signs=signs, jl_dim=m, residual_norm=norms.reshape(residual.shape[:-1]))


def bit_pack(signs: torch.Tensor) -> torch.Tensor:
    """bool [..., m] -> uint8 [..., ceil(m/8)], bit k of byte j = sign[8j + k]
    (qjl_kernel.py:72-92, 110-123)."""
    m = signs.shape[-1]
    pad = (-m) % 8
    if pad:
        signs = torch.nn.functional.pad(signs, (0, pad))
    grouped = signs.reshape(*signs.shape[:-1], -1, 8).to(torch.int32)
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=signs.device)
    return (grouped * weights).sum(dim=-1).to(torch.uint8)


def bit_unpack(packed: torch.Tensor, m: int) -> torch.Tensor:
    """Inverse of bit_pack (qjl_kernel.py:95-107, 126-135)."""
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=packed.device)
    bits = (packed.to(torch.int32).unsqueeze(-1) & weights) > 0
    return bits.reshape(*packed.shape[:-1], -1)[..., :m]


def compute_correction(query: torch.Tensor, packed_signs: torch.Tensor, residual_norms: torch.Tensor,
                       jl_matrix) -> torch.Tensor:
    """corr[..., q, s] = dot(2*signs[s]-1, P q) / m, zero where the residual norm is zero
    (qjl.py:38-57, qjl_kernel.py:40-69).  A checking utility in float64 torch ops; the
    decode kernel evaluates the same term in-kernel."""
    P = torch.as_tensor(np.asarray(jl_matrix, dtype=np.float64) if not isinstance(jl_matrix, torch.Tensor)
                        else jl_matrix, device=query.device).double()
    m = P.shape[0]
    sv = 2.0 * bit_unpack(packed_signs, m).double() - 1.0
    qp = query.double() @ P.T
    corr = qp @ sv.transpose(-2, -1) / m
    return torch.where(residual_norms.unsqueeze(-2) > 0, corr, torch.zeros_like(corr))
