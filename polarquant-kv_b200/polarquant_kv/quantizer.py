"""compress / decompress on the GPU, block_pq4 layout.

API of python/polarquant_kv/quantizer.py (compress, decompress, compress_batch,
decompress_batch) and of src/polarquant_kv_cuda/compress_kernel.py:100-189 /
decompress_kernel.py:10-51 (torch tensors, optional jl_matrix); the arithmetic runs in
pq_compress / pq_dequant of libpolarquant_b200.so.
"""

from __future__ import annotations

import ctypes

import torch

from . import _ext
from .codebook import block_codebook, decision_thresholds
from .rotation import device_plan
from .types import BLOCK, CompressedKV, block_bytes

_TABLES: dict = {}


def _validate_params(n_bits: int, group_size: int, d: int) -> None:
    """The reference's range checks (quantizer.py:15-22) plus what the kernels support."""
    if not (2 <= n_bits <= 8):
        raise ValueError(f"n_bits must be in [2, 8], got {n_bits}")
    if group_size <= 0:
        raise ValueError(f"group_size must be positive, got {group_size}")
    if group_size > d:
        raise ValueError(f"group_size ({group_size}) cannot exceed the vector dimension ({d})")
    if n_bits not in (2, 4):
        raise ValueError(f"the B200 kernels store 2- or 4-bit indices, got n_bits={n_bits}")
    if group_size != BLOCK:
        raise ValueError(f"block_pq4 uses blocks of {BLOCK} elements, got group_size={group_size}")
    if d not in (64, 128):
        raise ValueError(f"the B200 kernels support head_dim 64 or 128, got {d}")


def tables(n_bits: int):
    """(codebook, thresholds) as host float32 ctypes arrays for the ABI."""
    t = _TABLES.get(n_bits)
    if t is None:
        cb = block_codebook(n_bits)
        t = (_ext.float_array(cb), _ext.float_array(decision_thresholds(cb)), cb)
        _TABLES[n_bits] = t
    return t


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def compress(kv: torch.Tensor, rotation_matrix, n_bits: int = 4, group_size: int = 32,
             jl_matrix=None, out: CompressedKV | None = None, position: int = 0) -> CompressedKV:
    """kv float16 [batch, heads, seq, head_dim] (or [..., head_dim]) -> CompressedKV.

    With ``jl_matrix`` the QJL sign sketch and residual norms are produced as well.
    ``out``/``position`` write the new tokens in place into a preallocated cache at
    sequence offset ``position`` (append-on-write); otherwise a new cache is returned.  ``position``
    may be a one-element int64 tensor on the device: the kernel then reads the offset when it runs
    (pq_compress_rows_dynamic), which lets a decode step be recorded once as a CUDA graph.
    An empty input returns an empty cache (compress_kernel.py:108-124).
    """
    _require_cuda(kv, "kv")
    if kv.dim() < 1:
        raise ValueError("kv needs at least one dimension")
    d = kv.shape[-1]
    _validate_params(n_bits, group_size, d)
    shape4 = kv.shape if kv.dim() == 4 else (1, 1, kv.numel() // d, d)
    kv4 = kv.reshape(shape4)
    B, H, S, _ = shape4
    dev = kv.device
    plan = device_plan(rotation_matrix, dev, jl_matrix)
    if plan.head_dim != d:
        raise ValueError(f"rotation matrix is {plan.head_dim}x{plan.head_dim} but head_dim is {d}")
    nblk, bb = d // BLOCK, block_bytes(n_bits)
    jl_dim = plan.jl_dim

    if out is None:
        blocks = torch.empty((B, H, S, nblk, bb), dtype=torch.uint8, device=dev)
        signs = torch.empty((B, H, S, jl_dim // 8), dtype=torch.uint8, device=dev) if jl_dim else None
        norms = torch.empty((B, H, S), dtype=torch.float16, device=dev) if jl_dim else None
        out = CompressedKV(blocks, signs, norms, n_bits, group_size, d, S, S)
        capacity, position = S, 0
    else:
        if out.n_bits != n_bits or out.original_dim != d or tuple(out.blocks.shape[:2]) != (B, H):
            raise ValueError("preallocated cache does not match the input")
        if isinstance(position, torch.Tensor):
            # the offset lives on the device (a decode step replayed from a CUDA graph): the kernel checks
            # it against the capacity; the caller keeps out.seq_len up to date
            if position.dtype != torch.int64 or position.numel() != 1 or position.device != dev:
                raise ValueError("a device-side position must be a one-element int64 tensor on the cache's device")
        elif position < 0 or position + S > out.max_seq_len:
            raise RuntimeError(f"cache full: {position}+{S} > {out.max_seq_len}")   # kv_cache.py:76-79
        if jl_dim and (out.qjl_signs is None or out.qjl_signs.shape[-1] != jl_dim // 8):
            raise ValueError("preallocated cache has no sketch side band of this width")
        if not out.blocks.is_contiguous():
            raise ValueError("cache tensors must be contiguous")
        capacity = out.blocks.shape[2]
        if not isinstance(position, torch.Tensor):
            out.seq_len = max(out.seq_len, position + S)
    if kv4.numel() == 0:
        return out

    cb, thr, _ = tables(n_bits)
    x = kv4.to(torch.float16).contiguous()
    # one launch for all (batch, head) rows: row r of the input goes to tokens [position, position + S) of
    # row r of the cache
    dynamic = isinstance(position, torch.Tensor)
    fn = _ext.lib().pq_compress_rows_dynamic if dynamic else _ext.lib().pq_compress_rows
    st = fn(
        x.data_ptr(), B * H, S, capacity, position.data_ptr() if dynamic else position, d, n_bits,
        plan.rot_split.data_ptr(), thr, cb, out.blocks.data_ptr(),
        plan.jl_split.data_ptr() if jl_dim else None, jl_dim,
        out.qjl_signs.data_ptr() if jl_dim else None, out.residual_norms.data_ptr() if jl_dim else None, _stream(dev))
    _ext.check(st, "pq_compress_rows_dynamic" if dynamic else "pq_compress_rows")
    return out


def decompress(cache: CompressedKV, rotation_matrix, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """CompressedKV -> [batch, heads, seq_len, head_dim] in ``dtype`` (float32 like the numpy
    reference, or float16 like decompress_gpu, clamped to the float16 range)."""
    if dtype not in (torch.float32, torch.float16):
        raise ValueError("dtype must be float32 or float16")
    blocks = cache.blocks
    _require_cuda(blocks, "cache.blocks")
    B, H = blocks.shape[:2]
    S, d = cache.seq_len, cache.original_dim
    dev = blocks.device
    out = torch.empty((B, H, S, d), dtype=dtype, device=dev)
    if out.numel() == 0:
        return out
    plan = device_plan(rotation_matrix, dev)
    cb, _, _ = tables(cache.n_bits)
    lib = _ext.lib()
    src = blocks[:, :, :S]
    if not src.is_contiguous():
        src = src.contiguous()
    st = lib.pq_dequant(src.data_ptr(), B * H * S, d, cache.n_bits, cb, plan.rot.data_ptr(),
                        out.data_ptr(), 1 if dtype == torch.float16 else 0, _stream(dev))
    _ext.check(st, "pq_dequant")
    return out


def compress_batch(kv: torch.Tensor, rotation_matrix, n_bits: int = 4, group_size: int = 32,
                   jl_matrix=None) -> CompressedKV:
    """[batch, heads, seq, head_dim] -> CompressedKV (quantizer.py:161-195; one launch instead
    of a Python loop per vector)."""
    if kv.dim() != 4:
        raise ValueError(f"compress_batch expects [batch, heads, seq, head_dim], got {tuple(kv.shape)}")
    return compress(kv, rotation_matrix, n_bits, group_size, jl_matrix)


def decompress_batch(cache: CompressedKV, rotation_matrix, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """quantizer.py:198-219."""
    return decompress(cache, rotation_matrix, dtype)


def allocate_cache(batch: int, heads: int, max_seq_len: int, head_dim: int, n_bits: int = 4,
                   jl_dim: int = 0, device="cuda") -> CompressedKV:
    """Preallocated cache for append-in-place use (successor of KVCacheManager's
    concat-on-append, src/polarquant_kv_cuda/inference/kv_cache.py:68-116)."""
    _validate_params(n_bits, BLOCK, head_dim)
    blocks = torch.zeros((batch, heads, max_seq_len, head_dim // BLOCK, block_bytes(n_bits)),
                         dtype=torch.uint8, device=device)
    signs = torch.zeros((batch, heads, max_seq_len, jl_dim // 8), dtype=torch.uint8, device=device) if jl_dim else None
    norms = torch.zeros((batch, heads, max_seq_len), dtype=torch.float16, device=device) if jl_dim else None
    return CompressedKV(blocks, signs, norms, n_bits, BLOCK, head_dim, 0, max_seq_len)
