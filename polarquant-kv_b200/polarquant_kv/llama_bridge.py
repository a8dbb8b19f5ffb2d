"""The llama.cpp bridge's C entry points (include/polarquant_llama_abi.h) on torch tensors.

The reference reaches these through dlsym from llama.cpp (integration/polarquant-kv.patch,
decoded lines 1536-1560 and 1586-1607: llama_polarquant_compress_k / _v / _attention); this
module is the same call sequence for Python callers and for the tests.  It is the bridge's own
codec (one float32 radius per vector, nibble-packed indices), not block_pq4.
"""

from __future__ import annotations

import ctypes

import torch

from . import _ext

ERRORS = {1: "NULL pointer", 2: "head dim must be even and at most 1024", 3: "n_levels outside [1, 16]",
          4: "total_q_heads is not a multiple of total_kv_heads", 5: "a CUDA call failed"}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32")
    return t.contiguous()


def _raise_on_error(where: str) -> None:
    code = _ext.lib().polarquant_last_error_c()
    if code:
        raise ValueError(f"{where}: {ERRORS.get(code, code)}")


def compress(x: torch.Tensor, rotation: torch.Tensor, codebook: torch.Tensor):
    """x [N, D] float32 -> (radius float32 [N], packed uint8 [N, D/2])."""
    x, rotation, codebook = _f32(x, "x"), _f32(rotation, "rotation"), _f32(codebook, "codebook")
    n, d = x.shape
    radius = torch.empty(n, dtype=torch.float32, device=x.device)
    packed = torch.empty(n, d // 2, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _ext.lib().polarquant_compress_cuda_c(x.data_ptr(), rotation.data_ptr(), codebook.data_ptr(),
                                              radius.data_ptr(), packed.data_ptr(), n, d, codebook.numel(),
                                              _stream(x))
    _raise_on_error("polarquant_compress_cuda_c")
    return radius, packed


def rotate_query(q: torch.Tensor, rotation: torch.Tensor) -> torch.Tensor:
    """q [Hq, D] · Rᵀ."""
    q, rotation = _f32(q, "q"), _f32(rotation, "rotation")
    out = torch.empty_like(q)
    with torch.cuda.device(q.device):
        _ext.lib().polarquant_rotate_query_cuda_c(q.data_ptr(), rotation.data_ptr(), out.data_ptr(),
                                                  q.shape[0], q.shape[1], _stream(q))
    _raise_on_error("polarquant_rotate_query_cuda_c")
    return out


def inverse_rotate(y: torch.Tensor, rotation: torch.Tensor) -> torch.Tensor:
    """y [Hq, D] · R."""
    y, rotation = _f32(y, "y"), _f32(rotation, "rotation")
    out = torch.empty_like(y)
    with torch.cuda.device(y.device):
        _ext.lib().polarquant_inverse_rotate_cuda_c(y.data_ptr(), rotation.data_ptr(), out.data_ptr(),
                                                    y.shape[0], y.shape[1], _stream(y))
    _raise_on_error("polarquant_inverse_rotate_cuda_c")
    return out


def fused_attention(q_rot: torch.Tensor, packed_k: torch.Tensor, k_radius: torch.Tensor,
                    packed_v: torch.Tensor, v_radius: torch.Tensor, codebook: torch.Tensor,
                    scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """q_rot [Hq, D]; packed_* uint8 [Hkv, S, D/2]; *_radius [Hkv, S] -> [Hq, D] (rotated space)."""
    q_rot, k_radius, v_radius, codebook = (_f32(q_rot, "q_rot"), _f32(k_radius, "k_radius"),
                                           _f32(v_radius, "v_radius"), _f32(codebook, "codebook"))
    if packed_k.dtype != torch.uint8 or packed_v.dtype != torch.uint8:
        raise TypeError("packed_k and packed_v must be uint8")
    packed_k, packed_v = packed_k.contiguous(), packed_v.contiguous()
    hq, d = q_rot.shape
    hkv, s = packed_k.shape[0], packed_k.shape[1]
    if packed_k.shape[2] * 2 != d or packed_v.shape != packed_k.shape or tuple(k_radius.shape) != (hkv, s) \
            or tuple(v_radius.shape) != (hkv, s):
        raise ValueError("shape mismatch between q_rot, packed_k/v and the radii")
    if out is None:
        out = torch.empty_like(q_rot)
    with torch.cuda.device(q_rot.device):
        _ext.lib().polarquant_fused_attention_cuda_c(
            q_rot.data_ptr(), packed_k.data_ptr(), k_radius.data_ptr(), packed_v.data_ptr(), v_radius.data_ptr(),
            codebook.data_ptr(), out.data_ptr(), hq, hkv, s, d, codebook.numel(), ctypes.c_float(scale),
            _stream(q_rot))
    _raise_on_error("polarquant_fused_attention_cuda_c")
    return out


class PolarquantStateFields(ctypes.Structure):
    """Layout of struct polarquant_state (include/polarquant_llama_abi.h)."""
    _fields_ = [("enabled", ctypes.c_bool), ("n_bits", ctypes.c_int), ("n_levels", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("n_q_heads", ctypes.c_int),
                ("n_layers", ctypes.c_int), ("n_kv_max", ctypes.c_int), ("codebook", ctypes.c_void_p),
                ("rotation", ctypes.c_void_p), ("layers", ctypes.c_void_p)]


class State:
    """polarquant_init_c / polarquant_free_c as a context manager; `.fields` reads the struct."""

    def __init__(self, head_dim, n_kv_heads, n_q_heads, n_layers, n_kv_max, n_bits=4):
        self.handle = _ext.lib().polarquant_init_c(head_dim, n_kv_heads, n_q_heads, n_layers, n_kv_max, n_bits)
        if not self.handle:
            _raise_on_error("polarquant_init_c")
            raise MemoryError("polarquant_init_c returned NULL")
        self.fields = PolarquantStateFields.from_address(self.handle)

    def device_tensor(self, address: int, count: int, typestr: str = "<f4") -> torch.Tensor:
        """A copy of `count` elements at a device address owned by the state (float32 by default)."""
        return torch.as_tensor(_DeviceSpan(address, count, typestr), device="cuda").clone()

    def close(self):
        if self.handle:
            _ext.lib().polarquant_free_c(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class _DeviceSpan:
    """Device memory described through __cuda_array_interface__ so torch can view it."""

    def __init__(self, address: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (address, False),
                                         "version": 2}
