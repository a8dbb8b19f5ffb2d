"""ctypes binding of libpolarquant_b200.so (the C ABI in include/polarquant_b200.h).

The reference binds its native kernels through pybind with raw ``data_ptr()`` integers
(csrc/flash_turboquant.cu:180-230) or dlsym (integration/polarquant-kv.patch); here the
boundary is a plain C ABI loaded with ctypes, so any host language can bind it.
"""

from __future__ import annotations

import ctypes
import os

_LIB_NAME = "libpolarquant_b200.so"
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), _LIB_NAME)

c_void_p, c_int, c_int64, c_float, c_size_t = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                               ctypes.c_float, ctypes.c_size_t)
c_float_p = ctypes.POINTER(ctypes.c_float)

# name -> (restype, argtypes); must list every symbol the headers under include/ declare
SIGNATURES = {
    "pq_version": (c_int, []),
    "pq_strerror": (ctypes.c_char_p, [c_int]),
    "pq_poll_device_errors": (c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "pq_compress": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_float_p, c_float_p, c_void_p,
                            c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "pq_compress_rows": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_float_p,
                                 c_float_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "pq_dequant": (c_int, [c_void_p, c_int64, c_int, c_int, c_float_p, c_void_p, c_void_p, c_int, c_void_p]),
    "pq_compress_rows_dynamic": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p,
                                         c_float_p, c_float_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                         c_void_p]),
    "pq_decode_attn_dynamic": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_void_p, c_int64,
                                       c_int, c_int, c_int, c_float_p, c_float_p, c_void_p, c_float,
                                       c_void_p, c_int, c_void_p, c_void_p,
                                       c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "pq_decode_attn": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                               c_int, c_int, c_int, c_float_p, c_float_p, c_void_p, c_float,
                               c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "pq_decode_attn_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                      c_int, c_int, c_int, c_float_p, c_float_p, c_void_p, c_float,
                                      c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "pq_decode_attn_static_scratch_capacity": (c_size_t, []),
    "pq_decode_attn_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int64, c_int, c_int]),
    "pq_decode_attn_default_splits": (c_int, [c_int, c_int, c_int, c_int64, c_int]),
    "pq_lse_merge": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "pq_lse_exchange_bytes": (c_size_t, [c_int, c_int64, c_int]),
    "pq_lse_exchange_merge": (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), ctypes.c_uint64, c_int64,
                                      c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "pq_qjl_sketch": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pq_prefill_attn": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                c_int, c_int, c_int, c_float_p, c_float_p, c_void_p, c_float, c_int,
                                c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "pq_prefill_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int64, c_int]),
    # include/polarquant_llama_abi.h: the llama.cpp bridge's entry points
    "polarquant_init_c": (c_void_p, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "polarquant_free_c": (None, [c_void_p]),
    "polarquant_compress_cuda_c": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_void_p]),
    "polarquant_rotate_query_cuda_c": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "polarquant_fused_attention_cuda_c": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "polarquant_inverse_rotate_cuda_c": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "polarquant_last_error_c": (c_int, []),
}

_lib = None


class PQError(RuntimeError):
    """A non-zero pq_status from the native library."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().pq_strerror(status).decode()
        super().__init__(f"{where}: pq_status {status} ({msg})")


def library_path() -> str:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                f"{_LIB_NAME} not found at {_LIB_PATH}: build it with "
                "`python -m polarquant_kv._build` (needs nvcc); there is no fallback path")
        handle = ctypes.CDLL(_LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError here means a stale build
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise PQError(status, where)


def poll_device_errors() -> int:
    """Synchronising check of the device-side error flags (0 = none); raises on a set flag."""
    flags = ctypes.c_uint(0)
    check(lib().pq_poll_device_errors(ctypes.byref(flags)), "pq_poll_device_errors")
    if flags.value:
        raise RuntimeError(f"device-side error flags {flags.value:#x}: a bounded tensor-core wait gave up; "
                           "results of the affected launch are invalid")
    return flags.value


def float_array(values) -> ctypes.Array:
    """Host float32 table (thresholds, codebooks) for the ABI's HOST pointers."""
    vals = [float(v) for v in values]
    return (ctypes.c_float * len(vals))(*vals)
