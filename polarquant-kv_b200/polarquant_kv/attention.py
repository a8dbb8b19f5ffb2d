"""Attention over a block_pq4 cache.

``compressed_attention`` keeps the reference's GPU signature
(src/polarquant_kv_cuda/attention_kernel.py:11-36, compressor.py:19-25) and the semantics
of python/polarquant_kv/attention.py:83-191: non-causal softmax(q K^T / sqrt(d)) V on the
dequantised cache with GQA (query head h reads kv head h // (Hq/Hkv)) and the optional QJL
score correction.  seq_q == 1 runs pq_decode_attn, seq_q > 1 runs pq_prefill_attn.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _ext
from .quantizer import _require_cuda, _stream, compress, tables
from .rotation import device_plan
from .types import CompressedKV

_SCRATCH: dict = {}


def _scratch(device, nbytes: int, batch: int, q_heads: int, kv_heads: int) -> torch.Tensor:
    """Scratch for pq_decode_attn, one per (device, stream); grown on demand.

    The buffer starts with one ticket counter per (batch, kv head, head group), which must read zero when
    a launch starts; the segment records follow.  A kernel leaves its own counters at zero, so consecutive
    calls of one shape reuse the buffer as it is.  A call of another shape has another number of counters:
    where its counters lie, an earlier call with fewer of them may have written records, so the counter
    region is cleared whenever the shape differs from the previous call's on this buffer — and always
    while the stream is being captured into a CUDA graph: the graph is replayed later, after calls this
    function has not seen, so the clear has to be part of it."""
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    shape = (batch, q_heads, kv_heads)
    buf, last = _SCRATCH.get(key, (None, None))
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    elif last != shape or torch.cuda.is_current_stream_capturing():
        # at most one counter per (batch, query head); rounded up to the 256 bytes the records start on
        buf[:min(buf.numel(), (batch * q_heads * 4 + 255) // 256 * 256)].zero_()
    _SCRATCH[key] = (buf, shape)
    return buf


def standard_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                       num_kv_heads: int | None = None) -> torch.Tensor:
    """Uncompressed float64 reference on the GPU, for checks: [B, Hq, Sq, D] x [B, Hkv, S, D]
    (attention.py:20-73 of the reference; non-causal; GQA by repetition)."""
    B, Hq, Sq, D = query.shape
    Hkv = key.shape[1]
    if num_kv_heads is not None and num_kv_heads != Hkv:
        raise ValueError(f"key heads {Hkv} != num_kv_heads {num_kv_heads}")
    if key.shape[2] == 0:
        return torch.zeros((B, Hq, Sq, D), dtype=torch.float32, device=query.device)
    rep = Hq // Hkv
    k = key.double().repeat_interleave(rep, dim=1)
    v = value.double().repeat_interleave(rep, dim=1)
    s = query.double() @ k.transpose(-2, -1) / math.sqrt(D)
    return (torch.softmax(s, dim=-1) @ v).float()


def decode_attention(query: torch.Tensor, ck: CompressedKV, cv: CompressedKV, plan,
                     enable_qjl: bool = True, scale: float | None = None,
                     out_dtype: torch.dtype = torch.float32, n_splits: int = 0,
                     partial: bool = False, seq_range: tuple[int, int] | None = None,
                     seq_len_tensor: torch.Tensor | None = None) -> torch.Tensor:
    """One query token per sequence.  query [B, Hq, D] float16 -> [B, Hq, D] (or, with
    ``partial``, float32 [B, Hq, D+2] = (m, l, o_rotated) for a cross-GPU merge).
    ``seq_range`` restricts attention to tokens [begin, end) of the cache.  With ``seq_len_tensor``
    (one int64 on the device) the kernel reads the number of tokens when it runs, up to the cache's
    capacity (pq_decode_attn_dynamic): the launch can be replayed from a CUDA graph as the cache grows."""
    _require_cuda(query, "query")
    B, Hq, D = query.shape
    Hkv = ck.blocks.shape[1]
    if Hq % Hkv:
        raise ValueError(f"q heads {Hq} not a multiple of kv heads {Hkv}")
    dev = query.device
    kb, vb = ck.blocks, cv.blocks
    S, cap = ck.seq_len, ck.max_seq_len
    bits_t, norms_t = ck.qjl_signs, ck.residual_norms
    if seq_range is not None:
        lo, hi = seq_range
        kb, vb = kb[:, :, lo:hi], vb[:, :, lo:hi]
        if bits_t is not None:
            bits_t, norms_t = bits_t[:, :, lo:hi], norms_t[:, :, lo:hi]
        S = max(0, min(hi, S) - lo)
    if not kb.is_contiguous() or not vb.is_contiguous():
        kb, vb = kb.contiguous(), vb.contiguous()
        if bits_t is not None:
            bits_t, norms_t = bits_t.contiguous(), norms_t.contiguous()
    cap = kb.shape[2]
    use_qjl = bool(enable_qjl and plan.jl is not None and bits_t is not None)
    q = query.to(torch.float16).contiguous()
    lib = _ext.lib()
    n_splits = max(0, int(n_splits))     # 0: the library balances the work itself
    if seq_len_tensor is not None:
        if seq_range is not None:
            raise ValueError("seq_range and seq_len_tensor exclude each other")
        if seq_len_tensor.dtype != torch.int64 or seq_len_tensor.numel() != 1 or seq_len_tensor.device != dev:
            raise ValueError("seq_len_tensor must be a one-element int64 tensor on the query's device")
        S = cap                              # the work partition and the scratch cover the capacity
    need = lib.pq_decode_attn_scratch_bytes(B, Hq, Hkv, S, D, n_splits)
    scratch = _scratch(dev, need, B, Hq, Hkv)
    if partial:
        out = torch.empty((B, Hq, D + 2), dtype=torch.float32, device=dev)
    else:
        out = torch.empty((B, Hq, D), dtype=out_dtype, device=dev)
    cbk, _, _ = tables(ck.n_bits)
    cbv, _, _ = tables(cv.n_bits)
    fn, length = lib.pq_decode_attn, (S,)
    if seq_len_tensor is not None:
        fn, length = lib.pq_decode_attn_dynamic, (S, seq_len_tensor.data_ptr())
    st = fn(
        q.data_ptr(), kb.data_ptr(), vb.data_ptr(), B, Hq, Hkv, *length, cap, D, ck.n_bits, cv.n_bits,
        cbk, cbv, plan.rot.data_ptr(), ctypes.c_float(scale if scale is not None else 1.0 / math.sqrt(D)),
        plan.jl.data_ptr() if use_qjl else None, plan.jl_dim if use_qjl else 0,
        bits_t.data_ptr() if use_qjl else None, norms_t.data_ptr() if use_qjl else None,
        None if partial else out.data_ptr(), 1 if out_dtype == torch.float16 else 0,
        out.data_ptr() if partial else None, n_splits, scratch.data_ptr(), scratch.numel(), _stream(dev))
    _ext.check(st, "pq_decode_attn")
    return out


class PreparedDecode:
    """A decode-attention call with every argument resolved once (pointers, tables, scratch,
    output buffer), for serving loops where the Python-side set-up of ``decode_attention``
    would sit on the critical path of every token.  The cache objects and the query buffer
    are captured by reference: update ``ck.seq_len`` / the cache contents / the query buffer in
    place and call the object again.  Returns the (reused) output tensor.

    ``partial=True`` produces the float32 (m, l, o_rotated) records [B, Hq, D+2] of a
    sequence-sharded decode instead of the finished output.  The QJL score correction is applied
    when the plan carries a JL matrix, the key cache carries a sketch and ``enable_qjl`` is set
    (the defaults of ``decode_attention``).

    ``seq_len_tensor`` (a one-element int64 tensor on the device) makes the kernel read the number
    of tokens from device memory at every launch (pq_decode_attn_dynamic, clamped to the cache's
    capacity), so the call can be recorded once in a CUDA graph and replayed while the cache grows."""

    def __init__(self, query: torch.Tensor, ck: CompressedKV, cv: CompressedKV, plan,
                 scale: float | None = None, out_dtype: torch.dtype = torch.float32, n_splits: int = 0,
                 partial: bool = False, enable_qjl: bool = True, seq_len_tensor: torch.Tensor | None = None):
        _require_cuda(query, "query")
        if query.dtype != torch.float16 or not query.is_contiguous():
            raise ValueError("the query buffer must be a contiguous float16 tensor [B, Hq, D]")
        if not ck.blocks.is_contiguous() or not cv.blocks.is_contiguous():
            raise ValueError("cache tensors must be contiguous")
        self.query, self.ck, self.cv, self.plan = query, ck, cv, plan
        B, Hq, D = query.shape
        Hkv = ck.blocks.shape[1]
        self.dev = query.device
        if partial:
            self.out = torch.empty((B, Hq, D + 2), dtype=torch.float32, device=self.dev)
        else:
            self.out = torch.empty((B, Hq, D), dtype=out_dtype, device=self.dev)
        lib = _ext.lib()
        self._fn = lib.pq_decode_attn
        self.seq_len_tensor = seq_len_tensor
        if seq_len_tensor is not None:
            if seq_len_tensor.dtype != torch.int64 or seq_len_tensor.numel() != 1 or seq_len_tensor.device != self.dev:
                raise ValueError("seq_len_tensor must be a one-element int64 tensor on the query's device")
            self._fn = lib.pq_decode_attn_dynamic
        need = lib.pq_decode_attn_scratch_bytes(B, Hq, Hkv, ck.max_seq_len, D, max(0, n_splits))
        self.scratch = torch.zeros(max(need, 256), dtype=torch.uint8, device=self.dev)   # private: no sharing
        cbk, cbv = tables(ck.n_bits)[0], tables(cv.n_bits)[0]
        use_qjl = bool(enable_qjl and plan.jl is not None and ck.qjl_signs is not None)
        if use_qjl and (not ck.qjl_signs.is_contiguous() or not ck.residual_norms.is_contiguous()):
            raise ValueError("sketch tensors must be contiguous")
        self._head = (query.data_ptr(), ck.blocks.data_ptr(), cv.blocks.data_ptr(), B, Hq, Hkv)
        self._tail = (ck.max_seq_len, D, ck.n_bits, cv.n_bits, cbk, cbv, plan.rot.data_ptr(),
                      ctypes.c_float(scale if scale is not None else 1.0 / math.sqrt(D)),
                      plan.jl.data_ptr() if use_qjl else None, plan.jl_dim if use_qjl else 0,
                      ck.qjl_signs.data_ptr() if use_qjl else None,
                      ck.residual_norms.data_ptr() if use_qjl else None,
                      None if partial else self.out.data_ptr(), 1 if out_dtype == torch.float16 else 0,
                      self.out.data_ptr() if partial else None,
                      max(0, n_splits), self.scratch.data_ptr(), self.scratch.numel())
        self._stream = torch.cuda.current_stream(self.dev)

    def __call__(self, stream: torch.cuda.Stream | None = None) -> torch.Tensor:
        """Enqueue on the stream the object was prepared on, or on `stream`."""
        if self.seq_len_tensor is not None:
            st = self._fn(*self._head, self.ck.max_seq_len, self.seq_len_tensor.data_ptr(), *self._tail,
                          (stream or self._stream).cuda_stream)
        else:
            st = self._fn(*self._head, self.ck.seq_len, *self._tail, (stream or self._stream).cuda_stream)
        if st:
            _ext.check(st, "pq_decode_attn")
        return self.out

    def capture(self, query_host: torch.Tensor | None = None, out_host: torch.Tensor | None = None):
        """Record one decode step as a CUDA graph and return it (replay with ``graph.replay()``): optional
        copy of the pinned ``query_host`` into the query buffer, the attention kernel, optional copy of the
        output into the pinned ``out_host``.  One graph launch then replaces three stream operations.  The
        sequence length is frozen at capture time: re-capture after the cache has grown."""
        graph = torch.cuda.CUDAGraph()
        self()                                    # first launch outside the capture (function attributes)
        torch.cuda.current_stream(self.dev).synchronize()
        with torch.cuda.graph(graph):
            cur = torch.cuda.current_stream(self.dev)
            if query_host is not None:
                self.query.copy_(query_host, non_blocking=True)
            self(cur)
            if out_host is not None:
                out_host.copy_(self.out, non_blocking=True)
        return graph


def prepare_decode(query: torch.Tensor, ck: CompressedKV, cv: CompressedKV, plan, **kw) -> PreparedDecode:
    """See PreparedDecode."""
    return PreparedDecode(query, ck, cv, plan, **kw)


_PREFILL_WS: dict = {}
PREFILL_WORKSPACE_LIMIT = 1 << 30      # bytes; larger shapes use the fused (dequantise-in-kernel) path


def _prefill_workspace(dev: torch.device, need: int) -> torch.Tensor:
    """Per-(device, stream) buffer for the expanded K/V tiles, grown on demand."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    buf = _PREFILL_WS.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.uint8, device=dev)
        _PREFILL_WS[key] = buf
    return buf


def prefill_attention(query: torch.Tensor, ck: CompressedKV, cv: CompressedKV, plan,
                      scale: float | None = None, causal: bool = False,
                      out_dtype: torch.dtype = torch.float32, use_workspace: bool | None = None) -> torch.Tensor:
    """query [B, Hq, Sq, D] float16 -> [B, Hq, Sq, D]; K/V tiles are dequantised into shared
    memory and contracted on tensor cores (pq_prefill_attn).  `use_workspace`: True expands every
    K/V tile once into a device workspace first (1 KB per token and KV head at D = 128), False
    dequantises inside the attention kernel; None picks the workspace when more than one 128-row
    query tile shares a KV head and the workspace stays below PREFILL_WORKSPACE_LIMIT."""
    _require_cuda(query, "query")
    B, Hq, Sq, D = query.shape
    Hkv = ck.blocks.shape[1]
    dev = query.device
    out = torch.empty((B, Hq, Sq, D), dtype=out_dtype, device=dev)
    if out.numel() == 0:
        return out
    kb, vb = ck.blocks, cv.blocks
    if not kb.is_contiguous() or not vb.is_contiguous():
        kb, vb = kb.contiguous(), vb.contiguous()
    q = query.to(torch.float16).contiguous()
    cbk, _, _ = tables(ck.n_bits)
    cbv, _, _ = tables(cv.n_bits)
    lib = _ext.lib()
    need = lib.pq_prefill_attn_workspace_bytes(B, Hkv, ck.seq_len, D)
    if use_workspace is None:
        use_workspace = Sq * (Hq // Hkv) > 128 and 0 < need <= PREFILL_WORKSPACE_LIMIT
    ws = _prefill_workspace(dev, need) if (use_workspace and need > 0) else None
    st = lib.pq_prefill_attn(
        q.data_ptr(), kb.data_ptr(), vb.data_ptr(), B, Hq, Hkv, Sq, ck.seq_len, ck.max_seq_len, D,
        ck.n_bits, cv.n_bits, cbk, cbv, plan.rot.data_ptr(),
        ctypes.c_float(scale if scale is not None else 1.0 / math.sqrt(D)), 1 if causal else 0,
        out.data_ptr(), 1 if out_dtype == torch.float16 else 0,
        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream(dev))
    _ext.check(st, "pq_prefill_attn")
    return out


def compressed_attention(query: torch.Tensor, compressed_keys, compressed_values, rotation_matrix,
                         jl_matrix=None, enable_qjl: bool = True, num_kv_heads: int | None = None,
                         n_bits: int = 4, group_size: int = 32,
                         out_dtype: torch.dtype = torch.float32, return_scores: bool = False):
    """query [B, Hq, Sq, D] (or [Hq, Sq, D], or the reference's 2-D form [n_q, D] with keys/values
    [S, D]) float16 on the GPU; keys/values either
    CompressedKV caches (the GPU facade's signature) or raw float16 tensors
    [B, Hkv, S, D] / [Hkv, S, D], which are compressed first as the numpy reference does
    (attention.py:138-144).  Returns [B, Hq, Sq, D] (same rank as the query), float32 by
    default since float16 cannot hold the 2e-3 parity the path is checked to.
    An empty cache gives zeros (attention.py:127-131).  return_scores=True returns
    {"output", "scores"} like the reference's 2-D form (attention.py:157-160); the pre-softmax
    scores [.., Sq, S] come from a checking path (pq_dequant + a float32 matmul + the sketch
    correction in torch), not from the attention kernels."""
    _require_cuda(query, "query")
    if query.dim() == 2:                       # reference 2-D form: one head, n_q query rows
        def lift(x):
            return x if isinstance(x, CompressedKV) else x.reshape(1, 1, *x.shape)
        res = compressed_attention(query.reshape(1, 1, *query.shape), lift(compressed_keys), lift(compressed_values),
                                   rotation_matrix, jl_matrix, enable_qjl, num_kv_heads, n_bits, group_size,
                                   out_dtype, return_scores)
        if return_scores:
            return {"output": res["output"][0, 0], "scores": res["scores"][0, 0]}
        return res[0, 0]
    squeeze = query.dim() == 3
    q4 = query.unsqueeze(0) if squeeze else query
    if q4.dim() != 4:
        raise ValueError(f"unsupported query shape {tuple(query.shape)}")
    dev = query.device
    plan = device_plan(rotation_matrix, dev, jl_matrix if enable_qjl else None)

    def as_cache(x, with_qjl):
        if isinstance(x, CompressedKV):
            return x
        x4 = x.unsqueeze(0) if x.dim() == 3 else x
        return compress(x4, plan if not with_qjl else rotation_matrix, n_bits, group_size,
                        jl_matrix if with_qjl else None)

    ck = as_cache(compressed_keys, enable_qjl and jl_matrix is not None)
    cv = as_cache(compressed_values, False)
    Hkv = ck.blocks.shape[1]
    if num_kv_heads is not None and num_kv_heads != Hkv:
        raise ValueError(f"key heads {Hkv} != num_kv_heads {num_kv_heads}")
    B, Hq, Sq, D = q4.shape
    if ck.seq_len == 0 or q4.numel() == 0:
        out = torch.zeros((B, Hq, Sq, D), dtype=out_dtype, device=dev)
    elif Sq == 1:
        out = decode_attention(q4[:, :, 0], ck, cv, plan, enable_qjl, out_dtype=out_dtype).unsqueeze(2)
    else:
        if enable_qjl and jl_matrix is not None and ck.qjl_signs is not None:
            # The sketch correction lives in the decode kernel.  Every position sees the whole cache (non-causal,
            # as the reference), so the Sq positions of a query head are Sq more heads of its KV head's group:
            # one decode launch over Hq * Sq heads, [B, Hq, Sq, D] read as [B, Hq * Sq, D] (kv-head major as it is).
            out = decode_attention(q4.reshape(B, Hq * Sq, D).contiguous(), ck, cv, plan, True,
                                   out_dtype=out_dtype).reshape(B, Hq, Sq, D)
        else:
            out = prefill_attention(q4, ck, cv, plan, out_dtype=out_dtype)
    if return_scores:
        if ck.seq_len == 0:
            scores = torch.empty((B, Hq, Sq, 0), dtype=torch.float32, device=dev)
        else:
            from . import qjl as _qjl
            from .quantizer import decompress
            k_hat = decompress(ck, rotation_matrix).repeat_interleave(Hq // Hkv, dim=1)       # [B, Hq, S, D]
            scores = (q4.float() @ k_hat.transpose(-2, -1)) / math.sqrt(D)
            if enable_qjl and jl_matrix is not None and ck.qjl_signs is not None:
                S = ck.seq_len
                corr = _qjl.compute_correction(q4.float(), ck.qjl_signs[:, :, :S].repeat_interleave(Hq // Hkv, dim=1),
                                               ck.residual_norms[:, :, :S].repeat_interleave(Hq // Hkv, dim=1), jl_matrix)
                scores = scores + (corr / math.sqrt(D)).float()
        res = {"output": out[0] if squeeze else out, "scores": scores[0] if squeeze else scores}
        return res
    return out[0] if squeeze else out
