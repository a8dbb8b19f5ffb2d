"""Per-layer KV cache over block_pq4 storage.

Successor of KVCacheManager (src/polarquant_kv_cuda/inference/kv_cache.py:14-134 of the reference):
the same interface (append / get_kv / reset / seq_len / memory_bytes / compression_ratio, RuntimeError
when full), but the cache is preallocated at ``max_seq_len`` and a new step is written IN PLACE by one
launch per tensor (pq_compress_rows) instead of compressing into fresh tensors and concatenating every
cache tensor on every token (kv_cache.py:93-94, 107-116).  With ``enable_compression=False`` a plain
float16 cache of the same capacity is kept, for comparisons.
"""

from __future__ import annotations

import torch

from .. import quantizer
from ..attention import decode_attention, prefill_attention
from ..qjl import generate_jl_matrix
from ..rotation import device_plan, generate_rotation_matrix
from .config import PolarQuantConfig


class KVCacheManager:
    def __init__(self, config: PolarQuantConfig, max_seq_len: int, batch: int, num_heads: int, head_dim: int,
                 device: str | torch.device = "cuda", rotation_seed: int = 42, jl_seed: int = 1):
        self.config = config
        self.max_seq_len, self.batch, self.num_heads, self.head_dim = max_seq_len, batch, num_heads, head_dim
        self.device = torch.device(device)
        self.R = generate_rotation_matrix(head_dim, seed=rotation_seed)
        self.P = generate_jl_matrix(config.jl_dim, head_dim, seed=jl_seed) if config.enable_qjl else None
        self.plan = device_plan(self.R, self.device, self.P)          # keys (with the sketch matrices)
        self.plan_v = device_plan(self.R, self.device)                # values: no sketch
        self.k_bits = config.n_bits
        self.v_bits = config.v_bits if config.v_bits is not None else config.n_bits
        self._seq_len = 0
        self._compressed_keys = self._compressed_values = None
        self._key_cache = self._value_cache = None
        if config.enable_compression:
            jl = config.jl_dim if config.enable_qjl else 0
            self._compressed_keys = quantizer.allocate_cache(batch, num_heads, max_seq_len, head_dim, self.k_bits, jl, self.device)
            self._compressed_values = quantizer.allocate_cache(batch, num_heads, max_seq_len, head_dim, self.v_bits, 0, self.device)
        else:
            shape = (batch, num_heads, max_seq_len, head_dim)
            self._key_cache = torch.zeros(shape, dtype=torch.float16, device=self.device)
            self._value_cache = torch.zeros(shape, dtype=torch.float16, device=self.device)

    @property
    def seq_len(self) -> int:
        return self._seq_len

    @property
    def memory_bytes(self) -> int:
        """Bytes the tokens stored so far occupy (the reference's accounting: used, not reserved)."""
        per_token = self.batch * self.num_heads
        if not self.config.enable_compression:
            return per_token * self._seq_len * self.head_dim * 2 * 2
        nblk = self.head_dim // 32
        k = nblk * (2 + 4 * self.k_bits) + ((self.config.jl_dim // 8 + 2) if self.config.enable_qjl else 0)
        v = nblk * (2 + 4 * self.v_bits)
        return per_token * self._seq_len * (k + v)

    @property
    def compression_ratio(self) -> float:
        if self._seq_len == 0:
            return 0.0
        original = self.batch * self.num_heads * self._seq_len * self.head_dim * 2 * 2       # K+V, float16
        used = self.memory_bytes
        return original / used if used > 0 else 0.0

    def append(self, key: torch.Tensor, value: torch.Tensor, position: torch.Tensor | None = None) -> None:
        """key, value: [batch, num_heads, new_seq, head_dim] float16; written at the current length.

        With ``position`` (one int64 on the device) the offset is read by the kernels when they run and
        the host-side length is left alone: a decode step recorded once as a CUDA graph appends at a
        position that advances on the device; call ``advance`` afterwards for the bookkeeping."""
        new_seq = key.shape[2]
        if position is not None:
            if not self.config.enable_compression:
                raise ValueError("a device-side position needs the compressed cache")
            quantizer.compress(key, self.plan, self.k_bits, 32, self.P, out=self._compressed_keys, position=position)
            quantizer.compress(value, self.plan_v, self.v_bits, out=self._compressed_values, position=position)
            return
        if self._seq_len + new_seq > self.max_seq_len:
            raise RuntimeError(f"KV cache full: {self._seq_len} + {new_seq} > {self.max_seq_len}")
        pos = self._seq_len
        if self.config.enable_compression:
            quantizer.compress(key, self.plan, self.k_bits, 32, self.P, out=self._compressed_keys, position=pos)
            quantizer.compress(value, self.plan_v, self.v_bits, out=self._compressed_values, position=pos)
        else:
            self._key_cache[:, :, pos:pos + new_seq] = key
            self._value_cache[:, :, pos:pos + new_seq] = value
        self._seq_len += new_seq
        if self.config.enable_compression:
            self._compressed_keys.seq_len = self._compressed_values.seq_len = self._seq_len

    def advance(self, new_tokens: int) -> None:
        """Account for tokens that were appended with a device-side position."""
        if self._seq_len + new_tokens > self.max_seq_len:
            raise RuntimeError(f"KV cache full: {self._seq_len} + {new_tokens} > {self.max_seq_len}")
        self._seq_len += new_tokens
        if self.config.enable_compression:
            self._compressed_keys.seq_len = self._compressed_values.seq_len = self._seq_len

    def get_kv(self):
        """(CompressedKV, CompressedKV) in compressed mode, (key, value) float16 views otherwise."""
        if not self.config.enable_compression:
            return self._key_cache[:, :, :self._seq_len], self._value_cache[:, :, :self._seq_len]
        return self._compressed_keys, self._compressed_values

    def attend(self, query: torch.Tensor, causal: bool = True,
               seq_len_tensor: torch.Tensor | None = None) -> torch.Tensor:
        """query [batch, q_heads, seq_q, head_dim] float16 over everything stored so far -> float32
        [batch, q_heads, seq_q, head_dim].  The last seq_q tokens of the cache are the queries' own
        positions: with ``causal`` query i sees tokens [0, seq_len - seq_q + i].  ``seq_len_tensor``
        (one int64 on the device, seq_q == 1): the number of tokens is read by the kernel when it runs."""
        B, Hq, Sq, D = query.shape
        if seq_len_tensor is not None:
            if Sq != 1 or not self.config.enable_compression:
                raise ValueError("a device-side length serves single-token steps over the compressed cache")
            ck, cv = self.get_kv()
            return decode_attention(query[:, :, 0].contiguous(), ck, cv, self.plan,
                                    enable_qjl=self.config.enable_qjl, seq_len_tensor=seq_len_tensor).unsqueeze(2)
        if not self.config.enable_compression:
            k, v = self.get_kv()
            rep = Hq // self.num_heads
            k, v = k.float().repeat_interleave(rep, dim=1), v.float().repeat_interleave(rep, dim=1)
            mask = None
            if causal and Sq > 1:
                S = self._seq_len
                idx = torch.arange(S, device=query.device)[None, :] <= (S - Sq + torch.arange(Sq, device=query.device))[:, None]
                mask = idx
            return torch.nn.functional.scaled_dot_product_attention(query.float(), k, v, attn_mask=mask)
        ck, cv = self.get_kv()
        if Sq == 1:
            return decode_attention(query[:, :, 0].contiguous(), ck, cv, self.plan,
                                    enable_qjl=self.config.enable_qjl).unsqueeze(2)
        return prefill_attention(query, ck, cv, self.plan, causal=causal)

    def reset(self) -> None:
        self._seq_len = 0
        if self.config.enable_compression:
            self._compressed_keys.seq_len = self._compressed_values.seq_len = 0
