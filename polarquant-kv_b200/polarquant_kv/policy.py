"""Mixed-precision policies over block_pq4 caches: bit widths per layer, per KV head and per token range.

Successor of src/polarquant_kv_cuda/adaptive_bitwidth.py:15-68 (U-shaped widths per layer) and
token_importance.py:17-79 (sink + recent window at 4 bits, the middle at 2) of the reference, where
both are estimators: they count tokens and predict ratios, nothing is stored or attended.  Here a policy
is a *partition descriptor* — runs of KV heads or of tokens that share a width — and each run is a
block_pq4 cache of its own, so the existing kernels serve it: a head-partitioned cache is attended run
by run (the query heads of a run are independent of the others), a token-partitioned cache by one
partial decode per run (m, l, o_rotated) and a log-sum-exp merge (the machinery of the sequence-sharded
long-context path, on one GPU).  One launch per run; widths are 2 or 4.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import quantizer
from .attention import decode_attention
from .distributed import lse_merge
from .rotation import device_plan
from .types import CompressedKV


def compute_layer_bitwidths(num_layers: int, target_avg_bits: float = 3.0, min_bits: int = 2,
                            max_bits: int = 4) -> list[int]:
    """U-shaped widths per layer (adaptive_bitwidth.py:15-68): the first and last layers keep
    ``max_bits``, the middle gets ``min_bits``, and as many layers as the target average allows, taken
    from the ends inwards, stay at ``max_bits``.  Only the two packed widths exist here, so every layer is
    ``min_bits`` or ``max_bits`` (the reference also emits 3)."""
    if num_layers <= 2:
        return [max_bits] * num_layers
    mid = (num_layers - 1) / 2.0
    order = sorted(range(num_layers), key=lambda i: (-abs(i - mid), i))       # ends first
    n_high = int(round(num_layers * (target_avg_bits - min_bits) / max(max_bits - min_bits, 1)))
    n_high = max(2, min(num_layers, n_high))
    bits = [min_bits] * num_layers
    for i in order[:n_high]:
        bits[i] = max_bits
    return bits


def compute_token_bitwidths(seq_len: int, sink_size: int = 4, window_size: int = 64, high_bits: int = 4,
                            low_bits: int = 2) -> torch.Tensor:
    """[seq_len] int32: the first ``sink_size`` and the last ``window_size`` tokens at ``high_bits``, the
    rest at ``low_bits`` (token_importance.py:17-40)."""
    bits = torch.full((seq_len,), low_bits, dtype=torch.int32)
    bits[:min(sink_size, seq_len)] = high_bits
    if seq_len > sink_size + window_size:
        bits[-window_size:] = high_bits
    elif seq_len > sink_size:
        bits[sink_size:] = high_bits
    return bits


def runs_of(widths) -> list[tuple[int, int, int]]:
    """[(begin, end, bits)] maximal runs of equal width in a sequence of widths."""
    w = [int(x) for x in (widths.tolist() if isinstance(widths, torch.Tensor) else widths)]
    runs, start = [], 0
    for i in range(1, len(w) + 1):
        if i == len(w) or w[i] != w[start]:
            runs.append((start, i, w[start]))
            start = i
    return runs


@dataclass
class PartitionedKV:
    """Keys and values of one [batch, kv_heads, seq, head_dim] tensor pair, stored as one block_pq4 cache
    pair per run of the partition.  ``axis`` is "head" or "token"; ``runs`` = [(begin, end, bits)]."""
    axis: str
    runs: list[tuple[int, int, int]]
    keys: list[CompressedKV]
    values: list[CompressedKV]

    def memory_bytes(self) -> int:
        return sum(c.memory_bytes() for c in self.keys) + sum(c.memory_bytes() for c in self.values)

    @property
    def average_bits(self) -> float:
        total = sum((e - b) for b, e, _ in self.runs)
        return sum((e - b) * bits for b, e, bits in self.runs) / max(total, 1)


def mixed_precision_compress(key: torch.Tensor, value: torch.Tensor, rotation_matrix, widths, axis: str = "token"
                             ) -> PartitionedKV:
    """key, value float16 [batch, kv_heads, seq, head_dim]; ``widths`` = one width per token
    (compute_token_bitwidths) or per KV head.  Successor of token_importance.mixed_precision_compress
    (token_importance.py:43-79), which only counts the two classes."""
    if axis not in ("token", "head"):
        raise ValueError("axis must be 'token' or 'head'")
    dim = 2 if axis == "token" else 1
    if len(widths) != key.shape[dim]:
        raise ValueError(f"{len(widths)} widths for {key.shape[dim]} {axis}s")
    plan = device_plan(rotation_matrix, key.device)
    runs = runs_of(widths)
    ks, vs = [], []
    for b, e, bits in runs:
        sl = (slice(None), slice(None), slice(b, e)) if axis == "token" else (slice(None), slice(b, e))
        ks.append(quantizer.compress(key[sl].contiguous(), plan, bits))
        vs.append(quantizer.compress(value[sl].contiguous(), plan, bits))
    return PartitionedKV(axis, runs, ks, vs)


def mixed_precision_attention(query: torch.Tensor, cache: PartitionedKV, rotation_matrix,
                              out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """One query token per sequence, query [batch, q_heads, head_dim] float16 -> [batch, q_heads, head_dim]:
    non-causal attention over the whole partitioned cache."""
    plan = device_plan(rotation_matrix, query.device)
    B, Hq, D = query.shape
    if cache.axis == "head":
        Hkv = sum(e - b for b, e, _ in cache.runs)
        G = Hq // Hkv
        outs = [decode_attention(query[:, b * G:e * G].contiguous(), ck, cv, plan, enable_qjl=False, out_dtype=out_dtype)
                for (b, e, _), ck, cv in zip(cache.runs, cache.keys, cache.values)]
        return torch.cat(outs, dim=1)
    parts = [decode_attention(query, ck, cv, plan, enable_qjl=False, partial=True).reshape(B * Hq, D + 2)
             for ck, cv in zip(cache.keys, cache.values)]
    return lse_merge(torch.stack(parts), plan, out_dtype).reshape(B, Hq, D)


def estimate_mixed_compression_ratio(seq_len: int, sink_size: int = 4, window_size: int = 64, head_dim: int = 128) -> float:
    """float16 bytes over block_pq4 bytes for the sink + window policy (token_importance.py:82-90 counts
    index bits only; the two radius bytes per block are included here)."""
    bits = compute_token_bitwidths(seq_len, sink_size, window_size)
    per_tok = [(head_dim // 32) * (2 + 4 * int(b)) for b in bits.tolist()]
    return (2 * head_dim * seq_len) / max(sum(per_tok), 1)


def estimate_adaptive_compression_ratio(bitwidths, head_dim: int = 128) -> float:
    """float16 bits over the mean block_pq4 bits per value of a per-layer plan (adaptive_bitwidth.py:71-84
    amortises a float32 radius per vector; here every 32 values carry one float16 radius: 0.5 bit each)."""
    widths = [int(b) for b in bitwidths]
    if not widths:
        return 0.0
    return 16.0 / (sum(b + 16.0 / 32.0 for b in widths) / len(widths))
