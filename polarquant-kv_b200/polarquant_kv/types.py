"""Result containers, mirroring python/polarquant_kv/types.py and
src/polarquant_kv_cuda/types.py of the reference on the block_pq4 layout."""

from __future__ import annotations

from dataclasses import dataclass

import torch

BLOCK = 32


def block_bytes(n_bits: int) -> int:
    if n_bits not in (2, 4):
        raise ValueError(f"block_pq4 supports n_bits 2 or 4 on the GPU, got {n_bits}")
    return 2 + BLOCK * n_bits // 8


@dataclass
class CompressedKV:
    """A compressed K or V tensor on the GPU.

    blocks          uint8 [batch, heads, max_seq_len, head_dim/32, 2 + 32*n_bits/8]
                    = {float16 d, packed Lloyd-Max indices} per 32 elements
    qjl_signs       uint8 [batch, heads, max_seq_len, jl_dim/8] or None
    residual_norms  float16 [batch, heads, max_seq_len] or None
    The field names n_bits / group_size / original_dim / seq_len / max_seq_len are the
    reference's (CompressedKVCacheGPU); group_size is always 32 here.
    """

    blocks: torch.Tensor
    qjl_signs: torch.Tensor | None
    residual_norms: torch.Tensor | None
    n_bits: int
    group_size: int
    original_dim: int
    seq_len: int
    max_seq_len: int

    @property
    def radius(self) -> torch.Tensor:
        """float16 [batch, heads, seq, head_dim/32]: the per-block radii (a copy)."""
        b = self.blocks[..., :2].contiguous()
        return b.view(torch.float16).squeeze(-1)

    @property
    def quantized_direction(self) -> torch.Tensor:
        """uint8 [batch, heads, seq, head_dim * n_bits / 8]: packed indices (a copy)."""
        return self.blocks[..., 2:].reshape(*self.blocks.shape[:3], -1)

    def memory_bytes(self) -> int:
        total = self.blocks.numel()
        if self.qjl_signs is not None:
            total += self.qjl_signs.numel()
        if self.residual_norms is not None:
            total += self.residual_norms.numel() * 2
        return total


# the reference's GPU-side name for the same thing
CompressedKVCacheGPU = CompressedKV


@dataclass
class QJLSignatures:
    """Sign sketch of quantisation residuals (python/polarquant_kv/types.py:21-27 of the reference).

    signs          bool [..., jl_dim]: sign(P e) >= 0
    jl_dim         number of projections
    residual_norm  ||e||: a float for one vector (as in the reference) or a tensor [...] for a batch
    """

    signs: torch.Tensor
    jl_dim: int
    residual_norm: float | torch.Tensor = 0.0


@dataclass
class CompressedKVCache:
    """Key + value + optional key signatures (python/polarquant_kv/types.py:30-35).  On the GPU path
    the keys' sketch normally lives inside compressed_keys (qjl_signs / residual_norms);
    key_signatures is kept for code written against the reference's container."""

    compressed_keys: CompressedKV
    compressed_values: CompressedKV
    key_signatures: QJLSignatures | None = None
