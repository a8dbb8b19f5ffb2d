"""The reference's inference-side layers by name, over this package's cache manager.

``CompressedMultiHeadAttention`` has the interface of src/polarquant_kv_cuda/inference/attention.py:13-92
(bias-free q/k/v/o projections, an optional KVCacheManager per call, NON-causal attention over everything
the cache holds: the reference attends through compressed_attention_gpu, or scaled_dot_product_attention
without a mask).  ``SimpleTransformerLayer`` / ``SimpleTransformer`` are its test transformer
(inference/transformer.py:11-66): pre-norm layers of attention + GELU feed-forward, an embedding and an
output head, one cache manager per layer with rotation seeds 42 + layer.  Parameter names match, so a
state dict of the reference's modules loads.  The decoder in model.py is what the benchmark runs; these
exist so that code written against the reference's layers finds them."""

from __future__ import annotations

import torch
import torch.nn as nn

from .config import PolarQuantConfig
from .kv_cache import KVCacheManager


class CompressedMultiHeadAttention(nn.Module):
    def __init__(self, config: PolarQuantConfig, embed_dim: int, num_heads: int, num_kv_heads: int | None = None):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError(f"embed_dim {embed_dim} is not a multiple of num_heads {num_heads}")
        self.config, self.embed_dim, self.num_heads = config, embed_dim, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        if num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {self.num_kv_heads}")
        self.head_dim = embed_dim // num_heads
        kv_width = self.num_kv_heads * self.head_dim
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.k_proj = nn.Linear(embed_dim, kv_width, bias=False)
        self.v_proj = nn.Linear(embed_dim, kv_width, bias=False)
        self.o_proj = nn.Linear(embed_dim, embed_dim, bias=False)

    def _heads(self, t: torch.Tensor, n: int) -> torch.Tensor:
        b, s, _ = t.shape
        return t.view(b, s, n, self.head_dim).transpose(1, 2).to(torch.float16)

    def forward(self, x: torch.Tensor, cache_manager: KVCacheManager | None = None) -> torch.Tensor:
        """x [batch, seq, embed_dim] -> [batch, seq, embed_dim]; with a cache manager the new keys and
        values are appended first and the queries attend to the whole cache."""
        b, s, _ = x.shape
        q = self._heads(self.q_proj(x), self.num_heads)
        k = self._heads(self.k_proj(x), self.num_kv_heads)
        v = self._heads(self.v_proj(x), self.num_kv_heads)
        if cache_manager is None:
            rep = self.num_heads // self.num_kv_heads
            out = torch.nn.functional.scaled_dot_product_attention(
                q.float(), k.float().repeat_interleave(rep, dim=1), v.float().repeat_interleave(rep, dim=1))
        else:
            cache_manager.append(k.contiguous(), v.contiguous())
            out = cache_manager.attend(q.contiguous(), causal=False)
        out = out.transpose(1, 2).reshape(b, s, self.embed_dim)
        return self.o_proj(out.to(self.o_proj.weight.dtype))


class SimpleTransformerLayer(nn.Module):
    def __init__(self, config: PolarQuantConfig, embed_dim: int, num_heads: int,
                 num_kv_heads: int | None = None, ffn_dim: int | None = None):
        super().__init__()
        self.attn = CompressedMultiHeadAttention(config, embed_dim, num_heads, num_kv_heads)
        self.norm1, self.norm2 = nn.LayerNorm(embed_dim), nn.LayerNorm(embed_dim)
        hidden = ffn_dim or 4 * embed_dim
        self.ffn = nn.Sequential(nn.Linear(embed_dim, hidden, bias=False), nn.GELU(),
                                 nn.Linear(hidden, embed_dim, bias=False))

    def forward(self, x: torch.Tensor, cache_manager: KVCacheManager | None = None) -> torch.Tensor:
        x = x + self.attn(self.norm1(x.float()), cache_manager)
        return x + self.ffn(self.norm2(x.float()))


class SimpleTransformer(nn.Module):
    def __init__(self, config: PolarQuantConfig, num_layers: int, embed_dim: int, num_heads: int,
                 num_kv_heads: int | None = None, vocab_size: int = 1000):
        super().__init__()
        self.config = config
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads or num_heads
        self.head_dim = embed_dim // num_heads
        self.embed = nn.Embedding(vocab_size, embed_dim)
        self.layers = nn.ModuleList(SimpleTransformerLayer(config, embed_dim, num_heads, num_kv_heads)
                                    for _ in range(num_layers))
        self.head = nn.Linear(embed_dim, vocab_size, bias=False)

    def forward(self, input_ids: torch.Tensor, cache_managers: list[KVCacheManager] | None = None) -> torch.Tensor:
        x = self.embed(input_ids).float()
        for i, layer in enumerate(self.layers):
            x = layer(x, cache_managers[i] if cache_managers else None)
        return self.head(x.float())

    def create_cache_managers(self, max_seq_len: int, batch: int, device: str = "cuda") -> list[KVCacheManager]:
        return [KVCacheManager(self.config, max_seq_len, batch, self.num_kv_heads, self.head_dim, device,
                               rotation_seed=42 + i) for i in range(len(self.layers))]
