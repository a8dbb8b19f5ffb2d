"""Hugging Face `transformers` cache whose storage is block_pq4.

Successor of CompressedDynamicCache / patch_model / create_compressed_cache
(src/polarquant_kv_cuda/hf_integration.py:21-127 of the reference).  The reference's cache keeps the
full float16 cache and only shadows it with a compressed copy that never feeds attention
(hf_integration.py:43-62); here the compressed blocks ARE the cache: ``update`` compresses the new
keys / values in place (one pq_compress_rows launch per tensor) and hands the model the dequantised
tensors (pq_dequant) that its own attention implementation consumes, so any `transformers` decoder runs
over it unchanged.  Every layer has its own rotation, seeds 42 + layer (hf_integration.py:30-34).

`transformers` is imported lazily: the rest of the package does not depend on it.
"""

from __future__ import annotations

import torch

from . import quantizer
from .rotation import device_plan, generate_rotation_matrix


def _layer_base():
    from transformers.cache_utils import DynamicLayer
    return DynamicLayer


def make_layer_class():
    DynamicLayer = _layer_base()

    class PolarQuantLayer(DynamicLayer):
        """One layer's keys and values as block_pq4 caches of a fixed capacity, grown by doubling."""

        def __init__(self, layer_idx: int, n_bits: int = 4, v_bits: int | None = None, initial_capacity: int = 256):
            super().__init__()
            self.layer_idx, self.k_bits, self.v_bits = layer_idx, n_bits, v_bits or n_bits
            self.capacity = initial_capacity
            self.ck = self.cv = self.plan = None
            self.length = 0

        def lazy_initialization(self, key_states, value_states):
            self.dtype, self.device = key_states.dtype, key_states.device
            B, H, _, D = key_states.shape
            self.plan = device_plan(generate_rotation_matrix(D, seed=42 + self.layer_idx), self.device)
            self.ck = quantizer.allocate_cache(B, H, self.capacity, D, self.k_bits, 0, self.device)
            self.cv = quantizer.allocate_cache(B, H, self.capacity, D, self.v_bits, 0, self.device)
            self.keys = torch.tensor([], dtype=self.dtype, device=self.device)      # kept for the base class
            self.values = torch.tensor([], dtype=self.dtype, device=self.device)
            self.is_initialized = True

        def _grow(self, need: int):
            cap = self.capacity
            while cap < need:
                cap *= 2
            for name in ("ck", "cv"):
                old = getattr(self, name)
                B, H = old.blocks.shape[:2]
                new = quantizer.allocate_cache(B, H, cap, old.original_dim, old.n_bits, 0, self.device)
                new.blocks[:, :, :self.length].copy_(old.blocks[:, :, :self.length])
                new.seq_len = self.length
                setattr(self, name, new)
            self.capacity = cap

        def update(self, key_states, value_states, *args, **kwargs):
            if not self.is_initialized:
                self.lazy_initialization(key_states, value_states)
            new = key_states.shape[-2]
            if self.length + new > self.capacity:
                self._grow(self.length + new)
            quantizer.compress(key_states.to(torch.float16), self.plan, self.k_bits, out=self.ck, position=self.length)
            quantizer.compress(value_states.to(torch.float16), self.plan, self.v_bits, out=self.cv, position=self.length)
            self.length += new
            self.ck.seq_len = self.cv.seq_len = self.length
            keys = quantizer.decompress(self.ck, self.plan, torch.float16).to(self.dtype)
            values = quantizer.decompress(self.cv, self.plan, torch.float16).to(self.dtype)
            return keys, values

        def get_seq_length(self) -> int:
            return self.length

        def get_mask_sizes(self, query_length: int):
            return self.length + query_length, 0

        def compressed_bytes(self) -> int:
            if self.ck is None:
                return 0
            per_tok = self.ck.blocks.shape[0] * self.ck.blocks.shape[1]
            return per_tok * self.length * (self.ck.blocks.shape[3] * self.ck.blocks.shape[4] +
                                            self.cv.blocks.shape[3] * self.cv.blocks.shape[4])

    return PolarQuantLayer


def CompressedDynamicCache(n_bits: int = 4, group_size: int = 32, head_dim: int = 64, num_layers: int = 24,
                           v_bits: int | None = None):
    """A `transformers` Cache with one PolarQuantLayer per decoder layer (the reference's constructor
    signature, hf_integration.py:24).  head_dim is taken from the first update; it is accepted for
    signature compatibility.  Extra methods: get_compressed_memory_bytes(), get_standard_memory_bytes()."""
    if group_size != 32:
        raise ValueError("block_pq4 uses blocks of 32 elements")
    from transformers.cache_utils import Cache
    Layer = make_layer_class()

    class _Cache(Cache):
        def get_compressed_memory_bytes(self) -> int:
            return sum(layer.compressed_bytes() for layer in self.layers)

        def get_standard_memory_bytes(self) -> int:
            total = 0
            for layer in self.layers:
                if layer.ck is not None:
                    B, H = layer.ck.blocks.shape[:2]
                    total += 2 * B * H * layer.length * layer.ck.original_dim * 2
            return total

    return _Cache(layers=[Layer(i, n_bits, v_bits) for i in range(num_layers)])


def patch_model(model, n_bits: int = 4, group_size: int = 32):
    """Records the compression settings on the model (hf_integration.py:92-116); pass
    ``past_key_values=create_compressed_cache(model)`` to ``generate`` / ``forward``."""
    cfg = model.config
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    model._polarquant_config = {"n_bits": n_bits, "group_size": group_size, "head_dim": head_dim,
                                "num_layers": cfg.num_hidden_layers}
    return model


def create_compressed_cache(model):
    c = model._polarquant_config
    return CompressedDynamicCache(n_bits=c["n_bits"], group_size=c["group_size"], head_dim=c["head_dim"],
                                  num_layers=c["num_layers"])
