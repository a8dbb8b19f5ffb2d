"""A decoder-only language model that keeps its KV cache compressed.

Successor of CompressedMultiHeadAttention / SimpleTransformer
(src/polarquant_kv_cuda/inference/attention.py:13-92, transformer.py:11-66 of the reference), in the
shape of a current decoder: RMSNorm, rotary position embedding, grouped-query attention with biases on
the q/k/v projections, SwiGLU MLP.  Keys and values are compressed on write (after the rotary
embedding) and read by the fused attention kernels; every layer has its own rotation, seeds 42 + layer
as the reference's create_cache_managers (transformer.py:58-66).  The dense layers are plain torch
(library GEMMs): they are not part of the compressed-cache path.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import PolarQuantConfig
from .kv_cache import KVCacheManager


@dataclass
class DecoderConfig:
    """Defaults: the Qwen2.5-0.5B architecture."""
    num_layers: int = 24
    hidden: int = 896
    q_heads: int = 14
    kv_heads: int = 2
    head_dim: int = 64
    intermediate: int = 4864
    vocab: int = 151936
    rope_theta: float = 1.0e6
    rms_eps: float = 1.0e-6


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """positions [S] -> (cos, sin), each [S, head_dim] float32 (the rotate_half convention: the angle
    of pair i sits at columns i and i + head_dim / 2).  One pair of tables serves every layer of a step."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return torch.cos(ang).repeat(1, 2), torch.sin(ang).repeat(1, 2)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, S, D] -> float32 x * cos + rotate_half(x) * sin."""
    D = x.shape[-1]
    xf = x.float()
    rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], dim=-1)
    return torch.addcmul(xf * cos, rot, sin)


def rotary(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, H, S, D], positions [S] -> rotated halves (the rotate_half convention)."""
    return apply_rotary(x, *rotary_tables(positions, x.shape[-1], theta))


class _FusedLinear:
    """The weights (and biases) of several nn.Linear layers that read the same input, stacked so that one
    GEMM serves them all; rebuilt when a layer's parameters were modified in place or moved."""

    def __init__(self, *layers: nn.Linear):
        self.layers = layers
        self.key = None
        self.weight = self.bias = None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        key = tuple((l.weight._version, l.weight.data_ptr(), l.weight.dtype) for l in self.layers)
        if key != self.key:
            self.weight = torch.cat([l.weight.detach() for l in self.layers], dim=0)
            self.bias = (torch.cat([l.bias.detach() for l in self.layers], dim=0)
                         if self.layers[0].bias is not None else None)
            self.key = key
        return F.linear(x, self.weight, self.bias)


class CompressedAttention(nn.Module):
    """q/k/v projections, rotary embedding, cache append, attention over the cache, output projection."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.q_proj = nn.Linear(cfg.hidden, cfg.q_heads * cfg.head_dim, bias=True)
        self.k_proj = nn.Linear(cfg.hidden, cfg.kv_heads * cfg.head_dim, bias=True)
        self.v_proj = nn.Linear(cfg.hidden, cfg.kv_heads * cfg.head_dim, bias=True)
        self.o_proj = nn.Linear(cfg.q_heads * cfg.head_dim, cfg.hidden, bias=False)
        self._qkv = _FusedLinear(self.q_proj, self.k_proj, self.v_proj)

    def forward(self, x: torch.Tensor, cache: KVCacheManager, timers=None, device_step=None, rope=None) -> torch.Tensor:
        """``device_step`` = (position, length) one-element int64 device tensors: the step's token
        position and the number of cached tokens after the append, both read on the device.
        ``rope`` = (cos, sin) of the step's positions (rotary_tables); computed here when absent."""
        c = self.cfg
        B, S, _ = x.shape
        if rope is None:
            pos = device_step[0] if device_step is not None else \
                torch.arange(cache.seq_len, cache.seq_len + S, device=x.device)
            rope = rotary_tables(pos, c.head_dim, c.rope_theta)
        # one GEMM for the three projections; the rotary embedding runs over the query and key heads together
        qkv = self._qkv(x).view(B, S, c.q_heads + 2 * c.kv_heads, c.head_dim).transpose(1, 2)
        qk = apply_rotary(qkv[:, :c.q_heads + c.kv_heads], *rope).to(torch.float16)
        q, k = qk[:, :c.q_heads], qk[:, c.q_heads:]
        v = qkv[:, c.q_heads + c.kv_heads:].to(torch.float16)
        if timers is not None:
            timers.start()
        if device_step is not None:
            cache.append(k.contiguous(), v.contiguous(), position=device_step[0])
            out = cache.attend(q.contiguous(), seq_len_tensor=device_step[1])
        else:
            cache.append(k.contiguous(), v.contiguous())
            out = cache.attend(q.contiguous(), causal=True)
        if timers is not None:
            timers.stop()
        out = out.to(x.dtype).transpose(1, 2).reshape(B, S, c.q_heads * c.head_dim)
        return self.o_proj(out)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.attn = CompressedAttention(cfg)
        self.norm1, self.norm2 = RMSNorm(cfg.hidden, cfg.rms_eps), RMSNorm(cfg.hidden, cfg.rms_eps)
        self.gate = nn.Linear(cfg.hidden, cfg.intermediate, bias=False)
        self.up = nn.Linear(cfg.hidden, cfg.intermediate, bias=False)
        self.down = nn.Linear(cfg.intermediate, cfg.hidden, bias=False)
        self._gate_up = _FusedLinear(self.gate, self.up)

    def forward(self, x, cache, timers=None, device_step=None, rope=None):
        x = x + self.attn(self.norm1(x), cache, timers, device_step, rope)
        g, u = self._gate_up(self.norm2(x)).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


class KernelTimer:
    """Accumulates device time spent between start() and stop() (the compressed-cache kernels)."""

    def __init__(self):
        self.pairs = []

    def start(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open = e

    def stop(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs.append((self._open, e))

    def total_ms(self) -> float:
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.pairs)


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig, pq: PolarQuantConfig):
        super().__init__()
        self.cfg, self.pq = cfg, pq
        self.embed = nn.Embedding(cfg.vocab, cfg.hidden)
        self.layers = nn.ModuleList([DecoderLayer(cfg) for _ in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden, cfg.rms_eps)
        self.head = nn.Linear(cfg.hidden, cfg.vocab, bias=False)

    @torch.no_grad()
    def init_random(self, seed: int = 0, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        """Random weights (normal, std 0.02; norm weights one) drawn on ``device`` from ``seed``, in ``dtype``."""
        self.to(device=device, dtype=dtype)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        for name, prm in self.named_parameters():
            if name.endswith("norm1.weight") or name.endswith("norm2.weight") or name == "norm.weight":
                prm.fill_(1.0)
            else:
                prm.copy_((torch.randn(prm.shape, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype))
        return self

    def create_cache_managers(self, max_seq_len: int, batch: int, device="cuda") -> list[KVCacheManager]:
        c = self.cfg
        return [KVCacheManager(self.pq, max_seq_len, batch, c.kv_heads, c.head_dim, device, rotation_seed=42 + i)
                for i in range(c.num_layers)]

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, caches: list[KVCacheManager], timers=None, last_only: bool = True):
        """input_ids [B, S] (a prompt, or S == 1 for a decode step) -> logits of the last position
        [B, vocab] (or of every position with last_only=False)."""
        x = self.embed(input_ids)
        start = caches[0].seq_len
        rope = rotary_tables(torch.arange(start, start + input_ids.shape[1], device=input_ids.device),
                             self.cfg.head_dim, self.cfg.rope_theta)
        for layer, cache in zip(self.layers, caches):
            x = layer(x, cache, timers, None, rope)
        x = self.norm(x[:, -1:] if last_only else x)
        return self.head(x).float().squeeze(1) if last_only else self.head(x).float()

    @torch.no_grad()
    def _device_step(self, token: torch.Tensor, caches, state) -> None:
        """One greedy step whose position, cache length and output slot live on the device:
        ``token`` [B, 1] is consumed and overwritten with the next token."""
        position, length, step, out = state
        out.index_copy_(1, step, token)
        x = self.embed(token)
        rope = rotary_tables(position, self.cfg.head_dim, self.cfg.rope_theta)
        for layer, cache in zip(self.layers, caches):
            x = layer(x, cache, None, (position, length), rope)
        logits = self.head(self.norm(x)).float().squeeze(1)
        token.copy_(logits.argmax(-1, keepdim=True))
        position.add_(1)
        length.add_(1)
        step.add_(1)

    @torch.no_grad()
    def decode_graph(self, token: torch.Tensor, steps: int, caches: list[KVCacheManager]) -> torch.Tensor:
        """``steps`` greedy single-token steps after a prefill, starting from ``token`` [B, 1], replayed
        from ONE CUDA graph: the position and the cache length advance in device memory
        (pq_compress_rows_dynamic, pq_decode_attn_dynamic), so the 22 or so kernels per layer are launched by
        one graph launch per token instead of one Python call each.  The first step runs eagerly (it
        also warms the libraries up), the second is recorded, the rest are replays.  Returns the ids
        fed and generated, [B, steps]."""
        B = token.shape[0]
        start = caches[0].seq_len
        if start + steps > caches[0].max_seq_len:
            raise RuntimeError(f"KV cache full: {start} + {steps} > {caches[0].max_seq_len}")
        dev = token.device
        if steps == 0:
            return token[:, :0]
        token = token.clone()
        state = (torch.full((1,), start, dtype=torch.int64, device=dev),
                 torch.full((1,), start + 1, dtype=torch.int64, device=dev),
                 torch.zeros(1, dtype=torch.int64, device=dev),
                 torch.empty((B, steps), dtype=token.dtype, device=dev))
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._device_step(token, caches, state)
        torch.cuda.current_stream(dev).wait_stream(side)
        if steps > 1:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._device_step(token, caches, state)
            for _ in range(steps - 1):
                graph.replay()
        for cache in caches:
            cache.advance(steps)
        return state[3]

    @torch.no_grad()
    def generate_graph(self, prompt_ids: torch.Tensor, steps: int, caches: list[KVCacheManager]) -> torch.Tensor:
        """``generate`` with the single-token steps served by ``decode_graph``."""
        if prompt_ids.shape[1] + steps > caches[0].max_seq_len:
            raise RuntimeError(f"KV cache full: {prompt_ids.shape[1]} + {steps} > {caches[0].max_seq_len}")
        token = self.forward(prompt_ids, caches).argmax(-1, keepdim=True)
        return self.decode_graph(token, steps, caches)

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, steps: int, caches: list[KVCacheManager], timers=None) -> torch.Tensor:
        """Greedy decoding: one prefill pass over the prompt [B, S], then ``steps`` single-token steps.
        Returns the generated ids [B, steps]."""
        logits = self.forward(prompt_ids, caches, timers)
        out = []
        tok = logits.argmax(-1, keepdim=True)
        for _ in range(steps):
            out.append(tok)
            logits = self.forward(tok, caches, timers)
            tok = logits.argmax(-1, keepdim=True)
        return torch.cat(out, dim=1)
