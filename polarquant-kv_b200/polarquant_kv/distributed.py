"""Multi-GPU use of the path (one process per GPU, torch.distributed).

The reference has no multi-GPU code.  Two schemes cover the path:

* batch / KV-head sharding — rows are independent, every rank runs the plain kernels on its
  own sequences and nothing is exchanged (``batch_shard``);
* sequence sharding of ONE long sequence — every rank holds a contiguous slice of the
  cache, computes the partial softmax state (m, l, o_rot) of its slice with
  ``pq_decode_attn(partial_out=...)``, the ranks all-gather those records
  (``q_heads * (head_dim + 2)`` floats each) and every rank merges them with
  ``pq_lse_merge`` (log-sum-exp merge + inverse rotation); ``PeerExchange`` does the exchange and the
  merge in ONE kernel over NVLink peer memory instead (``pq_lse_exchange_merge``).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _ext


def batch_shard(batch: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the sequences rank ``rank`` owns; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def sequence_shard(seq_len: int, rank: int, world: int, align: int = 16) -> tuple[int, int]:
    """[begin, end) of the tokens rank ``rank`` owns when one sequence is cut into ``world``
    contiguous slices.  Slice boundaries are multiples of ``align`` tokens (the decode
    kernel's tile) except the last end; trailing ranks may get an empty slice."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if seq_len < 0 or align <= 0:
        raise ValueError("seq_len must be >= 0 and align > 0")
    tiles = (seq_len + align - 1) // align
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * align, seq_len), min(t1 * align, seq_len)


def gather_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-rank records: [rows, D+2] -> [world, rows, D+2] on every rank.
    Works on any backend (NCCL over NVLink on GPUs; gloo in the CPU tests)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(partial.shape), dtype=partial.dtype, device=partial.device)
    dist.all_gather([out[r] for r in range(world)], partial.contiguous(), group=group)
    return out


def lse_merge(partials: torch.Tensor, plan, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """[n_parts, rows, D+2] float32 CUDA records -> [rows, D] (pq_lse_merge)."""
    if not partials.is_cuda:
        raise TypeError("partials must be a CUDA tensor: this package has no CPU path")
    n_parts, rows, width = partials.shape
    D = width - 2
    out = torch.empty((rows, D), dtype=out_dtype, device=partials.device)
    st = _ext.lib().pq_lse_merge(partials.contiguous().data_ptr(), n_parts, rows, D, plan.rot.data_ptr(),
                                 out.data_ptr(), 1 if out_dtype == torch.float16 else 0,
                                 ctypes.c_void_p(torch.cuda.current_stream(partials.device).cuda_stream))
    _ext.check(st, "pq_lse_merge")
    return out


class PeerExchange:
    """Exchange of the partial records and their merge as one kernel over peer memory
    (pq_lse_exchange_merge): every rank's kernel stores its records into the peers' buffers with plain
    NVLink stores, counts itself in with a system-scope atomic, waits (bounded) for the peers' records
    and merges.  The buffers are symmetric allocations of torch.distributed (one per rank, addressable
    by every rank of the node).  Every rank must call ``merge`` the same number of times, in the same
    order; at most eight ranks.  ``close`` (or the end of the process) releases the buffers."""

    def __init__(self, rows: int, head_dim: int, device, group=None):
        import os
        # plain peer stores only: keep the allocation off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("PeerExchange serves at most eight ranks")
        self.rows, self.head_dim, self.device = rows, head_dim, torch.device(device)
        lib = _ext.lib()
        nbytes = lib.pq_lse_exchange_bytes(self.world, rows, head_dim)
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group.group_name)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)                     # every rank's counters read zero before anyone counts
        ptrs = [int(x) for x in self.handle.buffer_ptrs]
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self.epoch = 0

    def merge(self, partial: torch.Tensor, plan, out_dtype: torch.dtype = torch.float32,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """partial float32 [rows, D+2] of this rank -> merged, rotated-back [rows, D] on every rank."""
        if partial.dtype != torch.float32 or tuple(partial.shape) != (self.rows, self.head_dim + 2) \
                or not partial.is_contiguous() or partial.device != self.device:
            raise ValueError("partial must be a contiguous float32 [rows, head_dim + 2] tensor on the exchange's device")
        if out is None:
            out = torch.empty((self.rows, self.head_dim), dtype=out_dtype, device=self.device)
        self.epoch += 1
        st = _ext.lib().pq_lse_exchange_merge(
            partial.data_ptr(), self.world, self.rank, self._ptrs, self.epoch, self.rows, self.head_dim,
            plan.rot.data_ptr(), out.data_ptr(), 1 if out.dtype == torch.float16 else 0,
            ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        _ext.check(st, "pq_lse_exchange_merge")
        return out

    def close(self) -> None:
        self.handle = None
        self.buf = None


def sharded_decode_attention(query: torch.Tensor, ck_local, cv_local, plan, group=None,
                             enable_qjl: bool = True, scale: float | None = None,
                             out_dtype: torch.dtype = torch.float32,
                             exchange: PeerExchange | None = None) -> torch.Tensor:
    """Decode attention over a sequence whose cache is split across the ranks of ``group``.

    query [B, Hq, D] (replicated); ck_local / cv_local hold this rank's slice of the
    sequence (``seq_len`` may be 0).  Returns [B, Hq, D] on every rank.  With ``exchange`` (a
    PeerExchange for B * Hq rows) the records travel and merge in one kernel over peer memory;
    otherwise by an all-gather of the process group followed by ``pq_lse_merge``."""
    from .attention import decode_attention
    B, Hq, D = query.shape
    part = decode_attention(query, ck_local, cv_local, plan, enable_qjl=enable_qjl, scale=scale, partial=True)
    if exchange is not None:
        return exchange.merge(part.reshape(B * Hq, D + 2), plan, out_dtype).reshape(B, Hq, D)
    allp = gather_partials(part.reshape(B * Hq, D + 2), group)
    return lse_merge(allp, plan, out_dtype).reshape(B, Hq, D)
