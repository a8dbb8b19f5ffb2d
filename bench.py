"""Benchmark of the PQ4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload ("step" = one decode-attention pass over the batch): Llama-3-8B-shaped decode
over a PQ4 (4-bit block_pq4) cache — batch 32, 8 KV heads, 32 query heads, head_dim 128, context
8192, one query token per sequence, the batch SHARDED across the GPUs (32/N sequences per rank, no
collective; strong scaling).  Metric: compressed K/V bytes streamed per second (GB/s), each stored
byte counted once per KV head.  At N > 1 the line also carries `weak_scaling` (batch 32 on every
rank) for comparison.

Timing: W >= 3 warm-up steps, then blocks of exactly K steps, each bracketed by a barrier and a
device synchronisation; the block time is taken with CUDA events on the launching stream.  The block
is repeated (15 times by default) and every rank reports the MEDIAN block; the job's time is the
maximum of those medians over the ranks (`per_rank_ms` lists them).  Steps go through a prepared
call (all host-side set-up done once), two caches alternate so no step finds its data in L2.

Other objects on the JSON line: `roofline` (dominant kernel against the measured HBM copy
bandwidth), `e2e` (same step through the public API with host buffers: query copied from pinned host
memory, output copied back), `parity_sample_max_abs` (one (batch, kv-head) row of the very cache that
was timed, against the numpy oracle), `long_context` (one 131072-token sequence split along the
sequence across the ranks: partial decode, then the exchange and merge of the per-rank records as one kernel
over NVLink peer memory, with the all-gather + merge path timed beside it), `compress` (2^24 K vectors with the
QJL sketch + 2^24 V vectors, per variant), `dequant`, `prefill`, `llama_bridge` (the llama.cpp bridge's
entry points), `e2e_model` (a Qwen2.5-0.5B-shaped decoder over the compressed cache: 64 prompts of 4096
tokens, 256 greedy steps, one CUDA graph launch per token; the same steps issued kernel by kernel under
`eager`), `cpu_baseline` (the numpy oracle on a bounded sample, and the reference's own CPU functions as
shipped on its CPU-runnable case and on a 16384-vector sample of the bulk-compress workload) and the clocks
sampled during the timed region.

`--impl reference` times the CPU implementation of the same step (the numpy restatement of the
reference algorithm, oracle/pq_oracle.py, on all host cores, on a bounded sample per step).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "polarquant-kv_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOAD = dict(name="llama3-8b-shaped PQ4 decode attention", batch=32, kv_heads=8, q_heads=32,
                head_dim=128, context=8192, k_bits=4, v_bits=4)
LONG_CONTEXT = dict(name="single long sequence, sequence-sharded", batch=1, kv_heads=8, q_heads=64,
                    head_dim=128, context=131072, k_bits=4, v_bits=4)
COMPRESS_VECS = 1 << 24        # K vectors and V vectors per compress measurement
FALLBACK_HBM_GBS = 6650.0      # used only when MEASURED_PEAKS.json is absent
BLOCK_REPEATS = 15


def algorithmic_bytes(w, batch=None) -> int:
    """Compressed K + V bytes one decode step must read: B * Hkv * S * 2 * (D/32) * 18."""
    per_token = (w["head_dim"] // 32) * ((2 + 4 * w["k_bits"]) + (2 + 4 * w["v_bits"]))
    return (w["batch"] if batch is None else batch) * w["kv_heads"] * w["context"] * per_token


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s measured on this pool (burst figure: the prefill kernel is timed alone);
    falls back to the earlier pool measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax,
               "samples": len(sm), "reasons": sorted(reasons)}
        if not sm and self.lines:
            out["error"] = self.lines[0][:200]
        return out


# ----------------------------------------------------------------------------- CPU arm
def _cpu_rows(args):
    """Worker: decode attention of `n_rows` (batch, kv head) rows with the numpy oracle."""
    import numpy as np
    from oracle import pq_oracle as O
    n_rows, seed, w = args
    D, S, G = w["head_dim"], w["context"], w["q_heads"] // w["kv_heads"]
    rng = np.random.default_rng(seed)
    R = O.rotation_matrix(D, 0)
    cb, _ = O.lloyd_max_codebook(32, 4, n_iterations=50, grid_size=5000)
    nblk = D // 32
    kb = rng.integers(0, 256, (1, S, nblk, 18), dtype=np.uint8)
    vb = rng.integers(0, 256, (1, S, nblk, 18), dtype=np.uint8)
    one = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    kb[..., 0:2] = one
    vb[..., 0:2] = one
    q = rng.standard_normal((G, 1, D)).astype(np.float16)
    t0 = time.perf_counter()
    for _ in range(n_rows):
        O.attention_from_blocks(q, kb, vb, R, cb, cb)
    return time.perf_counter() - t0


def cpu_arm(pool, w, n_procs: int, rows_per_proc: int):
    """Rate (compressed GB/s) of the oracle port over n_procs worker processes (pool already
    started, so interpreter start-up is outside the timing); returns (GB/s, seconds)."""
    per_row = algorithmic_bytes(w) // (w["batch"] * w["kv_heads"])
    t0 = time.perf_counter()
    pool.map(_cpu_rows, [(rows_per_proc, i, w) for i in range(n_procs)])
    dt = time.perf_counter() - t0
    return per_row * rows_per_proc * n_procs / dt / 1e9, dt


def reference_as_shipped():
    """The reference's own numpy code (staged by oracle/build_ref.py, when present), unmodified, single
    process: compress_batch + compressed_attention on the CPU-runnable configuration (1 x 2 KV heads x
    512 tokens x 64 dims, 14 query heads).  Its quantizer is the reference's group-min/max one — the
    block_pq4 layout exists only as prose there — so this is the reference's CPU path as a user runs
    it, not the same codec."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "polarquant_kv")):
        return {"available": False, "why": "oracle/_ref not staged (no reference checkout at build time)"}
    script = (
        "import sys, time, json, numpy as np\n"
        f"sys.path.insert(0, {ref_dir!r}); sys.path.insert(0, {ROOT!r})\n"
        "from oracle import inputs\n"
        "from polarquant_kv.rotation import generate_rotation_matrix\n"
        "from polarquant_kv.quantizer import compress_batch\n"
        "from polarquant_kv.attention import compressed_attention\n"
        "K, V, q = inputs.make_kvq(**inputs.C0)\n"
        "R = generate_rotation_matrix(64, 0)\n"
        "t0 = time.perf_counter(); compress_batch(K.astype(np.float32), R, 4, 32); t1 = time.perf_counter()\n"
        "out = compressed_attention(q[0].astype(np.float32), K[0].astype(np.float32), V[0].astype(np.float32), R, None, 4, 32, False, 2)\n"
        "t2 = time.perf_counter()\n"
        # a fixed sub-sample of the bulk-compress workload: 16384 vectors of head dim 128, same distribution
        "K2, _, _ = inputs.make_kvq(1, 1, 1, 16384, 128, seed=0)\n"
        "R2 = generate_rotation_matrix(128, 0)\n"
        "t3 = time.perf_counter(); compress_batch(K2.astype(np.float32), R2, 4, 32); t4 = time.perf_counter()\n"
        "print(json.dumps({'compress_batch_s': t1 - t0, 'vectors': int(K.shape[1] * K.shape[2]), 'compressed_attention_s': t2 - t1,"
        " 'bulk_vectors': 16384, 'bulk_compress_s': t4 - t3}))\n")
    try:
        env = dict(os.environ, OMP_NUM_THREADS="1", OPENBLAS_NUM_THREADS="1")
        res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=120, env=env)
        d = json.loads(res.stdout.strip().splitlines()[-1])
    except Exception as e:   # the staged copy is optional: report, do not fail the benchmark
        return {"available": False, "why": f"{type(e).__name__}: {e}"[:200]}
    return {"available": True, "cores": 1, "config": "1 x 2 KV heads x 512 tokens x 64 dims, 14 query heads, 4-bit",
            "compress_vectors_per_s": round(d["vectors"] / d["compress_batch_s"], 1),
            "compressed_attention_s": round(d["compressed_attention_s"], 3),
            "kv_tokens_x_q_heads_per_s": round(512 * 14 / d["compressed_attention_s"], 1),
            "bulk_compress_sample": {"vectors": d["bulk_vectors"], "head_dim": 128,
                                     "vectors_per_s": round(d["bulk_vectors"] / d["bulk_compress_s"], 1)}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 64))
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    import multiprocessing as mp
    rows = 2
    steps = []
    with mp.get_context("spawn").Pool(procs) as pool:
        for _ in range(max(1, args.warmup)):
            cpu_arm(pool, w, procs, 1)           # warm-up (imports, codebook, BLAS start-up)
        for _ in range(max(1, args.steps)):
            steps.append(cpu_arm(pool, w, procs, rows))
    gbs = sum(g for g, _ in steps) / len(steps)
    ms_step = 1e3 * sum(t for _, t in steps) / len(steps)
    full_step_s = algorithmic_bytes(w) / 1e9 / gbs
    sample = (f"each step = {procs} processes x {rows} (batch, kv-head) rows of the workload "
              f"({procs * rows} of {w['batch'] * w['kv_heads']} rows), numpy oracle port of the reference "
              "algorithm (vectorised; the reference's own per-token Python loop is slower)")
    line = {
        "impl": "reference", "metric": "PQ4 decode-attn compressed-byte throughput", "value": round(gbs, 4),
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 2), "ms_per_full_workload_step_extrapolated": round(full_step_s * 1e3, 1),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"}},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": procs, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def synthetic_kv(shape, dev, gen):
    """The benchmark distribution: N(0,1) x per-channel lognormal(0,1), two channels x10, float16."""
    import torch
    D = shape[-1]
    scale = torch.exp(torch.randn(D, generator=gen, device=dev))
    hot = torch.randperm(D, generator=gen, device=dev)[:2]
    scale[hot] *= 10.0
    return (torch.randn(shape, generator=gen, device=dev) * scale).to(torch.float16)


def build_cache(w, dev, seed, batch=None, context=None):
    """Synthetic K/V with the benchmark distribution, compressed on the GPU into a cache."""
    import torch
    from polarquant_kv import quantizer
    from polarquant_kv.rotation import device_plan, generate_rotation_matrix

    B = w["batch"] if batch is None else batch
    S = w["context"] if context is None else context
    H, D = w["kv_heads"], w["head_dim"]
    R = generate_rotation_matrix(D, 0)
    plan = device_plan(R, dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    caches = []
    for bits in (w["k_bits"], w["v_bits"]):
        cache = quantizer.allocate_cache(B, H, max(S, 16), D, bits, 0, dev)
        for b in range(B):
            if S == 0:
                break
            x = synthetic_kv((1, H, S, D), dev, gen)
            c = quantizer.compress(x, plan, bits)
            cache.blocks[b:b + 1, :, :S].copy_(c.blocks)
        cache.seq_len = S
        caches.append(cache)
    return plan, caches[0], caches[1]


class Timer:
    """Blocks of `steps` steps, each bracketed by barrier + synchronize, timed with CUDA events; the
    rank's figure is the median block, the job's the maximum over ranks."""

    def __init__(self, dev, world, repeats):
        self.dev, self.world, self.repeats = dev, world, repeats

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(self, fn, steps, repeats=None):
        """-> (job ms per block = max over ranks of the per-rank median, [per-rank medians])"""
        import torch
        import torch.distributed as dist
        blocks = []
        for _ in range(repeats or self.repeats):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            blocks.append(e0.elapsed_time(e1))
        self.barrier()
        blocks.sort()
        med = blocks[len(blocks) // 2]
        per_rank = [med]
        if self.world > 1:
            t = torch.tensor([med], device=self.dev, dtype=torch.float64)
            allt = [torch.zeros_like(t) for _ in range(self.world)]
            dist.all_gather(allt, t)
            per_rank = [float(x.item()) for x in allt]
        return max(per_rank), per_rank


def decode_measurement(w, batch, dev, rank, timer, steps, warmup, n_splits, with_e2e=True, parity=True):
    """Decode attention over `batch` sequences of workload `w` on this rank; returns a dict of raw times."""
    import numpy as np
    import torch
    from polarquant_kv import attention

    Hq, D = w["q_heads"], w["head_dim"]
    res = {"batch_this_rank": batch}
    if batch == 0:                       # more ranks than sequences: this rank idles
        for key in ("ms_block", "ms_block_e2e"):
            res[key] = timer.run(lambda i: None, steps)
        return res
    sets = [build_cache(w, dev, 1000 * rank + i, batch=batch) for i in range(2)]
    plan = sets[0][0]
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    q_dev = torch.randn((batch, Hq, D), generator=gen, device=dev).to(torch.float16)
    q_host = q_dev.cpu().pin_memory()
    out_host = torch.empty((batch, Hq, D), dtype=torch.float32).pin_memory()
    prepared = [attention.prepare_decode(q_dev, sets[j][1], sets[j][2], plan, n_splits=n_splits) for j in range(2)]

    def step(i):
        prepared[i & 1]()

    # the serving-loop form of the public API: one CUDA graph per cache = copy of the query from pinned host
    # memory, the attention kernel, copy of the result back to pinned host memory
    q_stage = torch.empty_like(q_dev)
    prep_e2e = [attention.prepare_decode(q_stage, sets[j][1], sets[j][2], plan, n_splits=n_splits) for j in range(2)]
    graphs = [pd.capture(q_host, out_host) for pd in prep_e2e] if with_e2e else None

    def step_e2e(i):
        graphs[i & 1].replay()
        torch.cuda.current_stream().synchronize()     # the caller reads the result on the host

    for i in range(max(3, warmup)):
        step(i)
        if with_e2e:
            step_e2e(i)
    torch.cuda.synchronize()
    res["ms_block"] = timer.run(step, steps)
    if with_e2e:
        res["ms_block_e2e"] = timer.run(step_e2e, steps)
        res["h2d"], res["d2h"] = q_host.numel() * 2, out_host.numel() * 4
    if parity:
        # one row of the cache that was just timed, against the oracle
        from oracle import pq_oracle as O
        out = prepared[0]().clone()
        torch.cuda.synchronize()
        G = Hq // w["kv_heads"]
        b, h = batch - 1, w["kv_heads"] // 2
        cb, _ = O.lloyd_max_codebook(32, 4)
        R = O.rotation_matrix(D, 0)
        kb = sets[0][1].blocks[b, h:h + 1].cpu().numpy()
        vb = sets[0][2].blocks[b, h:h + 1].cpu().numpy()
        ref = O.attention_from_blocks(q_dev[b, h * G:(h + 1) * G].cpu().numpy()[:, None, :], kb, vb, R, cb, cb)[:, 0]
        res["parity_sample_max_abs"] = float(np.abs(out[b, h * G:(h + 1) * G].cpu().numpy() - ref).max())
    res["_keep"] = (sets, prepared)      # the prefill section reuses the caches
    return res


def long_context_measurement(dev, rank, world, timer, steps, peer_exchange="auto"):
    """One long sequence split along the sequence across the ranks: per-rank partial decode
    (m, l, o_rotated), exchange of the records and log-sum-exp merge + inverse rotation on every rank -
    as one kernel over NVLink peer memory (PeerExchange), with the all-gather + pq_lse_merge path beside it."""
    import torch
    import torch.distributed as dist
    from polarquant_kv import attention, distributed

    w = LONG_CONTEXT
    Hq, D, S = w["q_heads"], w["head_dim"], w["context"]
    lo, hi = distributed.sequence_shard(S, rank, world)
    sets = [build_cache(w, dev, 5000 + 10 * rank + i, context=hi - lo) for i in range(2)]
    plan = sets[0][0]
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    q = torch.randn((1, Hq, D), generator=gen, device=dev).to(torch.float16)
    out = {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"}, "tokens_this_rank": hi - lo}
    if world == 1:
        prepared = [attention.prepare_decode(q, sets[j][1], sets[j][2], plan) for j in range(2)]

        def step(i):
            prepared[i & 1]()
        for i in range(3):
            step(i)
        ms, per_rank = timer.run(step, steps)
        out["phases_us"] = {"decode_kernel": round(1e3 * ms / steps, 2)}
    else:
        prepared = [attention.prepare_decode(q, sets[j][1], sets[j][2], plan, partial=True) for j in range(2)]
        gathered = torch.empty((world, Hq, D + 2), dtype=torch.float32, device=dev)
        merged = torch.empty((Hq, D), dtype=torch.float32, device=dev)
        exchange = None
        # the exchange + merge as one kernel over NVLink peer memory (run at 2, 4 and 8 ranks); "off" and
        # any failure to map the peers' buffers fall back to the collective path
        if peer_exchange == "on" or (peer_exchange == "auto" and world <= 8):
            try:
                exchange = distributed.PeerExchange(Hq, D, dev)
            except Exception as exc:   # noqa: BLE001  (no peer mapping between these GPUs: the collective path serves)
                out["peer_exchange_unavailable"] = repr(exc)[:200]
        flags = torch.tensor([1 if exchange is not None else 0], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)          # every rank takes the same path
        if int(flags.item()) == 0:
            exchange = None

        def step_nccl(i):
            part = prepared[i & 1]()
            dist.all_gather_into_tensor(gathered, part.reshape(Hq, D + 2))
            return distributed.lse_merge(gathered, plan)

        def step_peer(i):
            return exchange.merge(prepared[i & 1]().reshape(Hq, D + 2), plan, out=merged)

        step = step_peer if exchange is not None else step_nccl
        for i in range(3):
            step(i)
        ms, per_rank = timer.run(step, steps)
        # phases, timed one at a time (events between the phases of a step would serialise them)
        ms_part, _ = timer.run(lambda i: prepared[i & 1](), steps, repeats=5)
        part = prepared[0]().reshape(Hq, D + 2)
        ms_gather, _ = timer.run(lambda i: dist.all_gather_into_tensor(gathered, part), steps, repeats=5)
        ms_merge, _ = timer.run(lambda i: distributed.lse_merge(gathered, plan), steps, repeats=5)
        out["phases_us"] = {"partial_decode_kernel": round(1e3 * ms_part / steps, 2)}
        if exchange is not None:
            ms_x, _ = timer.run(lambda i: exchange.merge(part, plan, out=merged), steps, repeats=5)
            ms_nccl, _ = timer.run(step_nccl, steps)
            out["phases_us"]["peer_exchange_merge_kernel"] = round(1e3 * ms_x / steps, 2)
            out["exchange"] = "one kernel over NVLink peer memory (pq_lse_exchange_merge): stores into the peers' " \
                              "buffers, system-scope arrival counters, merge + inverse rotation"
            out["collective_path"] = {"us_per_step": round(1e3 * ms_nccl / steps, 2),
                                      "all_gather": round(1e3 * ms_gather / steps, 2),
                                      "lse_merge_kernel": round(1e3 * ms_merge / steps, 2),
                                      "note": "the same step with torch.distributed all_gather_into_tensor (NCCL) + pq_lse_merge"}
            _ext_poll = __import__("polarquant_kv._ext", fromlist=["poll_device_errors"]).poll_device_errors
            _ext_poll()
        else:
            out["phases_us"]["all_gather"] = round(1e3 * ms_gather / steps, 2)
            out["phases_us"]["lse_merge_kernel"] = round(1e3 * ms_merge / steps, 2)
            out["all_gather_share_of_step"] = round(ms_gather / ms, 3)
        out["exchange_payload_bytes_per_rank"] = Hq * (D + 2) * 4
    bytes_total = algorithmic_bytes(w)
    us = 1e3 * ms / steps
    out.update({"us_per_step": round(us, 2), "per_rank_ms": [round(x / steps, 5) for x in per_rank],
                "value_gbs": round(bytes_total / us / 1e3, 1), "algorithmic_bytes": bytes_total,
                "scaling": "strong (sequence axis split across the ranks)"})
    return out


def compress_measurement(dev, world, timer, steps, n, peak):
    """2^24 K vectors (with the 128-projection QJL sketch) and 2^24 V vectors per variant."""
    import torch
    from polarquant_kv import quantizer
    from polarquant_kv.qjl import generate_jl_matrix
    from polarquant_kv.rotation import device_plan, generate_rotation_matrix

    D = 128
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    chunk = 1 << 20
    xk = torch.empty((1, 1, n, D), dtype=torch.float16, device=dev)
    xv = torch.empty((1, 1, n, D), dtype=torch.float16, device=dev)
    for x in (xk, xv):
        scale = torch.exp(torch.randn(D, generator=gen, device=dev))
        scale[torch.randperm(D, generator=gen, device=dev)[:2]] *= 10.0
        for lo in range(0, n, chunk):
            m = min(chunk, n - lo)
            x[0, 0, lo:lo + m] = (torch.randn((m, D), generator=gen, device=dev) * scale).to(torch.float16)
    R = generate_rotation_matrix(D, 0)
    plan = device_plan(R, dev)
    plan_q = device_plan(R, dev, generate_jl_matrix(D, D, 1))
    comp = {}
    # (label, [(bits, share of the vectors)]): "mixed" = first half of the heads at 4-bit, the rest at 2-bit
    variants = (("4bit", [(4, 1.0)]), ("2bit", [(2, 1.0)]), ("mixed_4bit_2bit_by_head", [(4, 0.5), (2, 0.5)]))
    k = max(3, min(steps, 5))
    for label, parts in variants:
        jobs, lo = [], 0
        for bits, share in parts:
            cnt = int(n * share)
            jobs.append((bits, lo, cnt, quantizer.allocate_cache(1, 1, cnt, D, bits, D, dev),
                         quantizer.allocate_cache(1, 1, cnt, D, bits, 0, dev)))
            lo += cnt

        def kstep(i, jobs=jobs):
            for bits, lo, cnt, ck, _ in jobs:
                quantizer.compress(xk[:, :, lo:lo + cnt], plan_q, bits, 32, plan_q.jl, out=ck, position=0)

        def vstep(i, jobs=jobs):
            for bits, lo, cnt, _, cv in jobs:
                quantizer.compress(xv[:, :, lo:lo + cnt], plan, bits, out=cv, position=0)

        for fn in (kstep, vstep):
            fn(0)
        torch.cuda.synchronize()
        time.sleep(0.25)           # every kernel is timed alone: let the previous one's power draw decay
        tv = timer.run(vstep, k, repeats=3)[0] / k
        time.sleep(0.25)
        tk = timer.run(kstep, k, repeats=3)[0] / k
        out_bytes = sum(share * (D // 32) * (2 + 4 * bits) for bits, share in parts)
        bk, bv = 2 * D + out_bytes + D // 8 + 2, 2 * D + out_bytes
        comp[label] = {
            "k_with_qjl": {"ms": round(tk, 4), "mvec_per_s": round(n * world / tk / 1e3, 1), "bytes_per_vector": bk,
                           "achieved_gbs": round(n * bk / tk / 1e6, 1), "frac_of_hbm_peak": round(n * bk / tk / 1e6 / peak, 4)},
            "v": {"ms": round(tv, 4), "mvec_per_s": round(n * world / tv / 1e3, 1), "bytes_per_vector": bv,
                  "achieved_gbs": round(n * bv / tv / 1e6, 1), "frac_of_hbm_peak": round(n * bv / tv / 1e6 / peak, 4)},
            "k_plus_v": {"ms": round(tk + tv, 4), "mvec_per_s": round(2 * n * world / (tk + tv) / 1e3, 1),
                         "achieved_gbs": round(n * (bk + bv) / (tk + tv) / 1e6, 1),
                         "frac_of_hbm_peak": round(n * (bk + bv) / (tk + tv) / 1e6 / peak, 4)},
            "vectors_per_tensor": n, "launches_per_tensor": len(jobs)}
        del jobs
    # dequantise (blocks -> float16 vectors): 72 B in, 256 B out per vector
    nd = min(n, 1 << 22)
    cache = quantizer.compress(xv[:, :, :nd], plan, 4)
    quantizer.decompress(cache, plan, torch.float16)
    td = timer.run(lambda i: quantizer.decompress(cache, plan, torch.float16), k, repeats=3)[0] / k
    dq = {"ms": round(td, 4), "vectors": nd, "bytes_per_vector": 72 + 256, "achieved_gbs": round(nd * 328 / td / 1e6, 1),
          "frac_of_hbm_peak": round(nd * 328 / td / 1e6 / peak, 4), "out_dtype": "float16"}
    return comp, dq


def prefill_measurement(w, sets, plan, dev, timer, steps):
    import torch
    from polarquant_kv import attention
    Hq, D = w["q_heads"], w["head_dim"]
    Sq, Sp, Bp = 512, 4096, 2
    _, ck0, cv0 = sets[0]
    if ck0.blocks.shape[0] < Bp:
        return None
    ckp = type(ck0)(ck0.blocks[:Bp, :, :Sp].contiguous(), None, None, 4, 32, D, Sp, Sp)
    cvp = type(cv0)(cv0.blocks[:Bp, :, :Sp].contiguous(), None, None, 4, 32, D, Sp, Sp)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    qp = torch.randn((Bp, Hq, Sq, D), generator=gen, device=dev).to(torch.float16)
    useful = 4.0 * Bp * Hq * Sq * Sp * D                       # QK^T and PV multiply-adds x2
    kp = max(3, min(steps, 10))
    tensor_peak = measured_tensor_peak()
    prefill = {"shape": {"batch": Bp, "q_heads": Hq, "kv_heads": w["kv_heads"], "seq_q": Sq, "seq_kv": Sp, "head_dim": D}}
    # "workspace": K/V tiles expanded once by a first kernel (two launches, the default for this shape);
    # "fused": the attention kernel dequantises the tiles itself (one launch, no workspace)
    for label, use_ws in (("workspace", True), ("fused", False)):
        def pstep(i, use_ws=use_ws):
            attention.prefill_attention(qp, ckp, cvp, plan, use_workspace=use_ws)
        for i in range(3):
            pstep(i)
        pms = timer.run(pstep, kp, repeats=3)[0] / kp
        prefill[label] = {"ms": round(pms, 4), "useful_tflops": round(useful / pms / 1e9, 1),
                          "frac_of_tensor_peak": round(useful / pms / 1e9 / tensor_peak, 4),
                          "issued_tflops_3_term_fp16": round(3 * useful / pms / 1e9, 1)}
    prefill["roofline"] = {"bound": "tensor", "achieved": prefill["workspace"]["useful_tflops"], "peak": tensor_peak,
                           "unit": "TFLOP/s", "frac": prefill["workspace"]["frac_of_tensor_peak"],
                           "note": "useful multiply-adds; the kernel issues three float16 product terms per useful one"}
    return prefill


def cache_kernels_per_step(model, caches, cfg, B, dev, timer):
    """Device time of one decode step's compressed-cache kernels alone (per layer: append of the new key
    and value rows, attention over the cache), replayed from a CUDA graph at the caches' current length."""
    import torch
    k = torch.randn(B, cfg.kv_heads, 1, cfg.head_dim, device=dev).to(torch.float16)
    q = torch.randn(B, cfg.q_heads, 1, cfg.head_dim, device=dev).to(torch.float16)
    position = torch.full((1,), caches[0].seq_len - 1, dtype=torch.int64, device=dev)
    length = torch.full((1,), caches[0].seq_len, dtype=torch.int64, device=dev)

    def one_step():
        for cache in caches:
            cache.append(k, k, position=position)          # overwrites the last token's slot
            cache.attend(q, seq_len_tensor=length)

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        one_step()
    torch.cuda.current_stream(dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_step()
    ms, _ = timer.run(lambda i: graph.replay(), 10, repeats=3)
    return ms / 10


def bridge_measurement(dev, timer, steps):
    """The llama.cpp bridge's entry points (include/polarquant_llama_abi.h; per-vector-radius codec): fused
    attention of 32 query / 8 kv heads over 65 536 tokens and compress of 2^20 float32 vectors, head dim 128.
    Two input sets alternate so that no step finds its data in L2 (151 MB per attention set)."""
    import torch
    from polarquant_kv import llama_bridge as LB
    hq, hkv, S, D, n = 32, 8, 65536, 128, 1 << 20
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    cb = torch.sort(torch.randn(16, generator=gen, device=dev) * 0.09).values.contiguous()
    sets = []
    for _ in range(2):
        pk = torch.randint(0, 256, (hkv, S, D // 2), dtype=torch.uint8, generator=gen, device=dev)
        pv = torch.randint(0, 256, (hkv, S, D // 2), dtype=torch.uint8, generator=gen, device=dev)
        kr = torch.rand(hkv, S, generator=gen, device=dev) + 0.5
        vr = torch.rand(hkv, S, generator=gen, device=dev) + 0.5
        sets.append((pk, kr, pv, vr))
    q = torch.randn(hq, D, generator=gen, device=dev)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(D)

    def attend(i):
        pk, kr, pv, vr = sets[i & 1]
        LB.fused_attention(q, pk, kr, pv, vr, cb, scale, out=out)

    attend(0), attend(1)
    t_att = timer.run(attend, steps, repeats=5)[0] / steps
    att_bytes = 2 * hkv * S * (D // 2 + 4)
    xs = [torch.randn(n, D, generator=gen, device=dev) for _ in range(2)]
    R = torch.linalg.qr(torch.randn(D, D, generator=gen, device=dev))[0].contiguous()
    LB.compress(xs[0], R, cb)
    t_cmp = timer.run(lambda i: LB.compress(xs[i & 1], R, cb), steps, repeats=5)[0] / steps
    cmp_bytes = n * (D * 4 + D // 2 + 4)
    peak, _ = measured_peak()
    return {"attention": {"q_heads": hq, "kv_heads": hkv, "tokens": S, "head_dim": D, "us": round(t_att * 1e3, 1),
                          "stored_bytes": att_bytes, "achieved_gbs": round(att_bytes / t_att / 1e6, 1),
                          "frac_of_hbm_peak": round(att_bytes / t_att / 1e6 / peak, 4)},
            "compress": {"vectors": n, "head_dim": D, "ms": round(t_cmp, 4), "mvec_per_s": round(n / t_cmp / 1e3, 1),
                         "bytes_per_vector": D * 4 + D // 2 + 4, "achieved_gbs": round(cmp_bytes / t_cmp / 1e6, 1),
                         "frac_of_hbm_peak": round(cmp_bytes / t_cmp / 1e6 / peak, 4)}}


def e2e_model_measurement(dev, rank, world, timer, steps=256):
    """End-to-end greedy decoding of a Qwen2.5-0.5B-architecture decoder with random bfloat16 weights
    (seed 0): 64 prompts of 4096 random token ids (sharded by batch across the ranks), one prefill pass,
    then `steps` single-token steps; keys and values are compressed on write and read by the fused
    attention kernels.  The dense layers are plain torch; `cache_kernel_share` is the part of the
    decode time spent between cache append and attention output (compress x2 + attention per layer)."""
    import torch
    from polarquant_kv import distributed
    from polarquant_kv.inference import DecoderConfig, DecoderLM, PolarQuantConfig
    from polarquant_kv.inference.model import KernelTimer
    cfg = DecoderConfig()
    B_total, S = 64, 4096
    lo, hi = distributed.batch_shard(B_total, rank, world)
    B = hi - lo
    model = DecoderLM(cfg, PolarQuantConfig(n_bits=4)).init_random(seed=0, dtype=torch.bfloat16, device=dev)
    gen = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (B_total, S), generator=gen)[lo:hi].to(dev)
    caches = model.create_cache_managers(S + steps, max(B, 1), dev)
    state = {}

    def prefill(i):
        for c in caches:
            c.reset()
        state["logits"] = model(prompt, caches)

    def decode(i):
        tok = state["logits"].argmax(-1, keepdim=True)
        for _ in range(steps):
            state["logits"] = model(tok, caches, state.get("timers"))
            tok = state["logits"].argmax(-1, keepdim=True)

    def decode_graph(i):
        # the same steps, launched as one CUDA graph replay per token (position and cache length on the
        # device); recording the graph is inside the timed region
        state["graph_tokens"] = model.decode_graph(state["logits"].argmax(-1, keepdim=True), steps, caches)

    if B == 0:
        prefill = decode = decode_graph = (lambda i: None)
    ms_prefill, _ = timer.run(prefill, 1, repeats=1)
    state["timers"] = KernelTimer()
    ms_decode, per_rank = timer.run(decode, 1, repeats=1)
    kernel_ms = state["timers"].total_ms() if B else 0.0
    mem = sum(c.memory_bytes for c in caches) if B else 0
    state["timers"] = None
    timer.run(prefill, 1, repeats=1)                       # fresh caches for the graph-replayed run
    ms_graph, _ = timer.run(decode_graph, 1, repeats=1)
    ms_cache_step = cache_kernels_per_step(model, caches, cfg, max(B, 1), dev, timer) if B else 0.0
    return {"model": "Qwen2.5-0.5B architecture, random bfloat16 weights (seed 0)", "batch": B_total, "prompt_len": S,
            "decode_steps": steps, "batch_this_rank": B,
            "prefill_s": round(ms_prefill / 1e3, 3),
            # the decode loop as the library runs it: one CUDA graph launch per token
            "launch_mode": "one CUDA graph launch per token (pq_compress_rows_dynamic + pq_decode_attn_dynamic read "
                           "position and length from device memory); recording the graph is inside the timed region",
            "decode_s": round(ms_graph / 1e3, 3),
            "decode_tokens_per_s": round(B_total * steps / (ms_graph / 1e3), 1),
            "ms_per_decode_step": round(ms_graph / steps, 3),
            "cache_kernels_ms_per_step": round(ms_cache_step, 3),
            "cache_kernel_share_of_decode": round(ms_cache_step / (ms_graph / steps), 3) if B else None,
            # the same steps issued kernel by kernel from Python (about 25 small launches per layer: host-launch bound)
            "eager": {"decode_s": round(ms_decode / 1e3, 3),
                      "decode_tokens_per_s": round(B_total * steps / (ms_decode / 1e3), 1),
                      "ms_per_decode_step": round(ms_decode / steps, 3),
                      "cache_kernel_share_of_decode": round(kernel_ms / ms_decode, 3) if B else None},
            "compressed_cache_bytes_this_rank": mem}


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from polarquant_kv import _ext, distributed
    _ext.lib()   # raises if the CUDA library is missing: there is no fallback

    w = WORKLOAD
    timer = Timer(dev, world, args.repeats)
    peak, peak_kind = measured_peak()
    if args.only_compress or args.only_bridge:
        # the compress and dequantise launches, or the bridge's, alone (for profiler captures of those kernels)
        if args.only_bridge:
            res = {"llama_bridge": bridge_measurement(dev, timer, args.steps)}
        else:
            comp, dequant = compress_measurement(dev, world, timer, args.steps, args.compress_vecs, peak)
            res = {"compress": comp, "dequant": dequant}
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            dist.destroy_process_group()
        return
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # nvidia-smi takes a moment to start: begin before the warm-up

    # ---- headline: the workload's 32 sequences sharded across the ranks
    b_lo, b_hi = distributed.batch_shard(w["batch"], rank, world)
    dec = decode_measurement(w, b_hi - b_lo, dev, rank, timer, args.steps, args.warmup, args.splits)
    clocks = sampler.stop() if rank == 0 else None
    sets = dec.get("_keep", (None, None))[0]
    ms_block, per_rank = dec["ms_block"]
    ms_step = ms_block / args.steps
    alg_bytes = algorithmic_bytes(w)                       # the whole job's bytes per step
    value = alg_bytes / (ms_step * 1e-3) / 1e9
    per_gpu_bytes = algorithmic_bytes(w, batch=max(1, math.ceil(w["batch"] / world)))
    achieved = per_gpu_bytes / (ms_step * 1e-3) / 1e9      # the most loaded rank's launch
    ms_e2e_block, per_rank_e2e = dec["ms_block_e2e"]
    e2e_val = alg_bytes / (ms_e2e_block / args.steps * 1e-3) / 1e9

    parity_err, h2d, d2h = dec.get("parity_sample_max_abs"), dec.get("h2d", 0), dec.get("d2h", 0)
    weak = None
    if world > 1 and not args.only_decode:
        dec.pop("_keep", None)           # free the sharded caches before building the per-rank full batch
        sets = None
        wdec = decode_measurement(w, w["batch"], dev, rank, timer, args.steps, args.warmup, args.splits,
                                  with_e2e=False, parity=False)
        wms, wper = wdec["ms_block"]
        weak = {"scaling": "weak", "batch_per_gpu": w["batch"], "ms_per_step": round(wms / args.steps, 5),
                "value": round(algorithmic_bytes(w) * world / (wms / args.steps * 1e-3) / 1e9, 1), "unit": "GB/s",
                "per_rank_ms": [round(x / args.steps, 5) for x in wper]}
        sets = wdec["_keep"][0]

    long_ctx = None if args.only_decode else long_context_measurement(dev, rank, world, timer, args.steps,
                                                                      args.peer_exchange)
    comp = dequant = None
    if not args.only_decode:
        comp, dequant = compress_measurement(dev, world, timer, args.steps, args.compress_vecs, peak)
    prefill = None
    if not args.only_decode and sets is not None:
        prefill = prefill_measurement(w, sets, sets[0][0], dev, timer, args.steps)
    sets = None
    bridge = None
    if not args.only_decode:
        torch.cuda.empty_cache()
        bridge = bridge_measurement(dev, timer, args.steps)     # per GPU, like the compress figures
    e2e_model = None
    if not args.only_decode and not args.skip_model:
        torch.cuda.empty_cache()
        e2e_model = e2e_model_measurement(dev, rank, world, timer)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- CPU baseline on a bounded sample (one process, as the oracle is written)
    cpu = None
    if world == 1:
        t0 = time.perf_counter()
        rows = 0
        while time.perf_counter() - t0 < (0.0 if args.only_decode else 10.0) or rows == 0:
            _cpu_rows((1, rows, w))
            rows += 1
        cpu_dt = time.perf_counter() - t0
        cpu_gbs = algorithmic_bytes(w) // (w["batch"] * w["kv_heads"]) * rows / cpu_dt / 1e9
        try:
            from threadpoolctl import threadpool_info
            blas_threads = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
        except Exception:
            blas_threads = 1
        cpu = {"value": round(cpu_gbs, 4), "unit": "GB/s", "cores": blas_threads, "kind": "port",
               "sample": f"{rows} (batch, kv-head) rows of the workload in {cpu_dt:.1f} s, numpy oracle, one process",
               "reference_as_shipped": None if args.only_decode else reference_as_shipped()}

    # DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum of a single-launch ncu capture of
    # this very shape on one GPU: 302 813 184 read + 4 269 312 written); any other shape reports none.
    captured_shape = world == 1 and (w["batch"], w["context"], w["q_heads"]) == (32, 8192, 32) and not args.splits
    traffic = 307_082_496 if captured_shape else None

    line = {
        "metric": "PQ4 decode-attn compressed-byte throughput", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 accumulate over f16x2-split operands", "data": "synthetic",
        "config": {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"},
                   "parallelism": f"the 32 sequences sharded across {world} GPU(s) by batch, no collective",
                   "l2": "two caches alternated between steps; at one GPU each is 302 MB (L2 is 126 MB); the "
                         "per-rank slice shrinks to 38 MB at eight GPUs, where two slices still exceed no L2 — "
                         "the strong-scaling figure at N >= 4 is L2-assisted and launch-bound, see weak_scaling",
                   "timing": f"median of {args.repeats} blocks of {args.steps} steps per rank, maximum over ranks"},
        "per_rank_ms": [round(x / args.steps, 5) for x in per_rank],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic, "peak_kind": f"of {peak_kind}",
                     "kernel": "pq_decode_attn_kernel<128,4,4,1,false>",
                     "algorithmic_bytes_per_launch": per_gpu_bytes,
                     "traffic_note": "dram bytes read + written by one launch of this shape in a single-launch ncu "
                                     "capture (1.017 x the algorithmic bytes); null for shapes that were not captured"},
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e_block / args.steps, 5),
                "per_rank_ms": [round(x / args.steps, 5) for x in per_rank_e2e]},
        "parity_sample_max_abs": parity_err,
        "gpu_launches": args.steps,
        "weak_scaling": weak,
        "long_context": long_ctx,
        "compress": comp,
        "dequant": dequant,
        "prefill": prefill,
        "llama_bridge": bridge,
        "e2e_model": e2e_model,
        "cpu_baseline": cpu,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=BLOCK_REPEATS, help="timed blocks per measurement (median is reported)")
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"],
                    help="sequences in the decode workload (default: the headline workload's 32; smaller for profiler captures)")
    ap.add_argument("--context", type=int, default=0, help="tokens per sequence (default: the headline workload's)")
    ap.add_argument("--q-heads", type=int, default=0, help="query heads (default: the headline workload's)")
    ap.add_argument("--only-decode", action="store_true",
                    help="only the headline decode measurement (profiler captures)")
    ap.add_argument("--only-compress", action="store_true",
                    help="run the compress and dequantise measurements alone and print them")
    ap.add_argument("--peer-exchange", default="auto", choices=["auto", "on", "off"],
                    help="long-context step: exchange + merge as one kernel over NVLink peer memory "
                         "(auto: up to 8 ranks of one node; the all-gather + merge path otherwise)")
    ap.add_argument("--only-bridge", action="store_true",
                    help="run the llama.cpp bridge measurement alone and print it")
    ap.add_argument("--skip-model", action="store_true", help="skip the end-to-end decoder measurement")
    ap.add_argument("--splits", type=int, default=0, help="sequence splits per (batch, kv head); 0 = library default")
    ap.add_argument("--compress-vecs", type=int, default=COMPRESS_VECS, help="vectors per tensor in the compress measurement")
    args = ap.parse_args()
    WORKLOAD["batch"] = args.batch
    if args.context or args.q_heads:           # other decode shapes: not the headline
        WORKLOAD["context"] = args.context or WORKLOAD["context"]
        WORKLOAD["q_heads"] = args.q_heads or WORKLOAD["q_heads"]
        WORKLOAD["name"] = "custom PQ4 decode attention shape"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
