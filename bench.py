"""Benchmark of the PQ4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload ("step" = one decode-attention pass over one batch): Llama-3-8B-shaped
decode over a PQ4 (4-bit block_pq4) cache — batch 32 per GPU, 8 KV heads, 32 query heads,
head_dim 128, context 8192, one query token per sequence.  Metric: compressed K/V bytes
streamed per second (GB/s), each stored byte counted once per KV head.  Multi-GPU runs
shard by batch with no collective (every rank owns its own 32 sequences: weak scaling).

The JSON line also carries: `roofline` (dominant kernel against the measured HBM copy
bandwidth), `e2e` (same step through the public API with host buffers: query copied from
pinned host memory, output copied back), `compress` (bulk compress throughput in Mvec/s
with its own roofline figure), `cpu_baseline` (the numpy oracle on a bounded sample, rank 0)
and the clocks sampled during the timed region.

`--impl reference` times the CPU implementation of the same step (the numpy restatement of
the reference algorithm, oracle/pq_oracle.py — the reference itself is Python and does not
travel to the GPU box) on all host cores, on a bounded sample.
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
COMPRESS_VECS = 1 << 22        # vectors per compress launch in the secondary measurement
FALLBACK_HBM_GBS = 6650.0      # used only when MEASURED_PEAKS.json is absent
DECODE_TRAFFIC_BYTES = 308_857_600   # ncu: 302.39 MB read + 6.46 MB written per launch of the headline workload


def algorithmic_bytes(w) -> int:
    """Compressed K + V bytes one decode step must read: B * Hkv * S * 2 * (D/32) * 18."""
    per_token = (w["head_dim"] // 32) * ((2 + 4 * w["k_bits"]) + (2 + 4 * w["v_bits"]))
    return w["batch"] * w["kv_heads"] * w["context"] * per_token


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
                 "--format=csv,noheader,nounits", "-lms", "100"],
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
    rows = 4
    steps_ms = []
    with mp.get_context("spawn").Pool(procs) as pool:
        for _ in range(max(1, args.warmup)):
            cpu_arm(pool, w, procs, 1)           # warm-up (imports, codebook, BLAS start-up)
        for _ in range(max(1, args.steps)):
            steps_ms.append(cpu_arm(pool, w, procs, rows))
    gbs = sum(g for g, _ in steps_ms) / len(steps_ms)
    full_step_s = algorithmic_bytes(w) / 1e9 / gbs
    sample = (f"{procs} processes x {rows} (batch, kv-head) rows of the workload per step "
              f"({procs * rows} of {w['batch'] * w['kv_heads']} rows), numpy oracle port of the reference "
              "algorithm (vectorised; the reference's own per-token Python loop is slower)")
    line = {
        "impl": "reference", "metric": "PQ4 decode-attn compressed-byte throughput", "value": round(gbs, 4),
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(full_step_s * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"}},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": procs, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def build_cache(w, dev, seed):
    """Synthetic K/V with the benchmark distribution, compressed on the GPU into a cache."""
    import torch
    from polarquant_kv import quantizer
    from polarquant_kv.rotation import device_plan, generate_rotation_matrix

    B, H, S, D = w["batch"], w["kv_heads"], w["context"], w["head_dim"]
    R = generate_rotation_matrix(D, 0)
    plan = device_plan(R, dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    caches = []
    for bits in (w["k_bits"], w["v_bits"]):
        scale = torch.exp(torch.randn(D, generator=gen, device=dev))
        hot = torch.randperm(D, generator=gen, device=dev)[:2]
        scale[hot] *= 10.0
        cache = quantizer.allocate_cache(B, H, S, D, bits, 0, dev)
        for b in range(B):
            x = (torch.randn((1, H, S, D), generator=gen, device=dev) * scale).to(torch.float16)
            c = quantizer.compress(x, plan, bits)
            cache.blocks[b:b + 1].copy_(c.blocks)
        cache.seq_len = S
        caches.append(cache)
    return plan, caches[0], caches[1]


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

    from polarquant_kv import _ext, attention, quantizer
    _ext.lib()   # raises if the CUDA library is missing: there is no fallback

    w = WORKLOAD
    B, Hq, D = w["batch"], w["q_heads"], w["head_dim"]
    if args.only_compress:
        w = dict(w, batch=1, context=256)        # a token-sized decode set-up; only compress is measured
        B = 1
    alg_bytes = algorithmic_bytes(w)
    # two independent caches, alternated between steps, so no step finds its data in L2
    sets = [build_cache(w, dev, 1000 * rank + i) for i in range(2)]
    plan = sets[0][0]
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    q_dev = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.float16)
    q_host = q_dev.cpu().pin_memory()
    out_host = torch.empty((B, Hq, D), dtype=torch.float32).pin_memory()
    q_stage = torch.empty_like(q_dev)

    def step(i):
        _, ck, cv = sets[i & 1]
        return attention.decode_attention(q_dev, ck, cv, plan, enable_qjl=False, n_splits=args.splits)

    prepared = [attention.prepare_decode(q_stage, sets[j][1], sets[j][2], plan, n_splits=args.splits) for j in range(2)]

    # the serving-loop form of the public API: one CUDA graph per cache = copy of the query from pinned host
    # memory, the attention kernel, copy of the result back to pinned host memory
    graphs = [pd.capture(q_host, out_host) for pd in prepared]

    def step_e2e(i):
        graphs[i & 1].replay()
        torch.cuda.current_stream().synchronize()     # the caller reads the result on the host

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # nvidia-smi takes a moment to start: begin before the warm-up
    for i in range(max(3, args.warmup)):
        step(i)
        step_e2e(i)
    torch.cuda.synchronize()
    t_busy = time.perf_counter()
    while rank == 0 and time.perf_counter() - t_busy < 0.6:   # keep the GPU loaded until samples arrive
        step(0)
        torch.cuda.synchronize()
    ms_total = timed(step, args.steps)
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # ---- secondary: bulk compress throughput (4-bit, with and without the QJL sketch)
    from polarquant_kv.qjl import generate_jl_matrix
    from polarquant_kv.rotation import device_plan, generate_rotation_matrix
    n = 1024 if args.only_decode else args.compress_vecs
    x = (torch.randn((n, D), generator=gen, device=dev) * torch.exp(torch.randn(D, generator=gen, device=dev))).to(torch.float16)
    x2 = x.flip(0).contiguous()
    Rm = generate_rotation_matrix(D, 0)
    plan_q = device_plan(Rm, dev, generate_jl_matrix(D, D, 1))
    comp = {}
    # variants: (label, [(bits, share of the vectors)], with QJL sketch); "mixed" = first half of the
    # vectors (heads) at 4-bit, the rest at 2-bit, as two launches
    variants = (("4bit", [(4, 1.0)], False), ("2bit", [(2, 1.0)], False),
                ("mixed_4bit_2bit", [(4, 0.5), (2, 0.5)], False), ("4bit_qjl", [(4, 1.0)], True))
    for label, parts, jl in (() if args.only_decode else variants):
        pl = plan_q if jl else plan
        jobs = []
        lo = 0
        for bits, share in parts:
            cnt = int(n * share)
            jobs.append((bits, lo, cnt, [quantizer.allocate_cache(1, 1, cnt, D, bits, D if jl else 0, dev)
                                          for _ in range(2)]))
            lo += cnt
        xs = [x.view(1, 1, n, D), x2.view(1, 1, n, D)]

        def cstep(i, pl=pl, jl=jl, jobs=jobs, xs=xs):
            for bits, lo, cnt, outs in jobs:
                quantizer.compress(xs[i & 1][:, :, lo:lo + cnt], pl, bits, 32, pl.jl if jl else None,
                                   out=outs[i & 1], position=0)

        for i in range(3):
            cstep(i)
        k = max(4, min(args.steps, 20))
        per_launch = timed(cstep, k) / k
        out_bytes = sum(share * (D // 32) * (2 + 4 * bits) for bits, share in parts)
        bytes_per_vec = 2 * D + out_bytes + ((D // 8 + 2) if jl else 0)
        comp[label] = {"mvec_per_s": round(n * world / per_launch / 1e3, 1), "ms_per_step": round(per_launch, 4),
                       "vectors_per_step": n, "launches_per_step": len(jobs), "bytes_per_vector": bytes_per_vec,
                       "achieved_gbs": round(n * bytes_per_vec / per_launch / 1e6, 1)}

    # ---- secondary: prefill-shape attention over the compressed cache (tensor-core bound)
    prefill = None
    if not args.only_decode and not args.only_compress:
        Sq, Sp, Bp = 512, 4096, 2
        _, ck0, cv0 = sets[0]
        ckp = type(ck0)(ck0.blocks[:Bp, :, :Sp].contiguous(), None, None, 4, 32, D, Sp, Sp)
        cvp = type(cv0)(cv0.blocks[:Bp, :, :Sp].contiguous(), None, None, 4, 32, D, Sp, Sp)
        qp = torch.randn((Bp, Hq, Sq, D), generator=gen, device=dev).to(torch.float16)

        useful = 4.0 * Bp * Hq * Sq * Sp * D                       # QK^T and PV multiply-adds x2
        kp = max(3, min(args.steps, 10))
        prefill = {"shape": {"batch": Bp, "q_heads": Hq, "kv_heads": w["kv_heads"], "seq_q": Sq, "seq_kv": Sp,
                             "head_dim": D}}
        tensor_peak = measured_tensor_peak()
        # "workspace": K/V tiles expanded once by a first kernel (two launches, the default for this shape);
        # "fused": the attention kernel dequantises the tiles itself (one launch, no workspace)
        for label, use_ws in (("workspace", True), ("fused", False)):
            def pstep(i, use_ws=use_ws):
                attention.prefill_attention(qp, ckp, cvp, plan, use_workspace=use_ws)

            for i in range(3):
                pstep(i)
            pms = timed(pstep, kp) / kp
            issued = 3 * useful / pms / 1e9
            prefill[label] = {"ms": round(pms, 4), "useful_tflops": round(useful / pms / 1e9, 1),
                              "issued_tflops_3_term_fp16": round(issued, 1),
                              "frac_of_tensor_peak": round(issued / tensor_peak, 4) if tensor_peak else None}
        prefill["tensor_peak_tflops"] = tensor_peak
        prefill["ms"] = prefill["workspace"]["ms"]
        prefill["useful_tflops"] = prefill["workspace"]["useful_tflops"]

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    if args.only_compress:
        for c in comp.values():
            c["frac_of_hbm_peak"] = round(c["achieved_gbs"] / peak, 4)
        print(json.dumps({"metric": "block_pq4 compress throughput", "unit": "Mvec/s", "n_gpus": world,
                          "compress": comp, "peak_gbs": peak, "peak_kind": f"of {peak_kind}"}))
        if world > 1:
            dist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9            # per GPU: one launch per step per GPU
    value = achieved * world
    e2e_val = alg_bytes * world / (ms_e2e / args.steps * 1e-3) / 1e9
    for c in comp.values():
        c["frac_of_hbm_peak"] = round(c["achieved_gbs"] / peak, 4)

    # ---- CPU baseline on a bounded sample (one process, as the oracle is written)
    t0 = time.perf_counter()
    rows = 0
    while time.perf_counter() - t0 < (0.0 if args.only_decode else 10.0) or rows == 0:
        _cpu_rows((1, rows, w))
        rows += 1
    cpu_dt = time.perf_counter() - t0
    cpu_gbs = alg_bytes // (w["batch"] * w["kv_heads"]) * rows / cpu_dt / 1e9
    try:
        from threadpoolctl import threadpool_info
        blas_threads = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        blas_threads = 1

    # DRAM bytes per launch from the ncu capture summarised in profiles/decode_attn_c1_ncu.md
    # (dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload)
    traffic = DECODE_TRAFFIC_BYTES if w["batch"] == 32 else None
    line = {
        "metric": "PQ4 decode-attn compressed-byte throughput", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over f16x2-split operands",
        "data": "synthetic",
        "config": {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"},
                   "batch_is_per_gpu": True, "parallelism": f"batch-sharded x{world}, no collective",
                   "l2": "two 302 MB caches alternated between steps (each larger than the 126 MB L2)"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic, "peak_kind": f"of {peak_kind}",
                     "kernel": "pq_decode_attn_kernel<128,4,4,1,false>", "algorithmic_bytes_per_launch": alg_bytes},
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": q_host.numel() * 2,
                "d2h_bytes_per_step": out_host.numel() * 4, "ms_per_step": round(ms_e2e / args.steps, 5)},
        "gpu_launches": args.steps,
        "compress": comp,
        "prefill": prefill,
        "cpu_baseline": {"value": round(cpu_gbs, 4), "unit": "GB/s", "cores": blas_threads, "kind": "port",
                         "sample": f"{rows} (batch, kv-head) rows of the workload in {cpu_dt:.1f} s, numpy oracle, one process"},
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"],
                    help="sequences per GPU (default: the headline workload's 32; smaller for profiler captures)")
    ap.add_argument("--context", type=int, default=0, help="tokens per sequence (default: the headline workload's)")
    ap.add_argument("--q-heads", type=int, default=0, help="query heads (default: the headline workload's)")
    ap.add_argument("--only-decode", action="store_true",
                    help="skip the compress and CPU-baseline measurements (profiler captures)")
    ap.add_argument("--splits", type=int, default=0, help="sequence splits per (batch, kv head); 0 = library default")
    ap.add_argument("--only-compress", action="store_true",
                    help="run only the bulk-compress measurement and print its JSON (profiler captures)")
    ap.add_argument("--compress-vecs", type=int, default=COMPRESS_VECS, help="vectors per compress launch")
    args = ap.parse_args()
    WORKLOAD["batch"] = args.batch
    if args.context or args.q_heads:           # other decode shapes (e.g. one long sequence): not the headline
        WORKLOAD["context"] = args.context or WORKLOAD["context"]
        WORKLOAD["q_heads"] = args.q_heads or WORKLOAD["q_heads"]
        WORKLOAD["name"] = "custom PQ4 decode attention shape"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
