"""Two-rank NCCL run of the sequence-sharded decode (needs >= 2 GPUs; skipped otherwise)."""

import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "polarquant-kv_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import inputs
        from oracle import pq_oracle as O
        from polarquant_kv import distributed
        from polarquant_kv.rotation import device_plan
        from polarquant_kv.types import CompressedKV
        Hkv, Hq, S, D = 2, 16, 3000, 128
        K, V, q = inputs.make_kvq(1, Hkv, Hq, S, D, seed=21)
        R = O.rotation_matrix(D, 0)
        cb, _ = O.lloyd_max_codebook(32, 4)
        kb, vb = O.compress(K[0], R, cb, 4), O.compress(V[0], R, cb, 4)
        lo, hi = distributed.sequence_shard(S, rank, world)
        n = hi - lo
        ck = CompressedKV(torch.from_numpy(kb[None, :, lo:hi].copy()).to(dev), None, None, 4, 32, D, n, n)
        cv = CompressedKV(torch.from_numpy(vb[None, :, lo:hi].copy()).to(dev), None, None, 4, 32, D, n, n)
        qd = torch.from_numpy(q[:, :, 0]).to(dev)
        plan = device_plan(R, dev)
        out = distributed.sharded_decode_attention(qd, ck, cv, plan)
        torch.cuda.synchronize()
        ref = O.attention_from_blocks(q[0], kb, vb, R, cb, cb)[:, 0]
        err = np.abs(out[0].cpu().numpy() - ref).max()
        # the same exchange and merge as one kernel over peer memory, several steps on the same buffers
        ex = distributed.PeerExchange(Hq, D, dev)
        err_peer = 0.0
        for step in range(5):
            got = distributed.sharded_decode_attention(qd, ck, cv, plan, exchange=ex)
            torch.cuda.synchronize()
            err_peer = max(err_peer, float(np.abs(got[0].cpu().numpy() - ref).max()))
            err_peer = max(err_peer, float((got - out).abs().max()) * 1e3 if step == 0 else 0.0)   # equal to the NCCL path to 2e-6
        from polarquant_kv import _ext
        _ext.poll_device_errors()
        ex.close()
        np.save(os.path.join(out_dir, f"err{rank}.npy"), np.array([max(err, err_peer)]))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_decode_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, 29600 + os.getpid() % 1000, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert float(np.load(tmp_path / f"err{r}.npy")[0]) <= 2e-3
