"""world_size-2 gloo test of the sequence-sharded decode plumbing on CPU.

The CUDA kernels cannot run here, so each rank produces the (m, l, o_rot) record of its
slice with the numpy oracle; the product code under test is the shard arithmetic and the
all-gather (polarquant_kv.distributed.sequence_shard / gather_partials).  The gathered
records are merged with a numpy log-sum-exp and must equal attention over the whole
sequence.
"""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _partial_record(q, kb, vb, R, cb, scale):
    """(m in log2 units, l, o in rotated space) per query head for a slice; numpy."""
    from oracle import pq_oracle as O
    Hq, D = q.shape[0], q.shape[-1]
    rep = Hq // kb.shape[0]
    rec = np.zeros((Hq, D + 2), dtype=np.float32)
    for h in range(Hq):
        g = h // rep
        if kb.shape[1] == 0:
            rec[h, 0] = 0.0
            continue
        k_rot = O.dequant_rotated(kb[g], cb, 4).astype(np.float64)
        v_rot = O.dequant_rotated(vb[g], cb, 4).astype(np.float64)
        q_rot = O.rotate(q[h, 0].astype(np.float64), R)
        s = k_rot @ q_rot * scale * np.log2(np.e)
        m = s.max()
        p = np.exp2(s - m)
        rec[h, 0], rec[h, 1] = m, p.sum()
        rec[h, 2:] = p @ v_rot
    return rec


def _worker(rank, world, port, result_dir):
    for p in (ROOT, os.path.join(ROOT, "polarquant-kv_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import inputs
        from oracle import pq_oracle as O
        from polarquant_kv.distributed import gather_partials, sequence_shard
        Hkv, Hq, S, D = 2, 8, 150, 64
        K, V, q = inputs.make_kvq(1, Hkv, Hq, S, D, seed=5)
        R = O.rotation_matrix(D, 0)
        cb, _ = O.lloyd_max_codebook(32, 4, n_iterations=20, grid_size=4000)
        kb, vb = O.compress(K[0], R, cb, 4), O.compress(V[0], R, cb, 4)
        lo, hi = sequence_shard(S, rank, world)
        rec = _partial_record(q[0], kb[:, lo:hi], vb[:, lo:hi], R, cb, 1.0 / np.sqrt(D))
        allrec = gather_partials(torch.from_numpy(rec)).numpy()
        assert allrec.shape == (world, Hq, D + 2)
        # numpy LSE merge + inverse rotation
        out = np.zeros((Hq, D))
        for h in range(Hq):
            live = allrec[:, h, 1] > 0
            m = allrec[live, h, 0].max()
            w = np.exp2(allrec[live, h, 0] - m)
            l = (w * allrec[live, h, 1]).sum()
            o = (w[:, None] * allrec[live, h, 2:]).sum(0) / l
            out[h] = O.inverse_rotate(o, R)
        ref = O.attention_from_blocks(q[0], kb, vb, R, cb, cb)[:, 0]
        err = float(np.abs(out - ref).max())
        np.save(os.path.join(result_dir, f"err{rank}.npy"), np.array([err, lo, hi]))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_sequence_sharded_decode_two_ranks_gloo(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    spans = []
    for r in range(world):
        err, lo, hi = np.load(tmp_path / f"err{r}.npy")
        assert err < 1e-4, (r, err)
        spans.append((int(lo), int(hi)))
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == 150
