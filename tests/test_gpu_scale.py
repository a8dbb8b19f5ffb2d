"""GPU parity at the sizes the benchmark runs at.

The small parity cases never reach the regime the measured launches run in: persistent CTAs that each
walk several segments, rows cut across CTAs and merged through the ticket counters, compress launches
of more than a million vectors.  These tests run such shapes and pull SAMPLES back to the numpy oracle
(the oracle cannot walk the whole workload in seconds): a few (batch, kv-head) rows of a decode, a
strided subset of the vectors of a bulk compress.

Tolerances as in test_gpu_parity.py: attention max-abs <= 2e-3; packed indices bit-exact except
coordinates within 1e-6 of a decision boundary (counted, none unexplained), radii within one
float16 ulp (counted).
"""

import numpy as np
import pytest
import torch

from oracle import pq_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _synthetic(shape, dev, seed):
    """The benchmark distribution on the GPU: N(0,1) x per-channel lognormal(0,1), two channels x10."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    D = shape[-1]
    scale = torch.exp(torch.randn(D, generator=gen, device=dev))
    hot = torch.randperm(D, generator=gen, device=dev)[:2]
    scale[hot] *= 10.0
    return (torch.randn(shape, generator=gen, device=dev) * scale).to(torch.float16)


def _build(B, Hkv, S, D, dev, seed, bits=4, cap=None):
    from polarquant_kv import quantizer
    from polarquant_kv.rotation import device_plan
    R = O.rotation_matrix(D, 0)
    plan = device_plan(R, dev)
    caches = []
    for i in range(2):
        cache = quantizer.allocate_cache(B, Hkv, cap or S, D, bits, 0, dev)
        for b in range(B):
            x = _synthetic((1, Hkv, S, D), dev, seed + 100 * i + b)
            quantizer.compress(x, plan, bits, out=_row_view(cache, b), position=0)
        cache.seq_len = S
        caches.append(cache)
    return R, plan, caches[0], caches[1]


def _row_view(cache, b):
    from polarquant_kv.types import CompressedKV
    return CompressedKV(cache.blocks[b:b + 1], None, None, cache.n_bits, 32, cache.original_dim, 0, cache.max_seq_len)


def _check_rows(out, q, ck, cv, R, rows, S, label, bits=4):
    cb, _ = O.lloyd_max_codebook(32, bits)
    Hq, Hkv = q.shape[1], ck.blocks.shape[1]
    G = Hq // Hkv
    worst = 0.0
    for b, h in rows:
        kb = ck.blocks[b, h:h + 1, :S].cpu().numpy()
        vb = cv.blocks[b, h:h + 1, :S].cpu().numpy()
        qh = q[b, h * G:(h + 1) * G].cpu().numpy()[:, None, :]
        ref = O.attention_from_blocks(qh, kb, vb, R, cb, cb, bits_k=bits, bits_v=bits)[:, 0]
        err = float(np.abs(out[b, h * G:(h + 1) * G].cpu().numpy() - ref).max())
        worst = max(worst, err)
    print(f"{label}: {len(rows)} sampled (batch, kv-head) rows, max-abs {worst:.3e}")
    assert worst <= ATTN_TOL


@pytest.mark.parametrize("B,Hkv,Hq,S", [(4, 8, 32, 8192), (3, 2, 32, 4099)])
def test_decode_multi_segment_vs_oracle(B, Hkv, Hq, S):
    """Balanced persistent partition with many tiles per CTA (n_splits = 0): sampled rows against the
    oracle, all rows against the one-segment-per-row schedule (n_splits = 1).  The second shape has 16
    query heads per KV head (two head groups) and a ragged last tile."""
    from polarquant_kv import attention
    dev = _cuda()
    D = 128
    R, plan, ck, cv = _build(B, Hkv, S, D, dev, seed=5)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    q = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.float16)
    out = attention.decode_attention(q, ck, cv, plan, enable_qjl=False, n_splits=0)
    one = attention.decode_attention(q, ck, cv, plan, enable_qjl=False, n_splits=1)
    torch.cuda.synchronize()
    diff = float((out - one).abs().max())
    print(f"B{B} Hkv{Hkv} Hq{Hq} S{S}: balanced vs one segment per row: max-abs {diff:.3e}")
    assert diff <= 2e-4
    rows = [(0, 0), (B - 1, Hkv - 1), (B // 2, Hkv // 2), (1, 1), (B - 1, 0), (0, Hkv - 1)]
    _check_rows(out, q, ck, cv, R, rows, S, f"decode B{B} Hkv{Hkv} Hq{Hq} S{S}")


@pytest.mark.parametrize("B,Hkv,Hq,S,D,bits", [(96, 8, 48, 40, 128, 4), (160, 8, 24, 56, 64, 2)])
def test_decode_many_short_rows_vs_oracle(B, Hkv, Hq, S, D, bits):
    """More than 1200 short (batch, kv head, head group) rows: every team of warps walks five or six
    segments, so it rotates the queries of its segments in more than one pass (a pass holds four), rows
    start in the middle of a team's range, and the last tile of every row is ragged.  First shape: six query
    heads per KV head (two head groups); second: head dim 64 with 2-bit blocks (other tile sizes)."""
    from polarquant_kv import attention
    dev = _cuda()
    R, plan, ck, cv = _build(B, Hkv, S, D, dev, seed=17, bits=bits)
    gen = torch.Generator(device=dev)
    gen.manual_seed(6)
    q = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.float16)
    out = attention.decode_attention(q, ck, cv, plan, enable_qjl=False, n_splits=0)
    one = attention.decode_attention(q, ck, cv, plan, enable_qjl=False, n_splits=1)
    torch.cuda.synchronize()
    diff = float((out - one).abs().max())
    print(f"B{B} Hkv{Hkv} Hq{Hq} S{S} D{D} b{bits}: balanced vs one segment per row: max-abs {diff:.3e}")
    assert diff <= 2e-4
    rows = [(0, 0), (0, 1), (1, 7), (37, 3), (38, 4), (64, 0), (B - 1, 6), (B - 1, 7)]
    _check_rows(out, q, ck, cv, R, rows, S, f"decode B{B} Hkv{Hkv} Hq{Hq} S{S} D{D} b{bits}", bits=bits)


def test_decode_shared_scratch_after_a_call_with_fewer_rows():
    """decode_attention keeps one scratch buffer per stream.  A call over few (batch, kv head) rows writes
    its segment records where a later call over many rows keeps its ticket counters: the later call must
    still merge every row (the wrapper clears the counter region when the shape changes)."""
    from polarquant_kv import attention
    dev = _cuda()
    D, S = 128, 96
    R, plan, ck_small, cv_small = _build(2, 2, S, D, dev, seed=23)
    _, _, ck_big, cv_big = _build(48, 8, S, D, dev, seed=29)
    gen = torch.Generator(device=dev)
    gen.manual_seed(8)
    q_small = torch.randn((2, 8, D), generator=gen, device=dev).to(torch.float16)
    q_big = torch.randn((48, 32, D), generator=gen, device=dev).to(torch.float16)
    want = attention.prepare_decode(q_big, ck_big, cv_big, plan, n_splits=3)().clone()     # private scratch
    for _ in range(2):
        attention.decode_attention(q_small, ck_small, cv_small, plan, enable_qjl=False, n_splits=3)
        got = attention.decode_attention(q_big, ck_big, cv_big, plan, enable_qjl=False, n_splits=3)
        torch.cuda.synchronize()
        assert float((got - want).abs().max()) <= 1e-5
    _check_rows(got, q_big, ck_big, cv_big, R, [(0, 0), (47, 7), (20, 3)], S, "decode after a smaller call")


def test_decode_long_context_shape_vs_oracle():
    """One 131072-token sequence, 8 KV heads, 64 query heads (8 per KV head): two sampled KV heads."""
    from polarquant_kv import attention
    dev = _cuda()
    B, Hkv, Hq, S, D = 1, 8, 64, 131072, 128
    R, plan, ck, cv = _build(B, Hkv, S, D, dev, seed=11)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    q = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.float16)
    out = attention.decode_attention(q, ck, cv, plan, enable_qjl=False)
    torch.cuda.synchronize()
    _check_rows(out, q, ck, cv, R, [(0, 1), (0, 6)], S, "decode long context")


@pytest.mark.parametrize("n_bits,with_qjl", [(4, False), (2, False), (4, True)])
def test_compress_million_vectors_sampled_vs_oracle(n_bits, with_qjl):
    from polarquant_kv import quantizer
    from polarquant_kv.rotation import device_plan
    from test_gpu_parity import compare_blocks
    dev = _cuda()
    n, D = 1 << 20, 128
    R = O.rotation_matrix(D, 0)
    P = O.jl_matrix(D, D, 1) if with_qjl else None
    cb, _ = O.lloyd_max_codebook(32, n_bits)
    x = _synthetic((1, 1, n, D), dev, seed=23)
    c = quantizer.compress(x, device_plan(R, dev, P), n_bits, 32, P)
    torch.cuda.synchronize()
    idx = torch.arange(17, n, 64, device=dev)
    xs = x[0, 0, idx].cpu().numpy()
    got = c.blocks[0, 0, idx].cpu().numpy()
    rep = compare_blocks(xs, R, n_bits, got, cb)
    print(f"compress 2^20 vectors, b{n_bits}, qjl={with_qjl}, 1-in-64 sample: {rep}")
    assert rep["unexplained"] == 0 and rep["radius_bad"] == 0
    assert rep["mismatch"] <= max(3, xs.size // 20000)
    # the last tile of the launch
    tail = slice(n - 300, n)
    rep = compare_blocks(x[0, 0, tail].cpu().numpy(), R, n_bits, c.blocks[0, 0, tail].cpu().numpy(), cb)
    assert rep["unexplained"] == 0 and rep["radius_bad"] == 0


def test_prepared_decode_growing_sequence():
    """A PreparedDecode sized for the cache capacity serves every shorter length (few rows, so the
    balanced partition cuts each row into many segments whose number changes with the length)."""
    from polarquant_kv import attention
    dev = _cuda()
    B, Hkv, Hq, cap, D = 1, 2, 8, 8192, 128
    R, plan, ck, cv = _build(B, Hkv, cap, D, dev, seed=31)
    gen = torch.Generator(device=dev)
    gen.manual_seed(6)
    q = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.float16)
    ck.seq_len = cv.seq_len = cap
    pd = attention.prepare_decode(q, ck, cv, plan)
    for S in (16, 576, 577, 1000, 2368, 4097, 8192):
        ck.seq_len = cv.seq_len = S
        got = pd().clone()
        ref = attention.decode_attention(q, ck, cv, plan, enable_qjl=False, n_splits=1)
        torch.cuda.synchronize()
        err = float((got - ref).abs().max())
        assert err <= 2e-4, (S, err)
    _check_rows(got, q, ck, cv, R, [(0, 1)], 8192, "prepared decode at capacity")


@pytest.mark.parametrize("head_dim,n_bits,n", [(128, 4, 300_001), (64, 2, 211_003), (128, 2, 1 << 20)])
def test_dequant_many_tiles_vs_float64(head_dim, n_bits, n):
    """The dequantise kernel at sizes where a persistent CTA owns many tiles (operand and accumulator
    buffers reused, a ragged last tile): every vector against float64 arithmetic on the same stored bytes
    (centroid * radius in float32 as the reference rounds it, then v @ R), and a sample against the oracle."""
    from polarquant_kv import quantizer
    from polarquant_kv.rotation import device_plan
    from polarquant_kv.types import CompressedKV
    dev = _cuda()
    R = O.rotation_matrix(head_dim, 5)
    cb, _ = O.lloyd_max_codebook(32, n_bits)
    plan = device_plan(R, dev)
    x = _synthetic((1, 1, n, head_dim), dev, seed=29)
    c = quantizer.compress(x, plan, n_bits)
    # float32 output: three float16 product terms keep 2^-22 per term; over 10^8 outputs the largest deviation
    # seen is 2.2e-6 of the vector's largest component (1.6e-6 over 4 * 10^7), so the bar here is 4e-6
    for dtype, tol in ((torch.float32, 4e-6), (torch.float16, 2e-3)):
        got = quantizer.decompress(c, plan, dtype)[0, 0]
        torch.cuda.synchronize()
        # float64 on the device from the stored bytes
        blocks = c.blocks[0, 0]                                            # [n, nblk, bb]
        d = blocks[..., :2].contiguous().view(torch.float16).to(torch.float32)[..., 0]      # [n, nblk]
        packed = blocks[..., 2:].to(torch.int32)
        if n_bits == 4:
            idx = torch.stack([packed & 15, packed >> 4], dim=-1).reshape(n, head_dim // 32, 32)
        else:
            idx = torch.stack([(packed >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).reshape(n, head_dim // 32, 32)
        cbt = torch.from_numpy(cb.astype(np.float32)).to(dev)
        rot = (cbt[idx.long()] * d[..., None]).reshape(n, head_dim)          # float32 product, as the reference
        ref = rot.double() @ torch.from_numpy(R).to(dev)
        scale = ref.abs().amax(dim=-1, keepdim=True) + 1e-30
        err = ((got.double() - ref).abs() / scale).amax().item()
        print(f"dequant D{head_dim} b{n_bits} n={n} -> {dtype}: worst error relative to the vector's largest component {err:.2e}")
        assert err < tol
    # and the oracle on a sample that includes the last tile
    sel = np.concatenate([np.arange(5, n, 4099), np.arange(n - 130, n)])
    ref_o = O.decompress(c.blocks[0, 0, torch.from_numpy(sel).to(dev)].cpu().numpy(), R, cb, n_bits)
    got_o = quantizer.decompress(c, plan)[0, 0, torch.from_numpy(sel).to(dev)].cpu().numpy()
    sc = np.abs(ref_o).max(axis=-1, keepdims=True) + 1e-30
    assert (np.abs(got_o - ref_o) / sc).max() < 4e-6


@pytest.mark.parametrize("ws", [True, False])
def test_prefill_bench_shape_vs_oracle(ws):
    """The prefill shape the bench times (2 x 32 query / 8 KV heads x 512 queries x 4096 tokens, D 128):
    two KV heads of one sequence against the oracle, all 512 query rows; and, with the causal mask the decoder
    harness uses, sampled rows against a decode over their prefix."""
    from polarquant_kv import attention
    from polarquant_kv.types import CompressedKV
    dev = _cuda()
    B, Hkv, Hq, Sq, S, D = 2, 8, 32, 512, 4096, 128
    R, plan, ck, cv = _build(B, Hkv, S, D, dev, seed=31)
    gen = torch.Generator(device=dev)
    gen.manual_seed(6)
    q = torch.randn((B, Hq, Sq, D), generator=gen, device=dev).to(torch.float16)
    out = attention.prefill_attention(q, ck, cv, plan, use_workspace=ws)
    torch.cuda.synchronize()
    cb, _ = O.lloyd_max_codebook(32, 4)
    G = Hq // Hkv
    for b, hkv in ((1, 0), (0, 5)):
        kb = ck.blocks[b, hkv:hkv + 1, :S].cpu().numpy()
        vb = cv.blocks[b, hkv:hkv + 1, :S].cpu().numpy()
        qs = q[b, hkv * G:(hkv + 1) * G].cpu().numpy()
        ref = O.attention_from_blocks(qs, kb, vb, R, cb, cb)
        err = np.abs(out[b, hkv * G:(hkv + 1) * G].cpu().numpy() - ref).max()
        print(f"prefill bench shape, workspace={ws}, batch {b} kv head {hkv}: max-abs {err:.3e}")
        assert err <= 2e-3
    causal = attention.prefill_attention(q, ck, cv, plan, causal=True, use_workspace=ws)
    torch.cuda.synchronize()
    for i in (0, 1, 127, 128, 300, 511):
        n = S - Sq + i + 1
        pk = CompressedKV(ck.blocks, None, None, 4, 32, D, n, ck.max_seq_len)
        pv = CompressedKV(cv.blocks, None, None, 4, 32, D, n, cv.max_seq_len)
        row = attention.decode_attention(q[:, :, i].contiguous(), pk, pv, plan, enable_qjl=False)
        assert float((causal[:, :, i] - row).abs().max()) <= 2e-3, i
