"""Calls of different shapes one after another on one stream.

Every other GPU test builds one shape and checks it.  A serving process interleaves shapes: the library and
its Python layer keep state between calls (a scratch buffer per stream, a prefill workspace, per-kernel
attributes, cached plans and tables), and that state must not leak from one shape into the next.  Each call
here is checked against a call of the same shape that owns fresh state (a PreparedDecode with a private,
zeroed scratch; a freshly allocated output), and sampled rows against the numpy oracle.
"""

import numpy as np
import pytest
import torch

from oracle import pq_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3

# (batch, kv heads, query heads per kv head, tokens, head dim, key bits, value bits, n_splits, sketch)
DECODE_SHAPES = [
    (2, 2, 4, 100, 128, 4, 4, 0, False),
    (40, 8, 4, 200, 128, 4, 4, 3, False),
    (3, 1, 7, 333, 64, 4, 4, 2, False),
    (64, 4, 2, 64, 64, 2, 2, 0, False),
    (1, 8, 8, 3000, 128, 4, 2, 0, False),
    (16, 2, 1, 500, 128, 2, 4, 3, False),
    (5, 2, 4, 77, 128, 4, 4, 2, True),       # an odd capacity with the sketch: side-band rows off the 16-byte grid
    (48, 8, 4, 96, 128, 4, 4, 3, False),
    (2, 2, 4, 100, 128, 4, 4, 4, False),
    (300, 4, 4, 40, 64, 4, 4, 0, False),
    (7, 3, 5, 1000, 128, 4, 4, 0, True),
]


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _case(shape, dev, seed):
    from polarquant_kv import quantizer
    from polarquant_kv.qjl import generate_jl_matrix
    from polarquant_kv.rotation import device_plan
    B, Hkv, G, S, D, kb, vb, n_splits, sketch = shape
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    R = O.rotation_matrix(D, seed % 5)
    P = generate_jl_matrix(D, D, 1) if sketch else None
    plan = device_plan(R, dev, P)
    scale = torch.exp(torch.randn(D, generator=gen, device=dev))
    k = (torch.randn((B, Hkv, S, D), generator=gen, device=dev) * scale).to(torch.float16)
    v = (torch.randn((B, Hkv, S, D), generator=gen, device=dev) * scale).to(torch.float16)
    ck = quantizer.compress(k, plan, kb, 32, plan.jl if sketch else None)
    cv = quantizer.compress(v, plan, vb)
    q = torch.randn((B, Hkv * G, D), generator=gen, device=dev).to(torch.float16)
    return R, plan, ck, cv, q


def test_decode_calls_of_many_shapes_share_one_stream():
    from polarquant_kv import attention
    dev = _cuda()
    worst = 0.0
    for rnd in range(2):                                   # the second round meets state left by every shape
        for i, shape in enumerate(DECODE_SHAPES):
            B, Hkv, G, S, D, kb, vb, n_splits, sketch = shape
            R, plan, ck, cv, q = _case(shape, dev, 100 * rnd + i)
            got = attention.decode_attention(q, ck, cv, plan, enable_qjl=sketch, n_splits=n_splits)
            want = attention.prepare_decode(q, ck, cv, plan, n_splits=n_splits, enable_qjl=sketch)().clone()
            torch.cuda.synchronize()
            assert torch.isfinite(got).all(), shape
            diff = float((got - want).abs().max())
            assert diff <= 1e-5 * max(1.0, float(want.abs().max())), (shape, diff)
            if not sketch:
                cbk, _ = O.lloyd_max_codebook(32, kb)
                cbv, _ = O.lloyd_max_codebook(32, vb)
                for b, h in ((0, 0), (B - 1, Hkv - 1)):
                    ref = O.attention_from_blocks(q[b, h * G:(h + 1) * G].cpu().numpy()[:, None, :],
                                                  ck.blocks[b, h:h + 1].cpu().numpy(), cv.blocks[b, h:h + 1].cpu().numpy(),
                                                  R, cbk, cbv, bits_k=kb, bits_v=vb)[:, 0]
                    err = float(np.abs(got[b, h * G:(h + 1) * G].cpu().numpy() - ref).max())
                    worst = max(worst, err / max(1.0, float(np.abs(ref).max())))
                    assert err <= ATTN_TOL * max(1.0, float(np.abs(ref).max())), (shape, b, h, err)
    print(f"{2 * len(DECODE_SHAPES)} decode calls over {len(DECODE_SHAPES)} shapes: worst oracle error "
          f"{worst:.2e} of max(1, largest output)")


def test_prefill_and_compress_calls_of_many_shapes_share_one_stream():
    """The prefill workspace grows and shrinks in use, compress re-encodes its tensor map per call, and both
    alternate with decode calls: every result equals the one a first call of that shape gives."""
    from polarquant_kv import attention, quantizer
    dev = _cuda()
    shapes = [(1, 2, 4, 300, 128, 4, 4, 0, False), (2, 8, 4, 1100, 128, 4, 4, 0, False),
              (3, 2, 7, 130, 64, 4, 4, 0, False), (1, 4, 2, 2050, 128, 2, 2, 0, False),
              (2, 2, 4, 65, 64, 4, 2, 0, False)]
    first = {}
    for rnd in range(2):
        for i, shape in enumerate(shapes):
            B, Hkv, G, S, D, kb, vb, _, _ = shape
            R, plan, ck, cv, q = _case(shape, dev, 7 + i)          # the same data in both rounds
            Sq = min(S, 70 + 30 * i)
            gen = torch.Generator(device=dev)
            gen.manual_seed(50 + i)
            qs = torch.randn((B, Hkv * G, Sq, D), generator=gen, device=dev).to(torch.float16)
            outs = [attention.prefill_attention(qs, ck, cv, plan, causal=True, use_workspace=ws) for ws in (True, False)]
            dec = attention.decode_attention(q, ck, cv, plan, enable_qjl=False)
            torch.cuda.synchronize()
            assert float((outs[0] - outs[1]).abs().max()) <= ATTN_TOL
            # the last query row of a causal prefill sees the whole cache, like a decode step with that query
            last = attention.decode_attention(qs[:, :, -1].contiguous(), ck, cv, plan, enable_qjl=False)
            assert float((outs[0][:, :, -1] - last).abs().max()) <= ATTN_TOL * max(1.0, float(last.abs().max()))
            key = i
            if rnd == 0:
                first[key] = (ck.blocks.clone(), cv.blocks.clone(), outs[0].clone(), dec.clone())
            else:
                fk, fv, fo, fd = first[key]
                assert torch.equal(ck.blocks, fk) and torch.equal(cv.blocks, fv)
                assert float((outs[0] - fo).abs().max()) <= 1e-5 * max(1.0, float(fo.abs().max()))
                assert float((dec - fd).abs().max()) <= 1e-5 * max(1.0, float(fd.abs().max()))
