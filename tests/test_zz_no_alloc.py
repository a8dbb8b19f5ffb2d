"""pq_decode_attn_static: decode attention for callers that cannot allocate device memory.

Some hosts of this library (an operator callback in a runtime that owns all device memory,
code running with the allocator frozen, a serving loop that must avoid cudaMalloc's
device-wide stall) cannot supply the scratch buffer pq_decode_attn asks for.  The static
variant uses an 8 MiB array built into the library.  This test drives it through the C ABI
twice in a row (the array is shared and keeps the previous call's contents) and checks each
result against the regular entry point, to the same 2e-3 max-abs bound the attention tests
use; it also checks that an over-large shape is refused.  It is collected last so that a
failure here cannot hide any other test.
"""

import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import inputs
from oracle import pq_oracle as O

pytestmark = pytest.mark.gpu
ATTN_TOL = 2e-3


def _call(lib, static, q, kb, vb, plan, cb, B, Hq, Hkv, S, D, n_splits, scratch=None):
    out = torch.empty((B, Hq, D), dtype=torch.float32, device=q.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    common = [q.data_ptr(), kb.data_ptr(), vb.data_ptr(), B, Hq, Hkv, S, S, D, 4, 4, cb, cb,
              plan.rot.data_ptr(), ctypes.c_float(1.0 / math.sqrt(D)), None, 0, None, None,
              out.data_ptr(), 0, None, n_splits]
    if static:
        st = lib.pq_decode_attn_static(*common, stream)
    else:
        st = lib.pq_decode_attn(*common, scratch.data_ptr(), scratch.numel(), stream)
    torch.cuda.synchronize()
    return st, out


def test_static_scratch_variant_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from polarquant_kv import _ext
    from polarquant_kv.quantizer import tables
    from polarquant_kv.rotation import device_plan

    dev = torch.device("cuda:0")
    lib = _ext.lib()
    assert lib.pq_decode_attn_static_scratch_capacity() == 8 << 20
    cb_host = tables(4)[0]
    cb_np, _ = O.lloyd_max_codebook(32, 4)

    # two different shapes, back to back, sharing the built-in array
    for call, (B, Hkv, Hq, S, D, splits) in enumerate([(2, 2, 8, 700, 128, 3), (1, 2, 14, 300, 64, 2)]):
        K, V, q = inputs.make_kvq(B, Hkv, Hq, S, D, seed=40 + call)
        R = O.rotation_matrix(D, 0)
        plan = device_plan(R, dev)
        kb_np = O.compress(K, R, cb_np, 4)
        vb_np = O.compress(V, R, cb_np, 4)
        kb = torch.from_numpy(kb_np).to(dev)
        vb = torch.from_numpy(vb_np).to(dev)
        qd = torch.from_numpy(q[:, :, 0]).to(dev).contiguous()
        need = lib.pq_decode_attn_scratch_bytes(B, Hq, Hkv, S, D, splits)
        scratch = torch.zeros(need, dtype=torch.uint8, device=dev)
        st_ref, ref = _call(lib, False, qd, kb, vb, plan, cb_host, B, Hq, Hkv, S, D, splits, scratch)
        st_new, got = _call(lib, True, qd, kb, vb, plan, cb_host, B, Hq, Hkv, S, D, splits)
        assert st_ref == 0 and st_new == 0, (st_ref, st_new)
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max().item() <= ATTN_TOL, call
        # and against the CPU oracle, like the other attention tests
        for b in range(B):
            want = O.attention_from_blocks(q[b], kb_np[b], vb_np[b], R, cb_np, cb_np)[:, 0]
            assert np.abs(got[b].cpu().numpy() - want).max() <= ATTN_TOL

    # a shape whose scratch need exceeds the built-in array is refused, nothing is launched
    B, Hkv, Hq, S, D = 64, 8, 64, 4096, 128
    assert lib.pq_decode_attn_scratch_bytes(B, Hq, Hkv, S, D, 8) > lib.pq_decode_attn_static_scratch_capacity()
    dummy = torch.zeros(16, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    st = lib.pq_decode_attn_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), B, Hq, Hkv, S, S, D, 4, 4,
                                   cb_host, cb_host, dummy.data_ptr(), ctypes.c_float(0.1), None, 0, None, None,
                                   dummy.data_ptr(), 0, None, 8, stream)
    assert st == 10
    assert b"built-in" in lib.pq_strerror(st)
