"""CPU-side checks: the C-ABI library loads and exports every declared symbol; host logic
(codebook, thresholds, operand splits, parameter validation, shard arithmetic)."""

import ctypes
import os
import re

import numpy as np
import pytest

from oracle import pq_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for header in ("polarquant_b200.h", "polarquant_llama_abi.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(pq_[a-z0-9_]+|polarquant_[a-z_]+_c)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from polarquant_kv import _ext
    names = declared_symbols()
    assert len(names) >= 10
    handle = ctypes.CDLL(_ext.library_path())
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"
        assert n in _ext.SIGNATURES, f"{n} has no ctypes signature"
    lib = _ext.lib()
    assert lib.pq_version() >= 100
    assert lib.pq_strerror(0) == b"ok"
    assert b"head_dim" in lib.pq_strerror(2)


def test_argument_validation_without_gpu():
    """Status codes for bad arguments are decided on the host before anything is launched."""
    from polarquant_kv import _ext
    lib = _ext.lib()
    f = _ext.float_array([0.0] * 16)
    assert lib.pq_compress(None, -1, 128, 4, None, f, f, None, None, 0, None, None, None) == 4
    assert lib.pq_compress(None, 8, 96, 4, None, f, f, None, None, 0, None, None, None) == 2
    assert lib.pq_compress(None, 8, 128, 3, None, f, f, None, None, 0, None, None, None) == 3
    assert lib.pq_compress(None, 8, 128, 4, None, f, f, None, None, 0, None, None, None) == 1
    assert lib.pq_compress(None, 0, 128, 4, None, f, f, None, None, 0, None, None, None) == 0
    assert lib.pq_dequant(None, 4, 128, 5, f, None, None, 0, None) == 3
    assert lib.pq_lse_merge(None, 0, 4, 128, None, None, 0, None) == 4
    assert lib.pq_decode_attn_scratch_bytes(32, 32, 8, 8192, 128, 4) == 256 * 4 + 256 * 4 * 8 * 130 * 4
    assert lib.pq_decode_attn_scratch_bytes(1, 7, 2, 10, 128, 1) == 0     # q heads not a multiple of kv heads


def test_package_codebook_matches_oracle_and_reference(golden):
    from polarquant_kv.codebook import block_codebook, build_lloyd_max_codebook
    for bits in (2, 4):
        c, b = build_lloyd_max_codebook(32, bits)
        assert np.array_equal(c, golden[f"codebook_dim32_b{bits}"])
        assert np.array_equal(b, golden[f"boundaries_dim32_b{bits}"])
        assert np.array_equal(block_codebook(bits), c)


@pytest.mark.parametrize("bits", [2, 4])
def test_decision_thresholds_reproduce_argmin(golden, bits):
    from polarquant_kv.codebook import decision_thresholds
    c = golden[f"codebook_dim32_b{bits}"]
    thr = decision_thresholds(c)
    assert np.all(np.diff(thr) > 0)
    rng = np.random.default_rng(0)
    v = rng.uniform(-1, 1, 300000).astype(np.float32)
    edge = []
    for t in thr:
        x = np.float32(t)
        for _ in range(4):
            edge.append(x)
            x = np.nextafter(x, np.float32(np.inf))
        x = np.float32(t)
        for _ in range(4):
            x = np.nextafter(x, np.float32(-np.inf))
            edge.append(x)
    tiny = np.float32(10.0) ** np.arange(-45, -5, 0.5)
    v = np.concatenate([v, np.array(edge, np.float32), c, tiny.astype(np.float32), -tiny.astype(np.float32),
                        np.array([0.0, -0.0, 1.0, -1.0], np.float32)])
    want = O.nearest_centroid(v, c)
    got = (v[:, None] > thr[None, :]).sum(-1).astype(np.uint8)
    assert np.array_equal(want, got)


def test_rotation_api_and_split_accuracy(golden):
    from polarquant_kv.rotation import ROT_SCALE, generate_rotation_matrix, inverse_rotate, rotate, split_fp16
    R = generate_rotation_matrix(128, 0)
    assert np.array_equal(R, golden["R_d128_seed0"])           # same scipy call as the reference
    assert np.allclose(R.T @ R, np.eye(128), atol=1e-6)
    with pytest.raises(ValueError):
        generate_rotation_matrix(0)
    with pytest.raises(ValueError):
        generate_rotation_matrix(1.5)
    assert generate_rotation_matrix(1, 7).shape == (1, 1)
    v = np.random.default_rng(1).standard_normal((5, 128)).astype(np.float32)
    assert np.allclose(inverse_rotate(rotate(v, R), R), v, atol=1e-5)
    s = split_fp16(R, ROT_SCALE).astype(np.float64)
    back = (s[:, :128] + s[:, 128:]) / ROT_SCALE
    assert np.abs(back - R).max() < 2.0 ** -22


def test_parameter_validation_messages():
    from polarquant_kv.quantizer import _validate_params
    for bad in (dict(n_bits=1, group_size=32, d=128), dict(n_bits=9, group_size=32, d=128),
                dict(n_bits=4, group_size=0, d=128), dict(n_bits=4, group_size=256, d=128),
                dict(n_bits=3, group_size=32, d=128), dict(n_bits=4, group_size=16, d=128),
                dict(n_bits=4, group_size=32, d=96)):
        with pytest.raises(ValueError):
            _validate_params(**bad)
    _validate_params(4, 32, 128)
    _validate_params(2, 32, 64)


def test_utils_formulas():
    from polarquant_kv import utils
    assert utils.compute_compression_ratio(128, 4, 32, 0) == pytest.approx(128 * 16 / (16 + 512 + 128))
    assert utils.block_pq4_bits_per_vector(128, 4) == 4 * 144
    assert utils.block_pq4_compression_ratio(128, 4) == pytest.approx(2048 / 576)
    assert utils.estimate_memory_bytes(32, 8, 8192, 128, 4) == 32 * 8 * 8192 * 72
    assert utils.cosine_similarity(np.ones(4), np.ones(4)) == pytest.approx(1.0)
    assert utils.cosine_similarity(np.zeros(4), np.ones(4)) == 0.0


def test_jl_matrix_and_bit_packing(golden):
    import torch
    from polarquant_kv import qjl
    assert np.array_equal(qjl.generate_jl_matrix(128, 128, 1), golden["P_m128_d128_seed1"])
    with pytest.raises(ValueError):
        qjl.generate_jl_matrix(0, 8)
    signs = torch.from_numpy(np.random.default_rng(0).integers(0, 2, (3, 5, 40)).astype(bool))
    packed = qjl.bit_pack(signs)
    assert packed.shape == (3, 5, 5)
    assert np.array_equal(packed.numpy(), O.pack_sign_bits(signs.numpy()))
    assert torch.equal(qjl.bit_unpack(packed, 40), signs)


def test_shard_arithmetic():
    from polarquant_kv.distributed import batch_shard, sequence_shard
    for n, w in ((32, 8), (33, 8), (5, 8), (0, 4)):
        parts = [batch_shard(n, r, w) for r in range(w)]
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    for S, w in ((131072, 8), (1000, 3), (17, 4), (0, 2), (16, 8)):
        parts = [sequence_shard(S, r, w) for r in range(w)]
        assert parts[0][0] == 0 and parts[-1][1] == S
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert all(a[0] % 16 == 0 or a[0] == S for a in parts)
    with pytest.raises(ValueError):
        sequence_shard(10, 3, 2)


def test_cuda_only_api_refuses_cpu_tensors():
    import torch
    from polarquant_kv import attention, quantizer
    R = O.rotation_matrix(64, 0)
    with pytest.raises(TypeError):
        quantizer.compress(torch.zeros((1, 1, 2, 64), dtype=torch.float16), R)
    with pytest.raises(TypeError):
        attention.compressed_attention(torch.zeros((1, 2, 1, 64), dtype=torch.float16), None, None, R)


def test_llama_bridge_entry_points_reject_before_touching_the_device():
    """include/polarquant_llama_abi.h: the void entry points record why they did not run."""
    from polarquant_kv import _ext
    lib = _ext.lib()
    assert lib.polarquant_last_error_c() == 0
    lib.polarquant_compress_cuda_c(None, None, None, None, None, 4, 128, 16, None)
    assert lib.polarquant_last_error_c() == 1
    assert lib.polarquant_last_error_c() == 0            # reading clears it
    lib.polarquant_compress_cuda_c(None, None, None, None, None, 0, 128, 16, None)   # nothing to do
    assert lib.polarquant_last_error_c() == 0
    one = ctypes.c_void_p(256)
    lib.polarquant_compress_cuda_c(one, one, one, one, one, 4, 127, 16, None)
    assert lib.polarquant_last_error_c() == 2
    lib.polarquant_compress_cuda_c(one, one, one, one, one, 4, 128, 17, None)
    assert lib.polarquant_last_error_c() == 3
    lib.polarquant_fused_attention_cuda_c(one, one, one, one, one, one, one, 6, 4, 10, 64, 16, 1.0, None)
    assert lib.polarquant_last_error_c() == 4
    lib.polarquant_rotate_query_cuda_c(one, one, one, 2, 2048, None)
    assert lib.polarquant_last_error_c() == 2
    lib.polarquant_free_c(None)


def test_llama_bridge_oracle_known_answers():
    from oracle import llama_bridge_oracle as LO
    cb = np.array([-0.75, -0.25, 0.25, 0.75])
    # ties go to the first centroid; directions are rotated / radius
    assert LO.nearest_level(np.array([0.0, 0.5, -0.5, 1.0, -1.0]), cb).tolist() == [1, 2, 0, 3, 0]
    x = np.array([[3.0, 0.0, -4.0, 0.0]])
    radius, packed, direction = LO.compress(x, np.eye(4), cb)
    assert radius[0] == 5.0 and direction[0].tolist() == [0.6, 0.0, -0.8, 0.0]
    assert packed[0].tolist() == [3 | (1 << 4), 0 | (1 << 4)]
    assert LO.unpack(packed, 4)[0].tolist() == [3, 1, 0, 1]
    zero_radius, zero_packed, _ = LO.compress(np.zeros((1, 4)), np.eye(4), cb)
    assert zero_radius[0] == 0.0 and zero_packed[0].tolist() == [1 | (1 << 4)] * 2
    # attention over one token returns that token's value whatever the score is
    out = LO.fused_attention(np.ones((2, 4)), packed[None], radius[None], packed[None], radius[None], cb, 4, 0.5)
    np.testing.assert_allclose(out, np.tile(cb[[3, 1, 0, 1]] * 5.0, (2, 1)))
    rng = np.random.default_rng(0)
    R, _ = np.linalg.qr(rng.standard_normal((8, 8)))
    y = rng.standard_normal((3, 8))
    np.testing.assert_allclose(LO.inverse_rotate(LO.rotate(y, R), R), y, atol=1e-12)


def test_mixed_precision_plans_host_logic():
    """policy.py: the per-layer and per-token width plans and their run-length form (no GPU)."""
    from polarquant_kv import policy
    assert policy.compute_layer_bitwidths(2) == [4, 4]
    assert policy.compute_layer_bitwidths(24, 3.0) == [4] * 6 + [2] * 12 + [4] * 6
    plan = policy.compute_layer_bitwidths(12, 2.5)
    assert plan == [4, 4] + [2] * 9 + [4]            # three layers stay wide: the ends first, then inwards
    assert sum(policy.compute_layer_bitwidths(32, 3.5)) / 32 == pytest.approx(3.5, abs=0.07)
    tok = policy.compute_token_bitwidths(333)
    assert policy.runs_of(tok) == [(0, 4, 4), (4, 269, 2), (269, 333, 4)]
    assert policy.runs_of(policy.compute_token_bitwidths(50)) == [(0, 50, 4)]            # shorter than sink + window
    assert policy.runs_of(policy.compute_token_bitwidths(3)) == [(0, 3, 4)]
    assert policy.runs_of([]) == [] and policy.runs_of([2, 2, 4, 2]) == [(0, 2, 2), (2, 3, 4), (3, 4, 2)]
    # 4 + 64 tokens at 72 bytes, 4028 at 40 bytes against 256 bytes of float16 per token
    ratio = policy.estimate_mixed_compression_ratio(4096)
    assert ratio == pytest.approx(256 * 4096 / (68 * 72 + 4028 * 40), rel=1e-12)


def test_peer_exchange_entry_rejects_bad_arguments_on_the_host():
    from polarquant_kv import _ext
    lib = _ext.lib()
    assert lib.pq_lse_exchange_bytes(2, 64, 128) == ((2 * 2 * 64 * 130 * 4 + 127) // 128) * 128 + 128
    assert lib.pq_lse_exchange_bytes(0, 64, 128) == 0
    one = ctypes.c_void_p(256)
    ptrs = (ctypes.c_void_p * 2)(256, 512)
    assert lib.pq_lse_exchange_merge(one, 9, 0, ptrs, 1, 4, 128, one, one, 0, None) == 4      # more than eight ranks
    assert lib.pq_lse_exchange_merge(one, 2, 2, ptrs, 1, 4, 128, one, one, 0, None) == 4      # rank outside the group
    assert lib.pq_lse_exchange_merge(one, 2, 0, ptrs, 0, 4, 128, one, one, 0, None) == 4      # epochs start at 1
    assert lib.pq_lse_exchange_merge(one, 2, 0, ptrs, 1, 4, 96, one, one, 0, None) == 2
    assert lib.pq_lse_exchange_merge(one, 2, 0, ptrs, 1, 0, 128, one, one, 0, None) == 0      # nothing to do
    assert lib.pq_lse_exchange_merge(None, 2, 0, ptrs, 1, 4, 128, one, one, 0, None) == 1
    bad = (ctypes.c_void_p * 2)(256, 520)
    assert lib.pq_lse_exchange_merge(one, 2, 0, bad, 1, 4, 128, one, one, 0, None) == 6       # 128-byte alignment


def test_decoder_harness_host_pieces():
    """The dense-layer helpers of the decoder harness on the CPU: rotary tables against the closed form,
    stacked projection weights that follow in-place edits of their layers, the RMS norm formula."""
    import torch
    from polarquant_kv.inference import model as M

    torch.manual_seed(0)
    x = torch.randn(2, 3, 4, 16)
    pos = torch.tensor([5, 6, 7, 8])
    cos, sin = M.rotary_tables(pos, 16, 1.0e6)
    inv = 1.0 / (1.0e6 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
    ang = pos.float()[:, None] * inv[None, :]
    want = torch.empty_like(x)
    want[..., :8] = x[..., :8] * torch.cos(ang) - x[..., 8:] * torch.sin(ang)
    want[..., 8:] = x[..., 8:] * torch.cos(ang) + x[..., :8] * torch.sin(ang)
    assert torch.allclose(M.apply_rotary(x, cos, sin), want, atol=1e-6)
    assert torch.allclose(M.rotary(x, pos, 1.0e6), want, atol=1e-6)

    a, b = torch.nn.Linear(8, 6), torch.nn.Linear(8, 4)
    fused = M._FusedLinear(a, b)
    v = torch.randn(5, 8)
    with torch.no_grad():
        out = fused(v)
        assert torch.allclose(out[:, :6], a(v), atol=1e-6) and torch.allclose(out[:, 6:], b(v), atol=1e-6)
        b.weight.mul_(3.0)                                  # an in-place edit is picked up
        assert torch.allclose(fused(v)[:, 6:], b(v), atol=1e-6)

    norm = M.RMSNorm(8, 1e-6)
    with torch.no_grad():
        norm.weight.copy_(torch.randn(8))
        want_n = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * norm.weight
        assert torch.allclose(norm(v), want_n, atol=1e-6)


def _walk_balanced_partition(n_vrows, tiles_per_row, n_workers):
    """The decode kernel's balanced work partition, restated: the tiles of all virtual rows form one
    sequence cut into n_workers equal contiguous ranges; a worker walks the pieces of rows ("segments")
    inside its range and derives, from its own numbers alone, which segment of the row it holds and how many
    the row has (the row's ticket counter and record slots depend on every worker agreeing).
    Yields (worker, virtual row, first tile, end tile, segment index, segments of the row)."""
    all_tiles = n_vrows * tiles_per_row
    for w in range(n_workers):
        cur, cur_end = w * all_tiles // n_workers, (w + 1) * all_tiles // n_workers
        while cur < cur_end:
            vrow = cur // tiles_per_row
            row_t0, row_t1 = vrow * tiles_per_row, (vrow + 1) * tiles_per_row
            seg_end = min(cur_end, row_t1)
            c_first = ((row_t0 + 1) * n_workers + all_tiles - 1) // all_tiles - 1
            c_last = (row_t1 * n_workers + all_tiles - 1) // all_tiles - 1
            yield w, vrow, cur - row_t0, seg_end - row_t0, w - c_first, c_last - c_first + 1
            cur = seg_end


def test_decode_partition_arithmetic():
    """Invariants the kernel and the host-side scratch layout rely on, over many shapes: every tile is covered
    once; the workers that share a row number their pieces 0..n-1 and agree on n; n never exceeds the number
    of record slots per row the scratch is sized for; a worker's pieces are consecutive rows and every piece
    after its first starts at tile 0 of its row (the query rotation of several pieces in one pass and the
    look-ahead for the next piece's first tiles assume both)."""
    from polarquant_kv import _ext
    lib = _ext.lib()
    rng = np.random.default_rng(3)
    shapes = [(256, 512), (32, 512), (8, 8192), (1536, 3), (1280, 4), (1, 1), (1, 7), (296, 1), (297, 1), (5, 59),
              (128, 272), (16, 272), (1000, 1), (3, 100000)]
    shapes += [(int(rng.integers(1, 2000)), int(rng.integers(1, 700))) for _ in range(40)]
    for n_vrows, tiles in shapes:
        # scratch layout for this shape: batch = n_vrows rows of one KV head with four query heads (one group)
        seq_len = tiles * 16
        need = lib.pq_decode_attn_scratch_bytes(n_vrows, 4, 1, seq_len, 128, 0)
        tickets = (n_vrows * 4 + 255) // 256 * 256
        slots = (need - tickets) // (n_vrows * 8 * 130 * 4)
        assert tickets + n_vrows * slots * 8 * 130 * 4 == need
        # (the library sizes the scratch for the device it runs on: 148 SMs when there is none)
        for sms, teams in ((148, 2), (148, 1), (132, 2)):
            n_workers = max(1, min(n_vrows * tiles, sms * teams))
            covered = np.zeros(n_vrows * tiles, dtype=np.int32)
            seen, last = {}, {}
            for w, vrow, t0, t1, idx, n in _walk_balanced_partition(n_vrows, tiles, n_workers):
                assert 0 <= t0 < t1 <= tiles and 0 <= idx < n
                covered[vrow * tiles + t0: vrow * tiles + t1] += 1
                seen.setdefault(vrow, []).append((idx, n))
                if w in last:
                    assert vrow == last[w] + 1 and t0 == 0, (n_vrows, tiles, n_workers, w)
                last[w] = vrow
            assert (covered == 1).all()
            for vrow, pieces in seen.items():
                n = pieces[0][1]
                assert sorted(i for i, _ in pieces) == list(range(n)) and all(m == n for _, m in pieces)
                if sms == 148:
                    assert n <= slots, (n_vrows, tiles, n_workers, n, slots)


def test_reference_gpu_package_paths_resolve():
    """Every module path and name the reference's tests import from polarquant_kv_cuda resolves (the functions
    themselves need a GPU); the layer classes build and run without a cache on the CPU."""
    import importlib

    import torch
    wanted = {
        "polarquant_kv_cuda.rotation": ["generate_rotation_matrix", "rotate", "inverse_rotate"],
        "polarquant_kv_cuda.lloyd_max": ["build_lloyd_max_codebook", "quantize_with_codebook",
                                         "dequantize_with_codebook", "get_codebook_torch"],
        "polarquant_kv_cuda.types": ["CompressedKVCacheGPU"],
        "polarquant_kv_cuda.compress_kernel": ["compress_gpu"],
        "polarquant_kv_cuda.decompress_kernel": ["decompress_gpu"],
        "polarquant_kv_cuda.attention_kernel": ["compressed_attention_gpu"],
        "polarquant_kv_cuda.qjl_kernel": ["compute_signatures_gpu", "compute_correction_gpu", "bit_pack", "bit_unpack"],
        "polarquant_kv_cuda.compressor": ["compress", "decompress", "compressed_attention", "get_memory_bytes"],
        "polarquant_kv_cuda.utils": ["cosine_similarity", "check_memory_warning", "cosine_similarity_gpu"],
        "polarquant_kv_cuda.adaptive_bitwidth": ["compute_layer_bitwidths", "estimate_adaptive_compression_ratio"],
        "polarquant_kv_cuda.token_importance": ["compute_token_bitwidths", "estimate_mixed_compression_ratio"],
        "polarquant_kv_cuda.hf_integration": ["CompressedDynamicCache", "patch_model", "create_compressed_cache"],
        "polarquant_kv_cuda.inference.config": ["PolarQuantConfig"],
        "polarquant_kv_cuda.inference.kv_cache": ["KVCacheManager"],
        "polarquant_kv_cuda.inference.attention": ["CompressedMultiHeadAttention"],
        "polarquant_kv_cuda.inference.transformer": ["SimpleTransformer", "SimpleTransformerLayer"],
    }
    for module, names in wanted.items():
        mod = importlib.import_module(module)
        assert [n for n in names if not hasattr(mod, n)] == [], module
    from polarquant_kv_cuda.inference.config import PolarQuantConfig
    from polarquant_kv_cuda.inference.transformer import SimpleTransformer
    from polarquant_kv_cuda.rotation import generate_rotation_matrix, inverse_rotate, rotate
    model = SimpleTransformer(PolarQuantConfig(), num_layers=2, embed_dim=64, num_heads=4, num_kv_heads=2, vocab_size=50)
    with torch.no_grad():
        assert model(torch.randint(0, 50, (2, 5))).shape == (2, 5, 50)
    assert {"layers.0.attn.q_proj.weight", "layers.1.ffn.2.weight", "layers.0.norm2.bias", "embed.weight",
            "head.weight"} <= set(model.state_dict())
    from polarquant_kv_cuda.adaptive_bitwidth import compute_layer_bitwidths, estimate_adaptive_compression_ratio
    plan = compute_layer_bitwidths(24, 3.0)
    assert plan[0] == plan[-1] == 4 and plan[12] == 2 and abs(sum(plan) / 24 - 3.0) <= 0.1
    assert abs(estimate_adaptive_compression_ratio([4, 2]) - 16.0 / 3.5) < 1e-9
    R = generate_rotation_matrix(64, 3, device="cpu")
    v = torch.randn(5, 64)
    assert R.dtype == torch.float32 and torch.allclose(inverse_rotate(rotate(v, R), R), v, atol=1e-5)
    assert np.allclose(R.numpy(), O.rotation_matrix(64, 3), atol=1e-7)


def test_decode_split_mode_partition_arithmetic():
    """n_splits >= 1, restated from the decode kernel: every row is cut into n_splits pieces of
    ceil(tiles / n_splits) tiles, the pieces of all rows are dealt round-robin to the workers.  Every
    tile is covered once, pieces past the end of a row are empty (they deliver an empty record), and the
    scratch holds n_splits record slots per row; the library's default split count stays within its bounds."""
    from polarquant_kv import _ext
    lib = _ext.lib()
    rng = np.random.default_rng(4)
    for _ in range(60):
        n_vrows, tiles = int(rng.integers(1, 300)), int(rng.integers(1, 600))
        n_splits = int(rng.integers(1, min(tiles, 40) + 1))
        per = -(-tiles // n_splits)
        covered = np.zeros(n_vrows * tiles, dtype=np.int32)
        n_workers = 2 * 148
        handled = 0
        for w in range(n_workers):
            for item in range(w, n_vrows * n_splits, n_workers):
                vrow, seg = divmod(item, n_splits)
                t0, t1 = seg * per, min(tiles, seg * per + per)
                handled += 1
                if t0 < t1:
                    covered[vrow * tiles + t0: vrow * tiles + t1] += 1
        assert handled == n_vrows * n_splits and (covered == 1).all()
        need = lib.pq_decode_attn_scratch_bytes(n_vrows, 4, 1, tiles * 16, 64, n_splits)
        assert need == (n_vrows * 4 + 255) // 256 * 256 + n_vrows * n_splits * 8 * 66 * 4
    for batch, hq, hkv, s in ((1, 64, 8, 131072), (32, 32, 8, 8192), (1, 8, 8, 16), (4, 14, 2, 5000)):
        d = lib.pq_decode_attn_default_splits(batch, hq, hkv, s, 128)
        assert 1 <= d <= max(1, min(64, -(-s // 16) // 32))
