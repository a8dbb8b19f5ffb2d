"""GPU tests of the inference-side users of the compressed cache: the in-place cache manager
(successor of the reference's KVCacheManager) and the decoder harness that attends through it."""

import numpy as np
import pytest
import torch

from oracle import inputs
from oracle import pq_oracle as O

pytestmark = pytest.mark.gpu


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def test_one_launch_append_equals_one_shot_compress():
    """Decode-style appends (one new token for every (batch, head) row, odd positions included) and a
    prompt-sized append write exactly the bytes of a one-shot compress of the whole tensor."""
    from polarquant_kv import quantizer
    dev = _cuda()
    B, H, S, D = 3, 2, 41, 128
    K, _, _ = inputs.make_kvq(B, H, 4, S, D, seed=5)
    R = O.rotation_matrix(D, 0)
    P = O.jl_matrix(128, D, 1)
    Kd = torch.from_numpy(K).to(dev)
    for bits, jl in ((4, P), (2, None)):
        full = quantizer.compress(Kd, R, bits, 32, jl)
        cache = quantizer.allocate_cache(B, H, 64, D, bits, 128 if jl is not None else 0, dev)
        quantizer.compress(Kd[:, :, :17], R, bits, 32, jl, out=cache, position=0)
        for pos in range(17, S):
            quantizer.compress(Kd[:, :, pos:pos + 1], R, bits, 32, jl, out=cache, position=pos)
        assert cache.seq_len == S
        assert torch.equal(cache.blocks[:, :, :S], full.blocks)
        assert not cache.blocks[:, :, S:].any()                    # nothing written past the end
        if jl is not None:
            assert torch.equal(cache.qjl_signs[:, :, :S], full.qjl_signs)
            assert torch.equal(cache.residual_norms[:, :, :S], full.residual_norms)


def test_cache_manager_interface():
    from polarquant_kv.inference import KVCacheManager, PolarQuantConfig
    dev = _cuda()
    B, H, D = 2, 2, 64
    K, V, q = inputs.make_kvq(B, H, 14, 40, D, seed=3)
    Kd, Vd = torch.from_numpy(K).to(dev), torch.from_numpy(V).to(dev)
    cm = KVCacheManager(PolarQuantConfig(n_bits=4), max_seq_len=48, batch=B, num_heads=H, head_dim=D, device=dev,
                        rotation_seed=42)
    assert cm.seq_len == 0 and cm.memory_bytes == 0 and cm.compression_ratio == 0.0
    cm.append(Kd[:, :, :39], Vd[:, :, :39])
    cm.append(Kd[:, :, 39:40], Vd[:, :, 39:40])
    assert cm.seq_len == 40
    assert cm.memory_bytes == B * H * 40 * 2 * 36
    assert abs(cm.compression_ratio - (D * 2 * 2) / 72) < 1e-9
    with pytest.raises(RuntimeError):
        cm.append(Kd[:, :, :9], Vd[:, :, :9])
    out = cm.attend(torch.from_numpy(q).to(dev))[:, :, 0]
    ck, cv = cm.get_kv()
    R = O.rotation_matrix(D, 42)
    cb, _ = O.lloyd_max_codebook(32, 4)
    for b in range(B):
        ref = O.attention_from_blocks(q[b], ck.blocks[b, :, :40].cpu().numpy(), cv.blocks[b, :, :40].cpu().numpy(), R, cb, cb)[:, 0]
        assert np.abs(out[b].cpu().numpy() - ref).max() <= 2e-3
    cm.reset()
    assert cm.seq_len == 0 and cm.get_kv()[0].seq_len == 0


class _OracleCache:
    """Stands in for KVCacheManager in the comparison run: every appended key / value goes through the
    numpy oracle's compress -> decompress, attention is float64 torch over the dequantised tensors."""

    def __init__(self, kv_heads, head_dim, seed):
        self.R = O.rotation_matrix(head_dim, seed)
        self.cb, _ = O.lloyd_max_codebook(32, 4)
        self.k = self.v = None
        self.num_heads = kv_heads

    @property
    def seq_len(self):
        return 0 if self.k is None else self.k.shape[2]

    def append(self, key, value):
        def qdq(x):
            xn = x.cpu().numpy()
            hat = O.decompress(O.compress(xn, self.R, self.cb, 4), self.R, self.cb, 4)
            return torch.from_numpy(hat).to(x.device).double()
        k, v = qdq(key), qdq(value)
        self.k = k if self.k is None else torch.cat([self.k, k], dim=2)
        self.v = v if self.v is None else torch.cat([self.v, v], dim=2)

    def attend(self, query, causal=True):
        B, Hq, Sq, D = query.shape
        rep = Hq // self.num_heads
        k, v = self.k.repeat_interleave(rep, dim=1), self.v.repeat_interleave(rep, dim=1)
        s = query.double() @ k.transpose(-2, -1) / np.sqrt(D)
        S = k.shape[2]
        if causal and Sq > 1:
            keep = torch.arange(S, device=query.device)[None, :] <= (S - Sq + torch.arange(Sq, device=query.device))[:, None]
            s = s.masked_fill(~keep, float("-inf"))
        return (torch.softmax(s, dim=-1) @ v).float()


def test_decoder_over_compressed_cache_matches_oracle_cache():
    """A small decoder (float32 weights, two layers) generates the same greedy tokens, and logits equal
    to 1e-3, whether its attention runs through the compressed cache kernels or through the oracle's
    quantise-dequantise + float64 attention."""
    from polarquant_kv.inference import DecoderConfig, DecoderLM, PolarQuantConfig
    dev = _cuda()
    cfg = DecoderConfig(num_layers=2, hidden=128, q_heads=4, kv_heads=2, head_dim=64, intermediate=256, vocab=503)
    model = DecoderLM(cfg, PolarQuantConfig(n_bits=4)).init_random(seed=0, dtype=torch.float32, device=dev)
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (2, 37), generator=gen).to(dev)
    caches = model.create_cache_managers(64, 2, dev)
    ref_caches = [_OracleCache(cfg.kv_heads, cfg.head_dim, 42 + i) for i in range(cfg.num_layers)]
    logits = model(prompt, caches)
    ref_logits = model(prompt, ref_caches)
    worst = float((logits - ref_logits).abs().max())
    toks = []
    for _ in range(6):
        tok, ref_tok = logits.argmax(-1, keepdim=True), ref_logits.argmax(-1, keepdim=True)
        assert torch.equal(tok, ref_tok)
        toks.append(tok)
        logits, ref_logits = model(tok, caches), model(tok, ref_caches)
        worst = max(worst, float((logits - ref_logits).abs().max()))
    print(f"decoder over compressed cache vs oracle cache: max logit difference {worst:.2e}")
    assert worst <= 1e-3
    assert caches[0].seq_len == 37 + 6


def test_hf_cache_adapter_serves_a_transformers_decoder():
    """A small random `transformers` Qwen2 decoder generates through the block_pq4-backed cache: the
    cache grows in place, its logits stay close to the float cache's (the codec is lossy: cosine), and
    greedy generation runs end to end."""
    transformers = pytest.importorskip("transformers")
    from polarquant_kv import hf_integration
    dev = _cuda()
    cfg = transformers.Qwen2Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512)
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(cfg).to(dev).eval()
    hf_integration.patch_model(model, n_bits=4)
    ids = torch.randint(0, 512, (2, 300), generator=torch.Generator().manual_seed(1)).to(dev)
    with torch.no_grad():
        ref = model(ids).logits[:, -1]
        cache = hf_integration.create_compressed_cache(model)
        got = model(ids, past_key_values=cache, use_cache=True).logits[:, -1]
        assert cache.get_seq_length() == 300 and cache.layers[0].capacity == 512       # grew 256 -> 512
        cos = torch.nn.functional.cosine_similarity(ref.float(), got.float(), dim=-1).min().item()
        step = model(ids[:, -1:], past_key_values=cache, use_cache=True).logits
        assert cache.get_seq_length() == 301 and tuple(step.shape) == (2, 1, 512)
        out = model.generate(ids[:, :40], max_new_tokens=8, do_sample=False,
                             past_key_values=hf_integration.create_compressed_cache(model))
    print(f"HF adapter: min cosine of last-token logits vs the float cache {cos:.4f}")
    assert cos > 0.98
    assert tuple(out.shape) == (2, 48)
    assert cache.get_compressed_memory_bytes() * 3 < cache.get_standard_memory_bytes()


def _oracle_mixed(q, K, V, R, runs, axis):
    """float64 attention over keys / values quantised-dequantised run by run with the oracle."""
    Hkv, S, D = K.shape
    Kh, Vh = np.zeros((Hkv, S, D)), np.zeros((Hkv, S, D))
    for b, e, bits in runs:
        cb, _ = O.lloyd_max_codebook(32, bits)
        sl = (slice(None), slice(b, e)) if axis == "token" else (slice(b, e),)
        Kh[sl] = O.decompress(O.compress(K[sl], R, cb, bits), R, cb, bits)
        Vh[sl] = O.decompress(O.compress(V[sl], R, cb, bits), R, cb, bits)
    G = q.shape[0] // Hkv
    out = np.zeros((q.shape[0], D))
    for h in range(q.shape[0]):
        s = Kh[h // G] @ q[h].astype(np.float64) / np.sqrt(D)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ Vh[h // G]
    return out


def test_mixed_precision_policies_vs_oracle():
    """Sink + window token policy (three runs merged by log-sum-exp) and a per-head policy, against the
    oracle's run-by-run quantise-dequantise + float64 attention (2e-3)."""
    from polarquant_kv import policy
    dev = _cuda()
    B, Hkv, Hq, S, D = 2, 4, 16, 333, 128
    K, V, q = inputs.make_kvq(B, Hkv, Hq, S, D, seed=8)
    R = O.rotation_matrix(D, 0)
    Kd, Vd, qd = torch.from_numpy(K).to(dev), torch.from_numpy(V).to(dev), torch.from_numpy(q[:, :, 0]).to(dev)
    tok_bits = policy.compute_token_bitwidths(S, sink_size=4, window_size=64)
    assert policy.runs_of(tok_bits) == [(0, 4, 4), (4, S - 64, 2), (S - 64, S, 4)]
    cache = policy.mixed_precision_compress(Kd, Vd, R, tok_bits, axis="token")
    out = policy.mixed_precision_attention(qd, cache, R).cpu().numpy()
    for b in range(B):
        ref = _oracle_mixed(q[b, :, 0], K[b], V[b], R, cache.runs, "token")
        assert np.abs(out[b] - ref).max() <= 2e-3
    assert 2.0 < cache.average_bits < 2.5 and cache.memory_bytes() < B * Hkv * S * 2 * 72
    head_bits = [4, 4, 2, 2]
    cache_h = policy.mixed_precision_compress(Kd, Vd, R, head_bits, axis="head")
    out_h = policy.mixed_precision_attention(qd, cache_h, R).cpu().numpy()
    for b in range(B):
        ref = _oracle_mixed(q[b, :, 0], K[b], V[b], R, cache_h.runs, "head")
        assert np.abs(out_h[b] - ref).max() <= 2e-3
    assert policy.compute_layer_bitwidths(24, 3.0) == [4] * 6 + [2] * 12 + [4] * 6
    assert policy.compute_layer_bitwidths(2) == [4, 4]


def test_device_side_position_and_length():
    """pq_compress_rows_dynamic / pq_decode_attn_dynamic: the offset of the append and the length of
    the attention come from device memory; results equal the host-argument entry points."""
    from polarquant_kv import _ext, quantizer, rotation
    from polarquant_kv.attention import PreparedDecode, decode_attention
    dev = _cuda()
    B, H, Hq, D, cap = 3, 2, 8, 128, 200
    R = rotation.generate_rotation_matrix(D, seed=5)
    plan = rotation.device_plan(R, dev)
    gen = torch.Generator().manual_seed(3)
    K = torch.randn(B, H, 150, D, generator=gen).to(dev, torch.float16)
    V = torch.randn(B, H, 150, D, generator=gen).to(dev, torch.float16)
    q = torch.randn(B, Hq, D, generator=gen).to(dev, torch.float16)
    pos = torch.zeros(1, dtype=torch.int64, device=dev)
    length = torch.zeros(1, dtype=torch.int64, device=dev)

    ref_k = quantizer.allocate_cache(B, H, cap, D, 4, 0, dev)
    ref_v = quantizer.allocate_cache(B, H, cap, D, 4, 0, dev)
    dyn_k = quantizer.allocate_cache(B, H, cap, D, 4, 0, dev)
    dyn_v = quantizer.allocate_cache(B, H, cap, D, 4, 0, dev)
    prepared = PreparedDecode(q, dyn_k, dyn_v, plan, seq_len_tensor=length)
    done = 0
    for chunk in (1, 33, 1, 100, 15):                      # appends of one token and of many
        ks, vs = K[:, :, done:done + chunk], V[:, :, done:done + chunk]
        quantizer.compress(ks, plan, 4, out=ref_k, position=done)
        quantizer.compress(vs, plan, 4, out=ref_v, position=done)
        pos.fill_(done)
        quantizer.compress(ks, plan, 4, out=dyn_k, position=pos)
        quantizer.compress(vs, plan, 4, out=dyn_v, position=pos)
        done += chunk
        length.fill_(done)
        assert torch.equal(ref_k.blocks, dyn_k.blocks) and torch.equal(ref_v.blocks, dyn_v.blocks)
        want = decode_attention(q, ref_k, ref_v, plan)
        got = decode_attention(q, dyn_k, dyn_v, plan, seq_len_tensor=length)
        assert float((got - want).abs().max()) <= 2e-5      # another work partition, same arithmetic
        assert float((prepared().clone() - want).abs().max()) <= 2e-5
    # a length beyond the capacity is clamped, zero gives zeros
    length.fill_(10 ** 6)
    dyn_k.seq_len = dyn_v.seq_len = cap
    full = decode_attention(q, dyn_k, dyn_v, plan)
    assert float((decode_attention(q, dyn_k, dyn_v, plan, seq_len_tensor=length) - full).abs().max()) <= 2e-5
    length.fill_(0)
    assert float(decode_attention(q, dyn_k, dyn_v, plan, seq_len_tensor=length).abs().max()) == 0.0
    # an append that would run past the capacity writes nothing and raises the device flag
    _ext.poll_device_errors()
    before = dyn_k.blocks.clone()
    pos.fill_(cap - 3)
    quantizer.compress(K[:, :, :4], plan, 4, out=dyn_k, position=pos)
    flags = ctypes_flags()
    assert flags & 32
    assert torch.equal(before, dyn_k.blocks)
    with pytest.raises(ValueError):
        quantizer.compress(K[:, :, :4], plan, 4, out=dyn_k, position=pos.to(torch.int32))


def ctypes_flags() -> int:
    """pq_poll_device_errors without the raising wrapper."""
    import ctypes
    from polarquant_kv import _ext
    flags = ctypes.c_uint(0)
    assert _ext.lib().pq_poll_device_errors(ctypes.byref(flags)) == 0
    return flags.value


def test_graph_replayed_decode_steps_equal_eager_steps():
    """generate_graph (one CUDA graph launch per token, position and length on the device) produces the
    greedy tokens of generate (one Python call per kernel), with and without the key sketch."""
    from polarquant_kv.inference import DecoderConfig, DecoderLM, PolarQuantConfig
    dev = _cuda()
    cfg = DecoderConfig(num_layers=3, hidden=128, q_heads=4, kv_heads=2, head_dim=64, intermediate=256, vocab=503)
    for pq in (PolarQuantConfig(n_bits=4), PolarQuantConfig(n_bits=4, enable_qjl=True, jl_dim=64)):
        model = DecoderLM(cfg, pq).init_random(seed=0, dtype=torch.float32, device=dev)
        prompt = torch.randint(0, cfg.vocab, (2, 41), generator=torch.Generator().manual_seed(7)).to(dev)
        eager_caches = model.create_cache_managers(96, 2, dev)
        graph_caches = model.create_cache_managers(96, 2, dev)
        eager = model.generate(prompt, 20, eager_caches)
        replayed = model.generate_graph(prompt, 20, graph_caches)
        assert torch.equal(eager, replayed)
        assert graph_caches[0].seq_len == eager_caches[0].seq_len == 61
        for a, b in zip(eager_caches, graph_caches):         # the prompt part is the same launch in both
            assert torch.equal(a.get_kv()[0].blocks[:, :, :41], b.get_kv()[0].blocks[:, :, :41])
            # the appended steps: same tokens in, inputs equal up to the attention's summation order
            same = (a.get_kv()[0].blocks[:, :, 41:61] == b.get_kv()[0].blocks[:, :, 41:61]).float().mean().item()
            assert same > 0.999
        assert ctypes_flags() == 0
        with pytest.raises(RuntimeError):
            model.generate_graph(prompt, 80, model.create_cache_managers(96, 2, dev))


def test_device_plan_cache_recognises_objects_and_edits():
    """rotation.device_plan: the same matrix objects give the cached plan without being hashed again; a
    copy with equal contents gives the same plan through the digest; an in-place edit gives a new one."""
    import numpy as np
    from polarquant_kv import qjl, rotation
    dev = _cuda()
    R = rotation.generate_rotation_matrix(64, seed=3)
    P = qjl.generate_jl_matrix(32, 64, seed=4)
    plan = rotation.device_plan(R, dev, P)
    assert rotation.device_plan(R, dev, P) is plan
    assert rotation.device_plan(R.copy(), dev, P.copy()) is plan
    assert rotation.device_plan(plan, dev) is plan
    assert rotation.device_plan(R, dev) is not plan and rotation.device_plan(R, dev).jl is None
    Rt = torch.from_numpy(R).to(dev)
    plan_t = rotation.device_plan(Rt, dev, P)
    assert plan_t is plan and rotation.device_plan(Rt, dev, P) is plan
    Rt.mul_(-1.0)                                            # version counter moves: not the cached object any more
    assert rotation.device_plan(Rt, dev, P) is not plan
    R2 = R.copy()
    first = rotation.device_plan(R2, dev)
    R2[0, 0], R2[-1, -1] = R2[-1, -1], R2[0, 0]
    assert rotation.device_plan(R2, dev) is not first
    assert np.allclose(first.rot.cpu().numpy(), R.astype(np.float32))


def test_reference_named_layers_and_gpu_package_functions():
    """The reference's GPU package by its own names: compress_gpu / decompress_gpu / compressed_attention_gpu
    give what the polarquant_kv functions give, and SimpleTransformer over compressed cache managers stays
    close to the same model over plain float16 caches (prompt, then two single-token steps)."""
    from polarquant_kv import quantizer, attention
    from polarquant_kv_cuda.attention_kernel import compressed_attention_gpu
    from polarquant_kv_cuda.compress_kernel import compress_gpu
    from polarquant_kv_cuda.compressor import get_memory_bytes
    from polarquant_kv_cuda.decompress_kernel import decompress_gpu
    from polarquant_kv_cuda.inference.config import PolarQuantConfig
    from polarquant_kv_cuda.inference.transformer import SimpleTransformer
    from polarquant_kv_cuda.rotation import generate_rotation_matrix
    dev = _cuda()
    torch.manual_seed(0)
    R = generate_rotation_matrix(64, 0)
    kv = torch.randn(2, 2, 50, 64, device=dev).half()
    q = torch.randn(2, 8, 1, 64, device=dev).half()
    cache = compress_gpu(kv, R, 4, 32)
    assert torch.equal(cache.blocks, quantizer.compress(kv, R, 4, 32).blocks)
    back = decompress_gpu(cache, R)
    assert back.dtype == torch.float16 and back.shape == kv.shape
    cos = torch.nn.functional.cosine_similarity(back.float().flatten(), kv.float().flatten(), dim=0)
    assert float(cos) > 0.99
    assert get_memory_bytes(cache) == 2 * 2 * 50 * 2 * 18
    out = compressed_attention_gpu(q, cache, cache, R)
    assert torch.equal(out, attention.compressed_attention(q, cache, cache, R))

    cfg_c, cfg_p = PolarQuantConfig(n_bits=4), PolarQuantConfig(enable_compression=False)
    model = SimpleTransformer(cfg_c, num_layers=2, embed_dim=256, num_heads=4, num_kv_heads=2, vocab_size=97).to(dev)
    plain = SimpleTransformer(cfg_p, num_layers=2, embed_dim=256, num_heads=4, num_kv_heads=2, vocab_size=97).to(dev)
    plain.load_state_dict(model.state_dict())
    ids = torch.randint(0, 97, (3, 20), device=dev)
    with torch.no_grad():
        cm_c, cm_p = model.create_cache_managers(32, 3, dev), plain.create_cache_managers(32, 3, dev)
        for chunk in (ids[:, :18], ids[:, 18:19], ids[:, 19:20]):
            a, b = model(chunk, cm_c), plain(chunk, cm_p)
            cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
            assert a.shape == (3, chunk.shape[1], 97) and float(cos) > 0.99, float(cos)
        assert cm_c[0].seq_len == 20 and cm_c[1].compression_ratio > 3.0
