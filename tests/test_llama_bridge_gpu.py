"""The llama.cpp bridge's entry points (include/polarquant_llama_abi.h) against the numpy
restatement of the bridge's kernels, through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import llama_bridge_oracle as LO

pytestmark = pytest.mark.gpu

# Indices may differ from the float64 restatement only where the direction sits this close to
# the midpoint of the two candidate centroids (float32 rotation and division on the device).
INDEX_WINDOW = 1e-6
# north_star tolerance for attention outputs.
ATTN_ATOL = 2e-3


def codebook_for(n_levels, rng):
    cb = np.sort(rng.normal(0.0, 0.09, n_levels)).astype(np.float32)
    return cb


def orthogonal(d, rng):
    q, _ = np.linalg.qr(rng.standard_normal((d, d)))
    return q.astype(np.float32)


def explained(direction, cb, got, want):
    """Mismatching indices whose two candidates are equally near within the window."""
    bad = np.argwhere(got != want)
    unexplained = 0
    worst = 0.0
    for n, j in bad:
        gap = abs(abs(direction[n, j] - cb[got[n, j]]) - abs(direction[n, j] - cb[want[n, j]]))
        worst = max(worst, gap)
        if gap > 2 * INDEX_WINDOW:
            unexplained += 1
    return len(bad), unexplained, worst


# n >= 4096 at head dim 64 / 128 takes the warp-per-four-vectors kernel (R transposed in shared memory), everything
# else the CTA-per-vector kernel
@pytest.mark.parametrize("d,n_levels,n", [(128, 16, 1000), (128, 4, 37), (64, 16, 513), (64, 8, 3),
                                          (96, 16, 200), (256, 16, 65), (130, 8, 9), (128, 16, 1),
                                          (128, 16, 20_003), (64, 4, 4096), (64, 16, 70_001), (128, 8, 4097)])
def test_compress_vs_oracle(d, n_levels, n):
    from polarquant_kv import llama_bridge as LB
    rng = np.random.default_rng(d * 131 + n_levels * 7 + n)
    x = (rng.standard_normal((n, d)) * rng.uniform(0.05, 30.0, (n, 1))).astype(np.float32)
    if n > 2:
        x[1] = 0.0                                         # radius 0: every direction is 0
    R, cb = orthogonal(d, rng), codebook_for(n_levels, rng)
    radius, packed = LB.compress(torch.from_numpy(x).cuda(), torch.from_numpy(R).cuda(), torch.from_numpy(cb).cuda())
    radius, packed = radius.cpu().numpy(), packed.cpu().numpy()
    want_radius, want_packed, direction = LO.compress(x, R, cb)
    np.testing.assert_allclose(radius, want_radius, rtol=2e-6, atol=1e-30)
    got_idx, want_idx = LO.unpack(packed, 16), LO.unpack(want_packed, 16)
    n_bad, n_unexplained, worst = explained(direction, cb.astype(np.float64), got_idx, want_idx)
    print(f"compress d={d} levels={n_levels} n={n}: {n_bad} of {got_idx.size} indices differ, "
          f"{n_unexplained} unexplained, widest gap {worst:.2e}")
    assert n_unexplained == 0
    assert n_bad <= max(2, got_idx.size // 2000)
    if n > 2:
        zero_level = int(np.argmin(np.abs(cb)))
        assert (got_idx[1] == zero_level).all() and radius[1] == 0.0


@pytest.mark.parametrize("d,rows", [(128, 32), (64, 7), (96, 3), (256, 40), (1024, 2)])
def test_rotate_and_inverse_vs_oracle(d, rows):
    from polarquant_kv import llama_bridge as LB
    rng = np.random.default_rng(d + rows)
    x = rng.standard_normal((rows, d)).astype(np.float32)
    R = orthogonal(d, rng)
    xr = LB.rotate_query(torch.from_numpy(x).cuda(), torch.from_numpy(R).cuda())
    np.testing.assert_allclose(xr.cpu().numpy(), LO.rotate(x, R), atol=2e-5)
    back = LB.inverse_rotate(xr, torch.from_numpy(R).cuda())
    np.testing.assert_allclose(back.cpu().numpy(), LO.inverse_rotate(xr.cpu().numpy(), R), atol=2e-5)
    np.testing.assert_allclose(back.cpu().numpy(), x, atol=1e-4)


def random_cache(hkv, s, d, n_levels, rng):
    idx = rng.integers(0, n_levels, (hkv, s, d), dtype=np.uint8)
    packed = (idx[..., 0::2] | (idx[..., 1::2] << 4)).astype(np.uint8)
    radius = rng.uniform(0.2, 12.0, (hkv, s)).astype(np.float32)
    return packed, radius


@pytest.mark.parametrize("hq,hkv,s,d,n_levels", [
    (8, 2, 1, 128, 16), (8, 2, 33, 128, 16), (32, 8, 1000, 128, 16), (32, 8, 20000, 128, 16),
    (4, 4, 4097, 64, 16), (16, 2, 777, 64, 4), (6, 2, 300, 96, 8), (12, 2, 2500, 128, 16),
    (8, 1, 5000, 256, 16), (2, 1, 260, 130, 16), (2, 2, 90, 512, 16), (1, 1, 70, 1024, 4),
    (16, 2, 131072, 128, 16)])
def test_fused_attention_vs_oracle(hq, hkv, s, d, n_levels):
    from polarquant_kv import llama_bridge as LB
    rng = np.random.default_rng(hq * 1009 + s * 13 + d + n_levels)
    cb = codebook_for(n_levels, rng)
    pk, kr = random_cache(hkv, s, d, n_levels, rng)
    pv, vr = random_cache(hkv, s, d, n_levels, rng)
    q = (rng.standard_normal((hq, d)) * 1.5).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    dev = lambda a: torch.from_numpy(a).cuda()
    out = LB.fused_attention(dev(q), dev(pk), dev(kr), dev(pv), dev(vr), dev(cb), scale).cpu().numpy()
    want = LO.fused_attention(q, pk, kr, pv, vr, cb, n_levels, scale)
    err = np.abs(out - want).max()
    print(f"attention hq={hq} hkv={hkv} s={s} d={d} levels={n_levels}: max abs err {err:.2e} "
          f"(output scale {np.abs(want).max():.3f})")
    assert err <= ATTN_ATOL
    assert err <= 1e-4 * max(1.0, np.abs(want).max())


def test_peaked_scores_and_large_radii():
    """One token dominates by far; the running maximum moves upward across tiles and slices."""
    from polarquant_kv import llama_bridge as LB
    rng = np.random.default_rng(5)
    hq, hkv, s, d, n_levels = 8, 2, 9000, 128, 16
    cb = codebook_for(n_levels, rng)
    pk, kr = random_cache(hkv, s, d, n_levels, rng)
    pv, vr = random_cache(hkv, s, d, n_levels, rng)
    kr = (kr * np.linspace(0.1, 40.0, s, dtype=np.float32)[None, :]).astype(np.float32)
    q = (rng.standard_normal((hq, d)) * 4.0).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).cuda()
    out = LB.fused_attention(dev(q), dev(pk), dev(kr), dev(pv), dev(vr), dev(cb), 1.0 / np.sqrt(d)).cpu().numpy()
    want = LO.fused_attention(q, pk, kr, pv, vr, cb, n_levels, 1.0 / np.sqrt(d))
    assert np.isfinite(out).all()
    assert np.abs(out - want).max() <= ATTN_ATOL


def test_state_and_whole_sequence_of_calls():
    """polarquant_init_c's state, then compress K and V, rotate q, attend, rotate back — the order
    the bridge calls them in — against float64 arithmetic on the same codes."""
    from polarquant_kv import llama_bridge as LB
    rng = np.random.default_rng(11)
    d, hkv, hq, s = 128, 4, 16, 700
    with LB.State(d, hkv, hq, n_layers=2, n_kv_max=1024, n_bits=4) as st:
        f = st.fields
        assert (f.enabled, f.n_bits, f.n_levels, f.head_dim, f.n_kv_heads, f.n_q_heads, f.n_layers, f.n_kv_max) == \
            (True, 4, 16, d, hkv, hq, 2, 1024)
        cb = st.device_tensor(f.codebook, 16)
        R = st.device_tensor(f.rotation, d * d).view(d, d)
        Rn = R.cpu().numpy().astype(np.float64)
        np.testing.assert_allclose(Rn @ Rn.T, np.eye(d), atol=2e-5)
        cbn = cb.cpu().numpy()
        assert cbn[0] == np.float32(-0.1547) and cbn[15] == np.float32(0.1947) and (np.diff(cbn) > 0).all()

        k = (rng.standard_normal((hkv * s, d)) * 2.0).astype(np.float32)
        v = rng.standard_normal((hkv * s, d)).astype(np.float32)
        q = rng.standard_normal((hq, d)).astype(np.float32)
        k_radius, k_packed = LB.compress(torch.from_numpy(k).cuda(), R, cb)
        v_radius, v_packed = LB.compress(torch.from_numpy(v).cuda(), R, cb)
        q_rot = LB.rotate_query(torch.from_numpy(q).cuda(), R)
        scale = 1.0 / np.sqrt(d)
        out_rot = LB.fused_attention(q_rot, k_packed.view(hkv, s, d // 2), k_radius.view(hkv, s),
                                     v_packed.view(hkv, s, d // 2), v_radius.view(hkv, s), cb, scale)
        out = LB.inverse_rotate(out_rot, R).cpu().numpy()

        want_rot = LO.fused_attention(LO.rotate(q, Rn), k_packed.view(hkv, s, d // 2).cpu().numpy(),
                                      k_radius.view(hkv, s).cpu().numpy(), v_packed.view(hkv, s, d // 2).cpu().numpy(),
                                      v_radius.view(hkv, s).cpu().numpy(), cbn, 16, scale)
        want = LO.inverse_rotate(want_rot, Rn)
        assert np.abs(out - want).max() <= ATTN_ATOL
        # and the codec does its job: close to exact attention over the uncompressed K and V
        kk, vv = k.reshape(hkv, s, d).astype(np.float64), v.reshape(hkv, s, d).astype(np.float64)
        exact = np.empty((hq, d))
        for h in range(hq):
            sc = kk[h // (hq // hkv)] @ q[h].astype(np.float64) * scale
            w = np.exp(sc - sc.max())
            exact[h] = (w / w.sum()) @ vv[h // (hq // hkv)]
        cos = (out * exact).sum() / (np.linalg.norm(out) * np.linalg.norm(exact))
        assert cos > 0.9
    for bits, levels in ((3, 8), (2, 4), (7, 16)):
        with LB.State(64, 2, 4, 1, 16, bits) as st:
            assert st.fields.n_levels == levels


def test_arguments_the_bridge_cannot_serve_are_reported():
    from polarquant_kv import llama_bridge as LB
    x = torch.zeros(4, 127, device="cuda")
    with pytest.raises(ValueError, match="even"):
        LB.compress(x, torch.zeros(127, 127, device="cuda"), torch.zeros(16, device="cuda"))
    q = torch.zeros(6, 64, device="cuda")
    pk = torch.zeros(4, 10, 32, dtype=torch.uint8, device="cuda")
    r = torch.ones(4, 10, device="cuda")
    with pytest.raises(ValueError, match="multiple"):
        LB.fused_attention(q, pk, r, pk, r, torch.zeros(16, device="cuda"), 1.0)
    with pytest.raises(ValueError, match="n_levels"):
        LB.fused_attention(torch.zeros(4, 64, device="cuda"), pk, r, pk, r, torch.zeros(17, device="cuda"), 1.0)
