"""The attention-side oracle (oracle/attention_oracle.c) against an independent float64 softmax
attention and against its own invariants.  luxcpp/webgpu holds no test vector for these shaders
(they are never dispatched), so this is what stands behind the restatement."""
import numpy as np
import pytest

from oracle import oracle as orc


def _ref_attention(q, k, v, scale, lens):
    """float64 softmax attention; q [R, D], k/v [T, D], lens[r] = keys row r sees."""
    out = np.zeros(q.shape, np.float64)
    lse = np.zeros(q.shape[0], np.float64)
    for r in range(q.shape[0]):
        n = lens[r]
        s = (k[:n].astype(np.float64) @ q[r].astype(np.float64)) * scale
        m = s.max()
        e = np.exp(s - m)
        out[r] = (e / e.sum()) @ v[:n].astype(np.float64)
        lse[r] = m + np.log(e.sum())
    return out, lse


def _ref_sdpa(q, k, v, scale, causal):
    B, H, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    out = np.zeros(q.shape, np.float64)
    lse = np.zeros((B, H, Sq), np.float64)
    for b in range(B):
        for h in range(H):
            lens = [min(i + 1, Skv) if causal else Skv for i in range(Sq)]
            out[b, h], lse[b, h] = _ref_attention(q[b, h], k[b, h // (H // Hkv)], v[b, h // (H // Hkv)], scale, lens)
    return out, lse


@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,D,causal", [
    (1, 2, 2, 5, 5, 16, False), (2, 4, 2, 7, 300, 64, False), (1, 4, 1, 33, 33, 32, True), (1, 8, 2, 3, 700, 128, True),
    (1, 1, 1, 1, 1, 8, False)])
def test_sdpa_matches_float64(B, H, Hkv, Sq, Skv, D, causal):
    rng = np.random.default_rng(7 + Skv)
    q = rng.standard_normal((B, H, Sq, D), np.float32)
    k = rng.standard_normal((B, Hkv, Skv, D), np.float32)
    v = rng.standard_normal((B, Hkv, Skv, D), np.float32)
    scale = 1.0 / np.sqrt(D)
    out, lse = orc.sdpa(q, k, v, scale, causal, want_lse=True)
    ref, ref_lse = _ref_sdpa(q, k, v, scale, causal)
    assert orc.rel_l2(out, ref) < 2e-6
    np.testing.assert_allclose(lse, ref_lse, rtol=1e-5, atol=1e-5)


def test_sdpa_causal_first_row_is_first_value():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 2, 4, 16), np.float32)
    k = rng.standard_normal((1, 2, 4, 16), np.float32)
    v = rng.standard_normal((1, 2, 4, 16), np.float32)
    out = orc.sdpa(q, k, v, 0.25, causal=True)
    np.testing.assert_array_equal(out[:, :, 0], v[:, :, 0])          # one key: weight exp(0) * (1 / 1)


def test_safe_exp_clamp_saturates_far_keys():
    # a key 200 below the max gets weight exp(-88), not 0, as the shader's clamp does
    q = np.ones((1, 1, 1, 4), np.float32)
    k = np.zeros((1, 1, 2, 4), np.float32)
    k[0, 0, 0] = 50.0
    k[0, 0, 1] = 0.0
    v = np.zeros((1, 1, 2, 4), np.float32)
    v[0, 0, 1] = 1.0
    out = orc.sdpa(q, k, v, 1.0)
    assert np.allclose(out[0, 0, 0], np.exp(np.float32(-88.0)), rtol=1e-5)


def test_kv_cache_append_then_attend():
    rng = np.random.default_rng(11)
    B, H, Hkv, D, max_len, cache_len, Sq = 2, 8, 2, 64, 96, 41, 3
    kc = np.zeros((B, Hkv, max_len, D), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :, :cache_len] = rng.standard_normal((B, Hkv, cache_len, D), np.float32)
    vc[:, :, :cache_len] = rng.standard_normal((B, Hkv, cache_len, D), np.float32)
    kn = rng.standard_normal((B, Hkv, Sq, D), np.float32)
    vn = rng.standard_normal((B, Hkv, Sq, D), np.float32)
    q = rng.standard_normal((B, H, Sq, D), np.float32)
    orc.update_kv_cache(kn, vn, kc, vc, cache_len)
    np.testing.assert_array_equal(kc[:, :, cache_len:cache_len + Sq], kn)
    np.testing.assert_array_equal(vc[:, :, cache_len:cache_len + Sq], vn)
    assert not kc[:, :, cache_len + Sq:].any()
    scale = 0.125
    full = orc.sdpa_kv_cache(q, kc, vc, cache_len, scale)
    # without a mask every row sees cache_len + Sq keys: the same as sdpa over the filled part
    ref = orc.sdpa(q, kc[:, :, :cache_len + Sq], vc[:, :, :cache_len + Sq], scale)
    np.testing.assert_allclose(full, ref, rtol=1e-6, atol=1e-7)
    causal = orc.sdpa_kv_cache(q, kc, vc, cache_len, scale, causal_append=True)
    for i in range(Sq):
        ref_i = orc.sdpa(q[:, :, i:i + 1], kc[:, :, :cache_len + i + 1], vc[:, :, :cache_len + i + 1], scale)
        np.testing.assert_allclose(causal[:, :, i:i + 1], ref_i, rtol=1e-6, atol=1e-7)
    np.testing.assert_array_equal(causal[:, :, Sq - 1], full[:, :, Sq - 1])


def test_kv_cache_overflow_is_dropped():
    kc = np.zeros((1, 1, 4, 8), np.float32)
    vc = np.zeros_like(kc)
    kn = np.ones((1, 1, 3, 8), np.float32)
    orc.update_kv_cache(kn, 2 * kn, kc, vc, 2)
    assert kc[0, 0, 2:].all() and not kc[0, 0, :2].any() and (vc[0, 0, 2:] == 2).all()


def _paged_case(rng, num_seqs, H, Hkv, D, block_size, lens, extra_blocks=3):
    max_blocks = max(1, max((n + block_size - 1) // block_size for n in lens))
    total = num_seqs * max_blocks + extra_blocks
    kc = rng.standard_normal((total, Hkv, block_size, D), np.float32)
    vc = rng.standard_normal((total, Hkv, block_size, D), np.float32)
    perm = rng.permutation(total)[:num_seqs * max_blocks].reshape(num_seqs, max_blocks).astype(np.int32)
    q = rng.standard_normal((num_seqs, H, D), np.float32)
    return q, kc, vc, perm, np.asarray(lens, np.int32)


def _gather(kc, table, n, kv_head):
    bs = kc.shape[2]
    return np.stack([kc[table[t // bs], kv_head, t % bs] for t in range(n)])


@pytest.mark.parametrize("lens,block_size,D,H,Hkv", [([37, 1, 300], 16, 64, 4, 2), ([129], 8, 128, 8, 8), ([600, 17], 32, 32, 2, 1)])
def test_paged_matches_float64_and_v2_matches_v1(lens, block_size, D, H, Hkv):
    rng = np.random.default_rng(len(lens) * 100 + D)
    q, kc, vc, table, cl = _paged_case(rng, len(lens), H, Hkv, D, block_size, lens)
    scale = 1.0 / np.sqrt(D)
    v1 = orc.paged_attention(q, kc, vc, table, cl, scale)
    for s, n in enumerate(lens):
        for h in range(H):
            kvh = h // (H // Hkv)
            ref, _ = _ref_attention(q[s, h][None], _gather(kc, table[s], n, kvh), _gather(vc, table[s], n, kvh), scale, [n])
            assert orc.rel_l2(v1[s, h], ref[0]) < 2e-6
    v2 = orc.paged_attention(q, kc, vc, table, cl, scale, partition_size=64)
    np.testing.assert_allclose(v2, v1, rtol=2e-5, atol=2e-6)


def test_paged_empty_sequence_leaves_output():
    rng = np.random.default_rng(5)
    q, kc, vc, table, _ = _paged_case(rng, 2, 2, 2, 16, 16, [20, 20])
    out = np.full(q.shape, 7.0, np.float32)
    orc.paged_attention(q, kc, vc, table, np.asarray([0, 20], np.int32), 0.25, out=out)
    assert (out[0] == 7.0).all() and not (out[1] == 7.0).any()


def test_rope_cache_and_rotation():
    D, S = 64, 40
    cos, sin = orc.rope_cache(S + 8, D, 10000.0)
    i = np.arange(D // 2)
    freq = 10000.0 ** (-2.0 * i / D)
    ang = np.arange(S + 8)[:, None] * freq[None, :]
    np.testing.assert_allclose(cos, np.cos(ang), atol=2e-5)           # f32 angle: |d angle| <= pos * 2^-24
    np.testing.assert_allclose(sin, np.sin(ang), atol=2e-5)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, S, 3, D), np.float32)
    y = orc.rope(x, cos, sin, position_offset=5)
    c, s = cos[5:5 + S][None, :, None, :], sin[5:5 + S][None, :, None, :]
    np.testing.assert_array_equal(y[..., 0::2], x[..., 0::2] * c - x[..., 1::2] * s)
    np.testing.assert_array_equal(y[..., 1::2], x[..., 0::2] * s + x[..., 1::2] * c)
    # without a cache the same angles are formed on the fly
    np.testing.assert_array_equal(orc.rope(x, theta_base=10000.0, position_offset=5), y)
    # backward undoes forward (rotation by the opposite angle)
    np.testing.assert_allclose(orc.rope(y, cos, sin, position_offset=5, backward=True), x, atol=1e-5)
    # custom positions
    pid = rng.integers(0, S + 8, (2, S)).astype(np.uint32)
    yp = orc.rope(x, cos, sin, position_ids=pid)
    cp, sp = cos[pid][:, :, None, :], sin[pid][:, :, None, :]
    np.testing.assert_array_equal(yp[..., 0::2], x[..., 0::2] * cp - x[..., 1::2] * sp)
    # norm of every pair is kept
    np.testing.assert_allclose(y[..., 0::2] ** 2 + y[..., 1::2] ** 2, x[..., 0::2] ** 2 + x[..., 1::2] ** 2, rtol=1e-5, atol=1e-6)


def test_rope_ntk_scaled_uses_scaled_base():
    D = 32
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1, 9, 2, D), np.float32)
    scaled = np.float32(10000.0) * np.float32(4.0) ** (np.float32(D) / np.float32(D - 2))
    np.testing.assert_allclose(orc.rope(x, theta_base=10000.0, ntk_scale=4.0), orc.rope(x, theta_base=float(scaled)), atol=1e-5)
