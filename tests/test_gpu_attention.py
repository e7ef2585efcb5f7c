"""GPU parity of the attention-side entry points (lux/gpu/attention_ext.h) against the oracle's
restatement of luxcpp/webgpu's shaders (kernels/wgsl/gpu/rope.wgsl, scaled_dot_product_attention.wgsl,
steel/attention/paged.wgsl, flash.wgsl).

Tolerance.  The rotation with a cos/sin cache and the cache append are bit-exact.  Attention sums in
a different order than the one-workgroup-per-row shaders (keys split over lanes, warps and thread
blocks), so it is held to relative L2 <= 2e-6 per call and 1e-5 absolute per element on N(0,1) data,
three orders below the 1e-3 limit for f32 outputs."""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B

pytestmark = pytest.mark.gpu
TOL = 2e-6


def _close(got, want):
    assert orc.rel_l2(got, want) < TOL, orc.rel_l2(got, want)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


# ---- rotary embedding -------------------------------------------------------------------------


@pytest.mark.parametrize("D,S,theta", [(64, 100, 10000.0), (128, 33, 500000.0), (2, 5, 10000.0), (80, 7, 10000.0)])
def test_rope_cache_matches_oracle(ctx, D, S, theta):
    cos, sin = orc.rope_cache(S, D, theta)
    cb, sb = ctx.alloc(cos.nbytes), ctx.alloc(sin.nbytes)
    ctx.rope_precompute_cache(cb, sb, S, D, theta)
    # the frequency is the same correctly rounded power on both sides; sinf / cosf differ in the last place
    np.testing.assert_allclose(cb.to_host(np.float32, cos.shape), cos, atol=3e-7, rtol=0)
    np.testing.assert_allclose(sb.to_host(np.float32, sin.shape), sin, atol=3e-7, rtol=0)


@pytest.mark.parametrize("B_,S,H,D,off", [(2, 40, 3, 64, 5), (1, 1, 32, 128, 4095), (3, 17, 5, 6, 0)])
def test_rope_with_cache_bit_exact(ctx, B_, S, H, D, off):
    rng = np.random.default_rng(S * D)
    cos, sin = orc.rope_cache(off + S + 3, D, 10000.0)
    x = rng.standard_normal((B_, S, H, D), np.float32)
    xb, ob, cb, sb = ctx.upload(x), ctx.alloc(x.nbytes), ctx.upload(cos), ctx.upload(sin)
    ctx.rope(xb, ob, B_, S, H, D, cos=cb, sin=sb, position_offset=off)
    want = orc.rope(x, cos, sin, position_offset=off)
    assert np.array_equal(ob.to_host(np.float32, x.shape).view(np.uint32), want.view(np.uint32))
    # backward, and in place (rope_inplace: out == x)
    ctx.rope(ob, ob, B_, S, H, D, cos=cb, sin=sb, position_offset=off, flags=B.FLAG_ROPE_BACKWARD)
    back = orc.rope(want, cos, sin, position_offset=off, backward=True)
    assert np.array_equal(ob.to_host(np.float32, x.shape).view(np.uint32), back.view(np.uint32))
    # custom positions
    pid = rng.integers(0, off + S + 3, (B_, S)).astype(np.uint32)
    ctx.rope(xb, ob, B_, S, H, D, cos=cb, sin=sb, position_ids=ctx.upload(pid))
    assert np.array_equal(ob.to_host(np.float32, x.shape).view(np.uint32), orc.rope(x, cos, sin, position_ids=pid).view(np.uint32))


def test_rope_without_cache_and_ntk(ctx):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 50, 4, 64), np.float32)
    xb, ob = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.rope(xb, ob, 2, 50, 4, 64, theta_base=10000.0, position_offset=7)
    np.testing.assert_allclose(ob.to_host(np.float32, x.shape), orc.rope(x, theta_base=10000.0, position_offset=7), atol=2e-6, rtol=0)
    ctx.rope(xb, ob, 2, 50, 4, 64, theta_base=10000.0, ntk_scale=4.0)
    np.testing.assert_allclose(ob.to_host(np.float32, x.shape), orc.rope(x, theta_base=10000.0, ntk_scale=4.0), atol=2e-6, rtol=0)


def test_rope_qk_fused_in_place(ctx):
    rng = np.random.default_rng(12)
    B_, S, H, Hkv, D, off = 2, 9, 8, 2, 128, 100
    cos, sin = orc.rope_cache(off + S, D, 500000.0)
    q = rng.standard_normal((B_, S, H, D), np.float32)
    k = rng.standard_normal((B_, S, Hkv, D), np.float32)
    qb, kb = ctx.upload(q), ctx.upload(k)
    ctx.rope_qk(qb, kb, ctx.upload(cos), ctx.upload(sin), B_, S, H, Hkv, D, position_offset=off)
    assert np.array_equal(qb.to_host(np.float32, q.shape), orc.rope(q, cos, sin, position_offset=off))
    assert np.array_equal(kb.to_host(np.float32, k.shape), orc.rope(k, cos, sin, position_offset=off))


def test_rope_arguments(ctx):
    x = ctx.alloc(4 * 64)
    lib, h = ctx.backend.lib, ctx.handle
    small = ctx.alloc(16)
    assert lib.lux_cuda_rope_f32(h, x.handle, x.handle, None, None, None, 1, 1, 1, 63, 10000.0, 0, 0.0, 0) == B.INVALID_ARGUMENT
    assert lib.lux_cuda_rope_f32(h, x.handle, x.handle, small.handle, None, None, 1, 1, 1, 64, 10000.0, 0, 0.0, 0) == B.INVALID_ARGUMENT
    # the cache holds 16 / 4 / 32 = 0 positions
    assert lib.lux_cuda_rope_f32(h, x.handle, x.handle, small.handle, small.handle, None, 1, 1, 1, 64, 10000.0, 0, 0.0, 0) == B.INVALID_ARGUMENT
    assert lib.lux_cuda_rope_f32(h, x.handle, x.handle, None, None, None, 1, 2, 1, 64, 10000.0, 0, 0.0, 0) == B.INVALID_ARGUMENT


# ---- scaled-dot-product attention ----------------------------------------------------------------


def _sdpa(ctx, q, k, v, scale, causal=False, lse=False):
    B_, H, Sq, D = q.shape
    qb, kb, vb, ob = ctx.upload(q), ctx.upload(k), ctx.upload(v), ctx.alloc(q.nbytes)
    lb = ctx.alloc(B_ * H * Sq * 4) if lse else None
    ctx.sdpa(qb, kb, vb, ob, B_, H, k.shape[1], Sq, k.shape[2], D, scale, lse=lb, flags=B.FLAG_ATTN_CAUSAL if causal else 0)
    out = ob.to_host(np.float32, q.shape)
    return (out, lb.to_host(np.float32, (B_, H, Sq))) if lse else out


@pytest.mark.parametrize("B_,H,Hkv,Sq,Skv,D,causal", [
    (1, 2, 2, 5, 5, 16, False),            # tiny, one row per KV head
    (2, 4, 2, 7, 300, 64, False),          # two heads per KV head, ragged chunk
    (1, 4, 1, 33, 33, 32, True),           # sdpa_mqa shape, causal, rows over several blocks
    (1, 8, 2, 3, 700, 128, True),
    (1, 32, 8, 1, 4096, 128, False),       # Llama-3-8B decode shape: keys split over CTAs
    (1, 8, 8, 128, 128, 128, True),        # prefill block, one head per KV head
    (2, 8, 2, 64, 200, 80, True),          # head_dim 80: partial last column
    (1, 2, 1, 4, 50, 256, False),          # head_dim 256
    (1, 3, 3, 6, 40, 20, False),           # head_dim 20
    (1, 1, 1, 1, 1, 8, False)])
def test_sdpa_matches_oracle(ctx, B_, H, Hkv, Sq, Skv, D, causal):
    rng = np.random.default_rng(Skv + D)
    q = rng.standard_normal((B_, H, Sq, D), np.float32)
    k = rng.standard_normal((B_, Hkv, Skv, D), np.float32)
    v = rng.standard_normal((B_, Hkv, Skv, D), np.float32)
    scale = 1.0 / np.sqrt(D)
    got, lse = _sdpa(ctx, q, k, v, scale, causal, lse=True)
    want, want_lse = orc.sdpa(q, k, v, scale, causal, want_lse=True)
    _close(got, want)
    np.testing.assert_allclose(lse, want_lse, rtol=1e-5, atol=1e-5)
    assert ctx.backend.last_kernel_name() in ("lux_attn_stream_f32", "lux_attn_merge_f32")


@pytest.mark.parametrize("D", [7, 30, 258])
def test_sdpa_plain_kernel_for_odd_head_dims(ctx, D):
    rng = np.random.default_rng(D)
    q = rng.standard_normal((1, 4, 3, D), np.float32)
    k = rng.standard_normal((1, 2, 300, D), np.float32)
    v = rng.standard_normal((1, 2, 300, D), np.float32)
    got = _sdpa(ctx, q, k, v, 0.3, causal=False)
    _close(got, orc.sdpa(q, k, v, 0.3))
    assert ctx.backend.last_kernel_name() == "lux_attn_plain_f32"


def test_sdpa_unaligned_view_takes_plain_kernel(ctx):
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 2, 2, 64), np.float32)
    k = rng.standard_normal((1, 2, 40, 64), np.float32)
    v = rng.standard_normal((1, 2, 40, 64), np.float32)
    big = ctx.upload(np.concatenate([np.zeros(1, np.float32), k.ravel()]))
    kb = ctx.wrap(big.device_ptr + 4, k.nbytes)
    qb, vb, ob = ctx.upload(q), ctx.upload(v), ctx.alloc(q.nbytes)
    ctx.sdpa(qb, kb, vb, ob, 1, 2, 2, 2, 40, 64, 0.125)
    _close(ob.to_host(np.float32, q.shape), orc.sdpa(q, k, v, 0.125))
    assert ctx.backend.last_kernel_name() == "lux_attn_plain_f32"


def test_sdpa_empty_keys_writes_zeros(ctx):
    q = np.ones((1, 2, 3, 16), np.float32)
    qb, ob = ctx.upload(q), ctx.upload(np.full(q.shape, 5.0, np.float32))
    dummy = ctx.alloc(64)
    ctx.sdpa(qb, dummy, dummy, ob, 1, 2, 2, 3, 0, 16, 1.0)
    assert not ob.to_host(np.float32, q.shape).any()


def test_sdpa_large_scores_do_not_overflow(ctx):
    # scores around +-2000: the running maximum keeps every exponent <= 0
    rng = np.random.default_rng(21)
    q = rng.standard_normal((1, 2, 2, 64), np.float32) * 30
    k = rng.standard_normal((1, 2, 500, 64), np.float32) * 30
    v = rng.standard_normal((1, 2, 500, 64), np.float32)
    got = _sdpa(ctx, q, k, v, 1.0)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, orc.sdpa(q, k, v, 1.0), rtol=1e-3, atol=1e-4)


def test_sdpa_arguments(ctx):
    lib, h = ctx.backend.lib, ctx.handle
    b = ctx.alloc(1024)
    assert lib.lux_cuda_sdpa_f32(h, b.handle, b.handle, b.handle, b.handle, None, 1, 3, 2, 1, 1, 8, 1.0, 0) == B.INVALID_ARGUMENT   # 3 % 2
    assert lib.lux_cuda_sdpa_f32(h, b.handle, b.handle, b.handle, b.handle, None, 1, 2, 2, 1, 1, 0, 1.0, 0) == B.INVALID_ARGUMENT   # head_dim 0
    assert lib.lux_cuda_sdpa_f32(h, b.handle, b.handle, b.handle, b.handle, None, 1, 2, 2, 100, 1, 8, 1.0, 0) == B.INVALID_ARGUMENT  # q too small
    assert lib.lux_cuda_sdpa_f32(h, None, b.handle, b.handle, b.handle, None, 1, 2, 2, 1, 1, 8, 1.0, 0) == B.INVALID_ARGUMENT


# ---- contiguous KV cache ----------------------------------------------------------------------------


@pytest.mark.parametrize("B_,H,Hkv,D,max_len,cache_len,Sq", [
    (2, 8, 2, 64, 96, 41, 3), (1, 32, 8, 128, 4096, 4000, 1), (4, 64, 8, 128, 1024, 1000, 1), (1, 4, 4, 128, 64, 0, 5),
    (1, 16, 2, 128, 300, 100, 16)])
def test_kv_cache_append_and_attend(ctx, B_, H, Hkv, D, max_len, cache_len, Sq):
    rng = np.random.default_rng(cache_len + D)
    kc = np.zeros((B_, Hkv, max_len, D), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :, :cache_len] = rng.standard_normal((B_, Hkv, cache_len, D), np.float32)
    vc[:, :, :cache_len] = rng.standard_normal((B_, Hkv, cache_len, D), np.float32)
    kn = rng.standard_normal((B_, Hkv, Sq, D), np.float32)
    vn = rng.standard_normal((B_, Hkv, Sq, D), np.float32)
    q = rng.standard_normal((B_, H, Sq, D), np.float32)
    kcb, vcb = ctx.upload(kc), ctx.upload(vc)
    ctx.update_kv_cache(ctx.upload(kn), ctx.upload(vn), kcb, vcb, B_, Hkv, Sq, cache_len, max_len, D)
    orc.update_kv_cache(kn, vn, kc, vc, cache_len)
    assert np.array_equal(kcb.to_host(np.float32, kc.shape), kc) and np.array_equal(vcb.to_host(np.float32, vc.shape), vc)
    scale = 1.0 / np.sqrt(D)
    qb, ob = ctx.upload(q), ctx.alloc(q.nbytes)
    for causal in (False, True):
        ctx.sdpa_kv_cache(qb, kcb, vcb, ob, B_, H, Hkv, Sq, cache_len, max_len, D, scale, flags=B.FLAG_ATTN_CAUSAL if causal else 0)
        _close(ob.to_host(np.float32, q.shape), orc.sdpa_kv_cache(q, kc, vc, cache_len, scale, causal_append=causal))


def test_kv_cache_overflow_is_dropped_and_attention_refuses(ctx):
    kc = np.zeros((1, 1, 4, 8), np.float32)
    kn = np.ones((1, 1, 3, 8), np.float32)
    kcb, vcb = ctx.upload(kc), ctx.upload(kc)
    ctx.update_kv_cache(ctx.upload(kn), ctx.upload(2 * kn), kcb, vcb, 1, 1, 3, 2, 4, 8)
    got = kcb.to_host(np.float32, kc.shape)
    assert got[0, 0, 2:].all() and not got[0, 0, :2].any() and (vcb.to_host(np.float32, kc.shape)[0, 0, 2:] == 2).all()
    q = ctx.alloc(3 * 8 * 4)
    rc = ctx.backend.lib.lux_cuda_sdpa_kv_cache_f32(ctx.handle, q.handle, kcb.handle, vcb.handle, q.handle, 1, 1, 1, 3, 2, 4, 8, 1.0, 0)
    assert rc == B.INVALID_ARGUMENT


def test_decode_steps_no_sync_chain(ctx):
    """rope -> append -> attend enqueued without waits, three decode steps in a row."""
    rng = np.random.default_rng(33)
    B_, H, Hkv, D, max_len, cache_len = 2, 8, 2, 64, 64, 10
    cos, sin = orc.rope_cache(max_len, D, 10000.0)
    cb, sb = ctx.upload(cos), ctx.upload(sin)
    kc = np.zeros((B_, Hkv, max_len, D), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :, :cache_len] = rng.standard_normal((B_, Hkv, cache_len, D), np.float32)
    vc[:, :, :cache_len] = rng.standard_normal((B_, Hkv, cache_len, D), np.float32)
    kcb, vcb = ctx.upload(kc), ctx.upload(vc)
    outs, wants = [], []
    for step in range(3):
        q = rng.standard_normal((B_, 1, H, D), np.float32)          # rope layout [batch, seq, heads, dim]
        k = rng.standard_normal((B_, 1, Hkv, D), np.float32)
        v = rng.standard_normal((B_, Hkv, 1, D), np.float32)
        qb, kb, vb, ob = ctx.upload(q), ctx.upload(k), ctx.upload(v), ctx.alloc(q.nbytes)
        pos = cache_len + step
        ctx.rope_qk(qb, kb, cb, sb, B_, 1, H, Hkv, D, position_offset=pos, flags=B.FLAG_NO_SYNC)
        # with one token per sequence [batch, 1, heads, dim] and [batch, heads, 1, dim] are the same bytes
        ctx.update_kv_cache(kb, vb, kcb, vcb, B_, Hkv, 1, pos, max_len, D, flags=B.FLAG_NO_SYNC)
        ctx.sdpa_kv_cache(qb, kcb, vcb, ob, B_, H, Hkv, 1, pos, max_len, D, 0.125, flags=B.FLAG_NO_SYNC)
        outs.append(ob)
        qr = orc.rope(q, cos, sin, position_offset=pos).reshape(B_, H, 1, D)
        kr = orc.rope(k, cos, sin, position_offset=pos).reshape(B_, Hkv, 1, D)
        orc.update_kv_cache(kr, v, kc, vc, pos)
        wants.append(orc.sdpa_kv_cache(qr, kc, vc, pos, 0.125))
    ctx.sync()
    for ob, want in zip(outs, wants):
        _close(ob.to_host(np.float32, want.shape), want)


# ---- paged KV cache -------------------------------------------------------------------------------


def _paged_case(rng, lens, H, Hkv, D, block_size, max_blocks=None, extra_blocks=3):
    n = len(lens)
    need = max(1, max((x + block_size - 1) // block_size for x in lens))
    max_blocks = max_blocks or need
    total = n * need + extra_blocks
    kc = rng.standard_normal((total, Hkv, block_size, D), np.float32)
    vc = rng.standard_normal((total, Hkv, block_size, D), np.float32)
    table = np.zeros((n, max_blocks), np.int32)
    table[:, :need] = rng.permutation(total)[:n * need].reshape(n, need)
    q = rng.standard_normal((n, H, D), np.float32)
    return q, kc, vc, table, np.asarray(lens, np.int32)


def _paged(ctx, q, kc, vc, table, lens, scale, out_init=None):
    S, H, D = q.shape
    ob = ctx.upload(out_init) if out_init is not None else ctx.alloc(q.nbytes)
    ctx.paged_attention(ctx.upload(q), ctx.upload(kc), ctx.upload(vc), ctx.upload(table), ctx.upload(lens), ob, S, H, kc.shape[1], D,
                        kc.shape[2], table.shape[1], scale)
    return ob.to_host(np.float32, q.shape)


@pytest.mark.parametrize("lens,block_size,D,H,Hkv,max_blocks", [
    ([37, 1, 300], 16, 64, 4, 2, None),
    ([129], 8, 128, 8, 8, None),
    ([600, 17], 32, 32, 2, 1, None),
    ([4096], 16, 128, 32, 8, None),          # one long sequence: keys split over CTAs
    ([1000, 3000, 5], 16, 128, 32, 8, 2048),  # table far wider than the contexts: most slices are empty
    ([50, 70], 5, 64, 4, 4, None),           # a block size that does not divide the chunk
    ([33], 1, 64, 2, 2, None),               # one key per page
    ([100], 64, 256, 4, 2, None),
    ([90, 10], 16, 18, 2, 2, None)])         # plain kernel
def test_paged_attention_matches_oracle(ctx, lens, block_size, D, H, Hkv, max_blocks):
    rng = np.random.default_rng(sum(lens) + D)
    q, kc, vc, table, cl = _paged_case(rng, lens, H, Hkv, D, block_size, max_blocks)
    scale = 1.0 / np.sqrt(D)
    _close(_paged(ctx, q, kc, vc, table, cl, scale), orc.paged_attention(q, kc, vc, table, cl, scale))


def test_paged_attention_long_context_many_partitions(ctx):
    """40k keys with 16-key pages: more pages than one CTA's table copy holds, so the keys must be
    sliced whatever the number of sequences (paged_attention_v2's reason to exist)."""
    rng = np.random.default_rng(40)
    q, kc, vc, table, cl = _paged_case(rng, [40000], 2, 1, 64, 16)
    scale = 0.125
    got = _paged(ctx, q, kc, vc, table, cl, scale)
    # the shader order adds 40000 f32 terms one after the other; its own rounding is what limits this comparison
    assert orc.rel_l2(got, orc.paged_attention(q, kc, vc, table, cl, scale)) < 1e-5
    np.testing.assert_allclose(got, orc.paged_attention(q, kc, vc, table, cl, scale, partition_size=512), rtol=1e-4, atol=1e-5)
    # against float64 the tolerance of the short cases holds
    bs = kc.shape[2]
    keys = np.stack([kc[table[0, t // bs], 0, t % bs] for t in range(40000)]).astype(np.float64)
    vals = np.stack([vc[table[0, t // bs], 0, t % bs] for t in range(40000)]).astype(np.float64)
    s = (keys @ q[0].astype(np.float64).T) * scale                   # [keys, heads]
    w = np.exp(s - s.max(axis=0))
    ref = (w / w.sum(axis=0)).T @ vals
    assert orc.rel_l2(got[0], ref) < TOL


def test_paged_attention_empty_sequence_untouched(ctx):
    rng = np.random.default_rng(6)
    q, kc, vc, table, _ = _paged_case(rng, [20, 20, 20], 4, 2, 64, 16)
    cl = np.asarray([20, 0, -3], np.int32)
    init = np.full(q.shape, 7.0, np.float32)
    got = _paged(ctx, q, kc, vc, table, cl, 0.125, out_init=init)
    assert (got[1:] == 7.0).all()
    want = orc.paged_attention(q, kc, vc, table, cl, 0.125, out=init.copy())
    _close(got, want)


def test_paged_attention_bad_block_is_reported_not_followed(ctx):
    rng = np.random.default_rng(2)
    q, kc, vc, table, cl = _paged_case(rng, [40], 2, 2, 64, 16)
    bad = table.copy()
    bad[0, 1] = 1 << 20
    # the entry is read as block 0 (no stray access), the call fails and the status word says why
    with pytest.raises(B.BackendError) as err:
        _paged(ctx, q, kc, vc, bad, cl, 0.125)
    assert err.value.code == B.DEVICE_LOST and ctx.last_device_status() == 0x7C050009
    _close(_paged(ctx, q, kc, vc, table, cl, 0.125), orc.paged_attention(q, kc, vc, table, cl, 0.125))      # the context still works


def test_decode_at_bench_size_properties(ctx):
    """The largest decode shape of the benchmark that a test can afford (8 sequences x 4096 keys, Llama-3-8B
    heads, 268 MB of KV cache): the oracle on every row, and properties that do not depend on the size --
    weights that sum to one, the paged kernel path giving the SAME BITS as the contiguous one when the
    pages hold the same keys in the same order, and independence of the sequences."""
    rng = np.random.default_rng(99)
    B_, H, Hkv, D, L = 8, 32, 8, 128, 4096
    kc = rng.standard_normal((B_, Hkv, L, D), np.float32)
    vc = rng.standard_normal((B_, Hkv, L, D), np.float32)
    q = rng.standard_normal((B_, H, 1, D), np.float32)
    scale = 1.0 / np.sqrt(D)
    kcb, vcb, qb, ob = ctx.upload(kc), ctx.upload(vc), ctx.upload(q), ctx.alloc(q.nbytes)
    ctx.sdpa_kv_cache(qb, kcb, vcb, ob, B_, H, Hkv, 1, L - 1, L, D, scale)
    out = ob.to_host(np.float32, q.shape)
    _close(out, orc.sdpa_kv_cache(q, kc, vc, L - 1, scale))
    # softmax weights sum to one: with V = 1 every output is 1
    ones = ctx.upload(np.ones_like(vc))
    ctx.sdpa_kv_cache(qb, kcb, ones, ob, B_, H, Hkv, 1, L - 1, L, D, scale)
    np.testing.assert_allclose(ob.to_host(np.float32, q.shape), 1.0, rtol=0, atol=2e-6)
    # the same keys as 16-token pages, in order: [seq, head, page, token, d] -> [seq * pages + page, head, token, d]
    bs = 16
    nblk = L // bs
    kp = np.ascontiguousarray(kc.reshape(B_, Hkv, nblk, bs, D).transpose(0, 2, 1, 3, 4)).reshape(B_ * nblk, Hkv, bs, D)
    vp = np.ascontiguousarray(vc.reshape(B_, Hkv, nblk, bs, D).transpose(0, 2, 1, 3, 4)).reshape(B_ * nblk, Hkv, bs, D)
    table = (np.arange(B_ * nblk, dtype=np.int32)).reshape(B_, nblk)
    lens = np.full(B_, L, np.int32)
    pb = ctx.alloc(q.nbytes)
    ctx.paged_attention(qb, ctx.upload(kp), ctx.upload(vp), ctx.upload(table), ctx.upload(lens), pb, B_, H, Hkv, D, bs, nblk, scale)
    paged = pb.to_host(np.float32, (B_, H, D))
    assert np.array_equal(paged.view(np.uint32), out.reshape(B_, H, D).view(np.uint32))
    # a sequence's output does not depend on the others: sequence 3 alone
    one = ctx.alloc(H * D * 4)
    ctx.sdpa_kv_cache(ctx.upload(q[3:4]), ctx.upload(kc[3:4]), ctx.upload(vc[3:4]), one, 1, H, Hkv, 1, L - 1, L, D, scale)
    _close(one.to_host(np.float32, (1, H, 1, D)), out[3:4])
