"""Seeded sweep over attention shapes the named cases do not hit: random head counts (grouped and
not), head sizes that take the streaming and the plain kernel, ragged key counts, causal and not,
paged caches with page sizes that do and do not divide a chunk, block tables wider than the
context, empty sequences, and the contiguous KV cache with and without the causal bit -- each
against the CPU oracle.  Fixed by its seed; there to catch a slicing or masking rule that fails on
a shape nobody wrote down.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B

pytestmark = pytest.mark.gpu


def _check(ctx, what, got, want):
    err = float(np.max(np.abs(got - want)))
    ref = float(np.max(np.abs(want)))
    assert np.isfinite(got).all(), what
    assert err <= 2e-5 * max(1.0, ref) + 2e-5, f"{what}: max error {err:.3e} against values up to {ref:.3e}"
    assert ctx.last_device_status() == 0, what


def _sdpa_case(ctx, rng, H, Hkv, D, scale):
    Bn = int(rng.integers(1, 4))
    Sq = int(rng.choice([1, 1, 2, 3, 5, 17, 64, 130]))
    causal = bool(rng.integers(0, 2))
    Skv = Sq if (causal and rng.integers(0, 2)) else int(rng.choice([1, 2, 31, 32, 33, 100, 257, 700, 1500, 5000]))
    if causal and Skv < Sq:
        Skv = Sq
    if Bn * H * Sq * Skv * D > 3e8:          # keeps the oracle's share of the test in seconds
        Skv = max(Sq, min(Skv, 300))
    q = rng.standard_normal((Bn, H, Sq, D), np.float32)
    k = rng.standard_normal((Bn, Hkv, Skv, D), np.float32)
    v = rng.standard_normal((Bn, Hkv, Skv, D), np.float32)
    qb, kb, vb, ob = ctx.upload(q), ctx.upload(k), ctx.upload(v), ctx.alloc(q.nbytes)
    ctx.sdpa(qb, kb, vb, ob, Bn, H, Hkv, Sq, Skv, D, scale, flags=B.FLAG_ATTN_CAUSAL if causal else 0)
    _check(ctx, f"sdpa B{Bn} H{H}/{Hkv} Sq{Sq} Skv{Skv} D{D} causal={causal}",
           ob.to_host(np.float32, q.shape), orc.sdpa(q, k, v, scale, causal))


def _paged_case(ctx, rng, H, Hkv, D, scale):
    n = int(rng.integers(1, 6))
    bs = int(rng.choice([1, 4, 5, 8, 16, 16, 32, 64, 128]))
    lens = [int(rng.choice([0, 1, 7, 33, 100, 500, 1000, 3000])) for _ in range(n)]
    if max(lens) == 0:
        lens[0] = 9
    if bs == 1:
        lens = [min(x, 200) for x in lens]
    need = max(1, max((x + bs - 1) // bs for x in lens))
    max_blocks = need if rng.integers(0, 2) else need + int(rng.integers(0, 40))
    total = n * need + 3
    kc = rng.standard_normal((total, Hkv, bs, D), np.float32)
    vc = rng.standard_normal((total, Hkv, bs, D), np.float32)
    table = np.zeros((n, max_blocks), np.int32)
    table[:, :need] = rng.permutation(total)[:n * need].reshape(n, need)
    q = rng.standard_normal((n, H, D), np.float32)
    cl = np.asarray(lens, np.int32)
    init = rng.standard_normal(q.shape, np.float32)
    ob = ctx.upload(init)
    ctx.paged_attention(ctx.upload(q), ctx.upload(kc), ctx.upload(vc), ctx.upload(table), ctx.upload(cl), ob, n, H, Hkv, D, bs,
                        max_blocks, scale)
    want = orc.paged_attention(q, kc, vc, table, cl, scale)
    for i, x in enumerate(lens):
        if x <= 0:
            want[i] = init[i]                # an empty sequence leaves its rows as they were
    _check(ctx, f"paged lens{lens} page{bs} H{H}/{Hkv} D{D} table{max_blocks}", ob.to_host(np.float32, q.shape), want)


def _kv_cache_case(ctx, rng, H, Hkv, D, scale):
    Bn = int(rng.integers(1, 3))
    Sq = int(rng.choice([1, 1, 1, 2, 5, 16]))
    cache_len = int(rng.choice([0, 1, 31, 100, 1000, 4000]))
    max_len = cache_len + Sq + int(rng.integers(0, 50))
    causal = bool(rng.integers(0, 2))
    kc = rng.standard_normal((Bn, Hkv, max_len, D), np.float32)
    vc = rng.standard_normal((Bn, Hkv, max_len, D), np.float32)
    q = rng.standard_normal((Bn, H, Sq, D), np.float32)
    qb, kb, vb, ob = ctx.upload(q), ctx.upload(kc), ctx.upload(vc), ctx.alloc(q.nbytes)
    ctx.sdpa_kv_cache(qb, kb, vb, ob, Bn, H, Hkv, Sq, cache_len, max_len, D, scale, flags=B.FLAG_ATTN_CAUSAL if causal else 0)
    total = cache_len + Sq
    if causal:                               # row i sees the cached keys and appended keys 0 .. i
        want = np.empty_like(q)
        for i in range(Sq):
            seen = cache_len + i + 1
            want[:, :, i:i + 1] = orc.sdpa(np.ascontiguousarray(q[:, :, i:i + 1]), np.ascontiguousarray(kc[:, :, :seen]),
                                           np.ascontiguousarray(vc[:, :, :seen]), scale, False)
    else:
        want = orc.sdpa(q, np.ascontiguousarray(kc[:, :, :total]), np.ascontiguousarray(vc[:, :, :total]), scale, False)
    _check(ctx, f"kv cache B{Bn} H{H}/{Hkv} Sq{Sq} cached{cache_len} of {max_len} D{D} causal={causal}",
           ob.to_host(np.float32, q.shape), want)


@pytest.mark.parametrize("seed", [21, 22])
def test_random_attention_shapes(ctx, seed):
    rng = np.random.default_rng(seed)
    for _ in range(60):
        kind = int(rng.integers(0, 3))
        D = int(rng.choice([4, 8, 16, 20, 32, 48, 64, 80, 96, 128, 128, 160, 256, 6, 30]))
        Hkv = int(rng.choice([1, 2, 3, 4, 8]))
        H = Hkv * int(rng.choice([1, 1, 2, 4, 7]))
        (_sdpa_case, _paged_case, _kv_cache_case)[kind](ctx, rng, H, Hkv, D, 1.0 / np.sqrt(D))
