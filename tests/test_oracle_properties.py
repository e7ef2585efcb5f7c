"""Properties of the oracle itself on seeded inputs (no GPU): agreement with a float64
numpy evaluation, linearity, sharding, and the accumulation modes."""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import synth, tp


def _ref64(x, layer):
    q = orc.qunpack(layer.w, layer.zeros, layer.bits, layer.group).astype(np.float64)
    s = np.repeat(orc.to_f32(layer.scales).astype(np.float64), layer.group, axis=1)
    return orc.to_f32(x).astype(np.float64) @ (q * s).T


@pytest.mark.parametrize("M", [1, 3])
def test_int4_matches_float64(M):
    x = synth.activations(M, 512, "f16", 3, "t.x")
    layer = synth.int4_layer(48, 512, 3, "t")
    ref = _ref64(x, layer)
    for mode in (0, 1, 2):
        y = orc.qmatmul(x, *layer.triple, bits=4, group=128, y_code=orc.F32, acc_mode=mode)
        assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 2e-6
    y16 = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert y16.dtype == np.float16
    assert orc.rel_l2(y16, ref.astype(np.float32)) < 1e-3


def test_int8_matches_float64():
    x = synth.activations(1, 256, "f32", 4, "t8.x")
    layer = synth.int8_layer(40, 256, 4, "t8")
    y = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    ref = _ref64(x, layer)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 2e-6


def test_dequant_is_unpack_times_scale():
    layer = synth.int4_layer(16, 256, 5, "dq")
    q = orc.qunpack(layer.w, layer.zeros, 4, 128)
    s = np.repeat(layer.scales.astype(np.float32), 128, axis=1)
    dq = orc.qdequant(layer.w, layer.scales, layer.zeros, 4, 128)
    assert np.array_equal(dq, q.astype(np.float32) * s)          # one f32 multiply, bit-exact
    assert np.array_equal(orc.qdequant(layer.w, layer.scales, layer.zeros, 4, 128, orc.BF16), orc.f32_to_bf16(dq))


def test_symmetric_int4_is_zero_point_8():
    layer = synth.int4_layer(8, 128, 6, "sym", symmetric=True)
    asym = synth.QLayer(4, 128, 8, 128, layer.w, layer.scales, np.full((8, 1), 0x88, np.uint8))
    assert np.array_equal(orc.qunpack(layer.w, None, 4, 128), orc.qunpack(asym.w, asym.zeros, 4, 128))


def test_linearity_in_x():
    layer = synth.int4_layer(32, 256, 7, "lin")
    a = synth.activations(1, 256, "f16", 7, "lin.a").astype(np.float32)
    b = synth.activations(1, 256, "f16", 7, "lin.b").astype(np.float32)
    f = lambda v: orc.qmatmul(v, *layer.triple, bits=4, group=128, y_code=orc.F32, acc_mode=2)
    assert np.allclose(f(a + b), f(a) + f(b), rtol=1e-5, atol=1e-6)


def test_bf16_weight_rounding_mode():
    x = synth.activations(4, 256, "bf16", 8, "bf.x")
    layer = synth.int4_layer(16, 256, 8, "bf")
    y = orc.qmatmul(x, *layer.triple, bits=4, group=128, w_round=orc.BF16)
    assert y.dtype == np.uint16
    wb = orc.bf16_to_f32(orc.qdequant(*layer.triple, 4, 128, orc.BF16)).astype(np.float64)
    ref = orc.bf16_to_f32(x).astype(np.float64) @ wb.T
    assert orc.rel_l2(y, ref.astype(np.float32)) < 5e-3


@pytest.mark.parametrize("world", [1, 2, 4])
def test_tp_sharding_reassembles(world):
    K, I, H, M = 256, 512, 128, 2
    gate_up, down = synth.mlp_layers(K, I, H, 9, "tp")
    x = synth.activations(M, K, "f16", 9, "tp.x")
    full = orc.mlp(x, gate_up.triple, down.triple, fused=True)
    shards = [tuple(l.triple for l in tp.shard_mlp(gate_up, down, r, world)) for r in range(world)]
    sharded = orc.tp_mlp(x, shards, fused=True)
    assert orc.rel_l2(sharded, full) < 5e-3
    # shards cover every weight exactly once
    assert sum(s[0][0].size + s[1][0].size for s in shards) == gate_up.w.size + down.w.size
    # the down shard's dequantized columns equal the matching slice of the full matrix
    dq_full = orc.qdequant(*down.triple, 4, 128)
    r = world - 1
    dq_sh = orc.qdequant(*shards[r][1], 4, 128)
    kl = I // world
    assert np.array_equal(dq_sh, dq_full[:, r * kl:(r + 1) * kl])


def test_mlp_fused_vs_layerwise_within_tolerance():
    gate_up, down = synth.mlp_layers(256, 256, 64, 10, "mlp")
    x = synth.activations(3, 256, "f16", 10, "mlp.x")
    a = orc.mlp(x, gate_up.triple, down.triple, fused=False)
    b = orc.mlp(x, gate_up.triple, down.triple, fused=True)
    assert orc.rel_l2(b, a) < 5e-3


def test_config_shapes():
    x, l = synth.config2()
    assert x.shape == (1, 4096) and l.w.shape == (14336, 2048) and l.scales.shape == (14336, 32)
    assert l.zeros.shape == (14336, 16) and l.weight_bytes == 29360128 + 917504 + 229376
    x1, l1 = synth.config1()
    assert l1.w.dtype == np.int8 and l1.scales.shape == (4096, 128) and l1.w.min() >= -127
    # determinism: same seed, same bytes
    assert np.array_equal(synth.config2()[1].w[:4], l.w[:4])


def test_cpu_baseline_agrees_with_the_oracle():
    """The timed CPU baseline (oracle/cpu_baseline.c: scale and zero-point hoisted per group,
    vectorised, multi-threaded) computes the oracle's arithmetic in another summation order."""
    from oracle import cpu_baseline as cb

    x = synth.activations(3, 1024, "f16", 9, "cb.x")
    for symmetric in (False, True):
        layer = synth.int4_layer(160, 1024, 9, "cb", symmetric=symmetric)
        ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
        for threads in (0, 1):
            assert orc.rel_l2(cb.qmatmul_i4(x, *layer.triple, threads=threads), ref) < 1e-3
    gate_up, down = synth.mlp_layers(512, 768, 256, 9, "cb.mlp")
    xm = synth.activations(2, 512, "f16", 9, "cb.xm")
    assert orc.rel_l2(cb.mlp_i4(xm, gate_up.triple, down.triple),
                      orc.mlp(xm, gate_up.triple, down.triple, fused=True)) < 1e-3
    assert cb.num_procs() >= 1
