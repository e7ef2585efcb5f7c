"""GPU parity of the tcgen05/TMEM int4 GEMM with the converted weights as the shared-memory B
operand (lux_qgemm_i4_tc; batch >= 33) against the CPU oracle.

The tensor-core path multiplies 16-bit operands: weights are dequantized to the
activation type with ONE rounding (the same bits lux_cuda_qdequant writes), so the
oracle is evaluated with weights rounded the same way (w_round) and the comparison
isolates accumulation order.  Tolerance: relative L2 <= 5e-3 (16-bit outputs).
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu
TOL_16 = 5e-3


@pytest.fixture(autouse=True)
def _b_operand_kernel(backend):
    """This file covers lux_qgemm_i4_tc (converted weights as the shared-memory B operand), which
    by default only takes the shapes lux_qgemm_i4_tc_wa does not: select it for every test here."""
    backend.tune("gemm_tc_kernel", 1)
    yield
    backend.tune("gemm_tc_kernel", 0)


def _run(ctx, x, layer, flags=0):
    L = ctx.upload_layer(layer)
    xb = ctx.upload(x)
    M = x.shape[0]
    n_out = layer.N // 2 if flags & B.FLAG_SWIGLU else layer.N
    yb = ctx.alloc(M * n_out * 2)
    ctx.qmatmul(xb, L, yb, M, B.np_dtype_code(x), flags=flags)
    return yb.to_host(x.dtype, (M, n_out))


def _oracle(x, layer, rows=None):
    code = orc.dtype_code(x)
    xs = x if rows is None else x[rows]
    return orc.qmatmul(xs, *layer.triple, bits=4, group=128, w_round=code, acc_mode=1 if xs.shape[0] == 1 else 0)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (64, 128, 256), (33, 64, 128), (200, 384, 1024), (130, 72, 512)])
def test_gemm_small_shapes(ctx, backend, dtype, M, N, K):
    x = synth.activations(M, K, dtype, 31, f"g.{M}.{K}")
    layer = synth.int4_layer(N, K, 31, f"g.{N}.{K}")
    y = _run(ctx, x, layer)
    err = orc.rel_l2(y, _oracle(x, layer))
    assert err < TOL_16, err
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("bn,stages", [(64, 2), (64, 4), (128, 3), (128, 6)])
@pytest.mark.parametrize("ma", [1, 2])
def test_gemm_tile_and_stage_choices(ctx, backend, bn, stages, ma):
    """Every weight-tile width, pipeline depth and number of batch tiles per CTA gives the same
    answer; 160 rows: the second batch tile of a CTA is partly (ma = 1) or mostly (ma = 2) empty."""
    x = synth.activations(160, 1024, "bf16", 32, "gt.x")
    layer = synth.int4_layer(256, 1024, 32, "gt")
    ref = _oracle(x, layer)
    backend.tune("gemm_tc_bn", bn)
    backend.tune("gemm_tc_stages", stages)
    backend.tune("gemm_tc_ma", ma)
    try:
        y = _run(ctx, x, layer)
    finally:
        backend.tune("gemm_tc_bn", 0)
        backend.tune("gemm_tc_stages", 0)
        backend.tune("gemm_tc_ma", 0)
    assert orc.rel_l2(y, ref) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("M", [129, 256, 300, 512])
def test_gemm_two_batch_tiles(ctx, backend, M):
    """Batches above 128 rows, ragged last tiles included, with whichever kernel and tile choice
    is the default for them."""
    x = synth.activations(M, 512, "f16", 33, f"g2.x{M}")
    layer = synth.int4_layer(192, 512, 33, "g2")
    ref = _oracle(x, layer)
    y = _run(ctx, x, layer)
    assert orc.rel_l2(y, ref) < TOL_16
    assert ctx.last_device_status() == 0


def test_config3_prefill_gemm(ctx, backend):
    x, layer = synth.config3()
    y = _run(ctx, x, layer)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_bf16"
    ref = _oracle(x, layer)
    err = orc.rel_l2(y, ref)
    assert err < TOL_16, err
    # and against weights kept in f32 (what the streaming path computes): still in tolerance
    ref32 = orc.qmatmul(x[:16], *layer.triple, bits=4, group=128)
    assert orc.rel_l2(y[:16], ref32) < TOL_16


@pytest.mark.parametrize("name", list(synth.SWEEP_LAYERS))
def test_config4_sweep_m64(ctx, name):
    x, layer = synth.config4(name, 64)
    y = _run(ctx, x, layer)
    rows = np.arange(0, 64, 8)                       # 8 of the 64 batch rows (rows are independent)
    assert orc.rel_l2(y[rows], _oracle(x, layer, rows)) < TOL_16


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_gemm_swiglu_epilogue(ctx, dtype):
    gate_up, _ = synth.mlp_layers(512, 384, 128, 33, "gsw")
    x = synth.activations(96, 512, dtype, 33, "gsw.x")
    h = _run(ctx, x, gate_up, flags=B.FLAG_SWIGLU)
    code = orc.dtype_code(x)
    gu = orc.qmatmul(x, *gate_up.triple, bits=4, group=128, y_code=orc.F32, w_round=code)
    assert orc.rel_l2(h, orc.swiglu(gu, h_code=code)) < TOL_16


def test_mlp_m64(ctx):
    gate_up, down = synth.mlp_layers(512, 768, 256, 34, "gmlp")
    x = synth.activations(64, 512, "f16", 34, "gmlp.x")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(64 * 768 * 2), ctx.alloc(64 * 256 * 2)
    ctx.qmlp(xb, G, D, hb, yb, 64, B.F16)
    y = yb.to_host(np.float16, (64, 256))
    assert orc.rel_l2(y, orc.mlp(x, gate_up.triple, down.triple, fused=True, w_round=orc.F16)) < TOL_16


def test_gemm_linearity_full_size(ctx):
    """Size-independent property at the full config-3 size: f(a) + f(b) ~= f(a + b)."""
    _, layer = synth.config3()
    a = synth.activations(512, 4096, "bf16", 35, "lin.a")
    b = synth.activations(512, 4096, "bf16", 35, "lin.b")
    s = orc.f32_to_bf16(orc.bf16_to_f32(a) + orc.bf16_to_f32(b))
    fa, fb, fs = (orc.bf16_to_f32(_run(ctx, v, layer)) for v in (a, b, s))
    assert np.linalg.norm(fs - (fa + fb)) / np.linalg.norm(fs) < 2e-2
