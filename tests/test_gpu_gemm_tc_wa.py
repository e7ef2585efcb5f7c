"""GPU parity of lux_qgemm_i4_tc_wa (converted weights as the tensor-memory A operand,
128 weight rows x 256 batch rows per CTA, optional split-K over a CTA pair) against the
CPU oracle, through the same C-ABI call as every other quantized matmul.

Tolerance: relative L2 <= 5e-3 (16-bit outputs), oracle evaluated with weights rounded
once to the activation type as the kernel does.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu
TOL_16 = 5e-3


def _run(ctx, x, layer):
    L = ctx.upload_layer(layer)
    xb = ctx.upload(x)
    M = x.shape[0]
    yb = ctx.alloc(M * layer.N * 2)
    ctx.qmatmul(xb, L, yb, M, B.np_dtype_code(x))
    return yb.to_host(x.dtype, (M, layer.N))


def _oracle(x, layer, rows=None):
    xs = x if rows is None else x[rows]
    return orc.qmatmul(xs, *layer.triple, bits=4, group=128, w_round=orc.dtype_code(x))


class _Tuned:
    def __init__(self, backend, **kv):
        self.b, self.kv = backend, kv

    def __enter__(self):
        for k, v in self.kv.items():
            self.b.tune(k, v)

    def __exit__(self, *exc):
        for k in self.kv:
            self.b.tune(k, 0)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("splitk", [1, 2, 4])
@pytest.mark.parametrize("M,N,K", [(256, 128, 256), (129, 128, 512), (300, 256, 512), (512, 384, 1024), (40, 128, 256),
                                   (33, 256, 512), (64, 128, 1024), (100, 256, 256), (128, 128, 512), (200, 128, 256)])
def test_wa_shapes(ctx, backend, dtype, splitk, M, N, K):
    """Whole and ragged batch tiles, one and several weight tiles, one, two and four K splits (a split K does not divide falls back to
    the built-in choice); the kernel is
    forced (gemm_tc_kernel = 2) so that batches of 128 rows and fewer run it too."""
    x = synth.activations(M, K, dtype, 41, f"wa.{M}.{K}")
    layer = synth.int4_layer(N, K, 41, f"wa.{N}.{K}")
    with _Tuned(backend, gemm_tc_kernel=2, gemm_tc_splitk=splitk):
        y = _run(ctx, x, layer)
        assert backend.last_kernel_name().startswith("lux_qgemm_i4_tc_wa")
    err = orc.rel_l2(y, _oracle(x, layer))
    assert err < TOL_16, err
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("groups,stages", [(2, 2), (2, 3), (3, 3), (3, 2)])
def test_wa_groups_and_stages(ctx, backend, groups, stages):
    """Every number of converter groups and ring depth gives the same bits (more groups than
    ring slots are clamped to the ring depth)."""
    x = synth.activations(384, 1024, "bf16", 42, "wag.x")
    layer = synth.int4_layer(256, 1024, 42, "wag")
    with _Tuned(backend, gemm_tc_kernel=2):
        base = _run(ctx, x, layer)
    with _Tuned(backend, gemm_tc_kernel=2, gemm_tc_groups=groups, gemm_tc_stages=stages):
        y = _run(ctx, x, layer)
    assert np.array_equal(y.view(np.uint16), base.view(np.uint16))
    assert orc.rel_l2(y, _oracle(x, layer)) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("splitk", [1, 2, 4])
@pytest.mark.parametrize("narrow", [1, 2])
@pytest.mark.parametrize("M,N,K", [(16, 256, 1024), (33, 128, 512), (64, 384, 512), (40, 128, 2048)])
def test_wa_narrow_and_wide_tiles_for_small_batches(ctx, backend, dtype, splitk, narrow, M, N, K):
    """Batches of up to 64 rows in both tile widths (narrow: 64 accumulator columns, 256 TMEM columns,
    two CTAs per SM; wide: 256 columns, one CTA per SM), every K split, plain and SwiGLU."""
    x = synth.activations(M, K, dtype, 47, f"wan.{M}.{K}")
    layer = synth.int4_layer(N, K, 47, f"wan.{N}.{K}")
    with _Tuned(backend, gemm_tc_kernel=2, gemm_tc_splitk=splitk, gemm_wa_narrow=narrow):
        y = _run(ctx, x, layer)
        assert backend.last_kernel_name().startswith("lux_qgemm_i4_tc_wa")
        h = _run_swiglu(ctx, x, layer)
    assert orc.rel_l2(y, _oracle(x, layer)) < TOL_16
    code = orc.dtype_code(x)
    gu = orc.qmatmul(x, *layer.triple, bits=4, group=128, y_code=orc.F32, w_round=code)
    assert orc.rel_l2(h, orc.swiglu(gu, h_code=code)) < TOL_16
    assert ctx.last_device_status() == 0


def test_wa_symmetric_weights(ctx, backend):
    """No zero-point table: the symmetric special case (zero-point 8)."""
    x = synth.activations(256, 512, "f16", 43, "was.x")
    layer = synth.int4_layer(128, 512, 43, "was", symmetric=True)
    with _Tuned(backend, gemm_tc_kernel=2):
        y = _run(ctx, x, layer)
    assert orc.rel_l2(y, _oracle(x, layer)) < TOL_16


def test_wa_is_default_for_plain_gemms(ctx, backend):
    """Config 3 (512 x 4096 x 4096, bf16) takes this kernel by default and agrees with the
    other tcgen05 kernel to accumulation order."""
    x, layer = synth.config3()
    y = _run(ctx, x, layer)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_bf16"
    rows = np.arange(0, 512, 37)
    assert orc.rel_l2(y[rows], _oracle(x, layer, rows)) < TOL_16
    with _Tuned(backend, gemm_tc_kernel=1):
        y_old = _run(ctx, x, layer)
        assert backend.last_kernel_name() == "lux_qgemm_i4_tc_bf16"
    assert orc.rel_l2(y, y_old) < 1e-3
    assert ctx.last_device_status() == 0


def _run_swiglu(ctx, x, gate_up):
    L = ctx.upload_layer(gate_up)
    xb = ctx.upload(x)
    M, n_out = x.shape[0], gate_up.N // 2
    hb = ctx.alloc(M * n_out * 2)
    ctx.qmatmul(xb, L, hb, M, B.np_dtype_code(x), flags=B.FLAG_SWIGLU)
    return hb.to_host(x.dtype, (M, n_out))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("splitk", [1, 2, 4])
@pytest.mark.parametrize("M,K,I", [(256, 512, 128), (96, 256, 64), (300, 512, 192), (33, 1024, 64)])
def test_wa_swiglu_epilogue(ctx, backend, dtype, splitk, M, K, I):
    """gate_up with the SwiGLU epilogue (steel_gemm_fused.wgsl:91-94, 452-558): gate rows on TMEM
    lanes 0..63, up rows on 64..127, combined in the write-out pass; whole and ragged batch tiles,
    one and several output tiles, both K splits."""
    gate_up, _ = synth.mlp_layers(K, I, 128, 44, f"wasw.{K}.{I}")
    x = synth.activations(M, K, dtype, 44, f"wasw.x.{M}.{K}")
    with _Tuned(backend, gemm_tc_kernel=2, gemm_tc_splitk=splitk):
        h = _run_swiglu(ctx, x, gate_up)
        assert backend.last_kernel_name().startswith("lux_qgemm_i4_tc_wa")
    code = orc.dtype_code(x)
    gu = orc.qmatmul(x, *gate_up.triple, bits=4, group=128, y_code=orc.F32, w_round=code)
    assert orc.rel_l2(h, orc.swiglu(gu, h_code=code)) < TOL_16
    assert ctx.last_device_status() == 0


def test_wa_mlp_m256(ctx, backend):
    """The FFN at 256 batch rows: both of its GEMMs take this kernel by default."""
    gate_up, down = synth.mlp_layers(512, 768, 256, 45, "wamlp")
    x = synth.activations(256, 512, "f16", 45, "wamlp.x")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(256 * 768 * 2), ctx.alloc(256 * 256 * 2)
    ctx.qmlp(xb, G, D, hb, yb, 256, B.F16)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    y = yb.to_host(np.float16, (256, 256))
    assert orc.rel_l2(y, orc.mlp(x, gate_up.triple, down.triple, fused=True, w_round=orc.F16)) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("M,expect", [(4, "lux_qgemv_i4_g128_units_fx"), (5, "lux_qgemm_i4_tc_wa_f16"), (8, "lux_qgemm_i4_tc_wa_f16"),
                                      (12, "lux_qgemm_i4_tc_wa_f16"), (32, "lux_qgemm_i4_tc_wa_f16")])
def test_small_batches_cross_over_at_5(ctx, backend, M, expect):
    """Up to four batch rows the GEMV kernels keep the shape, from five up the tensor-core
    kernel takes it (config 4's `o` layer); both agree with the oracle."""
    x, layer = synth.config4("o", M)
    y = _run(ctx, x, layer)
    assert backend.last_kernel_name() == expect
    rows = np.arange(0, M, max(1, M // 4))
    assert orc.rel_l2(y[rows], orc.qmatmul(x[rows], *layer.triple, bits=4, group=128)) < TOL_16
    assert ctx.last_device_status() == 0


def test_programmatic_dependent_launch_is_transparent(ctx, backend):
    """The same bits with and without the programmatic stream serialization attribute, for a chain
    of dependent launches (each FFN's down projection reads what its gate_up wrote)."""
    gate_up, down = synth.mlp_layers(512, 768, 256, 46, "pdl")
    x = synth.activations(256, 512, "f16", 46, "pdl.x")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(256 * 768 * 2), ctx.alloc(256 * 256 * 2)
    outs = []
    for pdl in (0, 2):
        with _Tuned(backend, pdl=pdl):
            for _ in range(3):
                ctx.qmlp(xb, G, D, hb, yb, 256, B.F16)
        outs.append(yb.to_host(np.float16, (256, 256)).copy())
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))
    assert ctx.last_device_status() == 0

