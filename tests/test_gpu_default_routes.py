"""The kernels the library picks BY DEFAULT on the benchmark configurations' own shapes (no
tunable set): configuration 4's four layers at batch 16 and 64 (lux_qgemm_i4_tc_wa, including
the four-way split-K of `o` and `down` at their real K), configuration 5's full-size gate_up
+ SwiGLU and down at batch 32 and 256, the FFN chain at those batches, and two contracts of the
C boundary that need a device but launch nothing or little.

Oracle comparisons use a subset of the batch rows (rows are independent); tolerance: relative
L2 <= 5e-3 for 16-bit outputs, weights rounded once to f16 as the tensor-core kernels do.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu
TOL_16 = 5e-3


def _rows(M, n=4):
    return np.unique(np.linspace(0, M - 1, n).astype(int))


@pytest.mark.parametrize("M", [5, 8, 11, 16, 64])
@pytest.mark.parametrize("name", list(synth.SWEEP_LAYERS))
def test_config4_default_route(ctx, backend, name, M):
    x, layer = synth.config4(name, M)
    L, xb = ctx.upload_layer(layer), ctx.upload(x)
    yb = ctx.alloc(M * layer.N * 2)
    ctx.qmatmul(xb, L, yb, M, B.F16)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    y = yb.to_host(np.float16, (M, layer.N))
    rows = _rows(M)
    ref = orc.qmatmul(np.ascontiguousarray(x[rows]), *layer.triple, bits=4, group=128, w_round=orc.F16)
    assert orc.rel_l2(y[rows], ref) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.fixture(scope="module")
def ffn70b(ctx):
    d = synth.MLP70B
    gate_up, down = synth.mlp_layers(d["K"], d["I"], d["H"], 0, "cfg5")
    return d, gate_up, down, ctx.upload_layer(gate_up), ctx.upload_layer(down)


@pytest.mark.parametrize("M", [3, 4])
@pytest.mark.parametrize("name", list(synth.SWEEP_LAYERS))
def test_config4_batches_3_and_4_default_route(ctx, backend, name, M):
    """Batches of three and four rows take the block-fixed-point kernel (two 8-column MMA tiles per
    weight fragment, a three-row batch padded to four) wherever the activations at three or four
    byte planes fit beside the weight FIFOs: the K = 4096 layers.  `down` (K = 14336) stays with the
    ring kernel."""
    x, layer = synth.config4(name, M)
    xb, L = ctx.upload(x), ctx.upload_layer(layer)
    yb = ctx.alloc(M * layer.N * 2)
    ctx.qmatmul(xb, L, yb, M, B.F16)
    want = "lux_qgemv_i4_g128_stream" if layer.K > 8192 else "lux_qgemv_i4_g128_units_fx"
    assert backend.last_kernel_name() == want
    y = yb.to_host(np.float16, (M, layer.N))
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert orc.rel_l2(y, ref) < 5e-3
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("M", [32, 256])
def test_config5_full_size_default_route(ctx, backend, ffn70b, M):
    """gate_up 8192 -> 57344 with the SwiGLU epilogue, down 28672 -> 8192, and the two chained
    through lux_cuda_qmlp, all at full size on one GPU."""
    d, gate_up, down, G, D = ffn70b
    x = synth.activations(M, d["K"], "f16", 0, "cfg5.x")
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(M * d["I"] * 2), ctx.alloc(M * d["H"] * 2)
    rows = _rows(M)
    # gate_up + SwiGLU alone
    ctx.qmatmul(xb, G, hb, M, B.F16, flags=B.FLAG_SWIGLU)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    h = hb.to_host(np.float16, (M, d["I"]))
    gu = orc.qmatmul(np.ascontiguousarray(x[rows]), *gate_up.triple, bits=4, group=128, y_code=orc.F32, w_round=orc.F16)
    assert orc.rel_l2(h[rows], orc.swiglu(gu, h_code=orc.F16)) < TOL_16
    # down alone, on the GPU's own h (K = 28672: the longest reduction any configuration has)
    ctx.qmatmul(hb, D, yb, M, B.F16)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    y = yb.to_host(np.float16, (M, d["H"]))
    ref = orc.qmatmul(np.ascontiguousarray(h[rows]), *down.triple, bits=4, group=128, w_round=orc.F16)
    assert orc.rel_l2(y[rows], ref) < TOL_16
    # the chain through the FFN entry point gives the same bits as the two calls
    y2b = ctx.alloc(M * d["H"] * 2)
    ctx.qmlp(xb, G, D, hb, y2b, M, B.F16)
    assert np.array_equal(y2b.to_host(np.float16, (M, d["H"])).view(np.uint16), y.view(np.uint16))
    # and agrees with the oracle's FFN end to end
    ref_ffn = orc.mlp(np.ascontiguousarray(x[rows]), gate_up.triple, down.triple, fused=True, w_round=orc.F16)
    assert orc.rel_l2(y[rows], ref_ffn) < TOL_16
    assert ctx.last_device_status() == 0


def test_misaligned_zero_points_are_refused_before_any_launch(ctx, backend):
    """Several kernels fetch zero-point rows with 16-byte bulk copies; a zero-point buffer that is
    a view at an odd offset must be answered with INVALID_ARGUMENT, not launched."""
    x, layer = synth.activations(1, 512, "f16", 5, "mz.x"), synth.int4_layer(64, 512, 5, "mz")
    L, xb = ctx.upload_layer(layer), ctx.upload(x)
    yb = ctx.alloc(64 * 2)
    padded = ctx.upload(np.concatenate([np.zeros(8, np.uint8), layer.zeros.ravel()]))
    view = ctx.wrap(padded.device_ptr + 8, layer.zeros.nbytes)
    before = backend.launch_count()
    d = B.make_desc(1, 64, 512, 4, 128, B.F16, B.F16, B.F16)
    code = backend.lib.lux_cuda_qmatmul(ctx.handle, C.byref(d), xb.handle, L.w.handle, L.scales.handle, view.handle, yb.handle)
    assert code == B.INVALID_ARGUMENT
    assert backend.launch_count() == before


def test_matmul_behind_an_unsynchronised_unpack_sees_its_output(ctx, backend):
    """lux_cuda_qunpack with NO_SYNC writes an int8 matrix that the next call binds as WEIGHTS.
    The matmul kernels request weights before griddepcontrol.wait, so the library must launch
    that matmul fully ordered: same bits as the synchronous sequence."""
    N, K = 4096, 4096
    x = synth.activations(1, K, "f32", 6, "pw.x")
    layer = synth.int4_layer(N, K, 6, "pw")                     # source of the int8 values
    L = ctx.upload_layer(layer)
    scales = ctx.upload(np.abs(np.random.default_rng(6).standard_normal((N, K // 32))).astype(np.float32) * 1e-3)
    xb, yb = ctx.upload(x), ctx.alloc(N * 4)
    w8 = ctx.alloc(N * K)
    du = B.make_desc(0, N, K, 4, 128, B.F32, B.F16, B.F32)
    dm = B.make_desc(1, N, K, 8, 32, B.F32, B.F32, B.F32)
    lib = backend.lib

    def run(no_sync):
        w8.from_host(np.zeros(N * K, np.int8))                  # stale contents the matmul must not see
        du.flags = B.FLAG_NO_SYNC if no_sync else 0
        assert lib.lux_cuda_qunpack(ctx.handle, C.byref(du), L.w.handle, L.zeros.handle, w8.handle) == B.OK
        assert lib.lux_cuda_qmatmul(ctx.handle, C.byref(dm), xb.handle, w8.handle, scales.handle, None, yb.handle) == B.OK
        return yb.to_host(np.float32, (1, N))

    ref = run(False)
    assert np.abs(ref).max() > 0
    for _ in range(3):
        assert np.array_equal(run(True).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("name", ["qkv", "gate_up"])
def test_bf16_decode_takes_the_fixed_point_gemv(ctx, backend, name, M):
    """bf16 activations at decode batches run on the same fixed-point GEMV as f16 ones (exact
    weights, f32 sums, one rounding to bf16), not on the tensor-core kernels that round the weights."""
    x16, layer = synth.config4(name, M)
    x = synth.f32_to_bf16_bits(x16.astype(np.float32))
    L, xb = ctx.upload_layer(layer), ctx.upload(x)
    yb = ctx.alloc(M * layer.N * 2)
    ctx.qmatmul(xb, L, yb, M, B.BF16)
    assert backend.last_kernel_name() == "lux_qgemv_i4_g128_units_fx"
    y = synth.bf16_bits_to_f32(yb.to_host(np.uint16, (M, layer.N)))
    ref = synth.bf16_bits_to_f32(orc.qmatmul(x, *layer.triple, bits=4, group=128))
    assert orc.rel_l2(y, ref) < 2.5e-3          # the output's own rounding to 8 bits; the weights are exact
    assert ctx.last_device_status() == 0
    # the f16 run on the same activation values (a bf16 value is an f16 value unless it is tiny) gives the
    # same sums; the two differ by their output roundings only
    yh = ctx.alloc(M * layer.N * 2)
    ctx.qmatmul(ctx.upload(synth.bf16_bits_to_f32(x).astype(np.float16)), L, yh, M, B.F16)
    assert orc.rel_l2(y, yh.to_host(np.float16, (M, layer.N)).astype(np.float32)) < 2.5e-3
