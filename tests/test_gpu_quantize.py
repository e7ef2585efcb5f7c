"""GPU parity of lux_cuda_qquantize against the oracle's restatement of compute_group_scales and
the quantize shaders (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:157-232, 236-259, 288-310,
336-362): packed bytes, scales and zero-points BIT-EXACT, for every format, on small, ragged and
full-size matrices and on the edge cases the arithmetic has (constant groups, groups of zeros, one
sign only, values beyond the clamp), and the round trip quantize -> lux_cuda_qdequant /
lux_cuda_qmatmul through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu


def _matrix(N, K, seed, kind="normal"):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, K)).astype(np.float32)
    if kind == "edges":
        g = 128
        x[0, :g] = 0.0                          # a group of zeros (asymmetric: -0/0)
        x[1, :g] = 2.5                          # a constant positive group (range 0, -min/0 = -inf)
        x[2, :g] = -1.25                        # a constant negative group (+inf)
        x[3] = np.abs(x[3])                     # one sign only
        x[4] = -np.abs(x[4])
        if N > 6:
            x[5, 7] = 3.0e38                    # near the f32 limit
            x[6, :32] *= 1e-30                  # tiny values: scale far below f16's range
    return x


def _to_host(layer, N, K, bits, scale_dtype):
    G = K // (128 if bits == 4 else 32)
    w = layer.w.to_host(np.uint8 if bits == 4 else np.int8, (N, K * bits // 8))
    s = layer.scales.to_host(np.float32 if scale_dtype == B.F32 else np.float16, (N, G))
    z = layer.zeros.to_host(np.uint8, (N, (G + 1) // 2)) if layer.zeros is not None else None
    return w, s, z


@pytest.mark.parametrize("kind", ["normal", "edges"])
@pytest.mark.parametrize("bits,symmetric,scale_dtype", [(4, False, B.F32), (4, True, B.F32), (4, False, B.F16),
                                                        (4, True, B.F16), (8, True, B.F32)])
@pytest.mark.parametrize("N,K", [(8, 256), (33, 384), (16, 4096), (5, 128)])
def test_quantize_bit_exact(ctx, N, K, bits, symmetric, scale_dtype, kind):
    x = _matrix(N, K, 7, kind)
    L = ctx.qquantize(x, bits, symmetric, scale_dtype)
    w, s, z = _to_host(L, N, K, bits, scale_dtype)
    rw, rs, rz = orc.quantize(x, bits, 128 if bits == 4 else 32, symmetric, orc.F32 if scale_dtype == B.F32 else orc.F16)
    assert np.array_equal(s.view(np.uint32 if scale_dtype == B.F32 else np.uint16),
                          rs.view(np.uint32 if scale_dtype == B.F32 else np.uint16)), "scales"
    if rz is not None:
        assert np.array_equal(z, rz), "zero-points"
    assert np.array_equal(w.view(np.uint8), rw.view(np.uint8)), "packed values"


def test_quantize_shifted_extension_bit_exact(ctx):
    x = _matrix(16, 1024, 8, "edges")
    L = ctx.qquantize(x, 4, False, B.F16, flags=B.FLAG_QUANT_SHIFTED)
    w, s, z = _to_host(L, 16, 1024, 4, B.F16)
    rw, rs, rz = orc.quantize(x, 4, 128, False, orc.F16, shifted=True)
    assert np.array_equal(s.view(np.uint16), rs.view(np.uint16)) and np.array_equal(z, rz) and np.array_equal(w, rw)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_quantize_16_bit_inputs_are_widened_exactly(ctx, dtype):
    x16 = synth.activations(24, 512, dtype, 9, "q16")
    x32 = orc.to_f32(x16)
    for bits, symmetric in ((4, False), (4, True), (8, True)):
        sd = B.F16 if bits == 4 else B.F32
        a = _to_host(ctx.qquantize(x16, bits, symmetric, sd), 24, 512, bits, sd)
        b = _to_host(ctx.qquantize(x32, bits, symmetric, sd), 24, 512, bits, sd)
        assert all(u is None and v is None or np.array_equal(u.view(np.uint8), v.view(np.uint8)) for u, v in zip(a, b))


def test_quantize_full_size_then_dequantize_and_matmul(ctx, backend):
    """Configuration 2's layer shape quantized on the device from an f32 matrix (symmetric int4,
    f16 scales), checked bit-exactly against the oracle; the device-resident result is then used as
    it is by lux_cuda_qdequant (bit-exact against the oracle's dequantize of the oracle's quantize)
    and by lux_cuda_qmatmul with NO wait in between (the matmul must be ordered behind the
    quantize kernel although its prologue prefetches weights)."""
    N, K = 14336, 4096
    wf = (np.random.default_rng(10).standard_normal((N, K)) * 0.02).astype(np.float32)
    x = synth.activations(1, K, "f16", 10, "qfull.x")
    rw, rs, _ = orc.quantize(wf, 4, 128, True, orc.F16)
    xb, yb = ctx.upload(x), ctx.alloc(N * 2)
    L = ctx.qquantize(wf, 4, True, B.F16, flags=B.FLAG_NO_SYNC)
    ctx.qmatmul(xb, L, yb, 1, B.F16)                      # enqueued straight behind the quantize kernel
    y = yb.to_host(np.float16, (1, N))
    w, s, _ = _to_host(L, N, K, 4, B.F16)
    assert np.array_equal(w, rw) and np.array_equal(s.view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(ctx.qdequant(L, B.F32).view(np.uint32), orc.qdequant(rw, rs, None, 4, 128).view(np.uint32))
    assert orc.rel_l2(y, orc.qmatmul(x, rw, rs, None, bits=4, group=128)) < 5e-3
    # the quantized layer reproduces the f32 product to the quantization error (one step is
    # max|w| / 7 per group; the error averages out over K)
    exact = (x.astype(np.float32) @ wf.T).astype(np.float16)
    assert orc.rel_l2(y, exact) < 0.15


def test_quantize_argument_checks(ctx, backend):
    import ctypes as C
    x = ctx.upload(np.zeros((4, 256), np.float32))
    w, s, z = ctx.alloc(4 * 128), ctx.alloc(4 * 2 * 4), ctx.alloc(4)
    lib = backend.lib

    def call(d, zz=z, ww=w):
        return lib.lux_cuda_qquantize(ctx.handle, C.byref(d), x.handle, ww.handle, s.handle, zz.handle if zz else None)

    assert call(B.make_desc(0, 4, 256, 4, 128, B.F32, B.F32, B.F32)) == B.OK
    assert call(B.make_desc(0, 4, 256, 4, 64, B.F32, B.F32, B.F32)) == B.NOT_SUPPORTED       # group size
    assert call(B.make_desc(0, 4, 256, 8, 32, B.F32, B.F32, B.F32)) == B.NOT_SUPPORTED       # int8 with zero-points
    assert call(B.make_desc(0, 4, 200, 4, 128, B.F32, B.F32, B.F32)) == B.INVALID_ARGUMENT   # K % group
    assert call(B.make_desc(0, 4, 256, 4, 128, B.F32, B.F32, B.F32), ww=ctx.alloc(16)) == B.INVALID_ARGUMENT
    assert lib.lux_cuda_qquantize(ctx.handle, None, x.handle, w.handle, s.handle, None) == B.INVALID_ARGUMENT
