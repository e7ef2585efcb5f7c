"""GPU parity of the activation-quantized integer path (W8A8 / W4A8) against the oracle's
restatement of the shaders (luxcpp/webgpu kernels/wgsl/gpu/quantized.wgsl:497-647,
quantized_nax.wgsl:644-718): exact integer arithmetic, so every comparison is BIT-EXACT -- int32
products, requantized values, packed activations and the dynamic scale.  Shapes cover the
tensor-core kernel (K % 16 == 0, N % 16 == 0), ragged tiles, and the plain kernel's any-shape path;
values cover the extremes (-128 x -128 over the whole K)."""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(23)


def _pack_int4_twos(v):
    """[M, K] ints in [-8, 7] -> flat bytes, element 2j in the low nibble (two's complement)."""
    flat = (np.asarray(v, np.int8).ravel().astype(np.uint8)) & 0xF
    if flat.size % 2:
        flat = np.concatenate([flat, np.zeros(1, np.uint8)])
    return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)


@pytest.mark.parametrize("M,N,K", [(1, 16, 16), (16, 128, 64), (130, 144, 208), (512, 4096, 4096), (33, 48, 4112),
                                   (7, 5, 13), (64, 30, 64), (20, 64, 50),
                                   # the tcgen05 kernel: one tile, ragged M / N, a K tail, N not a multiple of 4
                                   (128, 256, 256), (130, 300, 272), (1000, 1000, 1008), (257, 513, 4096)])
def test_matmul_int8_bit_exact(ctx, backend, M, N, K):
    a = RNG.integers(-128, 128, size=(M, K), dtype=np.int8)
    b = RNG.integers(-128, 128, size=(K, N), dtype=np.int8)
    ab, bb, cb = ctx.upload(a), ctx.upload(b), ctx.alloc(M * N * 4)
    ctx.matmul_int8(ab, bb, cb, M, N, K)
    got = cb.to_host(np.int32, (M, N))
    want = a.astype(np.float64) @ b.astype(np.float64)      # |sum| <= K * 2^14 < 2^53: exact in f64 (and fits int32)
    assert np.array_equal(got, want.astype(np.int32))
    if M * N >= 128 * 256 and K >= 256 and K % 16 == 0:
        assert backend.last_kernel_name() == "lux_matmul_int8_tcgen05"
        # the mma.sync kernel gives the same bits, and so does the tcgen05 kernel fed through a
        # transposed copy of B (what it does by itself when N is not a multiple of 16) instead of
        # reading B as it lies
        for choice, name in ((1, "lux_matmul_int8"), (2, "lux_matmul_int8_tcgen05")):
            backend.tune("int_matmul_kernel", choice)
            try:
                ctx.matmul_int8(ab, bb, cb, M, N, K)
                assert backend.last_kernel_name() == name
            finally:
                backend.tune("int_matmul_kernel", 0)
            assert np.array_equal(cb.to_host(np.int32, (M, N)), got)
    if M * N * K <= 1 << 22:
        assert np.array_equal(got, orc.matmul_int(a, b, M, N, K, 8))


@pytest.mark.parametrize("M,N", [(32, 32), (128, 256)])
def test_matmul_int8_extremes(ctx, M, N):
    K = 4096
    a = np.full((M, K), -128, np.int8)
    b = np.full((K, N), -128, np.int8)
    ab, bb, cb = ctx.upload(a), ctx.upload(b), ctx.alloc(M * N * 4)
    ctx.matmul_int8(ab, bb, cb, M, N, K)
    assert (cb.to_host(np.int32, (M, N)) == K * 16384).all()
    b[:] = 127
    bb.from_host(b)
    ctx.matmul_int8(ab, bb, cb, M, N, K)
    assert (cb.to_host(np.int32, (M, N)) == -K * 128 * 127).all()


@pytest.mark.parametrize("M,N,K", [(16, 16, 16), (128, 256, 128), (100, 80, 96), (4096, 512, 4096), (9, 7, 10), (3, 16, 24), (200, 260, 304)])
def test_matmul_int4_int8_bit_exact(ctx, M, N, K):
    w = RNG.integers(-8, 8, size=(M, K), dtype=np.int8)
    b = RNG.integers(-128, 128, size=(K, N), dtype=np.int8)
    wp = _pack_int4_twos(w)
    wb, bb, cb = ctx.upload(wp), ctx.upload(b), ctx.alloc(M * N * 4)
    ctx.matmul_int8(wb, bb, cb, M, N, K, a_bits=4)
    got = cb.to_host(np.int32, (M, N))
    assert np.array_equal(got, (w.astype(np.float64) @ b.astype(np.float64)).astype(np.int32))
    if M * N * K <= 1 << 22:
        assert np.array_equal(got, orc.matmul_int(wp, b, M, N, K, 4))


@pytest.mark.parametrize("n", [1, 255, 4096, 100003])
def test_requantize_bit_exact(ctx, n):
    x = RNG.integers(-(1 << 24), 1 << 24, size=n, dtype=np.int32)
    x[:min(n, 4)] = [0, 2 ** 31 - 1, -2 ** 31, 12345][:min(n, 4)]
    xb, ob = ctx.upload(x), ctx.alloc(n * 4)
    for in_s, out_s, zp in ((3.1e-4, 0.05, 0), (1.0, 7.0, -3), (2.5e-6, 1e-3, 100)):
        ctx.requantize(xb, ob, n, in_s, out_s, zp)
        assert np.array_equal(ob.to_host(np.int32, (n,)), orc.requantize_int32_to_int8(x, in_s, out_s, zp))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n", [1, 8, 13, 4096, 1 << 20, (1 << 20) + 5])
def test_dynamic_quantize_bit_exact(ctx, n, bits):
    x = (RNG.standard_normal(n) * 2).astype(np.float32)
    xb = ctx.upload(x)
    nbytes = n if bits == 8 else (n + 1) // 2
    ob, sb = ctx.alloc((nbytes + 3) // 4 * 4), ctx.alloc(4)
    ctx.dynamic_quantize(xb, ob, sb, n, bits)
    want, scale = orc.dynamic_quantize(x, bits)
    assert sb.to_host(np.float32, (1,)).view(np.uint32)[0] == np.float32(scale).view(np.uint32)
    assert np.array_equal(ob.to_host(np.uint8, ((nbytes + 3) // 4 * 4,))[:nbytes], want)
    # a tensor of zeros: the scale falls back to 1
    zb = ctx.upload(np.zeros(n, np.float32))
    ctx.dynamic_quantize(zb, ob, sb, n, bits)
    assert sb.to_host(np.float32, (1,))[0] == 1.0


def test_w8a8_linear_layer_end_to_end(ctx):
    """dynamic_quantize -> matmul_int8 -> scale back: the W8A8 linear layer the shaders compose,
    against the f32 product (quantization error only)."""
    M, K, N = 64, 1024, 256
    x = RNG.standard_normal((M, K)).astype(np.float32)
    w = RNG.standard_normal((K, N)).astype(np.float32) * 0.05
    wq, ws = orc.dynamic_quantize(w, 8)
    xb, qb, sb = ctx.upload(x), ctx.alloc(M * K), ctx.alloc(4)
    ctx.dynamic_quantize(xb, qb, sb, M * K, 8)
    xs = float(sb.to_host(np.float32, (1,))[0])
    wb, cb = ctx.upload(wq), ctx.alloc(M * N * 4)
    ctx.matmul_int8(qb, wb, cb, M, N, K)
    y = cb.to_host(np.int32, (M, N)).astype(np.float32) * np.float32(xs * ws)
    assert orc.rel_l2(y, x @ w) < 2e-2


def test_argument_checks(ctx, backend):
    a = ctx.upload(np.zeros(64, np.int8))
    c = ctx.alloc(16)
    lib = backend.lib
    assert lib.lux_cuda_matmul_int8(ctx.handle, a.handle, a.handle, c.handle, 8, 8, 8) == B.INVALID_ARGUMENT      # c too small
    assert lib.lux_cuda_matmul_int8(ctx.handle, a.handle, a.handle, c.handle, 0, 8, 8) == B.INVALID_ARGUMENT
    assert lib.lux_cuda_dynamic_quantize(ctx.handle, a.handle, a.handle, c.handle, 16, 5) == B.INVALID_ARGUMENT
    assert lib.lux_cuda_matmul_int8(None, a.handle, a.handle, c.handle, 1, 1, 1) == B.INVALID_ARGUMENT
