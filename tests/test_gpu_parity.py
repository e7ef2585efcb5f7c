"""GPU parity: every CUDA kernel, called through the C ABI, against the CPU oracle on the
same seeded inputs.

Bars (from the benchmark specification): integer unpack and dequantized weights
BIT-EXACT; matmul outputs within relative L2 error 1e-3 for f32 outputs and 5e-3 for
f16/bf16 outputs.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_16 = 5e-3

# The int4 decode path has two kernels computing the same thing: 1 = register-staged
# lux_qskinny_i4_g128 (any shape), 2 = bulk-copy ring lux_qgemv_i4_g128_stream (batch <= 16,
# at least 8 groups per row), 3 = warp-autonomous lux_qgemv_i4_g128_units (batch <= 16, group
# count a multiple of 4).  0 lets the library choose.
I4_KERNELS = [0, 1, 2, 3]


def _units_supported(M, K, n_out=16, swiglu=False, sms=148, f16_variant=False):
    """Mirror of the units kernel's shape rule: batch <= 16, an even group count, output rows a
    multiple of the 16-row tile, and room in 227 KB of shared memory for the staged
    activations, their group sums, the CTA's scale / zero-point tables, the partial-sum slots,
    the unit table and one (fixed-point variant) or two chunks of FIFO per warp."""
    G = K // 128
    if M > 16 or G < 2 or G % 2 or n_out % 16:
        return False
    mt, nacc = (1 if M <= 8 else 2), (2 if swiglu else 1)
    cg = 2 if G % 4 else 4
    tiles = n_out // 16
    per_cta = -(-tiles // min(sms, tiles))
    best, KS = 1e30, 0
    for ks in range(cg, min(G, 32) + 1, cg):
        if G % ks:
            continue
        cost = -(-(per_cta * nacc * (G // ks)) // 16) * (ks + 0.25)
        if cost < best - 1e-9:
            best, KS = cost, ks
    if not KS:
        return False
    cap = per_cta * nacc * (G // KS)
    rows = per_cta * 16 * nacc
    tmax = (min(M, 8) + 1) // 2
    zs = (G + 1) // 2
    meta = rows * G * 2 + ((rows * zs + 15) & ~15) + cap * 16
    if M <= 2 and not f16_variant:      # block-fixed-point variant: at least three byte planes of x
        fixed = G * 3 * M * 128 + G * 64 + meta + cap * 16 * M * 4 + 16 * 8 * 8 + 16 + 1024   # + barriers, slack
    else:
        fixed = M * (2 * K + 64) + G * 8 * mt * 8 + meta + cap * mt * 8 * tmax * 16
    min_stages = 1 if (M <= 2 and not f16_variant) else 2
    return fixed + min_stages * 16 * cg * 1024 <= 227 * 1024


def _kernel_supported(kernel, M, K, n_out, swiglu=False):
    if kernel == 2:
        return _stream_supported(M, K, n_out, swiglu)
    if kernel == 3:
        return _units_supported(M, K, n_out, swiglu)
    return True


def _stream_supported(M, K, n_out=16, swiglu=False, sms=148):
    """Mirror of the ring kernel's shape rule: batch <= 16, an even number (>= 8) of groups
    per row, output rows a multiple of the 16-row tile, and room in 227 KB of shared memory
    for the staged activations, their group sums, eight scale blocks, one batch of partial
    sums and at least three minimal stages."""
    G = K // 128
    if M > 16 or G < 8 or G % 2 or n_out % 16:
        return False
    cw = 16 if G >= 16 else 8
    mt, nacc = (1 if M <= 8 else 2), (2 if swiglu else 1)
    meta = (32 * G + 15) // 16 * 16 + (16 * ((G + 1) // 2) + 15) // 16 * 16
    tiles = n_out // 16
    per_cta = -(-tiles // min(sms, tiles))
    part_tile = cw * nacc * mt * 8 * ((min(M, 8) + 1) // 2) * 16
    part = max(1, min(per_cta, 16384 // part_tile)) * part_tile
    fixed = 1024 + M * (2 * K + 64) + G * 8 * mt * 8 + part + 8 * meta + 1024
    return fixed + 3 * (cw * 1024 + 16) <= 227 * 1024


class _kernel:
    def __init__(self, backend, which):
        self.backend, self.which = backend, which

    def __enter__(self):
        self.backend.tune("gemv_i4_kernel", self.which)

    def __exit__(self, *exc):
        self.backend.tune("gemv_i4_kernel", 0)


def _run(ctx, x, layer, flags=0):
    L = ctx.upload_layer(layer)
    xb = ctx.upload(x)
    M = x.shape[0]
    n_out = layer.N // 2 if flags & B.FLAG_SWIGLU else layer.N
    code = B.np_dtype_code(x)
    yb = ctx.alloc(M * n_out * x.itemsize)
    ctx.qmatmul(xb, L, yb, M, code, flags=flags)
    return yb.to_host(x.dtype, (M, n_out))


# -- unpack / dequant: bit-exact ----------------------------------------------------------

@pytest.mark.parametrize("shape", [(16, 128), (48, 512), (14336, 4096)])
@pytest.mark.parametrize("symmetric", [False, True])
def test_int4_unpack_and_dequant_bit_exact(ctx, shape, symmetric):
    N, K = shape
    if symmetric and N > 1000:
        pytest.skip("full size covered by the asymmetric case")
    layer = synth.int4_layer(N, K, 21, f"dq{N}x{K}", symmetric=symmetric)
    L = ctx.upload_layer(layer)
    assert np.array_equal(ctx.qunpack(L), orc.qunpack(layer.w, layer.zeros, 4, 128))
    assert np.array_equal(ctx.qdequant(L, B.F32).view(np.uint32),
                          orc.qdequant(*layer.triple, 4, 128, orc.F32).view(np.uint32))
    assert np.array_equal(ctx.qdequant(L, B.BF16), orc.qdequant(*layer.triple, 4, 128, orc.BF16))
    assert np.array_equal(ctx.qdequant(L, B.F16).view(np.uint16),
                          orc.qdequant(*layer.triple, 4, 128, orc.F16).view(np.uint16))


@pytest.mark.parametrize("shape", [(16, 64), (4096, 4096)])
def test_int8_unpack_and_dequant_bit_exact(ctx, shape):
    N, K = shape
    layer = synth.int8_layer(N, K, 22, f"dq8{N}")
    L = ctx.upload_layer(layer)
    assert np.array_equal(ctx.qunpack(L), orc.qunpack(layer.w, None, 8, 32))
    assert np.array_equal(ctx.qdequant(L, B.F32).view(np.uint32),
                          orc.qdequant(*layer.triple, 8, 32, orc.F32).view(np.uint32))


# -- config 1: int8 g32 GEMV, f32 ---------------------------------------------------------

class _kernel8:
    """Forces one int8 GEMV kernel: 1 = lux_qgemv_i8_g32_f32 (any shape), 2 = warp-autonomous
    lux_qgemv_i8_g32_units_fx (batch <= 2, K % 256 == 0, N % 16 == 0), 0 = the library's choice."""

    def __init__(self, backend, which):
        self.backend, self.which = backend, which

    def __enter__(self):
        self.backend.tune("gemv_i8_kernel", self.which)

    def __exit__(self, *exc):
        self.backend.tune("gemv_i8_kernel", 0)


@pytest.mark.parametrize("kernel", [0, 1, 2])
def test_config1_int8_gemv(ctx, backend, kernel):
    x, layer = synth.config1()
    with _kernel8(backend, kernel):
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    exact = orc.qmatmul(x, *layer.triple, bits=8, group=32, acc_mode=2)
    err = orc.rel_l2(y, ref)
    assert err < TOL_F32, err
    # the tensor-core order is at least as close to the exact sum as f32-sequential is
    assert orc.rel_l2(y, exact) <= max(2 * orc.rel_l2(ref, exact), 2e-6)
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("N,K,M", [(16, 64, 1), (40, 192, 1), (100, 1024, 3), (16, 16384, 1)])
def test_int8_gemv_shapes(ctx, backend, N, K, M):
    x = synth.activations(M, K, "f32", 23, f"i8.{N}.{K}")
    layer = synth.int8_layer(N, K, 23, f"i8.{N}.{K}")
    with _kernel8(backend, 1):
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    assert orc.rel_l2(y, ref) < TOL_F32


@pytest.mark.parametrize("N,K,M", [(16, 256, 1), (48, 512, 2), (16, 16384, 1), (4800, 256, 1), (4096, 4096, 2),
                                   (1008, 3072, 1)])
def test_int8_units_shapes(ctx, backend, N, K, M):
    """The warp-autonomous int8 kernel: one tile, several tiles per CTA (4800 rows = 300 tiles),
    long rows, batch 2."""
    x = synth.activations(M, K, "f32", 24, f"i8u.{N}.{K}")
    layer = synth.int8_layer(N, K, 24, f"i8u.{N}.{K}")
    with _kernel8(backend, 2):
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    assert orc.rel_l2(y, ref) < TOL_F32
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("ks,stages", [(8, 1), (8, 3), (16, 2), (32, 2), (96, 4)])
@pytest.mark.parametrize("M", [1, 2])
def test_int8_units_geometries(ctx, backend, ks, stages, M):
    """Every K-slice width and FIFO depth of the int8 units kernel gives the same answer
    (96 groups per row; 63 tiles)."""
    x = synth.activations(M, 3072, "f32", 26, "i8g.x")
    layer = synth.int8_layer(1008, 3072, 26, "i8g")
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    backend.tune("gemv_units_ks", ks)
    backend.tune("gemv_units_stages", stages)
    try:
        with _kernel8(backend, 2):
            y = _run(ctx, x, layer)
    finally:
        backend.tune("gemv_units_ks", 0)
        backend.tune("gemv_units_stages", 0)
    assert orc.rel_l2(y, ref) < TOL_F32
    assert ctx.last_device_status() == 0


def test_int8_units_fixed_point_ranges(ctx, backend):
    """Block fixed point per group of 32 activations: groups of zeros, of tiny values (flushed
    below 2^-96), of huge values and of magnitudes 2^20 apart must all agree with the oracle;
    an infinity makes every output non-finite."""
    K, N = 1024, 64
    rng = np.random.default_rng(91)
    x = rng.standard_normal((1, K)).astype(np.float32)
    x[:, 0:32] = 0.0
    x[:, 32:64] *= np.float32(1e-35)                              # below 2^-96: counts as zero
    x[:, 64:96] *= np.float32(1e20)
    x[:, 96:128] *= np.where(np.arange(32) % 5 == 0, np.float32(2.0 ** 20), np.float32(1.0))
    x[:, 128:160] *= np.float32(1e-20)
    layer = synth.int8_layer(N, K, 92, "i8r")
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    with _kernel8(backend, 2):
        y = _run(ctx, x, layer)
    assert orc.rel_l2(y, ref) < TOL_F32
    x2 = x.copy()
    x2[:, 64:96] = 0                                              # without the huge group
    ref2 = orc.qmatmul(x2, *layer.triple, bits=8, group=32)
    with _kernel8(backend, 2):
        y2 = _run(ctx, x2, layer)
    assert orc.rel_l2(y2, ref2) < TOL_F32
    x2[0, 700] = np.inf
    with _kernel8(backend, 2):
        y3 = _run(ctx, x2, layer)
    assert not np.isfinite(y3).any()


# -- config 2: int4 g128 GEMV, f16 ---------------------------------------------------------

@pytest.mark.parametrize("kernel", I4_KERNELS)
def test_config2_int4_gemv(ctx, backend, kernel):
    x, layer = synth.config2()
    with _kernel(backend, kernel):
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    err = orc.rel_l2(y, ref)
    assert err < TOL_16, err
    ref32 = orc.qmatmul(x, *layer.triple, bits=4, group=128, y_code=orc.F32, acc_mode=2)
    assert orc.rel_l2(y, ref32) < 1e-3          # f16 output rounding only


@pytest.mark.parametrize("N,K,M,symmetric", [
    (16, 128, 1, False), (16, 128, 1, True), (24, 384, 2, False), (1000, 1152, 5, False),
    (64, 4096, 8, False), (48, 2048, 9, False), (80, 1024, 16, False), (32, 512, 17, True),
    (64, 8192, 32, False), (40, 14336, 16, False), (16, 28672, 1, False),
])
@pytest.mark.parametrize("kernel", I4_KERNELS)
def test_int4_skinny_shapes(ctx, backend, N, K, M, symmetric, kernel):
    x = synth.activations(M, K, "f16", 24, f"i4.{N}.{K}.{M}")
    layer = synth.int4_layer(N, K, 24, f"i4.{N}.{K}", symmetric=symmetric)
    with _kernel(backend, kernel):
        if not _kernel_supported(kernel, M, K, N):
            with pytest.raises(B.BackendError) as e:
                _run(ctx, x, layer)
            assert e.value.code == B.NOT_SUPPORTED
            return
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert orc.rel_l2(y, ref) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("warps,cg,stages", [(8, 1, 3), (8, 2, 5), (8, 4, 2), (8, 4, 64), (16, 1, 1), (16, 2, 4), (16, 1, 64)])
def test_int4_stream_ring_shapes(ctx, backend, warps, cg, stages):
    """Every ring geometry (consumer warps, groups per stage, ring depth) gives the same answer."""
    x = synth.activations(5, 2560, "f16", 28, "ring.x")
    layer = synth.int4_layer(1008, 2560, 28, "ring")
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    backend.tune("gemv_stream_warps", warps)
    backend.tune("gemv_stream_cg", cg)
    backend.tune("gemv_stream_stages", stages)
    try:
        with _kernel(backend, 2):
            y = _run(ctx, x, layer)
    finally:
        backend.tune("gemv_stream_warps", 0)
        backend.tune("gemv_stream_cg", 0)
        backend.tune("gemv_stream_stages", 0)
    assert orc.rel_l2(y, ref) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("cg,ks,stages,pre", [(4, 4, 2, 1), (4, 8, 3, 3), (4, 12, 1, 1), (4, 24, 8, 2), (2, 2, 6, 1),
                                              (2, 6, 2, 2), (2, 8, 3, 1)])
@pytest.mark.parametrize("M,fx", [(1, 1), (1, 2), (2, 1), (2, 2), (3, 0), (4, 1), (4, 2), (11, 0)])
def test_int4_units_geometries(ctx, backend, cg, ks, stages, pre, M, fx):
    """Every chunk size, K-slice width, FIFO depth and pre-request count of the units kernel
    gives the same answer, in both arithmetic variants (fx 1: block fixed point + int8 mma,
    fx 2: f16 mma).  24 groups per row; 63 tiles, so the FIFO wraps many times."""
    x = synth.activations(M, 3072, "f16", 29, "units.x")
    layer = synth.int4_layer(1008, 3072, 29, "units")
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    tunes = {"gemv_units_cg": cg, "gemv_units_ks": ks, "gemv_units_stages": stages, "gemv_units_pre": pre,
             "gemv_units_fx": fx}
    for k, v in tunes.items():
        backend.tune(k, v)
    try:
        with _kernel(backend, 3):
            y = _run(ctx, x, layer)
    finally:
        for k in tunes:
            backend.tune(k, 0)
    assert orc.rel_l2(y, ref) < TOL_16
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("warps", [8, 16])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_units_fixed_point_both_cta_geometries(ctx, backend, M, warps):
    """The fixed-point kernels in their half-SM (8 warps, two CTAs per SM) and whole-SM (16 warps)
    geometries: plain int4, int4 with the SwiGLU epilogue, and int8, each against the oracle."""
    backend.tune("gemv_units_warps", warps)
    try:
        x = synth.activations(M, 2048, "f16", 31, "geo.x")
        layer = synth.int4_layer(1200, 2048, 31, "geo")
        with _kernel(backend, 3):
            y = _run(ctx, x, layer)
            assert backend.last_kernel_name() == "lux_qgemv_i4_g128_units_fx"
        assert orc.rel_l2(y, orc.qmatmul(x, *layer.triple, bits=4, group=128)) < 1e-3
        gate_up, _ = synth.mlp_layers(2048, 592, 128, 31, "geo.mlp")
        with _kernel(backend, 3):
            h = _run(ctx, x, gate_up, flags=B.FLAG_SWIGLU)
        gu = orc.qmatmul(x, *gate_up.triple, bits=4, group=128, y_code=orc.F32)
        assert orc.rel_l2(h, orc.swiglu(gu, h_code=orc.F16)) < TOL_16
        if M <= 2:                                   # the int8 twin takes one or two batch rows
            x8 = synth.activations(M, 2048, "f32", 31, "geo.x8")
            l8 = synth.int8_layer(1200, 2048, 31, "geo8")
            with _kernel8(backend, 2):
                y8 = _run(ctx, x8, l8)
                assert backend.last_kernel_name() == "lux_qgemv_i8_g32_units_fx"
            assert orc.rel_l2(y8, orc.qmatmul(x8, *l8.triple, bits=8, group=32)) < 1e-5
    finally:
        backend.tune("gemv_units_warps", 0)
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_int4_units_fixed_point_ranges(ctx, backend, M):
    """Block fixed point per group of 128 activations: groups of all zeros, of f16 denormals,
    of large values, and groups mixing magnitudes 2^12 apart must all agree with
    the oracle (elements more than 2^11 below their group's maximum lose low bits, at most
    2^-23 of that maximum each)."""
    K, N = 2048, 256
    rng = np.random.default_rng(77)
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[:, 0:128] = 0.0                                            # an all-zero group
    x[:, 128:256] *= 3e-7                                        # f16 denormals
    x[:, 256:384] = np.sign(x[:, 256:384]) * 30000.0             # large: the products still fit f16
    x[:, 384:512] *= np.where(np.arange(128) % 7 == 0, 4096.0, 1.0)   # mixed magnitudes
    x[:, 512:640] = -x[:, 512:640] * 1e-3
    x = x.astype(np.float16)
    layer = synth.int4_layer(N, K, 78, "fxr")
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert np.isfinite(ref).all()
    with _kernel(backend, 3):
        y = _run(ctx, x, layer)
    assert orc.rel_l2(y, ref) < TOL_16
    # without the huge group, the small groups must be resolved on their own
    x2 = x.copy()
    x2[:, 256:384] = 0
    ref2 = orc.qmatmul(x2, *layer.triple, bits=4, group=128)
    with _kernel(backend, 3):
        y2 = _run(ctx, x2, layer)
    assert orc.rel_l2(y2, ref2) < TOL_16


@pytest.mark.parametrize("warps", [8, 16])
@pytest.mark.parametrize("k_out", [130, 131])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_int4_units_fixed_point_outlier_group(ctx, backend, M, k_out, warps):
    """The "massive activation" case: one activation 2^15 times larger than everything else in its
    group, sitting on a weight whose (q - zp) is 0 in every row, at an even and at an odd k.  The
    outlier sets the group's block exponent and contributes nothing, so the outputs are made of
    the SMALL elements alone: with four byte planes (30 bits below the block exponent for even
    k, 26 for odd k) every f16 within 2^15 of the outlier is still exact, and the result must
    meet the 16-bit tolerance with room to spare, in both CTA geometries."""
    K, N = 1024, 512
    rng = np.random.default_rng(91)
    x = (rng.standard_normal((M, K)) * 0.5).astype(np.float32)
    x[:, k_out] = 0.9 * 32768.0 * np.sign(x[:, k_out])
    x = x.astype(np.float16)
    layer = synth.int4_layer(N, K, 91, "outl")
    zp = synth.unpack_nibbles(layer.zeros, K // 128)[:, k_out // 128]
    byte = layer.w[:, k_out // 2]
    layer.w[:, k_out // 2] = (byte & 0xF0) | zp if k_out % 2 == 0 else (byte & 0x0F) | (zp << 4)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    x0 = x.copy()
    x0[:, k_out] = 0
    assert orc.rel_l2(orc.qmatmul(x0, *layer.triple, bits=4, group=128), ref) < 1e-6     # the outlier is inert
    backend.tune("gemv_units_warps", warps)
    try:
        with _kernel(backend, 3):
            y = _run(ctx, x, layer)
        assert backend.last_kernel_name() == "lux_qgemv_i4_g128_units_fx"
        # rows too long for four planes keep three (22 / 18 bits): the same case then carries the
        # rounding of the small odd-k elements, 2^-19 of the outlier each, and stays within 3e-2
        backend.tune("gemv_units_planes", 3)
        with _kernel(backend, 3):
            y3 = _run(ctx, x, layer)
    finally:
        backend.tune("gemv_units_warps", 0)
        backend.tune("gemv_units_planes", 0)
    assert orc.rel_l2(y, ref) < 1e-3, orc.rel_l2(y, ref)
    assert orc.rel_l2(y3, ref) < 3e-2, orc.rel_l2(y3, ref)


@pytest.mark.parametrize("M", [1, 2])
def test_int8_units_fixed_point_outlier_group(ctx, backend, M):
    """The same for the int8 kernel (groups of 32, f32 activations, 30 bits below the block
    exponent): an activation 2^15 times the rest on weights that are 0."""
    K, N = 1024, 512
    rng = np.random.default_rng(92)
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[:, 77] = 32768.0 * 1.7
    layer = synth.int8_layer(N, K, 92, "outl8")
    layer.w[:, 77] = 0
    ref = orc.qmatmul(x, *layer.triple, bits=8, group=32)
    with _kernel8(backend, 2):
        y = _run(ctx, x, layer)
        assert backend.last_kernel_name() == "lux_qgemv_i8_g32_units_fx"
    assert orc.rel_l2(y, ref) < 1e-5, orc.rel_l2(y, ref)


def test_int4_units_fixed_point_nonfinite(ctx, backend):
    """An infinity or NaN among the activations makes every output non-finite, as it does in
    the oracle (each output multiplies every activation)."""
    x = synth.activations(1, 1024, "f16", 5, "nf.x").copy()
    x[0, 300] = np.float16(np.inf)
    layer = synth.int4_layer(64, 1024, 5, "nf")
    with _kernel(backend, 3):
        y = _run(ctx, x, layer)
    assert not np.isfinite(y.astype(np.float32)).any()


def test_int4_units_many_tiles_per_cta(ctx, backend):
    """More tiles than SMs (CTAs own several tiles, unevenly), symmetric weights (no zero-point
    tensor) and a group count that only allows two-group chunks."""
    x = synth.activations(2, 128 * 6, "f16", 31, "units2.x")
    layer = synth.int4_layer(16 * 500, 128 * 6, 31, "units2", symmetric=True)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    with _kernel(backend, 3):
        y = _run(ctx, x, layer)
    assert orc.rel_l2(y, ref) < TOL_16


@pytest.mark.parametrize("wpc,rt", [(1, 1), (2, 2), (4, 4), (8, 1), (8, 4)])
def test_int4_skinny_launch_shapes(ctx, backend, wpc, rt):
    """Every warps-per-CTA / row-tiles-per-CTA combination gives the same answer."""
    x = synth.activations(3, 1536, "f16", 25, "tune.x")
    layer = synth.int4_layer(208, 1536, 25, "tune")
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    backend.tune("gemv_i4_warps", wpc)
    backend.tune("gemv_i4_row_tiles", rt)
    try:
        with _kernel(backend, 1):
            y = _run(ctx, x, layer)
    finally:
        backend.tune("gemv_i4_warps", 0)
        backend.tune("gemv_i4_row_tiles", 0)
    assert orc.rel_l2(y, ref) < TOL_16


# -- config 4: Llama-3-8B decode sweep ----------------------------------------------------

@pytest.mark.parametrize("name", list(synth.SWEEP_LAYERS))
@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("kernel", [1, 2, 3])
def test_config4_sweep_streaming(ctx, backend, name, M, kernel):
    x, layer = synth.config4(name, M)
    if not _kernel_supported(kernel, M, layer.K, layer.N):
        pytest.skip("activations too large for this kernel's shared memory")
    with _kernel(backend, kernel):
        y = _run(ctx, x, layer)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert orc.rel_l2(y, ref) < TOL_16


# -- SwiGLU epilogue and the FFN ------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 8, 12, 20])
@pytest.mark.parametrize("kernel", [1, 2, 3])
def test_swiglu_epilogue_streaming(ctx, backend, M, kernel):
    gate_up, _ = synth.mlp_layers(1024, 384, 128, 26, "sw")
    x = synth.activations(M, 1024, "f16", 26, "sw.x")
    if not _kernel_supported(kernel, M, 1024, 384, swiglu=True):
        pytest.skip("this kernel covers batch <= 16")
    with _kernel(backend, kernel):
        h = _run(ctx, x, gate_up, flags=B.FLAG_SWIGLU)
    gu = orc.qmatmul(x, *gate_up.triple, bits=4, group=128, y_code=orc.F32)
    ref = orc.swiglu(gu, h_code=orc.F16)
    assert orc.rel_l2(h, ref) < TOL_16


@pytest.mark.parametrize("M", [1, 4])
def test_mlp_small(ctx, M):
    gate_up, down = synth.mlp_layers(512, 768, 256, 27, "mlp")
    x = synth.activations(M, 512, "f16", 27, "mlp.x")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(M * 768 * 2), ctx.alloc(M * 256 * 2)
    ctx.qmlp(xb, G, D, hb, yb, M, B.F16)
    y = yb.to_host(np.float16, (M, 256))
    for fused in (True, False):
        assert orc.rel_l2(y, orc.mlp(x, gate_up.triple, down.triple, fused=fused)) < TOL_16


def test_config5_mlp_70b_m1(ctx):
    d = synth.MLP70B
    gate_up, down = synth.mlp_layers(d["K"], d["I"], d["H"], 0, "cfg5")
    x = synth.activations(1, d["K"], "f16", 0, "cfg5.x")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(x)
    hb, yb = ctx.alloc(d["I"] * 2), ctx.alloc(d["H"] * 2)
    ctx.qmlp(xb, G, D, hb, yb, 1, B.F16)
    y = yb.to_host(np.float16, (1, d["H"]))
    assert orc.rel_l2(y, orc.mlp(x, gate_up.triple, down.triple, fused=True)) < TOL_16


# -- host-pointer variant, f32 slots, error behaviour ---------------------------------------

def test_host_pointer_variant_matches_device_variant(ctx):
    x, layer = synth.config4("o", 4)
    L = ctx.upload_layer(layer)
    a = ctx.qmatmul_host(x, L)
    b = _run(ctx, x, layer)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    # the bound form (arguments marshalled once) reads x and fills `out` at every call
    xs = x.copy()
    out = np.zeros_like(a)
    call = ctx.qmatmul_host_bound(xs, L, out)
    assert call() is out and np.array_equal(out.view(np.uint16), a.view(np.uint16))
    xs[:] = 2 * x
    call()
    assert np.array_equal(out.view(np.uint16), ctx.qmatmul_host(2 * x, L).view(np.uint16))


def test_f32_slots(ctx):
    rng = np.random.default_rng(5)
    a = rng.standard_normal(1000).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    ba, bb, bo = ctx.upload(a), ctx.upload(b), ctx.alloc(4000)
    for op, f in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply)):
        ctx.binary_f32(op, ba, bb, bo, 1000)
        assert np.array_equal(bo.to_host(np.float32, (1000,)), f(a, b))
    A = rng.standard_normal((37, 53)).astype(np.float32)
    Bm = rng.standard_normal((53, 29)).astype(np.float32)
    bA, bB, bC = ctx.upload(A), ctx.upload(Bm), ctx.alloc(37 * 29 * 4)
    ctx.matmul_f32(bA, bB, bC, 37, 53, 29)
    assert np.allclose(bC.to_host(np.float32, (37, 29)), A @ Bm, rtol=1e-4, atol=1e-4)


def test_buffer_rules(ctx, backend):
    buf = ctx.upload(np.arange(16, dtype=np.uint8))
    out = np.full(32, 0xEE, np.uint8)
    # copies clamp to the buffer size (src/webgpu_plugin.cpp:1495)
    assert backend.vt["buffer_copy_to_host"](ctx.handle, buf.handle, out.ctypes.data, 32) == B.OK
    assert out[:16].tolist() == list(range(16)) and out[16] == 0xEE
    assert backend.vt["buffer_get_host_ptr"](ctx.handle, buf.handle) is None
    info = ctx.device_info()
    assert info["vendor"] == "NVIDIA" and info["compute_units"] > 0 and info["is_discrete"]
    assert backend.create_context(0).handle            # a second context on the same device


def test_errors_on_device(ctx):
    x, layer = synth.config4("o", 1)
    L = ctx.upload_layer(layer)
    xb = ctx.upload(x)
    small = ctx.alloc(16)
    with pytest.raises(B.BackendError) as e:
        ctx.qmatmul(xb, L, small, 1, B.F16)             # output buffer too small
    assert e.value.code == B.INVALID_ARGUMENT
    with pytest.raises(B.BackendError) as e:
        ctx.qmatmul(xb, L, small, 1, B.F32)             # unsupported dtype combination
    assert e.value.code == B.NOT_SUPPORTED
    # an absurd allocation reports failure instead of raising a CUDA error later
    assert ctx.backend.vt["buffer_alloc"](ctx.handle, 1 << 50) is None
    ctx.sync()


def test_kernel_attributes(ctx, backend):
    import ctypes as C
    k = backend.lib.lux_cuda_kernel_get(b"lux_qskinny_i4_g128")
    attrs = B.KernelAttributes()
    assert backend.lib.lux_cuda_kernel_attributes(k, C.byref(attrs)) == B.OK
    assert attrs.binary_arch == 100 and attrs.registers_per_thread > 0 and attrs.local_bytes == 0
    backend.lib.lux_cuda_kernel_destroy(k)
