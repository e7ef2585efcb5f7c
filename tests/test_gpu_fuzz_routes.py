"""Seeded sweep over shapes the named configurations do not hit: random batch (1..513), output
count, row length, activation type, SwiGLU, symmetric / asymmetric int4 and int8 g32 layers, each
sent through lux_cuda_qmatmul on the DEFAULT route and compared with the CPU oracle on a subset of
the batch rows.  The sweep is fixed by its seed; it is there to catch a dispatch rule that sends a
shape to a kernel that mishandles it (ragged tiles, odd group counts, tiny K, batch just past a
crossover), not to measure anything.

Bars as everywhere: relative L2 error 1e-3 for f32 outputs, 5e-3 for f16 / bf16 outputs, and the
context's device status stays clear.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu

BATCHES = [1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 12, 13, 16, 17, 24, 31, 32, 33, 47, 64, 65, 100, 127, 128, 129,
           200, 255, 256, 257, 300, 513]
ROW_LENGTHS = [128, 256, 384, 512, 640, 768, 1024, 1280, 1536, 2048, 2560, 3072, 4096, 5120, 8192]


def _case(rng):
    M, K = int(rng.choice(BATCHES)), int(rng.choice(ROW_LENGTHS))
    step = int(rng.choice([16, 16, 32, 64, 128, 128, 256]))
    N = step * int(rng.integers(1, max(2, 4096 // step // int(rng.choice([1, 2, 4, 8])))))
    swiglu = bool(rng.integers(0, 3) == 0)
    if swiglu:
        N = (N // 32) * 32 or 32
    symmetric = bool(rng.integers(0, 4) == 0)
    dtype = str(rng.choice(["f16", "f16", "bf16"]))
    bits = 8 if rng.integers(0, 4) == 0 else 4
    if bits == 8:                       # the int8 g32 path is f32 in, f32 out, no epilogue
        swiglu, dtype = False, "f32"
    return M, N, K, bits, dtype, swiglu, symmetric


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_on_the_default_route(ctx, backend, seed):
    rng = np.random.default_rng(seed)
    kernels = set()
    for case in range(100):
        M, N, K, bits, dtype, swiglu, symmetric = _case(rng)
        if bits == 8:
            layer = synth.int8_layer(N, K, 1000 * seed + case, "fz8")
        else:
            layer = synth.int4_layer(N, K, 1000 * seed + case, "fz4", symmetric=symmetric)
        x = synth.activations(M, K, dtype, 1000 * seed + case, "fz.x")
        L, xb = ctx.upload_layer(layer), ctx.upload(x)
        n_out = N // 2 if swiglu else N
        yb = ctx.alloc(M * n_out * x.itemsize)
        ctx.qmatmul(xb, L, yb, M, B.np_dtype_code(x), flags=B.FLAG_SWIGLU if swiglu else 0)
        name = backend.last_kernel_name()
        kernels.add(name)
        y = yb.to_host(x.dtype, (M, n_out))
        rows = np.unique(np.linspace(0, M - 1, 6).astype(int))
        xr = np.ascontiguousarray(x[rows])
        if swiglu:
            gu = orc.qmatmul(xr, *layer.triple, bits=4, group=128, y_code=orc.F32)
            ref = orc.swiglu(gu, h_code=orc.dtype_code(x))
        else:
            ref = orc.qmatmul(xr, *layer.triple, bits=bits, group=128 if bits == 4 else 32)
        got = y[rows]
        if dtype == "bf16":
            got, ref = synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref)
        what = f"case {case}: M={M} N={N} K={K} int{bits} {dtype} swiglu={swiglu} symmetric={symmetric} -> {name}"
        assert orc.rel_l2(got, ref) < (1e-3 if dtype == "f32" else 5e-3), what
        assert ctx.last_device_status() == 0, what
        for b in (xb, yb, L.w, L.scales, L.zeros):
            if b is not None:
                b.free()
    # the sweep is only worth its time if it keeps reaching the GEMV, the skinny and both GEMM kernels
    assert len(kernels) >= 7, sorted(kernels)


@pytest.mark.parametrize("seed", [31])
def test_random_integer_matmul_shapes_bit_exact(ctx, backend, seed):
    """int8 x int8 and packed int4 x int8 -> int32 over random ragged shapes: every one bit-exact
    against an exact f64 product, whichever of the tcgen05 and the mma.sync kernel takes it."""
    rng = np.random.default_rng(seed)
    kernels = set()
    for case in range(120):
        M = int(rng.choice([1, 3, 16, 33, 100, 127, 128, 129, 255, 256, 300, 513, 1000, 1500]))
        N = int(rng.choice([1, 5, 16, 30, 64, 100, 255, 256, 257, 300, 512, 513, 1000, 2048]))
        K = int(rng.choice([16, 48, 50, 64, 208, 256, 272, 304, 512, 1008, 1024, 2048, 4096, 4112]))
        bits = 4 if rng.integers(0, 3) == 0 else 8
        lo, hi = (-8, 8) if bits == 4 else (-128, 128)
        a = rng.integers(lo, hi, size=(M, K), dtype=np.int8)
        b = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
        if bits == 4:
            flat = a.ravel().astype(np.uint8) & 0xF
            packed = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
        else:
            packed = a
        ab, bb, cb = ctx.upload(packed), ctx.upload(b), ctx.alloc(M * N * 4)
        ctx.matmul_int8(ab, bb, cb, M, N, K, a_bits=bits)
        kernels.add(backend.last_kernel_name())
        want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.int32)      # exact: |sum| < 2^53
        what = f"case {case}: M={M} N={N} K={K} a_bits={bits} -> {backend.last_kernel_name()}"
        assert np.array_equal(cb.to_host(np.int32, (M, N)), want), what
        assert ctx.last_device_status() == 0, what
        for buf in (ab, bb, cb):
            buf.free()
    assert "lux_matmul_int8_tcgen05" in kernels and len(kernels) >= 2, sorted(kernels)


@pytest.mark.parametrize("seed", [41])
def test_random_ffn_shapes(ctx, backend, seed):
    """lux_cuda_qmlp and lux_cuda_qmlp_noalloc over random (batch, K, I, H): the two entry points
    agree bit for bit, and the result meets the oracle's FFN with the SwiGLU applied to the f32 sums.
    f16: 5e-3 against the oracle with f32 weights.  bf16 from five rows up: the tensor-core kernels
    multiply weights rounded to bf16, so the bar of one layer is not the bar of two in a row; the
    check is 1e-3 against the oracle doing exactly that (weights rounded, f32 accumulate) and 8e-3
    against f32 weights (measured 3e-3 .. 6e-3: two weight roundings and two output roundings of
    8 bits).  bf16 up to four rows runs on the fixed-point GEMV with exact weights."""
    rng = np.random.default_rng(seed)
    for case in range(60):
        M = int(rng.choice([1, 2, 3, 4, 5, 8, 9, 16, 17, 32, 33, 64, 65, 128, 200, 256, 300]))
        K, I = 128 * int(rng.integers(1, 17)), 128 * int(rng.integers(1, 17))
        H = 16 * int(rng.integers(1, 65))
        if rng.integers(0, 2):
            H = 128 * ((H + 127) // 128)
        dtype = str(rng.choice(["f16", "bf16"]))
        gate_up, down = synth.mlp_layers(K, I, H, 1000 * seed + case, "fzm")
        x = synth.activations(M, K, dtype, 1000 * seed + case, "fzm.x")
        G, D, xb = ctx.upload_layer(gate_up), ctx.upload_layer(down), ctx.upload(x)
        hb, yb, yb2 = ctx.alloc(M * I * 2), ctx.alloc(M * H * 2), ctx.alloc(M * H * 2)
        code = B.np_dtype_code(x)
        ctx.qmlp(xb, G, D, hb, yb, M, code)
        y = yb.to_host(x.dtype, (M, H))
        what = f"case {case}: M={M} K={K} I={I} H={H} {dtype} -> {backend.last_kernel_name()}"
        if M * I * 2 <= B.NOALLOC_MAX_BYTES:
            ctx.qmlp_noalloc(xb, G, D, yb2, M, code)
            assert np.array_equal(y, yb2.to_host(x.dtype, (M, H))), what
        else:                                # larger than the built-in scratch: refused, nothing launched
            with pytest.raises(B.BackendError):
                ctx.qmlp_noalloc(xb, G, D, yb2, M, code)
        assert ctx.last_device_status() == 0, what
        rows = np.unique(np.linspace(0, M - 1, 5).astype(int))
        xr = np.ascontiguousarray(x[rows])
        exact = orc.mlp(xr, gate_up.triple, down.triple, fused=True)
        if dtype == "f16":
            assert orc.rel_l2(y[rows], exact) < 5e-3, what
        else:
            got = synth.bf16_bits_to_f32(y[rows])
            assert orc.rel_l2(got, synth.bf16_bits_to_f32(exact)) < 8e-3, what
            if M >= 5:                       # up to four rows the fixed-point GEMV keeps the weights exact
                rounded = orc.mlp(xr, gate_up.triple, down.triple, fused=True, w_round=orc.BF16)
                assert orc.rel_l2(got, synth.bf16_bits_to_f32(rounded)) < 1e-3, what
        for buf in (xb, hb, yb, yb2, G.w, G.scales, G.zeros, D.w, D.scales, D.zeros):
            if buf is not None:
                buf.free()
