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
