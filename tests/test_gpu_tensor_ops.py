"""GPU parity of the f32 tensor slots either side of a linear layer against the oracle's
restatement of the shaders that back them (luxcpp/webgpu kernels/wgsl/gpu/unary.wgsl, copy.wgsl,
softmax.wgsl, logsumexp.wgsl, layer_norm.wgsl, rms_norm.wgsl), through the vtable like add / sub /
mul / matmul.  Tolerance: relative L2 <= 1e-6 (the limit for f32 outputs is 1e-3): integer-exact ops
(neg, abs, relu, copy, transpose) must match bit for bit, the rest differ only by the last-place
differences between the device's and the host's exp / log / tanh."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(17)


def _unary(ctx, op, x):
    xb, ob = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.unary_f32(op, xb, ob, x.size)
    return ob.to_host(np.float32, x.shape)


@pytest.mark.parametrize("n", [1, 255, 4096, 1 << 20, (1 << 20) + 3])
@pytest.mark.parametrize("op", ["exp", "log", "sqrt", "neg", "abs", "tanh", "sigmoid", "relu", "gelu", "silu", "copy"])
def test_unary_ops(ctx, op, n):
    x = RNG.standard_normal(n).astype(np.float32) * 3
    if op in ("log", "sqrt"):
        x = np.abs(x) + np.float32(1e-3)
    got, want = _unary(ctx, op, x), orc.unary_f32(op, x)
    if op in ("neg", "abs", "relu", "copy", "sqrt"):
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    else:
        assert orc.rel_l2(got, want) < 1e-6
        assert np.allclose(got, want, rtol=1e-4, atol=1e-6)      # gelu and tanh cancel to almost 0 for x << 0


def test_div_and_unaligned_views(ctx, backend):
    a = RNG.standard_normal(10007).astype(np.float32)
    b = (RNG.standard_normal(10007).astype(np.float32) + np.float32(3.0))
    ab, bb, ob = ctx.upload(a), ctx.upload(b), ctx.alloc(a.nbytes)
    assert backend.vt["op_div_f32"](ctx.handle, ab.handle, bb.handle, ob.handle, a.size) == B.OK
    assert np.array_equal(ob.to_host(np.float32, a.shape).view(np.uint32), (a / b).view(np.uint32))
    # a view that is not 16-byte aligned takes the scalar path
    big = ctx.upload(np.concatenate([np.zeros(1, np.float32), a]))
    view = ctx.wrap(big.device_ptr + 4, a.nbytes)
    ctx.unary_f32("gelu", view, ob, a.size)
    assert orc.rel_l2(ob.to_host(np.float32, a.shape), orc.unary_f32("gelu", a)) < 1e-6


@pytest.mark.parametrize("rows,cols", [(1, 1), (32, 32), (33, 65), (1000, 37), (4096, 4096), (64, 192), (128, 64), (4160, 4096)])
def test_transpose(ctx, rows, cols):
    x = RNG.standard_normal((rows, cols)).astype(np.float32)
    xb, ob = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.transpose_f32(xb, ob, rows, cols)
    assert np.array_equal(ob.to_host(np.float32, (cols, rows)), x.T)


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("batch,dim", [(1, 1), (3, 7), (16, 256), (5, 1000), (64, 4096), (2, 32000), (4, 128256)])
def test_softmax(ctx, batch, dim, log):
    x = (RNG.standard_normal((batch, dim)) * 4).astype(np.float32)
    xb, ob = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.softmax_f32(xb, ob, batch, dim, log=log)
    got, want = ob.to_host(np.float32, x.shape), orc.softmax_f32(x, log=log)
    assert orc.rel_l2(got, want) < 1e-6
    if not log:
        assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("batch,dim", [(1, 64), (7, 1000), (32, 4096), (3, 8192), (2, 20000)])
def test_rms_norm_and_layer_norm(ctx, batch, dim):
    x = (RNG.standard_normal((batch, dim)) * 2 + 0.5).astype(np.float32)
    g = RNG.standard_normal(dim).astype(np.float32)
    b = RNG.standard_normal(dim).astype(np.float32)
    xb, gb, bb, ob = ctx.upload(x), ctx.upload(g), ctx.upload(b), ctx.alloc(x.nbytes)
    ctx.rms_norm_f32(xb, gb, ob, batch, dim, 1e-6)
    assert orc.rel_l2(ob.to_host(np.float32, x.shape), orc.rms_norm_f32(x, g, 1e-6)) < 1e-6
    ctx.layer_norm_f32(xb, gb, bb, ob, batch, dim, 1e-5)
    assert orc.rel_l2(ob.to_host(np.float32, x.shape), orc.layer_norm_f32(x, g, b, 1e-5)) < 1e-6


def test_argument_checks(ctx, backend):
    x = ctx.upload(np.zeros(64, np.float32))
    small = ctx.alloc(16)
    assert backend.vt["op_exp_f32"](ctx.handle, x.handle, small.handle, 64) == B.INVALID_ARGUMENT
    assert backend.vt["op_softmax_f32"](ctx.handle, x.handle, x.handle, 0, 8) == B.INVALID_ARGUMENT
    assert backend.vt["op_transpose_f32"](ctx.handle, x.handle, x.handle, 8, 8) == B.INVALID_ARGUMENT    # in place
    assert backend.vt["op_rms_norm_f32"](ctx.handle, x.handle, small.handle, x.handle, 1, 64, 1e-6) == B.INVALID_ARGUMENT
    assert backend.vt["op_exp_f32"](ctx.handle, x.handle, x.handle, 0) == B.OK


def test_decoder_block_pieces_chain(ctx):
    """rms_norm -> int4 linear -> silu, the sequence around a quantized layer, device-resident."""
    from webgpu_b200 import synth
    K, N = 1024, 512
    x = RNG.standard_normal((1, K)).astype(np.float32)
    w = RNG.standard_normal(K).astype(np.float32)
    layer = synth.int4_layer(N, K, 3, "blk")
    xb, wb, nb = ctx.upload(x), ctx.upload(w), ctx.alloc(K * 4)
    ctx.rms_norm_f32(xb, wb, nb, 1, K, 1e-6)
    xn = nb.to_host(np.float32, (1, K)).astype(np.float16)
    L, hb = ctx.upload_layer(layer), ctx.upload(xn)
    yb = ctx.alloc(N * 2)
    ctx.qmatmul(hb, L, yb, 1, B.F16)
    y = yb.to_host(np.float16, (1, N)).astype(np.float32)
    got = _unary(ctx, "silu", y)
    ref = orc.unary_f32("silu", orc.to_f32(orc.qmatmul(orc.rms_norm_f32(x, w, 1e-6).astype(np.float16), *layer.triple, bits=4, group=128)))
    assert orc.rel_l2(got, ref) < 5e-3
