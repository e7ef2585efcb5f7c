"""The f32 tensor-op oracle (oracle/tensor_ops_oracle.c) without a GPU: agreement with float64
numpy evaluations of the same formulas, and the properties each op has by definition.  The
shaders these restate are never run on data by the reference's own tests (parity unpinned), so
this only guards the restatement against slips."""
import numpy as np
import pytest

from oracle import oracle as orc

RNG = np.random.default_rng(5)


@pytest.mark.parametrize("op,fn", [
    ("exp", np.exp), ("log", np.log), ("sqrt", np.sqrt), ("neg", np.negative), ("abs", np.abs), ("tanh", np.tanh),
    ("sigmoid", lambda x: 1 / (1 + np.exp(-x))), ("relu", lambda x: np.maximum(x, 0)), ("copy", lambda x: x),
    ("silu", lambda x: x / (1 + np.exp(-x))),
    ("gelu", lambda x: 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))),
])
def test_unary_against_float64(op, fn):
    x = RNG.standard_normal(4099).astype(np.float32) * 3
    if op in ("log", "sqrt"):
        x = np.abs(x) + np.float32(1e-3)
    got = orc.unary_f32(op, x)
    want = fn(x.astype(np.float64))
    assert np.allclose(got, want, rtol=2e-6, atol=1e-7)


def test_transpose():
    x = RNG.standard_normal((37, 101)).astype(np.float32)
    assert np.array_equal(orc.transpose_f32(x), x.T)


@pytest.mark.parametrize("dim", [7, 256, 1000, 4096])
def test_softmax_and_log_softmax(dim):
    x = RNG.standard_normal((5, dim)).astype(np.float32) * 4
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(axis=1, keepdims=True))
    want = e / e.sum(axis=1, keepdims=True)
    got = orc.softmax_f32(x)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-9)
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)
    assert np.allclose(orc.softmax_f32(x, log=True), np.log(want), rtol=1e-5, atol=2e-6)
    # the shader clamps exp's argument to [-88, 88]: a row with a huge spread stays finite
    wide = np.array([[0.0, -200.0, 100.0]], np.float32)
    assert np.isfinite(orc.softmax_f32(wide)).all()


@pytest.mark.parametrize("dim", [64, 1000, 8192])
def test_norms(dim):
    x = (RNG.standard_normal((3, dim)) * 2 + 0.5).astype(np.float32)
    g = RNG.standard_normal(dim).astype(np.float32)
    b = RNG.standard_normal(dim).astype(np.float32)
    x64 = x.astype(np.float64)
    rms = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * g
    assert np.allclose(orc.rms_norm_f32(x, g, 1e-6), rms, rtol=1e-5, atol=1e-6)
    mean = x64.mean(axis=1, keepdims=True)
    var = (x64 ** 2).mean(axis=1, keepdims=True) - mean ** 2
    ln = g * ((x64 - mean) / np.sqrt(var + 1e-5)) + b
    assert np.allclose(orc.layer_norm_f32(x, g, b, 1e-5), ln, rtol=1e-4, atol=1e-5)
