"""The quantize side of the oracle (no GPU): the C restatement of compute_group_scales and the
three quantize shaders (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:157-232, 236-259,
288-310, 336-362) against the known-answer cases of tests/golden/wgsl_kat.json (a second, pure
Python restatement plus one case worked out by hand), and the properties that characterise the
reference's formats, including the asymmetric int4 shader's missing zero-point shift."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc

KAT = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "wgsl_kat.json")))


def _f32(bits):
    return np.array(bits, np.uint32).view(np.float32)


@pytest.mark.parametrize("case", KAT["quantize"], ids=lambda c: f"fmt{c['format']}_g{c['group']}_{len(c['x_bits'])}")
def test_known_answers(case):
    x = _f32(case["x_bits"])
    gs = orc.group_scales(x, case["group"], case["format"])
    assert gs["scale"].view(np.uint32).tolist() == case["scale_bits"]
    assert gs["zero_point"].tolist() == case["zero_points"]
    assert gs["group_min"].view(np.uint32).tolist() == case["min_bits"]
    assert gs["group_max"].view(np.uint32).tolist() == case["max_bits"]
    with np.errstate(all="ignore"):
        words = orc.quantize_packed(x, case["group"], case["format"], gs)
    assert words.tolist() == case["words"]


def test_symmetric_formats_round_trip_within_half_a_step():
    x = np.random.default_rng(1).standard_normal((8, 512)).astype(np.float32) * 3
    for bits, group in ((4, 128), (8, 32)):
        w, s, z = orc.quantize(x, bits, group, symmetric=True)
        assert z is None
        dq = orc.qdequant(w, s, None, bits, group)
        step = np.repeat(s, group, axis=1)
        assert np.all(np.abs(dq - x) <= 0.5 * step * (1 + 1e-6))


def test_asymmetric_int4_as_the_reference_writes_it():
    """quantize_nax_int4_asym stores clamp(round(v / scale), 0, 15): the zero-point is subtracted
    (:303) and added back inside the pack (:118) around two clamps and never shifts v.  So
      * every negative input is stored as nibble 0,
      * non-negative inputs v <= 15 * scale are stored as round(v / scale), and the round trip
        through dequantize, (nibble - zp) * scale, comes back lower by exactly zp * scale."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((4, 256)).astype(np.float32)
    w, s, z = orc.quantize(x, 4, 128, symmetric=False)
    nib = orc.qunpack(w, None, 4, 128).astype(np.int32) + 8          # stored nibbles (symmetric unpack subtracts 8)
    scale = np.repeat(s, 128, axis=1)
    zp = np.repeat(((z[:, :, None] >> np.array([0, 4])) & 15).reshape(4, -1)[:, :2], 128, axis=1).astype(np.int32)
    assert np.all(nib[x < 0] == 0)
    with np.errstate(all="ignore"):
        want = np.clip(np.rint(x / scale), 0, 15).astype(np.int32)
    assert np.array_equal(nib, want)
    dq = orc.qdequant(w, s, z, 4, 128)
    assert np.array_equal(dq, ((nib - zp).astype(np.float32) * scale))
    # a group that spans both signs has zp >= 1, so the round trip is NOT the identity
    assert zp.min() >= 1 and np.abs(dq - x).max() > scale.max()


def test_shifted_extension_round_trips():
    """The non-reference variant clamp(round(v / scale) + zp, 0, 15) reproduces v to within one step
    (the zero-point is itself rounded)."""
    x = np.random.default_rng(3).standard_normal((4, 256)).astype(np.float32)
    w, s, z = orc.quantize(x, 4, 128, symmetric=False, shifted=True)
    dq = orc.qdequant(w, s, z, 4, 128)
    assert np.all(np.abs(dq - x) <= np.repeat(s, 128, axis=1) * 1.01)


def test_f16_scale_table_quantizes_with_the_rounded_scale():
    x = np.random.default_rng(4).standard_normal((2, 256)).astype(np.float32)
    w, s, z = orc.quantize(x, 4, 128, symmetric=True, scale_code=orc.F16)
    assert s.dtype == np.float16
    with np.errstate(all="ignore"):
        want = np.clip(np.rint(x / np.repeat(s.astype(np.float32), 128, axis=1)), -8, 7).astype(np.int8)
    assert np.array_equal(orc.qunpack(w, None, 4, 128), want)
