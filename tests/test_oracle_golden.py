"""The C oracle against the known-answer fixture tests/golden/wgsl_kat.json.

The fixture is produced by tests/golden/make_kat.py, an independent pure-Python
restatement of the same WGSL lines, plus literal cases checked by hand.  The reference
itself holds no golden vectors for this path, so this is the strongest pin available.
"""
import json
import os
import struct

import numpy as np
import pytest

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "wgsl_kat.json")


@pytest.fixture(scope="module")
def kat():
    with open(GOLDEN) as f:
        return json.load(f)


def _f32(bits):
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def _bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_unpack_int4_asym(kat):
    for c in kat["unpack_int4_asym"]:
        assert orc.unpack_int4_asym_x8(c["word"], c["zp"]) == c["out"]


def test_unpack_int4_sym(kat):
    for c in kat["unpack_int4_sym"]:
        assert orc.unpack_int4_sym_x8(c["word"]) == c["out"]
        # symmetric is the asymmetric unpack with zero-point 8
        assert orc.unpack_int4_asym_x8(c["word"], 8) == c["out"]


def test_unpack_int8(kat):
    for c in kat["unpack_int8"]:
        assert orc.unpack_int8_x4(c["word"]) == c["out"]


def test_pack_int4_asym(kat):
    for c in kat["pack_int4_asym"]:
        assert orc.pack_int4_asym_x8(c["vals"], c["zp"]) == c["word"]


def test_low_nibble_first():
    # byte j holds element 2j in the low nibble: word 0x000000A5 -> elements (5, 10, 0, ...)
    assert orc.unpack_int4_asym_x8(0x000000A5, 0)[:2] == [5, 10]


def test_f16_widening(kat):
    for c in kat["f16_to_f32"]:
        assert _bits(orc.f16_bits_to_f32(c["bits"])) == c["f32_bits"]
    # exhaustive: the software widening equals IEEE for every non-NaN pattern
    allbits = np.arange(1 << 16, dtype=np.uint16)
    ieee = allbits.view(np.float16).astype(np.float32)
    for b in range(0, 1 << 16, 97):
        if np.isnan(ieee[b]):
            continue
        assert _bits(orc.f16_bits_to_f32(b)) == _bits(float(ieee[b])), hex(b)


def test_f16_narrowing_wgsl(kat):
    for c in kat["f32_to_f16_wgsl"]:
        assert orc.f32_to_f16_bits_wgsl(_f32(c["f32_bits"])) == c["bits"]


def test_f16_narrowing_wgsl_equals_rne_for_normals():
    rng = np.random.default_rng(1)
    vals = (rng.standard_normal(4000) * 10.0 ** rng.uniform(-4, 4, 4000)).astype(np.float32)
    for v in vals:
        r = orc.f32_to_f16_rne(float(v))
        exp = (r >> 10) & 0x1F
        if 0 < exp < 31:          # result normal in f16: shader narrowing == IEEE RNE
            assert orc.f32_to_f16_bits_wgsl(float(v)) == r


def test_bf16_rne(kat):
    for c in kat["bf16_rne"]:
        assert orc.f32_to_bf16_rne(_f32(c["f32_bits"])) == c["bits"]
    v = np.array([_f32(c["f32_bits"]) for c in kat["bf16_rne"]], np.float32)
    assert list(orc.f32_to_bf16(v)) == [c["bits"] for c in kat["bf16_rne"]]


def _case_arrays(c):
    bits, N, K, M = c["bits"], c["N"], c["K"], c["M"]
    if bits == 4:
        w = np.array(c["w_bytes"], np.uint8)
        z = np.array(c["zeros"], np.uint8)
        zeros = (z[:, 0::2] | (np.pad(z, ((0, 0), (0, z.shape[1] % 2)))[:, 1::2] << 4)).astype(np.uint8)
        scales = np.array(c["scale_bits"], np.uint16).view(np.float16)
        x = np.array(c["x_bits"], np.uint16).view(np.float16)
    else:
        w = np.array(c["w_bytes"], np.uint8).view(np.int8)
        zeros = None
        scales = np.array(c["scale_bits"], np.uint32).view(np.float32)
        x = np.array(c["x_bits"], np.uint32).view(np.float32)
    return w, scales, zeros, x


def test_matmul_cases(kat):
    for c in kat["matmul"]:
        w, scales, zeros, x = _case_arrays(c)
        q = orc.qunpack(w, zeros, c["bits"], c["group"])
        assert q.tolist() == c["q"]
        dq = orc.qdequant(w, scales, zeros, c["bits"], c["group"], orc.F32)
        assert dq.view(np.uint32).tolist() == c["dequant_f32_bits"]
        dqb = orc.qdequant(w, scales, zeros, c["bits"], c["group"], orc.BF16)
        assert dqb.tolist() == c["dequant_bf16_bits"]
        y = orc.qmatmul(x, w, scales, zeros, c["bits"], c["group"], y_code=orc.F32, acc_mode=0)
        assert y.view(np.uint32).tolist() == c["y_f32_bits"]
        # the other accumulation orders stay within f32 rounding of the sequential one
        for mode in (1, 2):
            y2 = orc.qmatmul(x, w, scales, zeros, c["bits"], c["group"], y_code=orc.F32, acc_mode=mode)
            assert orc.rel_l2(y2, y) < 1e-5


def test_silu():
    for v in (-3.0, -0.5, 0.0, 0.5, 4.0):
        assert abs(orc.silu(v) - v / (1.0 + np.exp(-v))) < 1e-6
