"""Writes tests/golden/wgsl_kat.json: known-answer cases for the quantized-matmul math.

luxcpp/webgpu ships no golden vectors for its quantized kernels, so these cases are
derived from the WGSL text by a SECOND, independent restatement: plain Python integers
and ``struct``-level float handling below, written line by line from the shader (paths
inside luxcpp/webgpu are cited at each function).  The C oracle
(oracle/qmatmul_oracle.c) must reproduce every case; a disagreement means one of the
two restatements misreads the shader.  The literal cases at the top of ``main`` were
also checked by hand.

Run:  python tests/golden/make_kat.py      (needs nothing but the standard library)
"""
import json
import os
import random
import struct


# kernels/wgsl/gpu/quantized_nax.wgsl:125-132
def unpack_int4_asym_x8(packed, zp):
    return [((packed >> (i * 4)) & 0xF) - zp for i in range(8)]


# kernels/wgsl/gpu/quantized_nax.wgsl:105-112
def unpack_int4_sym_x8(packed):
    return [((packed >> (i * 4)) & 0xF) - 8 for i in range(8)]


# kernels/wgsl/gpu/quantized_nax.wgsl:143-151
def unpack_int8_x4(packed):
    out = []
    for i in range(4):
        v = (packed >> (i * 8)) & 0xFF
        if v >= 128:
            v -= 256
        out.append(v)
    return out


# kernels/wgsl/gpu/quantized_nax.wgsl:115-122
def pack_int4_asym_x8(vals, zp):
    r = 0
    for i in range(8):
        a = max(0, min(15, vals[i] + zp))
        r |= (a & 0xF) << (i * 4)
    return r


def f32_bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def bits_f32(u):
    return struct.unpack("<f", struct.pack("<I", u & 0xFFFFFFFF))[0]


def f32(x):
    """Round a Python float to f32 (what every WGSL f32 operation does)."""
    return bits_f32(f32_bits(x))


# kernels/wgsl/gpu/fp_quantized.wgsl:131-165
def f16_bits_to_f32(bits):
    sign = (bits & 0x8000) << 16
    exp = (bits >> 10) & 0x1F
    mant = bits & 0x3FF
    if exp == 0:
        if mant == 0:
            return bits_f32(sign)
        m, e = mant, 0
        while (m & 0x400) == 0:
            m <<= 1
            e -= 1
        m &= 0x3FF
        return bits_f32(sign | ((127 - 15 + 1 + e) << 23) | (m << 13))
    if exp == 31:
        return bits_f32(sign | 0x7F800000 | (0 if mant == 0 else (0x400000 | (mant << 13))))
    return bits_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13))


# kernels/wgsl/gpu/fp_quantized.wgsl:65-128
def f32_to_f16_bits_wgsl(val):
    bits = f32_bits(val)
    sign = (bits >> 16) & 0x8000
    exp = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    if exp == 255:
        return sign | (0x7E00 if mant else 0x7C00)
    if exp == 0:
        return sign
    new_exp = exp - 127 + 15
    if new_exp >= 31:
        return sign | 0x7C00
    if new_exp <= 0:
        if new_exp < -10:
            return sign
        shift = 1 - new_exp
        mi = mant | 0x800000
        return sign | ((mi >> (13 + shift)) + ((mi >> (12 + shift)) & 1))
    trunc = mant >> 13
    rb = (mant >> 12) & 1
    sticky = (mant & 0xFFF) != 0
    r = trunc
    if rb and (sticky or (trunc & 1)):
        r += 1
        if r >= 0x400:
            return sign | ((new_exp + 1) << 10) if new_exp < 30 else sign | 0x7C00
    return sign | (new_exp << 10) | r


def bf16_rne_bits(val):
    u = f32_bits(val)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def wgsl_i32(v):
    """i32(f32): toward zero, clamped to the i32 range; NaN -> 0 (indeterminate in WGSL)."""
    if v != v:
        return 0
    if v >= 2147483648.0:
        return 2147483647
    if v <= -2147483648.0:
        return -2147483648
    return int(v)


def f32_div(a, b):
    """IEEE f32 division with the f32 results for a zero divisor."""
    if b == 0.0:
        if a == 0.0 or a != a:
            return float("nan")
        return float("inf") if (a > 0) == (str(b)[0] != "-") else float("-inf")
    return f32(a / b)


def clamp(v, lo, hi):
    return max(lo, min(hi, v))


# kernels/wgsl/gpu/quantized_nax.wgsl:157-232 (format 0 = int4 sym, 1 = int4 asym, 2 = int8 sym)
def compute_group_scales(vals, group, fmt):
    out = []
    for b in range(0, len(vals), group):
        mx, mn = f32(-1e30), f32(1e30)
        for v in vals[b:b + group]:
            mx = max(mx, v)
            mn = min(mn, v)
        if fmt in (0, 2):
            amax = max(abs(mx), abs(mn))
            scale = f32_div(amax, 7.0 if fmt == 0 else 127.0)
            zp = 0
        else:
            scale = f32_div(f32(mx - mn), 15.0)
            r = f32_div(-mn, scale)
            zp = clamp(wgsl_i32(float(round(r)) if r == r and abs(r) != float("inf") else r), 0, 15)
        if scale == 0.0:
            scale = 1.0
        out.append((scale, zp, mn, mx))
    return out


# kernels/wgsl/gpu/quantized_nax.wgsl:236-259, 288-310 (+ :115-122), 336-362 (+ :135-140)
def quantize_words(vals, group, fmt, gs):
    per = 4 if fmt == 2 else 8
    words = []
    for w in range(len(vals) // per):
        scale, zp, _, _ = gs[(w * per) // group]
        word = 0
        for i in range(per):
            r = f32_div(vals[w * per + i], scale)
            scaled = float(round(r)) if r == r and abs(r) != float("inf") else r
            if fmt == 0:
                word |= ((clamp(wgsl_i32(scaled), -8, 7) + 8) & 0xF) << (4 * i)
            elif fmt == 1:
                q = clamp(wgsl_i32(scaled), 0, 15) - zp
                word |= (clamp(q + zp, 0, 15) & 0xF) << (4 * i)
            else:
                word |= (clamp(wgsl_i32(scaled), -128, 127) & 0xFF) << (8 * i)
        words.append(word)
    return words


def main():
    rnd = random.Random(20240607)
    kat = {"unpack_int4_asym": [], "unpack_int4_sym": [], "unpack_int8": [], "pack_int4_asym": [],
           "f16_to_f32": [], "f32_to_f16_wgsl": [], "bf16_rne": [], "matmul": []}

    # literal cases, checked by hand
    kat["unpack_int4_asym"].append({"word": 0x76543210, "zp": 0, "out": [0, 1, 2, 3, 4, 5, 6, 7]})
    kat["unpack_int4_asym"].append({"word": 0x76543210, "zp": 3, "out": [-3, -2, -1, 0, 1, 2, 3, 4]})
    kat["unpack_int4_asym"].append({"word": 0xFFFFFFFF, "zp": 15, "out": [0] * 8})
    kat["unpack_int4_asym"].append({"word": 0x000000F0, "zp": 0, "out": [0, 15, 0, 0, 0, 0, 0, 0]})
    kat["unpack_int4_sym"].append({"word": 0x76543210, "out": [-8, -7, -6, -5, -4, -3, -2, -1]})
    kat["unpack_int4_sym"].append({"word": 0xFEDCBA98, "out": [0, 1, 2, 3, 4, 5, 6, 7]})
    kat["unpack_int8"].append({"word": 0x80FF7F01, "out": [1, 127, -1, -128]})
    kat["unpack_int8"].append({"word": 0x00000081, "out": [-127, 0, 0, 0]})
    kat["f16_to_f32"].append({"bits": 0x3C00, "f32_bits": f32_bits(1.0)})
    kat["f16_to_f32"].append({"bits": 0x0001, "f32_bits": f32_bits(2.0 ** -24)})
    kat["f16_to_f32"].append({"bits": 0xC000, "f32_bits": f32_bits(-2.0)})
    kat["f16_to_f32"].append({"bits": 0x7BFF, "f32_bits": f32_bits(65504.0)})
    kat["f32_to_f16_wgsl"].append({"f32_bits": f32_bits(1.0), "bits": 0x3C00})
    kat["f32_to_f16_wgsl"].append({"f32_bits": f32_bits(65520.0), "bits": 0x7C00})   # rounds up to inf
    kat["f32_to_f16_wgsl"].append({"f32_bits": f32_bits(1.0 + 2.0 ** -11), "bits": 0x3C00})  # tie -> even
    kat["f32_to_f16_wgsl"].append({"f32_bits": f32_bits(1.0 + 3 * 2.0 ** -11), "bits": 0x3C02})  # tie -> even (up)

    for _ in range(64):
        w = rnd.getrandbits(32)
        zp = rnd.randrange(16)
        kat["unpack_int4_asym"].append({"word": w, "zp": zp, "out": unpack_int4_asym_x8(w, zp)})
        kat["unpack_int4_sym"].append({"word": w, "out": unpack_int4_sym_x8(w)})
        kat["unpack_int8"].append({"word": w, "out": unpack_int8_x4(w)})
        vals = [rnd.randrange(-20, 20) for _ in range(8)]
        kat["pack_int4_asym"].append({"vals": vals, "zp": zp, "word": pack_int4_asym_x8(vals, zp)})
    for _ in range(128):
        b = rnd.getrandbits(16)
        if (b >> 10) & 0x1F == 31 and b & 0x3FF:
            continue                                        # NaN payloads are not compared
        kat["f16_to_f32"].append({"bits": b, "f32_bits": f32_bits(f16_bits_to_f32(b))})
        v = f32(rnd.gauss(0.0, 1.0) * 10.0 ** rnd.uniform(-6, 5))
        kat["f32_to_f16_wgsl"].append({"f32_bits": f32_bits(v), "bits": f32_to_f16_bits_wgsl(v)})
        kat["bf16_rne"].append({"f32_bits": f32_bits(v), "bits": bf16_rne_bits(v)})

    # small matmuls: y = x . dequant(W)^T, f32 accumulate in ascending k with a rounded
    # multiply then a rounded add (kernels/wgsl/gpu/quantized_nax.wgsl:577-621 for the
    # loop, :312-330 / :364-381 for the weight value).
    for bits, group, N, K, M in [(4, 128, 2, 128, 1), (4, 128, 3, 256, 2), (8, 32, 2, 64, 1), (8, 32, 4, 96, 3)]:
        G = K // group
        if bits == 4:
            wbytes = [[rnd.randrange(256) for _ in range(K // 2)] for _ in range(N)]
            zp = [[rnd.randrange(16) for _ in range(G)] for _ in range(N)]
            sc_bits = [[f32_to_f16_bits_wgsl(f32(abs(rnd.gauss(0, 0.02)) / 7.0)) for _ in range(G)] for _ in range(N)]
            sc = [[f16_bits_to_f32(b) for b in row] for row in sc_bits]
            q = [[((wbytes[n][k // 2] >> (4 * (k & 1))) & 0xF) - zp[n][k // group] for k in range(K)] for n in range(N)]
            x_bits = [[f32_to_f16_bits_wgsl(f32(rnd.gauss(0, 1))) for _ in range(K)] for _ in range(M)]
            x = [[f16_bits_to_f32(b) for b in row] for row in x_bits]
        else:
            wbytes = [[rnd.randrange(-127, 128) & 0xFF for _ in range(K)] for _ in range(N)]
            zp = None
            sc = [[f32(abs(rnd.gauss(0, 0.02)) / 127.0) for _ in range(G)] for _ in range(N)]
            sc_bits = [[f32_bits(v) for v in row] for row in sc]
            q = [[(b - 256 if b >= 128 else b) for b in row] for row in wbytes]
            x = [[f32(rnd.gauss(0, 1)) for _ in range(K)] for _ in range(M)]
            x_bits = [[f32_bits(v) for v in row] for row in x]
        wdq = [[f32(float(q[n][k]) * sc[n][k // group]) for k in range(K)] for n in range(N)]
        y = []
        for m in range(M):
            row = []
            for n in range(N):
                acc = 0.0
                for k in range(K):
                    acc = f32(acc + f32(wdq[n][k] * x[m][k]))
                row.append(f32_bits(acc))
            y.append(row)
        kat["matmul"].append({
            "bits": bits, "group": group, "M": M, "N": N, "K": K,
            "w_bytes": wbytes, "zeros": zp, "scale_bits": sc_bits, "x_bits": x_bits,
            "q": q, "dequant_f32_bits": [[f32_bits(v) for v in r] for r in wdq],
            "dequant_bf16_bits": [[bf16_rne_bits(v) for v in r] for r in wdq],
            "y_f32_bits": y,
        })

    # quantize side: group statistics and packed words.  A literal case first (checked by hand):
    # eight values 0..7 in one int4-asym group of 8: max 7, min 0, scale 7/15, zp 0, and
    # round(v / (7/15)) = 0, 2, 4, 6, 9, 11, 13, 15.
    kat["quantize"] = []
    lit = [float(i) for i in range(8)]
    gs = compute_group_scales(lit, 8, 1)
    assert quantize_words(lit, 8, 1, gs) == [0xFDB96420] and gs[0][1] == 0
    cases = [(lit, 8, 1)]
    for fmt, group in ((0, 128), (1, 128), (2, 32)):
        n = 2 * group
        cases.append(([f32(rnd.gauss(0, 1)) for _ in range(n)], group, fmt))
        cases.append(([f32(rnd.gauss(0.5, 0.1)) for _ in range(n)], group, fmt))          # all positive
        cases.append(([f32(-abs(rnd.gauss(0, 3))) for _ in range(n)], group, fmt))         # all negative
        cases.append(([0.0] * group + [f32(rnd.uniform(-1, 1)) for _ in range(group)], group, fmt))   # a group of zeros
        cases.append(([f32(2.5)] * group + [f32(-1.25)] * group, group, fmt))               # constant groups
    for vals, group, fmt in cases:
        gs = compute_group_scales(vals, group, fmt)
        kat["quantize"].append({
            "format": fmt, "group": group, "x_bits": [f32_bits(v) for v in vals],
            "scale_bits": [f32_bits(g[0]) for g in gs], "zero_points": [g[1] for g in gs],
            "min_bits": [f32_bits(g[2]) for g in gs], "max_bits": [f32_bits(g[3]) for g in gs],
            "words": quantize_words(vals, group, fmt, gs)})

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "wgsl_kat.json")
    with open(out, "w") as f:
        json.dump(kat, f, separators=(",", ":"))
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
