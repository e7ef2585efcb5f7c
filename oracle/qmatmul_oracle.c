/*
 * qmatmul_oracle.c -- CPU restatement of luxcpp/webgpu's group-quantized matmul math.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls
 * this file; it exists so that tests can compare the CUDA kernels with the
 * reference's arithmetic, and so that the benchmark can time the same arithmetic on
 * host cores as a CPU baseline.
 *
 * PARITY UNPINNED: luxcpp/webgpu holds no test, fixture or golden vector for its
 * quantized kernels, and its WGSL cannot be executed without a WebGPU runtime.  The
 * functions below are therefore written from the shader text alone; each one cites
 * the lines it restates (paths inside luxcpp/webgpu).  The known-answer cases in
 * tests/golden/ were worked out by hand from the same lines.
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off).  Contraction is
 * off so that "sum += a * b" is a rounded multiply followed by a rounded add, as the
 * WGSL text says, not a fused multiply-add.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_F32  0
#define ORC_F16  1
#define ORC_BF16 2

/* ------------------------------------------------------------------------------------
 * Integer unpack
 * ---------------------------------------------------------------------------------- */

/* unpack_nax_int4_asym_x8, kernels/wgsl/gpu/quantized_nax.wgsl:125-132:
 *   val = i32((packed >> (i*4)) & 0xF); result[i] = val - zero_point               */
void orc_unpack_int4_asym_x8(uint32_t packed, int32_t zero_point, int32_t out[8]) {
    for (uint32_t i = 0; i < 8u; i++) {
        int32_t val = (int32_t)((packed >> (i * 4u)) & 0xFu);
        out[i] = val - zero_point;
    }
}

/* unpack_nax_int4_sym_x8, quantized_nax.wgsl:105-112: stored [0,15] maps to [-8,7]. */
void orc_unpack_int4_sym_x8(uint32_t packed, int32_t out[8]) {
    for (uint32_t i = 0; i < 8u; i++) {
        uint32_t mapped = (packed >> (i * 4u)) & 0xFu;
        out[i] = (int32_t)mapped - 8;
    }
}

/* unpack_nax_int8_x4, quantized_nax.wgsl:143-151 (same convention as
 * gpu/quantized.wgsl:167-178): byte i, and "if (val >= 128) val -= 256".             */
void orc_unpack_int8_x4(uint32_t packed, int32_t out[4]) {
    for (uint32_t i = 0; i < 4u; i++) {
        int32_t val = (int32_t)((packed >> (i * 8u)) & 0xFFu);
        if (val >= 128) val -= 256;
        out[i] = val;
    }
}

/* pack_nax_int4_asym_x8, quantized_nax.wgsl:115-122 (store side; used to build
 * known-answer inputs).                                                             */
uint32_t orc_pack_int4_asym_x8(const int32_t vals[8], int32_t zero_point) {
    uint32_t result = 0u;
    for (uint32_t i = 0; i < 8u; i++) {
        int32_t a = vals[i] + zero_point;
        if (a < 0) a = 0;
        if (a > 15) a = 15;
        result |= ((uint32_t)a & 0xFu) << (i * 4u);
    }
    return result;
}

/* ------------------------------------------------------------------------------------
 * 16-bit float conversions
 * ---------------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* f16_bits_to_f32, kernels/wgsl/gpu/fp_quantized.wgsl:131-165: exact widening
 * (subnormals are normalised, so nothing is lost).                                  */
float orc_f16_bits_to_f32(uint32_t bits) {
    uint32_t sign = (bits & 0x8000u) << 16;
    uint32_t exp = (bits >> 10) & 0x1Fu;
    uint32_t mant = bits & 0x3FFu;
    if (exp == 0u) {
        if (mant == 0u) return bits_f32(sign);
        uint32_t m = mant;
        int32_t e = 0;
        while ((m & 0x400u) == 0u) { m <<= 1; e -= 1; }
        m &= 0x3FFu;
        uint32_t new_exp = (uint32_t)(127 - 15 + 1 + e);
        return bits_f32(sign | (new_exp << 23) | (m << 13));
    }
    if (exp == 31u) {
        if (mant == 0u) return bits_f32(sign | 0x7F800000u);
        return bits_f32(sign | 0x7FC00000u | (mant << 13));
    }
    return bits_f32(sign | ((exp + 127u - 15u) << 23) | (mant << 13));
}

/* f32_to_f16_bits, fp_quantized.wgsl:65-128, restated as written: round-to-nearest-
 * even for results in the f16 normal range, f32 subnormals flushed to zero, and
 * f16-subnormal results rounded half-UP (:96-107).  Kept to document where the
 * shader's software narrowing departs from IEEE; the matmul oracle narrows with
 * orc_f32_to_f16_rne, which equals this function whenever the result is normal.      */
uint32_t orc_f32_to_f16_bits_wgsl(float val) {
    uint32_t bits = f32_bits(val);
    uint32_t sign = (bits >> 16) & 0x8000u;
    uint32_t exp = (bits >> 23) & 0xFFu;
    uint32_t mant = bits & 0x7FFFFFu;
    if (exp == 255u) return mant != 0u ? (sign | 0x7E00u) : (sign | 0x7C00u);
    if (exp == 0u) return sign;
    int32_t new_exp = (int32_t)exp - 127 + 15;
    if (new_exp >= 31) return sign | 0x7C00u;
    if (new_exp <= 0) {
        if (new_exp < -10) return sign;
        uint32_t shift = (uint32_t)(1 - new_exp);
        uint32_t mi = mant | 0x800000u;
        uint32_t denorm = (mi >> (13u + shift)) + ((mi >> (12u + shift)) & 1u);
        return sign | denorm;
    }
    uint32_t trunc = mant >> 13;
    uint32_t round_bit = (mant >> 12) & 1u;
    int sticky = (mant & 0xFFFu) != 0u;
    uint32_t rounded = trunc;
    if (round_bit != 0u && (sticky || (trunc & 1u) != 0u)) {
        rounded += 1u;
        if (rounded >= 0x400u) {
            if (new_exp < 30) return sign | ((uint32_t)(new_exp + 1) << 10);
            return sign | 0x7C00u;
        }
    }
    return sign | ((uint32_t)new_exp << 10) | rounded;
}

/* IEEE round-to-nearest-even narrowing (what a native f16() cast does,
 * fp_quantized.wgsl:383-389).                                                        */
uint32_t orc_f32_to_f16_rne(float val) {
    _Float16 h = (_Float16)val;
    uint16_t u; memcpy(&u, &h, 2);
    return u;
}

/* bf16 does not occur in the reference (no "bf16" anywhere under kernels/); the
 * build's definition is IEEE round-to-nearest-even of the f32 value.                */
uint32_t orc_f32_to_bf16_rne(float val) {
    uint32_t u = f32_bits(val);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x7FFFFFu)) return (u >> 16) | 0x40u;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return u >> 16;
}
float orc_bf16_bits_to_f32(uint32_t bits) { return bits_f32(bits << 16); }

static inline float load_as_f32(const void* p, size_t i, int dtype) {
    switch (dtype) {
        case ORC_F32:  return ((const float*)p)[i];
        case ORC_F16:  return orc_f16_bits_to_f32(((const uint16_t*)p)[i]);
        default:       return orc_bf16_bits_to_f32(((const uint16_t*)p)[i]);
    }
}
static inline float round_to(float v, int dtype) {
    switch (dtype) {
        case ORC_F32:  return v;
        case ORC_F16:  return orc_f16_bits_to_f32(orc_f32_to_f16_rne(v));
        default:       return orc_bf16_bits_to_f32(orc_f32_to_bf16_rne(v));
    }
}
static inline void store_as(void* p, size_t i, float v, int dtype) {
    switch (dtype) {
        case ORC_F32:  ((float*)p)[i] = v; break;
        case ORC_F16:  ((uint16_t*)p)[i] = (uint16_t)orc_f32_to_f16_rne(v); break;
        default:       ((uint16_t*)p)[i] = (uint16_t)orc_f32_to_bf16_rne(v); break;
    }
}

/* ------------------------------------------------------------------------------------
 * Whole-matrix unpack and dequantize
 *   W int4 [N, K/2] bytes, low nibble first; W int8 [N, K]
 *   scales [N, G]; zeros [N, ceil(G/2)] nibbles low first, or NULL (symmetric)
 *   group of element (n, k) = (n*K + k) / group  (quantized_nax.wgsl:587-589), which
 *   is column k/group of row n because K % group == 0.
 * ---------------------------------------------------------------------------------- */

static inline int32_t zero_point_of(const uint8_t* zeros, int bits, size_t n, size_t g, size_t G) {
    if (!zeros) return bits == 4 ? 8 : 0;        /* symmetric: quantized_nax.wgsl:105-112 */
    size_t zstride = (G + 1) / 2;
    uint8_t b = zeros[n * zstride + g / 2];
    return (int32_t)((b >> ((g & 1u) * 4u)) & 0xFu);
}

/* Integer q - zp for one row (R1/R2/R3 of the scope table). */
static void unpack_row(int bits, int group, const uint8_t* w, const uint8_t* zeros,
                       size_t n, size_t K, int32_t* out) {
    size_t G = K / (size_t)group;
    if (bits == 4) {
        const uint8_t* row = w + n * (K / 2);
        for (size_t o = 0; o < K / 8; o++) {
            uint32_t word;
            memcpy(&word, row + o * 4, 4);       /* little-endian u32, as the WGSL array<u32> */
            int32_t zp = zero_point_of(zeros, 4, n, (o * 8) / (size_t)group, G);
            orc_unpack_int4_asym_x8(word, zp, out + o * 8);
        }
    } else {
        const uint8_t* row = w + n * K;
        for (size_t o = 0; o < K / 4; o++) {
            uint32_t word;
            memcpy(&word, row + o * 4, 4);
            orc_unpack_int8_x4(word, out + o * 4);
        }
    }
}

int orc_qunpack(int N, int K, int bits, int group, const uint8_t* w, const uint8_t* zeros, int8_t* out) {
    if (K % group || K % 8) return -1;
    #pragma omp parallel
    {
        int32_t* tmp = (int32_t*)malloc((size_t)K * sizeof(int32_t));
        #pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            unpack_row(bits, group, w, zeros, (size_t)n, (size_t)K, tmp);
            for (int k = 0; k < K; k++) out[(size_t)n * K + k] = (int8_t)tmp[k];
        }
        free(tmp);
    }
    return 0;
}

/* dequantize_nax_int4_asym (:312-330) / dequantize_nax_int8_group symmetric branch
 * (:364-381): output = f32(q_vals[i]) * gs.scale -- integer subtract first, then ONE
 * f32 multiply.  w_round then optionally rounds the f32 weight once more to f16/bf16. */
static void dequant_row(int bits, int group, const uint8_t* w, const void* scales, int s_dtype,
                        const uint8_t* zeros, size_t n, size_t K, int w_round,
                        int32_t* itmp, float* out) {
    size_t G = K / (size_t)group;
    unpack_row(bits, group, w, zeros, n, K, itmp);
    for (size_t k = 0; k < K; k++) {
        float scale = load_as_f32(scales, n * G + k / (size_t)group, s_dtype);
        float v = (float)itmp[k] * scale;
        out[k] = round_to(v, w_round);
    }
}

int orc_qdequant(int N, int K, int bits, int group, const uint8_t* w, const void* scales, int s_dtype,
                 const uint8_t* zeros, void* out, int out_dtype) {
    if (K % group || K % 8) return -1;
    #pragma omp parallel
    {
        int32_t* itmp = (int32_t*)malloc((size_t)K * sizeof(int32_t));
        float* ftmp = (float*)malloc((size_t)K * sizeof(float));
        #pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            dequant_row(bits, group, w, scales, s_dtype, zeros, (size_t)n, (size_t)K, ORC_F32, itmp, ftmp);
            for (int k = 0; k < K; k++) store_as(out, (size_t)n * K + k, ftmp[k], out_dtype);
        }
        free(itmp); free(ftmp);
    }
    return 0;
}

/* ------------------------------------------------------------------------------------
 * y[M,N] = x[M,K] . dequant(W[N,K])^T
 *
 * matmul_nax_grouped, quantized_nax.wgsl:568-626: each output element is
 * "sum += tile_a[..k] * tile_b[k..]" over k ascending, f32.  (The shader's operand
 * order is C[Mw,Nact] = W . A with the weights on the left, :583-610; that is the
 * same contraction with Mw = N and Nact = M.)  The shader hard-wires the symmetric
 * int4 unpack (:594); the asymmetric and int8 cases use the dequantize functions
 * cited above for the weight value.
 *
 * acc_mode 0: f32, strictly ascending k (the shader's order)
 *          1: f32, k split into 16 interleaved partial sums (vectorisable; used only
 *             as the timed CPU baseline)
 *          2: f64 accumulation of the same f32 products' exact values (tie-breaker:
 *             shows which f32 result is nearer the exact sum)
 * w_round: ORC_F32 keeps weights in f32; ORC_BF16/ORC_F16 round them once more first
 *          (the tensor-core prefill path multiplies 16-bit operands).
 * threads <= 0 uses every core.
 * ---------------------------------------------------------------------------------- */
int orc_qmatmul(int M, int N, int K, int bits, int group,
                const void* x, int x_dtype,
                const uint8_t* w, const void* scales, int s_dtype, const uint8_t* zeros,
                void* y, int y_dtype, int w_round, int acc_mode, int threads) {
    if (M <= 0 || N <= 0 || K <= 0 || K % group || K % 8) return -1;
    if (bits != 4 && bits != 8) return -1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
    else omp_set_num_threads(omp_get_num_procs());
#endif
    /* widen x once: xt[k*M + m] so that the inner loop over m is contiguous */
    float* xt = (float*)malloc((size_t)M * K * sizeof(float));
    if (!xt) return -2;
    for (int m = 0; m < M; m++)
        for (int k = 0; k < K; k++)
            xt[(size_t)k * M + m] = load_as_f32(x, (size_t)m * K + k, x_dtype);

    #pragma omp parallel
    {
        int32_t* itmp = (int32_t*)malloc((size_t)K * sizeof(int32_t));
        float* wrow = (float*)malloc((size_t)K * sizeof(float));
        float* acc = (float*)malloc((size_t)M * sizeof(float));
        double* acc64 = (double*)malloc((size_t)M * sizeof(double));
        #pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            dequant_row(bits, group, w, scales, s_dtype, zeros, (size_t)n, (size_t)K, w_round, itmp, wrow);
            if (acc_mode == 2) {
                for (int m = 0; m < M; m++) acc64[m] = 0.0;
                for (int k = 0; k < K; k++) {
                    double wk = (double)wrow[k];
                    const float* xk = xt + (size_t)k * M;
                    for (int m = 0; m < M; m++) acc64[m] += wk * (double)xk[m];
                }
                for (int m = 0; m < M; m++) store_as(y, (size_t)m * N + n, (float)acc64[m], y_dtype);
            } else if (acc_mode == 1 && M == 1) {
                float part[16] = {0};
                int k = 0;
                for (; k + 16 <= K; k += 16)
                    for (int j = 0; j < 16; j++) part[j] += wrow[k + j] * xt[k + j];
                for (; k < K; k++) part[k & 15] += wrow[k] * xt[k];
                float s = 0.0f;
                for (int j = 0; j < 16; j++) s += part[j];
                store_as(y, (size_t)n, s, y_dtype);
            } else {
                for (int m = 0; m < M; m++) acc[m] = 0.0f;
                for (int k = 0; k < K; k++) {
                    float wk = wrow[k];
                    const float* xk = xt + (size_t)k * M;
                    for (int m = 0; m < M; m++) acc[m] += wk * xk[m];   /* ascending k per (m,n) */
                }
                for (int m = 0; m < M; m++) store_as(y, (size_t)m * N + n, acc[m], y_dtype);
            }
        }
        free(itmp); free(wrow); free(acc); free(acc64);
    }
    free(xt);
    return 0;
}

/* silu, kernels/wgsl/steel/gemm/steel_gemm_fused.wgsl:91-94: x / (1 + exp(-x)). */
float orc_silu(float x) { return x / (1.0f + expf(-x)); }

/* h[m, i] = silu(gate[m, i]) * up[m, i] where gu = [gate | up] on the column axis
 * (steel_gemm_silu_mul reads `up` at column offset +N, steel_gemm_fused.wgsl:525,
 * and combines at :553-555).  gu is [M, 2*I]; h is [M, I]; both of dtype `dtype`
 * (values are widened to f32, combined, and narrowed once).                          */
int orc_swiglu(int M, int I, const void* gu, int gu_dtype, void* h, int h_dtype) {
    for (int m = 0; m < M; m++)
        for (int i = 0; i < I; i++) {
            float g = load_as_f32(gu, (size_t)m * 2 * I + i, gu_dtype);
            float u = load_as_f32(gu, (size_t)m * 2 * I + I + i, gu_dtype);
            store_as(h, (size_t)m * I + i, orc_silu(g) * u, h_dtype);
        }
    return 0;
}

int orc_num_procs(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------
 * Quantize side: f32 matrix -> group statistics -> packed integers
 * ---------------------------------------------------------------------------------- */

#define ORC_NAX_INT4_SYM  0     /* quantized_nax.wgsl:31-34 */
#define ORC_NAX_INT4_ASYM 1
#define ORC_NAX_INT8_SYM  2
/* NOT a reference format: asymmetric int4 with the zero-point applied before the clamp,
 * clamp(round(v / scale) + zp, 0, 15) -- the library's LUX_QQUANT_FLAG_SHIFTED extension. */
#define ORC_EXT_INT4_ASYM_SHIFTED 101

/* GroupScale, quantized_nax.wgsl:49-54 */
typedef struct { float scale; int32_t zero_point; float group_min; float group_max; } OrcGroupScale;

/* WGSL i32(f32): truncation toward zero, out-of-range values clamp to the i32 range.  The
 * result for NaN is indeterminate in WGSL; 0 is used here (UNPINNED choice, reached only by a
 * group of zeros in the asymmetric format: -0/0). */
static int32_t wgsl_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}
static int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* compute_group_scales, quantized_nax.wgsl:157-232.  Groups are runs of group_size consecutive
 * elements of the flat array (:165-166); with a row-major [N, K] matrix and K % group_size == 0
 * they lie along K inside a row.  min / max start from +-1e30 (:169-170).  round() is
 * round-half-to-even.  The zero-point is computed BEFORE the "scale == 0 -> 1" guard (:217-218
 * vs :227), so a constant group divides by zero there; IEEE results are used. */
int orc_compute_group_scales(const float* in, size_t size, int group_size, int format, OrcGroupScale* out) {
    if (group_size <= 0 || format < 0 || format > 2) return -1;
    const size_t groups = (size + (size_t)group_size - 1) / (size_t)group_size;
    #pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; g++) {
        const size_t b = g * (size_t)group_size;
        const size_t e = b + (size_t)group_size < size ? b + (size_t)group_size : size;
        float mx = -1e30f, mn = 1e30f;
        for (size_t i = b; i < e; i++) {
            const float v = in[i];
            mx = mx > v ? mx : v;       /* max(local_max, val) */
            mn = mn < v ? mn : v;
        }
        float scale;
        int32_t zp;
        if (format == ORC_NAX_INT4_SYM || format == ORC_NAX_INT8_SYM) {
            const float amax = fabsf(mx) > fabsf(mn) ? fabsf(mx) : fabsf(mn);
            scale = format == ORC_NAX_INT4_SYM ? amax / 7.0f : amax / 127.0f;
            zp = 0;
        } else {
            const float range = mx - mn;
            scale = range / 15.0f;
            zp = clampi(wgsl_i32(rintf(-mn / scale)), 0, 15);
        }
        if (scale == 0.0f) scale = 1.0f;
        out[g].scale = scale; out[g].zero_point = zp; out[g].group_min = mn; out[g].group_max = mx;
    }
    return 0;
}

/* quantize_nax_int4_sym (:236-259), quantize_nax_int4_asym (:288-310) with
 * pack_nax_int4_asym_x8 (:115-122), quantize_nax_int8_group symmetric branch (:336-362) with
 * pack_nax_int8_x4 (:135-140).  `size` must be a multiple of 8 (int4) or 4 (int8).
 *
 * The asymmetric int4 shader is restated AS WRITTEN: q = clamp(i32(round(val / scale)), 0, 15)
 * - zp (:303), and the pack adds zp back and clamps again (:118), so the stored nibble is
 * clamp(round(val / scale), 0, 15).  The zero-point never shifts the value before the clamp:
 * negative inputs are stored as 0 and the round trip through dequantize (nibble - zp) * scale
 * is offset by -zp * scale.  See tests/test_oracle_quantize.py for the characterisation. */
int orc_quantize(const float* in, size_t size, int group_size, int format, const OrcGroupScale* gs, uint32_t* out_packed) {
    if (group_size <= 0 || format < 0 || (format > 2 && format != ORC_EXT_INT4_ASYM_SHIFTED)) return -1;
    const int per = format == ORC_NAX_INT8_SYM ? 4 : 8;
    if (size % (size_t)per) return -1;
    #pragma omp parallel for schedule(static)
    for (size_t w = 0; w < size / (size_t)per; w++) {
        const size_t e0 = w * (size_t)per;
        const OrcGroupScale g = gs[e0 / (size_t)group_size];
        uint32_t word = 0;
        for (int i = 0; i < per; i++) {
            const float scaled = rintf(in[e0 + (size_t)i] / g.scale);
            if (format == ORC_NAX_INT4_SYM) {
                const int32_t q = clampi(wgsl_i32(scaled), -8, 7);
                word |= ((uint32_t)(q + 8) & 0xFu) << (4 * i);
            } else if (format == ORC_EXT_INT4_ASYM_SHIFTED) {
                const int32_t q = clampi(clampi(wgsl_i32(scaled), -32, 32) + g.zero_point, 0, 15);
                word |= ((uint32_t)q & 0xFu) << (4 * i);
            } else if (format == ORC_NAX_INT4_ASYM) {
                const int32_t q = clampi(wgsl_i32(scaled), 0, 15) - g.zero_point;
                word |= ((uint32_t)clampi(q + g.zero_point, 0, 15) & 0xFu) << (4 * i);
            } else {
                const int32_t q = clampi(wgsl_i32(scaled), -128, 127);
                word |= ((uint32_t)q & 0xFFu) << (8 * i);
            }
        }
        out_packed[w] = word;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Activation-quantized integer path (gpu/quantized.wgsl, gpu/quantized_nax.wgsl)
 * ---------------------------------------------------------------------------------- */

/* unpack_int4x8, kernels/wgsl/gpu/quantized.wgsl:150-158: TWO'S COMPLEMENT nibbles ("if (val >= 8)
 * val -= 16"), unlike the +8 offset of the weight-only format above. */
void orc_unpack_int4x8_twos(uint32_t packed, int32_t out[8]) {
    for (uint32_t i = 0; i < 8u; i++) {
        int32_t val = (int32_t)((packed >> (i * 4u)) & 0xFu);
        if (val >= 8) val -= 16;
        out[i] = val;
    }
}

/* matmul_int8 (quantized.wgsl:497-555) and matmul_int4_int8 (:590-647): C[M,N] (i32) = A[M,K] . B[K,N].
 * A is read as element flat_idx = row*K + col of a flat packed array (four int8 or eight int4 per
 * u32); B is int8, row-major [K, N].  a_bits = 8 or 4. */
int orc_matmul_int(int M, int N, int K, int a_bits, const uint8_t* a, const int8_t* b, int32_t* c) {
    if (M <= 0 || N <= 0 || K <= 0 || (a_bits != 4 && a_bits != 8)) return -1;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < M; r++)
        for (int col = 0; col < N; col++) {
            int32_t sum = 0;
            for (int k = 0; k < K; k++) {
                const size_t flat = (size_t)r * K + k;
                int32_t av;
                if (a_bits == 8) {
                    av = (int32_t)((a[flat]) & 0xFFu);
                    if (av >= 128) av -= 256;                    /* unpack_int8x4, :167-178 */
                } else {
                    av = (int32_t)((a[flat >> 1] >> ((flat & 1) * 4)) & 0xFu);
                    if (av >= 8) av -= 16;
                }
                sum += av * (int32_t)b[(size_t)k * N + col];
            }
            c[(size_t)r * N + col] = sum;
        }
    return 0;
}

/* requantize_int32_to_int8, quantized.wgsl:573-588 (the output array holds i32 values in [-128, 127]) */
int orc_requantize_int32_to_int8(const int32_t* in, int32_t* out, size_t n, float input_scale, float output_scale, int32_t zp) {
    for (size_t i = 0; i < n; i++) {
        const float v = (float)in[i] * input_scale;
        const float r = rintf(v / output_scale) + (float)zp;
        out[i] = clampi(wgsl_i32(r), -128, 127);
    }
    return 0;
}

/* dynamic_quantize, quantized_nax.wgsl:644-718: ONE scale for the whole tensor, max|x| / 127 (bits 8)
 * or / 7 (bits 4), 1 if that is 0; q = clamp(i32(round(x / scale)), MIN, MAX); int8 packed four per
 * word, int4 as pack_nax_int4_sym_x8 (stored nibble = q + 8, padding elements q = 0).  `out` holds
 * n bytes (bits 8) or ceil(n / 2) bytes (bits 4). */
int orc_dynamic_quantize(const float* x, size_t n, int bits, uint8_t* out, float* scale_out) {
    if (bits != 4 && bits != 8) return -1;
    float mx = 0.0f;
    for (size_t i = 0; i < n; i++) { const float a = fabsf(x[i]); mx = mx > a ? mx : a; }
    float scale = bits == 4 ? mx / 7.0f : mx / 127.0f;
    if (scale == 0.0f) scale = 1.0f;
    *scale_out = scale;
    if (bits == 8) {
        for (size_t i = 0; i < n; i++) out[i] = (uint8_t)(clampi(wgsl_i32(rintf(x[i] / scale)), -128, 127) & 0xFF);
    } else {
        for (size_t b = 0; b < (n + 1) / 2; b++) {
            const int32_t lo = clampi(wgsl_i32(rintf(x[2 * b] / scale)), -8, 7);
            const int32_t hi = 2 * b + 1 < n ? clampi(wgsl_i32(rintf(x[2 * b + 1] / scale)), -8, 7) : 0;
            out[b] = (uint8_t)(((uint32_t)(lo + 8) & 0xFu) | (((uint32_t)(hi + 8) & 0xFu) << 4));
        }
    }
    return 0;
}
