/*
 * cpu_baseline.c -- the timed CPU baseline of the int4 g128 quantized matmul.
 *
 * TEST / BENCHMARK INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file.  qmatmul_oracle.c is the parity oracle: it follows the shader text
 * operation by operation and is built without contraction or vectorisation-friendly
 * reordering, which makes it a poor baseline to quote a speed-up against.  This file is the
 * same arithmetic written the way a CPU backend would write it, and is what bench.py times:
 *
 *   w = f32(q - zp) * scale          dequantize_nax_int4_asym, quantized_nax.wgsl:312-330
 *   y = sum_k w * x, f32 accumulate  matmul_nax_grouped, quantized_nax.wgsl:577-621
 *   h = silu(gate) * up              steel_gemm_silu_mul, steel_gemm_fused.wgsl:91-94, 452-558
 *
 * with the scale and the zero-point hoisted out of the group (sum_k (q - zp) x_k * s =
 * s * (sum_k q x_k - zp * sum_k x_k)), x widened and de-interleaved once per call, 8-wide
 * partial sums per group, OpenMP over output rows.  Its results differ from the oracle's only in
 * summation order; tests/test_oracle_properties.py holds it to the oracle within 1e-3.
 *
 * Build: oracle/Makefile (gcc -O3 -march=x86-64-v3 -fopenmp; x86-64-v3 rather than native
 * because the library is built on one machine and timed on another).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f;       /* round to nearest even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

int cpub_num_procs(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* y[M, N] (f32) = x[M, K] (f16) . dequant(W[N, K])^T, int4 g128 asymmetric (zeros may be NULL:
 * zero-point 8).  threads <= 0: every core. */
int cpub_qmatmul_i4_f32out(int M, int N, int K, const uint16_t* x, const uint8_t* w, const uint16_t* scales,
                           const uint8_t* zeros, float* y, int threads) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 128) return -1;
    const int G = K / 128, ZS = (G + 1) / 2;
#ifdef _OPENMP
    omp_set_num_threads(threads > 0 ? threads : omp_get_num_procs());
#endif
    /* x widened once, even and odd k apart (a byte holds k = 2j in its low nibble, 2j + 1 in
     * its high nibble), plus the per-group sums for the zero-point term */
    float* xe = (float*)malloc((size_t)M * K / 2 * sizeof(float));
    float* xo = (float*)malloc((size_t)M * K / 2 * sizeof(float));
    float* xs = (float*)malloc((size_t)M * G * sizeof(float));
    if (!xe || !xo || !xs) { free(xe); free(xo); free(xs); return -2; }
    for (int m = 0; m < M; m++)
        for (int g = 0; g < G; g++) {
            float s = 0.0f;
            for (int j = 0; j < 64; j++) {
                const float a = h2f(x[(size_t)m * K + g * 128 + 2 * j]), b = h2f(x[(size_t)m * K + g * 128 + 2 * j + 1]);
                xe[(size_t)m * K / 2 + g * 64 + j] = a;
                xo[(size_t)m * K / 2 + g * 64 + j] = b;
                s += a + b;
            }
            xs[(size_t)m * G + g] = s;
        }
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint8_t* row = w + (size_t)n * (K / 2);
        for (int m = 0; m < M; m++) {
            const float* xem = xe + (size_t)m * K / 2;
            const float* xom = xo + (size_t)m * K / 2;
            float acc = 0.0f;
            for (int g = 0; g < G; g++) {
                const uint8_t* b = row + g * 64;
                float s0 = 0.0f, s1 = 0.0f;
                #pragma omp simd reduction(+ : s0, s1)
                for (int j = 0; j < 64; j++) {
                    s0 += (float)(b[j] & 15) * xem[g * 64 + j];
                    s1 += (float)(b[j] >> 4) * xom[g * 64 + j];
                }
                const int zp = zeros ? (zeros[(size_t)n * ZS + (g >> 1)] >> ((g & 1) * 4)) & 15 : 8;
                acc += h2f(scales[(size_t)n * G + g]) * ((s0 + s1) - (float)zp * xs[(size_t)m * G + g]);
            }
            y[(size_t)m * N + n] = acc;
        }
    }
    free(xe); free(xo); free(xs);
    return 0;
}

/* f16 output of the same product */
int cpub_qmatmul_i4(int M, int N, int K, const uint16_t* x, const uint8_t* w, const uint16_t* scales,
                    const uint8_t* zeros, uint16_t* y, int threads) {
    float* t = (float*)malloc((size_t)M * N * sizeof(float));
    if (!t) return -2;
    const int rc = cpub_qmatmul_i4_f32out(M, N, K, x, w, scales, zeros, t, threads);
    if (rc == 0)
        for (size_t i = 0; i < (size_t)M * N; i++) y[i] = f2h(t[i]);
    free(t);
    return rc;
}

/* The Llama FFN: h = silu(x . gate^T) * (x . up^T) narrowed to f16 (gate rows then up rows in
 * w_gu, 2*I rows), y = h . down^T, f16 out. */
int cpub_mlp_i4(int M, int K, int I, int H, const uint16_t* x, const uint8_t* w_gu, const uint16_t* s_gu,
                const uint8_t* z_gu, const uint8_t* w_dn, const uint16_t* s_dn, const uint8_t* z_dn, uint16_t* y,
                int threads) {
    float* gu = (float*)malloc((size_t)M * 2 * I * sizeof(float));
    uint16_t* h = (uint16_t*)malloc((size_t)M * I * sizeof(uint16_t));
    if (!gu || !h) { free(gu); free(h); return -2; }
    int rc = cpub_qmatmul_i4_f32out(M, 2 * I, K, x, w_gu, s_gu, z_gu, gu, threads);
    if (rc == 0) {
        for (int m = 0; m < M; m++)
            for (int i = 0; i < I; i++) {
                const float g = gu[(size_t)m * 2 * I + i], u = gu[(size_t)m * 2 * I + I + i];
                h[(size_t)m * I + i] = f2h(g / (1.0f + expf(-g)) * u);
            }
        rc = cpub_qmatmul_i4(M, H, I, h, w_dn, s_dn, z_dn, y, threads);
    }
    free(gu); free(h);
    return rc;
}
