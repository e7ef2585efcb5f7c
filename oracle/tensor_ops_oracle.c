/*
 * tensor_ops_oracle.c -- CPU restatement of the f32 shaders that back the tensor slots either side
 * of a linear layer (element-wise ops, transpose, softmax, log-softmax, layer norm, RMS norm).
 *
 * TEST INFRASTRUCTURE ONLY, like qmatmul_oracle.c: nothing in the shipped library links or calls it.
 * PARITY UNPINNED: luxcpp/webgpu's tests never run these shaders on data (its f32 tests cover
 * add / sub / mul / matmul only), so the functions follow the shader text; each cites its lines
 * (paths inside luxcpp/webgpu).  Built without contraction, so "a += b * c" is two roundings.
 *
 * The row-wise shaders reduce with one 256-thread workgroup per row: thread t accumulates
 * elements t, t + 256, ... and a binary tree (stride 128, 64, ... 1) combines the 256 partials.
 * That ORDER is restated here, because it decides the f32 sums.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#define WG 256

/* kernels/wgsl/gpu/unary.wgsl: neg :47, abs :54, sqrt :68, exp :109, log :137, tanh :235, relu :306,
 * gelu :347-355 (tanh form), sigmoid :367-372, silu :375-381; copy is the identity. */
enum { T_EXP, T_LOG, T_SQRT, T_NEG, T_ABS, T_TANH, T_SIGMOID, T_RELU, T_GELU, T_SILU, T_COPY };

int orc_unary_f32(int op, const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        const float x = in[i];
        float y;
        switch (op) {
            case T_EXP: y = expf(x); break;
            case T_LOG: y = logf(x); break;
            case T_SQRT: y = sqrtf(x); break;
            case T_NEG: y = -x; break;
            case T_ABS: y = fabsf(x); break;
            case T_TANH: y = tanhf(x); break;
            case T_SIGMOID: y = 1.0f / (1.0f + expf(-x)); break;
            case T_RELU: y = x > 0.0f ? x : 0.0f; break;
            case T_GELU: {
                const float c = 0.7978845608028654f;
                const float inner = c * (x + 0.044715f * x * x * x);
                y = 0.5f * x * (1.0f + tanhf(inner));
                break;
            }
            case T_SILU: y = x / (1.0f + expf(-x)); break;
            case T_COPY: y = x; break;
            default: return -1;
        }
        out[i] = y;
    }
    return 0;
}

/* transpose_2d, kernels/wgsl/gpu/copy.wgsl:283-293 */
int orc_transpose_f32(const float* in, float* out, int rows, int cols) {
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) out[(size_t)c * rows + r] = in[(size_t)r * cols + c];
    return 0;
}

static float tree_sum(float* p) {
    for (int s = WG / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) p[t] = p[t] + p[t + s];
    return p[0];
}
static float tree_max(float* p) {
    for (int s = WG / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) p[t] = p[t] > p[t + s] ? p[t] : p[t + s];
    return p[0];
}
static float safe_exp(float x) {                       /* softmax.wgsl:53-55, logsumexp.wgsl:55-57 */
    x = x < -88.0f ? -88.0f : (x > 88.0f ? 88.0f : x);
    return expf(x);
}

/* softmax, kernels/wgsl/gpu/softmax.wgsl:61-136 (temperature 1); log_softmax,
 * kernels/wgsl/gpu/logsumexp.wgsl:151-221 (stride 1) */
int orc_softmax_f32(const float* in, float* out, size_t batch, size_t dim, int log_form) {
    float part[WG];
    for (size_t b = 0; b < batch; b++) {
        const float* x = in + b * dim;
        float* y = out + b * dim;
        for (int t = 0; t < WG; t++) {
            float m = -3.402823466e+38f;
            for (size_t i = (size_t)t; i < dim; i += WG) m = m > x[i] ? m : x[i];
            part[t] = m;
        }
        const float mx = tree_max(part);
        for (int t = 0; t < WG; t++) {
            float s = 0.0f;
            for (size_t i = (size_t)t; i < dim; i += WG) s += safe_exp(x[i] - mx);
            part[t] = s;
        }
        const float sum = tree_sum(part);
        if (log_form) {
            const float lse = logf(sum);
            for (size_t i = 0; i < dim; i++) y[i] = x[i] - mx - lse;
        } else {
            const float inv = 1.0f / sum;
            for (size_t i = 0; i < dim; i++) y[i] = safe_exp(x[i] - mx) * inv;
        }
    }
    return 0;
}

/* layer_norm, kernels/wgsl/gpu/layer_norm.wgsl:97-159: variance = E[x^2] - mean^2,
 * y = gamma * ((x - mean) * rstd) + beta */
int orc_layer_norm_f32(const float* in, const float* gamma, const float* beta, float* out, size_t batch, size_t dim, float eps) {
    float p1[WG], p2[WG];
    for (size_t b = 0; b < batch; b++) {
        const float* x = in + b * dim;
        float* y = out + b * dim;
        for (int t = 0; t < WG; t++) {
            float s1 = 0.0f, s2 = 0.0f;
            for (size_t i = (size_t)t; i < dim; i += WG) { s1 += x[i]; s2 += x[i] * x[i]; }
            p1[t] = s1; p2[t] = s2;
        }
        const float mean = tree_sum(p1) / (float)dim;
        const float var = tree_sum(p2) / (float)dim - mean * mean;
        const float rstd = 1.0f / sqrtf(var + eps);
        for (size_t i = 0; i < dim; i++) y[i] = gamma[i] * ((x[i] - mean) * rstd) + beta[i];
    }
    return 0;
}

/* rms_norm, kernels/wgsl/gpu/rms_norm.wgsl:54-113: y = x * (1 / sqrt(mean(x^2) + eps)) * gamma */
int orc_rms_norm_f32(const float* in, const float* gamma, float* out, size_t batch, size_t dim, float eps) {
    float p2[WG];
    for (size_t b = 0; b < batch; b++) {
        const float* x = in + b * dim;
        float* y = out + b * dim;
        for (int t = 0; t < WG; t++) {
            float s2 = 0.0f;
            for (size_t i = (size_t)t; i < dim; i += WG) s2 += x[i] * x[i];
            p2[t] = s2;
        }
        const float rms = 1.0f / sqrtf(tree_sum(p2) / (float)dim + eps);
        for (size_t i = 0; i < dim; i++) y[i] = x[i] * rms * gamma[i];
    }
    return 0;
}
