// The f32 tensor slots either side of a linear layer, which the WebGPU plugin leaves unwired
// (luxcpp/webgpu src/webgpu_plugin.cpp:4044-4072 are nullptr) although its shader library holds
// them: element-wise unary ops and division, copy, transpose, softmax, log-softmax, layer norm and
// RMS norm, plus SiLU as an extension symbol (the vtable has no slot for it).  Arithmetic follows
// the shaders:
//
//   unary ops ............ kernels/wgsl/gpu/unary.wgsl:47-58 (neg, abs), 68-72 (sqrt), 109-113 (exp),
//                          137-141 (log), 235-239 (tanh), 306-310 (relu), 347-355 (gelu, tanh form),
//                          367-372 (sigmoid), 375-381 (silu)
//   transpose ............ kernels/wgsl/gpu/copy.wgsl:283-293
//   softmax .............. kernels/wgsl/gpu/softmax.wgsl:53-136 (temperature 1; exp clamped to +-88)
//   log-softmax .......... kernels/wgsl/gpu/logsumexp.wgsl:151-221
//   layer norm ........... kernels/wgsl/gpu/layer_norm.wgsl:97-159 (variance = E[x^2] - mean^2)
//   RMS norm ............. kernels/wgsl/gpu/rms_norm.wgsl:54-113 (x * rsqrt(mean(x^2) + eps) * gamma)
//
// The row-wise kernels keep the shaders' reduction ORDER -- one 256-thread group per row, each
// thread a strided partial, then a binary tree over the 256 partials -- so that their sums are
// the same f32 numbers a conforming run of the shader produces; the loads are what differs
// (the row is read once into registers when it fits, not three times).  All of these are
// HBM-bound: 4 bytes read and 4 written per element.
#include "common.cuh"

#include <algorithm>

namespace luxcuda {

namespace {

constexpr int ROW_THREADS = 256;       // the shaders' workgroup size: the reduction order depends on it
constexpr int ROW_CACHE = 16;          // elements per thread kept in registers (rows up to 4096)

enum UnaryOp { U_EXP, U_LOG, U_SQRT, U_NEG, U_ABS, U_TANH, U_SIGMOID, U_RELU, U_GELU, U_SILU, U_COPY };

template <int OP>
__device__ __forceinline__ float unary(float x) {
    switch (OP) {
        case U_EXP: return expf(x);
        case U_LOG: return logf(x);
        case U_SQRT: return sqrtf(x);
        case U_NEG: return -x;
        case U_ABS: return fabsf(x);
        case U_TANH: return tanhf(x);
        case U_SIGMOID: return __fdiv_rn(1.0f, 1.0f + expf(-x));
        case U_RELU: return fmaxf(x, 0.0f);
        case U_GELU: {
            const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
            return 0.5f * x * (1.0f + tanhf(inner));
        }
        case U_SILU: return __fdiv_rn(x, 1.0f + expf(-x));
        default: return x;
    }
}

template <int OP>
__global__ void __launch_bounds__(256) lux_unary_f32(const float* __restrict__ in, float* __restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n4 = n / 4;
    const bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (vec) {
        for (; i < n4; i += stride) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(in) + i);
            reinterpret_cast<float4*>(out)[i] = make_float4(unary<OP>(v.x), unary<OP>(v.y), unary<OP>(v.z), unary<OP>(v.w));
        }
        for (size_t j = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) out[j] = unary<OP>(in[j]);
    } else {
        for (; i < n; i += stride) out[i] = unary<OP>(in[i]);
    }
}

__global__ void __launch_bounds__(256) lux_div_f32(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = __fdiv_rn(a[i], b[i]);
}

// out[c, r] = in[r, c] through a 32 x 33 tile: coalesced on both sides
__global__ void __launch_bounds__(256) lux_transpose_f32(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = in[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) out[(size_t)c * rows + r] = tile[threadIdx.x][j];
    }
}

// The same for matrices made of whole 64 x 64 tiles with 16-byte aligned rows: 16-byte loads and
// stores, 256-byte runs on both sides (the 32 x 32 version moves 128-byte runs with 4-byte accesses)
__global__ void __launch_bounds__(256) lux_transpose64_f32(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float tile[64][65];
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64, t = threadIdx.x;
    const int q = t & 15, j0 = t >> 4;                      // 16 threads per row of 64 floats, 16 rows per pass
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int j = j0 + 16 * p;
        const float4 v = __ldg(reinterpret_cast<const float4*>(in + (size_t)(r0 + j) * cols + c0) + q);
        tile[j][4 * q] = v.x; tile[j][4 * q + 1] = v.y; tile[j][4 * q + 2] = v.z; tile[j][4 * q + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int c = j0 + 16 * p;                          // output row c0 + c, elements r0 + 4 q .. + 3
        const float4 v = make_float4(tile[4 * q][c], tile[4 * q + 1][c], tile[4 * q + 2][c], tile[4 * q + 3][c]);
        *(reinterpret_cast<float4*>(out + (size_t)(c0 + c) * rows + r0) + q) = v;
    }
}

// the shaders' tree over 256 partials: stride 128, 64, ... 1; every thread ends up with element 0
template <bool MAX>
__device__ __forceinline__ float tree256(float v, float* sh) {
    const int t = threadIdx.x;
    sh[t] = v;
    __syncthreads();
#pragma unroll
    for (int s = ROW_THREADS / 2; s > 0; s >>= 1) {
        if (t < s) sh[t] = MAX ? fmaxf(sh[t], sh[t + s]) : sh[t] + sh[t + s];
        __syncthreads();
    }
    const float r = sh[0];
    __syncthreads();
    return r;
}

__device__ __forceinline__ float safe_exp(float x) { return expf(fminf(fmaxf(x, -88.0f), 88.0f)); }

// element i of the thread: column threadIdx.x + i * 256 (the shader's strided walk)
template <bool LOG>
__global__ void __launch_bounds__(ROW_THREADS) lux_softmax_f32(const float* __restrict__ in, float* __restrict__ out, int dim) {
    __shared__ float sh[ROW_THREADS];
    const float* x = in + (size_t)blockIdx.x * dim;
    float* y = out + (size_t)blockIdx.x * dim;
    const int t = threadIdx.x;
    float cache[ROW_CACHE];
    float mx = -3.402823466e+38f;
    int cnt = 0;
    for (int i = t; i < dim; i += ROW_THREADS, cnt++) {
        const float v = x[i];
        if (cnt < ROW_CACHE) cache[cnt] = v;
        mx = fmaxf(mx, v);
    }
    mx = tree256<true>(mx, sh);
    float sum = 0.0f;
    cnt = 0;
    for (int i = t; i < dim; i += ROW_THREADS, cnt++) sum += safe_exp((cnt < ROW_CACHE ? cache[cnt] : x[i]) - mx);
    sum = tree256<false>(sum, sh);
    cnt = 0;
    if (LOG) {
        const float lse = logf(sum);
        for (int i = t; i < dim; i += ROW_THREADS, cnt++) y[i] = (cnt < ROW_CACHE ? cache[cnt] : x[i]) - mx - lse;
    } else {
        const float inv = __fdiv_rn(1.0f, sum);
        for (int i = t; i < dim; i += ROW_THREADS, cnt++) y[i] = safe_exp((cnt < ROW_CACHE ? cache[cnt] : x[i]) - mx) * inv;
    }
}

template <bool LAYER>
__global__ void __launch_bounds__(ROW_THREADS) lux_norm_f32(const float* __restrict__ in, const float* __restrict__ gamma,
                                                           const float* __restrict__ beta, float* __restrict__ out, int dim, float eps) {
    __shared__ float sh[ROW_THREADS];
    const float* x = in + (size_t)blockIdx.x * dim;
    float* y = out + (size_t)blockIdx.x * dim;
    const int t = threadIdx.x;
    float cache[ROW_CACHE];
    float s1 = 0.0f, s2 = 0.0f;
    int cnt = 0;
    for (int i = t; i < dim; i += ROW_THREADS, cnt++) {
        const float v = x[i];
        if (cnt < ROW_CACHE) cache[cnt] = v;
        if (LAYER) s1 += v;
        s2 = __fadd_rn(s2, __fmul_rn(v, v));           // a rounded product then a rounded sum, as the shader text says
    }
    float mean = 0.0f;
    if (LAYER) mean = __fdiv_rn(tree256<false>(s1, sh), (float)dim);
    const float msq = __fdiv_rn(tree256<false>(s2, sh), (float)dim);
    const float r = LAYER ? __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fsub_rn(msq, __fmul_rn(mean, mean)), eps)))
                          : __fdiv_rn(1.0f, sqrtf(__fadd_rn(msq, eps)));
    cnt = 0;
    for (int i = t; i < dim; i += ROW_THREADS, cnt++) {
        const float v = cnt < ROW_CACHE ? cache[cnt] : x[i];
        if (LAYER) y[i] = __fadd_rn(__fmul_rn(gamma[i], __fmul_rn(__fsub_rn(v, mean), r)), beta[i]);
        else y[i] = __fmul_rn(__fmul_rn(v, r), gamma[i]);
    }
}

template <int OP>
LuxBackendError unary_op(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n, const char* what) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!ctx || !bi || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bi->size < n * 4 || bo->size < n * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((n / 4 + 255) / 256 + 1, (size_t)ctx->sm_count * 16);
    lux_unary_f32<OP><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)bi->ptr, (float*)bo->ptr, n);
    count_launch();
    return finish_op(ctx, false, what);
}

bool rows_ok(size_t batch, size_t dim) { return batch > 0 && dim > 0 && batch <= 0x7fffffffu && dim <= 0x7fffffffu; }

}  // namespace

LuxBackendError op_exp_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_EXP>(c, i, o, n, "op_exp_f32"); }
LuxBackendError op_log_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_LOG>(c, i, o, n, "op_log_f32"); }
LuxBackendError op_sqrt_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_SQRT>(c, i, o, n, "op_sqrt_f32"); }
LuxBackendError op_neg_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_NEG>(c, i, o, n, "op_neg_f32"); }
LuxBackendError op_abs_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_ABS>(c, i, o, n, "op_abs_f32"); }
LuxBackendError op_tanh_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_TANH>(c, i, o, n, "op_tanh_f32"); }
LuxBackendError op_sigmoid_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_SIGMOID>(c, i, o, n, "op_sigmoid_f32"); }
LuxBackendError op_relu_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_RELU>(c, i, o, n, "op_relu_f32"); }
LuxBackendError op_gelu_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_GELU>(c, i, o, n, "op_gelu_f32"); }
LuxBackendError op_copy_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_COPY>(c, i, o, n, "op_copy_f32"); }
LuxBackendError op_silu_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary_op<U_SILU>(c, i, o, n, "op_silu_f32"); }

LuxBackendError op_div_f32(LuxBackendContext* context, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n) {
    Context* ctx = as_ctx(context);
    Buffer *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
    if (!ctx || !ba || !bb || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (ba->size < n * 4 || bb->size < n * 4 || bo->size < n * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
    lux_div_f32<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)ba->ptr, (const float*)bb->ptr, (float*)bo->ptr, n);
    count_launch();
    return finish_op(ctx, false, "op_div_f32");
}

LuxBackendError op_transpose_f32(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* out, int rows, int cols) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!ctx || !bi || !bo || rows <= 0 || cols <= 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t bytes = (size_t)rows * cols * 4;
    if (bi->size < bytes || bo->size < bytes || bi->ptr == bo->ptr) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((rows + 31) / 32 > 65535) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    const bool whole = rows % 64 == 0 && cols % 64 == 0 && rows / 64 <= 65535 &&
                       ((reinterpret_cast<uintptr_t>(bi->ptr) | reinterpret_cast<uintptr_t>(bo->ptr)) & 15u) == 0;
    if (whole) lux_transpose64_f32<<<dim3(cols / 64, rows / 64), 256, 0, ctx->stream>>>((const float*)bi->ptr, (float*)bo->ptr, rows, cols);
    else lux_transpose_f32<<<dim3((cols + 31) / 32, (rows + 31) / 32), dim3(32, 8), 0, ctx->stream>>>((const float*)bi->ptr, (float*)bo->ptr, rows, cols);
    count_launch();
    return finish_op(ctx, false, "op_transpose_f32");
}

static LuxBackendError softmax_op(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim, bool log) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!ctx || !bi || !bo || !rows_ok(batch, dim)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bi->size < batch * dim * 4 || bo->size < batch * dim * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    if (log) lux_softmax_f32<true><<<(unsigned)batch, ROW_THREADS, 0, ctx->stream>>>((const float*)bi->ptr, (float*)bo->ptr, (int)dim);
    else lux_softmax_f32<false><<<(unsigned)batch, ROW_THREADS, 0, ctx->stream>>>((const float*)bi->ptr, (float*)bo->ptr, (int)dim);
    count_launch();
    return finish_op(ctx, false, log ? "op_log_softmax_f32" : "op_softmax_f32");
}
LuxBackendError op_softmax_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t batch, size_t dim) { return softmax_op(c, i, o, batch, dim, false); }
LuxBackendError op_log_softmax_f32(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t batch, size_t dim) { return softmax_op(c, i, o, batch, dim, true); }

LuxBackendError op_layer_norm_f32(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* gamma, LuxBackendBuffer* beta,
                                  LuxBackendBuffer* out, size_t batch, size_t dim, float eps) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bg = as_buf(gamma), *bb = as_buf(beta), *bo = as_buf(out);
    if (!ctx || !bi || !bg || !bb || !bo || !rows_ok(batch, dim)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bi->size < batch * dim * 4 || bo->size < batch * dim * 4 || bg->size < dim * 4 || bb->size < dim * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    lux_norm_f32<true><<<(unsigned)batch, ROW_THREADS, 0, ctx->stream>>>((const float*)bi->ptr, (const float*)bg->ptr, (const float*)bb->ptr,
                                                                        (float*)bo->ptr, (int)dim, eps);
    count_launch();
    return finish_op(ctx, false, "op_layer_norm_f32");
}

LuxBackendError op_rms_norm_f32(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* weight, LuxBackendBuffer* out,
                                size_t batch, size_t dim, float eps) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bg = as_buf(weight), *bo = as_buf(out);
    if (!ctx || !bi || !bg || !bo || !rows_ok(batch, dim)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bi->size < batch * dim * 4 || bo->size < batch * dim * 4 || bg->size < dim * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    lux_norm_f32<false><<<(unsigned)batch, ROW_THREADS, 0, ctx->stream>>>((const float*)bi->ptr, (const float*)bg->ptr, nullptr,
                                                                         (float*)bo->ptr, (int)dim, eps);
    count_launch();
    return finish_op(ctx, false, "op_rms_norm_f32");
}

}  // namespace luxcuda

extern "C" LuxBackendError lux_cuda_op_silu_f32(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n) {
    return luxcuda::op_silu_f32(ctx, in, out, n);
}
