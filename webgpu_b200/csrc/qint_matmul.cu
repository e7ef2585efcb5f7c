// The activation-quantized integer path: dynamic per-tensor quantization of activations, int8 x int8
// and int4 x int8 matmuls with int32 results, and requantization back to int8.  Exact integer
// arithmetic, so every result is bit-identical to the shaders these replace:
//
//   dynamic_quantize            luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:644-718
//   matmul_int8                 kernels/wgsl/gpu/quantized.wgsl:497-555   C[M,N] = A[M,K] . B[K,N], i32
//   requantize_int32_to_int8    kernels/wgsl/gpu/quantized.wgsl:573-588
//   matmul_int4_int8            kernels/wgsl/gpu/quantized.wgsl:590-647   A int4, TWO'S COMPLEMENT nibbles
//                               (unpack_int4x8, :150-158: not the +8 offset of the weight-only format)
//
// The shaders walk 16 x 16 tiles with one scalar multiply-add per thread and k.  Here a CTA owns a
// 128 x 128 tile of C; A (row-major, K contiguous) and B (row-major [K, N] as in the shaders, N
// contiguous) are staged in shared memory 64 k at a time, B transposed on the way in (4 x 4 byte
// blocks through prmt) so that both operands of mma.sync.m16n8k32.s8.s8.s32 are plain 32-bit reads;
// int4 weights are sign-extended to bytes while they are staged.  Shapes the tiled kernel does not
// take (K % 16, N % 16, unaligned views) run in a plain one-thread-per-output kernel.
#include "common.cuh"

#include <algorithm>

namespace luxcuda {

namespace {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma16832_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// four two's-complement nibbles (one per byte, low 4 bits) -> four signed bytes
__device__ __forceinline__ uint32_t sext4(uint32_t x) { return x | (((x >> 3) & 0x01010101u) * 0xF0u); }

constexpr int TM = 128, TN = 128, TK = 64;
constexpr int PITCH = TK + 16;                 // bytes per staged row (80: 16-byte aligned, conflict-free 32-bit reads)

// A4 = false: A is int8 [M, K].  A4 = true: A is int4 [M, K/2 bytes], element 2j in the low nibble.
// B is int8 [K, N].  M, N any; K % 16 == 0, N % 16 == 0, 16-byte aligned bases.
template <bool A4>
__global__ void __launch_bounds__(256) lux_matmul_int8_tc(const uint8_t* __restrict__ A, const int8_t* __restrict__ B,
                                                         int* __restrict__ C, int M, int N, int K) {
    __shared__ __align__(16) unsigned char sa[TM * PITCH];
    __shared__ __align__(16) unsigned char sb[TN * PITCH];     // B transposed: [n][k]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;      // 2 x 4 warps, 64 x 32 each
    int acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[i][j][c] = 0;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // ---- stage A: 128 rows x 64 k, 16 bytes (int8) or 8 bytes (int4) of source per piece ----
        for (int p = tid; p < TM * (TK / 16); p += 256) {
            const int r = p >> 2, kc = (p & 3) * 16;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m0 + r < M && k0 + kc < K) {
                if (A4) {
                    const uint2 w = __ldg(reinterpret_cast<const uint2*>(A + ((size_t)(m0 + r) * K + k0 + kc) / 2));
                    const uint32_t l0 = sext4(w.x & 0x0F0F0F0Fu), h0 = sext4((w.x >> 4) & 0x0F0F0F0Fu);
                    const uint32_t l1 = sext4(w.y & 0x0F0F0F0Fu), h1 = sext4((w.y >> 4) & 0x0F0F0F0Fu);
                    v = make_uint4(prmt(l0, h0, 0x5140), prmt(l0, h0, 0x7362), prmt(l1, h1, 0x5140), prmt(l1, h1, 0x7362));
                } else {
                    v = __ldg(reinterpret_cast<const uint4*>(A + (size_t)(m0 + r) * K + k0 + kc));
                }
            }
            *reinterpret_cast<uint4*>(sa + r * PITCH + kc) = v;
        }
        // ---- stage B transposed: a thread takes 4 k x 4 n, four coalesced 32-bit loads ----
        for (int p = tid; p < (TK / 4) * (TN / 4); p += 256) {
            const int kq = p / (TN / 4), nq = p - kq * (TN / 4);
            uint32_t r0 = 0, r1 = 0, r2 = 0, r3 = 0;
            const int n = n0 + nq * 4, k = k0 + kq * 4;
            if (n < N && k < K) {
                const int8_t* src = B + (size_t)k * N + n;
                r0 = __ldg(reinterpret_cast<const uint32_t*>(src));
                r1 = __ldg(reinterpret_cast<const uint32_t*>(src + N));
                r2 = __ldg(reinterpret_cast<const uint32_t*>(src + 2 * (size_t)N));
                r3 = __ldg(reinterpret_cast<const uint32_t*>(src + 3 * (size_t)N));
            }
            // byte j of the output word for column c is row j's byte c
            const uint32_t a01 = prmt(r0, r1, 0x5140), a23 = prmt(r2, r3, 0x5140);   // [r0.b0 r1.b0 r0.b1 r1.b1], ..
            const uint32_t c01 = prmt(r0, r1, 0x7362), c23 = prmt(r2, r3, 0x7362);   // [r0.b2 r1.b2 r0.b3 r1.b3], ..
            unsigned char* dst = sb + (nq * 4) * PITCH + kq * 4;
            *reinterpret_cast<uint32_t*>(dst) = prmt(a01, a23, 0x5410);
            *reinterpret_cast<uint32_t*>(dst + PITCH) = prmt(a01, a23, 0x7632);
            *reinterpret_cast<uint32_t*>(dst + 2 * PITCH) = prmt(c01, c23, 0x5410);
            *reinterpret_cast<uint32_t*>(dst + 3 * PITCH) = prmt(c01, c23, 0x7632);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < TK; ks += 32) {
            uint32_t bf[4][2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const unsigned char* bp = sb + (wn + j * 8 + g) * PITCH + ks + t * 4;
                bf[j][0] = *reinterpret_cast<const uint32_t*>(bp);
                bf[j][1] = *reinterpret_cast<const uint32_t*>(bp + 16);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const unsigned char* ap = sa + (wm + i * 16 + g) * PITCH + ks + t * 4;
                const uint32_t a0 = *reinterpret_cast<const uint32_t*>(ap);
                const uint32_t a1 = *reinterpret_cast<const uint32_t*>(ap + 8 * PITCH);
                const uint32_t a2 = *reinterpret_cast<const uint32_t*>(ap + 16);
                const uint32_t a3 = *reinterpret_cast<const uint32_t*>(ap + 8 * PITCH + 16);
#pragma unroll
                for (int j = 0; j < 4; j++) mma16832_s8(acc[i][j], a0, a1, a2, a3, bf[j][0], bf[j][1]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = m0 + wm + i * 16 + g, c = n0 + wn + j * 8 + 2 * t;
            if (c < N) {                                   // N % 16 == 0: c + 1 < N too
                if (r < M) *reinterpret_cast<int2*>(C + (size_t)r * N + c) = make_int2(acc[i][j][0], acc[i][j][1]);
                if (r + 8 < M) *reinterpret_cast<int2*>(C + (size_t)(r + 8) * N + c) = make_int2(acc[i][j][2], acc[i][j][3]);
            }
        }
}

// any shape: one thread per output, ascending k (the shaders' order; integer sums do not depend on it)
template <bool A4>
__global__ void __launch_bounds__(256) lux_matmul_int8_plain(const uint8_t* __restrict__ A, const int8_t* __restrict__ B,
                                                            int* __restrict__ C, int M, int N, int K) {
    const size_t o = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (o >= (size_t)M * N) return;
    const int r = (int)(o / N), c = (int)(o - (size_t)r * N);
    int sum = 0;
    for (int k = 0; k < K; k++) {
        int a;
        if (A4) {
            const size_t flat = (size_t)r * K + k;
            int nib = (A[flat >> 1] >> ((flat & 1) * 4)) & 0xF;
            a = nib >= 8 ? nib - 16 : nib;
        } else {
            a = (int)(int8_t)A[(size_t)r * K + k];
        }
        sum += a * (int)B[(size_t)k * N + c];
    }
    C[o] = sum;
}

__global__ void __launch_bounds__(256) lux_requantize_i32_i8(const int* __restrict__ in, int* __restrict__ out, size_t n,
                                                            float in_scale, float out_scale, int zp) {
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float v = __fmul_rn((float)in[i], in_scale);
        const float r = __fadd_rn(rintf(__fdiv_rn(v, out_scale)), (float)zp);
        out[i] = min(max(__float2int_rz(r), -128), 127);
    }
}

// phase 1 of dynamic_quantize: max |x| over the tensor, as the bit pattern of a non-negative float
__global__ void __launch_bounds__(256) lux_absmax_f32(const float* __restrict__ x, size_t n, uint32_t* __restrict__ out_bits) {
    float m = 0.0f;
    const size_t stride = (size_t)gridDim.x * 256, t0 = (size_t)blockIdx.x * 256 + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        // 16-byte loads, two in flight per thread
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const size_t n4 = n / 4;
        size_t i = t0;
        for (; i + stride < n4; i += 2 * stride) {
            const float4 a = __ldg(x4 + i), b = __ldg(x4 + i + stride);
            m = fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                               fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w)))));
        }
        if (i < n4) {
            const float4 a = __ldg(x4 + i);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
        }
        for (size_t j = n4 * 4 + t0; j < n; j += stride) m = fmaxf(m, fabsf(x[j]));
    } else {
        for (size_t i = t0; i < n; i += stride) m = fmaxf(m, fabsf(x[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));
}

// phase 2: scale = max / 127 (or / 7), 1 if that is 0; q = clamp(i32(round(x / scale))); eight values per thread
template <int BITS>
__global__ void __launch_bounds__(256) lux_dynamic_quantize(const float* __restrict__ x, size_t n, const uint32_t* __restrict__ max_bits,
                                                           uint8_t* __restrict__ out, float* __restrict__ scale_out) {
    float scale = __fdiv_rn(__uint_as_float(*max_bits), BITS == 4 ? 7.0f : 127.0f);
    if (scale == 0.0f) scale = 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const size_t octets = (n + 7) / 8;
    const size_t stride = (size_t)gridDim.x * 256;
    // 16-byte loads and (int8) 8-byte stores where the views allow them
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0;
    for (size_t o = (size_t)blockIdx.x * 256 + threadIdx.x; o < octets; o += stride) {
        int q[8];
        if (vec && o * 8 + 8 <= n) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * o), b = __ldg(reinterpret_cast<const float4*>(x) + 2 * o + 1);
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 8; j++) q[j] = __float2int_rz(rintf(__fdiv_rn(v[j], scale)));
            if (BITS == 8) {
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    lo |= (uint32_t)(min(max(q[j], -128), 127) & 0xFF) << (8 * j);
                    hi |= (uint32_t)(min(max(q[4 + j], -128), 127) & 0xFF) << (8 * j);
                }
                *reinterpret_cast<uint2*>(out + o * 8) = make_uint2(lo, hi);
                continue;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const size_t i = o * 8 + j;
                q[j] = i < n ? __float2int_rz(rintf(__fdiv_rn(x[i], scale))) : 0;
            }
        }
        if (BITS == 4) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) w |= (uint32_t)((min(max(q[j], -8), 7) + 8) & 0xF) << (4 * j);   // pack_nax_int4_sym_x8
            if (o * 4 + 4 <= (n + 1) / 2) *reinterpret_cast<uint32_t*>(out + o * 4) = w;
            else for (size_t b = o * 4; b < (n + 1) / 2; b++) out[b] = (uint8_t)(w >> (8 * (b - o * 4)));
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (o * 8 + j < n) out[o * 8 + j] = (uint8_t)(min(max(q[j], -128), 127) & 0xFF);
        }
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <bool A4>
LuxBackendError matmul_int(LuxBackendContext* context, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* c, int M, int N, int K,
                           const char* what) {
    Context* ctx = as_ctx(context);
    Buffer *ba = as_buf(a), *bb = as_buf(b), *bc = as_buf(c);
    if (!ctx || !ba || !bb || !bc || M <= 0 || N <= 0 || K <= 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t a_bytes = A4 ? ((size_t)M * K + 1) / 2 : (size_t)M * K;
    if (ba->size < a_bytes || bb->size < (size_t)K * N || bc->size < (size_t)M * N * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    // matmuls with at least a 128 x 256 tile of outputs go to the tcgen05 kernel (qint_gemm_tc.cu);
    // int_matmul_kernel = 1 keeps everything on the mma.sync kernels below
    if (g_tune.int_matmul_kernel != 1) {
        LuxBackendError e = launch_matmul_int8_tcgen05(ctx, ba->ptr, bb->ptr, (int*)bc->ptr, M, N, K, A4);
        if (e == LUX_BACKEND_OK) return finish_op(ctx, false, what);
        if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED) return e;
    }
    const bool tiled = K % 16 == 0 && N % 16 == 0 && aligned16(ba->ptr) && aligned16(bb->ptr) && aligned16(bc->ptr) &&
                       (N + TN - 1) / TN <= 65535 * 32 && (M + TM - 1) / TM <= 65535;
    if (tiled) {
        dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
        lux_matmul_int8_tc<A4><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)ba->ptr, (const int8_t*)bb->ptr, (int*)bc->ptr, M, N, K);
    } else {
        const size_t outs = (size_t)M * N;
        lux_matmul_int8_plain<A4><<<(unsigned)((outs + 255) / 256), 256, 0, ctx->stream>>>((const uint8_t*)ba->ptr, (const int8_t*)bb->ptr,
                                                                                        (int*)bc->ptr, M, N, K);
    }
    count_launch(A4 ? "lux_matmul_int4_int8" : "lux_matmul_int8");
    return finish_op(ctx, false, what);
}

}  // namespace

const void* kernel_addr_matmul_int8() { return (const void*)lux_matmul_int8_tc<false>; }
const void* kernel_addr_matmul_int4_int8() { return (const void*)lux_matmul_int8_tc<true>; }

}  // namespace luxcuda

using namespace luxcuda;

extern "C" {

LuxBackendError lux_cuda_matmul_int8(LuxBackendContext* ctx, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* c, int M, int N, int K) {
    return matmul_int<false>(ctx, a, b, c, M, N, K, "lux_cuda_matmul_int8");
}

LuxBackendError lux_cuda_matmul_int4_int8(LuxBackendContext* ctx, LuxBackendBuffer* w4, LuxBackendBuffer* b, LuxBackendBuffer* c, int M, int N,
                                          int K) {
    return matmul_int<true>(ctx, w4, b, c, M, N, K, "lux_cuda_matmul_int4_int8");
}

LuxBackendError lux_cuda_requantize_int32_to_int8(LuxBackendContext* context, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n,
                                                  float input_scale, float output_scale, int32_t output_zero_point) {
    Context* ctx = as_ctx(context);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!ctx || !bi || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bi->size < n * 4 || bo->size < n * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
    lux_requantize_i32_i8<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const int*)bi->ptr, (int*)bo->ptr, n, input_scale, output_scale,
                                                                      output_zero_point);
    count_launch();
    return finish_op(ctx, false, "lux_cuda_requantize_int32_to_int8");
}

LuxBackendError lux_cuda_dynamic_quantize(LuxBackendContext* context, LuxBackendBuffer* x, LuxBackendBuffer* out, LuxBackendBuffer* scale_out,
                                          size_t n, uint32_t bits) {
    Context* ctx = as_ctx(context);
    Buffer *bx = as_buf(x), *bo = as_buf(out), *bs = as_buf(scale_out);
    if (!ctx || !bx || !bo || !bs || n == 0 || (bits != 4 && bits != 8)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t out_bytes = bits == 4 ? (n + 1) / 2 : n;
    if (bx->size < n * 4 || bo->size < out_bytes || bs->size < 4 || !ctx->d_absmax) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(bo->ptr) & 3u) != 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    std::lock_guard<std::mutex> lock(ctx->mu);                 // the max word belongs to the context
    LUX_CUDA_TRY(cudaMemsetAsync(ctx->d_absmax, 0, sizeof(uint32_t), ctx->stream));
    const size_t blocks = std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 8);
    lux_absmax_f32<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)bx->ptr, n, ctx->d_absmax);
    const size_t qblocks = std::min<size_t>(((n + 7) / 8 + 255) / 256, (size_t)ctx->sm_count * 8);
    if (bits == 4)
        lux_dynamic_quantize<4><<<(unsigned)qblocks, 256, 0, ctx->stream>>>((const float*)bx->ptr, n, ctx->d_absmax, (uint8_t*)bo->ptr, (float*)bs->ptr);
    else
        lux_dynamic_quantize<8><<<(unsigned)qblocks, 256, 0, ctx->stream>>>((const float*)bx->ptr, n, ctx->d_absmax, (uint8_t*)bo->ptr, (float*)bs->ptr);
    count_launch(2);
    ctx->writer_pending = true;
    return finish_op(ctx, false, "lux_cuda_dynamic_quantize");
}

}  // extern "C"
