// Standalone unpack and dequantize kernels.  They exist so that the integer unpack and
// the dequantized weights can be compared BIT-EXACTLY with the reference arithmetic,
// independent of how the matmul kernels reorder their sums:
//   unpack_nax_int4_asym_x8 / unpack_nax_int8_x4 ..... kernels/wgsl/gpu/quantized_nax.wgsl:125-151
//   dequantize_nax_int4_asym / _int8_group (sym) ...... kernels/wgsl/gpu/quantized_nax.wgsl:312-330, 364-381
// One thread handles 16 packed bytes (32 int4 or 16 int8 weights), all within one group.
#include "common.cuh"

namespace luxcuda {

namespace {

template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename S> __device__ __forceinline__ float widen(S v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ int zero_point_at(const uint8_t* zeros, int bits, size_t n, int g, int ZS) {
    if (!zeros) return bits == 4 ? 8 : 0;
    return (zeros[n * ZS + (g >> 1)] >> ((g & 1) * 4)) & 0xF;
}

// OUT = int8_t: integer (q - zp).  Otherwise f32(q - zp) * scale narrowed once to OUT.
template <int BITS, typename S, typename OUT, bool INTEGER>
__global__ void lux_qdequant(const uint8_t* __restrict__ w, const S* __restrict__ scales,
                             const uint8_t* __restrict__ zeros, OUT* __restrict__ out,
                             int N, int K, int group) {
    constexpr int PER = BITS == 4 ? 32 : 16;            // weights per 16 packed bytes
    const size_t units_per_row = (size_t)K / PER;
    const size_t total = (size_t)N * units_per_row;
    const int G = K / group, ZS = (G + 1) / 2;
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (size_t)gridDim.x * blockDim.x) {
        const size_t n = u / units_per_row;
        const int k0 = (int)(u - n * units_per_row) * PER;
        const int g = k0 / group;
        const uint4 q = *reinterpret_cast<const uint4*>(w + n * ((size_t)K * BITS / 8) + (size_t)k0 * BITS / 8);
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        const int zp = zero_point_at(zeros, BITS, n, g, ZS);
        float scale = 0.0f;
        if constexpr (!INTEGER) scale = widen<S>(scales[n * G + g]);
        OUT* o = out + n * (size_t)K + k0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (BITS == 4) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int v = (int)((words[j] >> (4 * i)) & 0xFu) - zp;          // integer subtract first
                    if constexpr (INTEGER) o[j * 8 + i] = (OUT)v;
                    else o[j * 8 + i] = narrow<OUT>(__fmul_rn((float)v, scale));     // one f32 multiply
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int v = (int)((words[j] >> (8 * i)) & 0xFFu);
                    if (v >= 128) v -= 256;
                    v -= zp;
                    if constexpr (INTEGER) o[j * 4 + i] = (OUT)v;
                    else o[j * 4 + i] = narrow<OUT>(__fmul_rn((float)v, scale));
                }
            }
        }
    }
}

template <int BITS, typename S, typename OUT, bool INTEGER>
cudaError_t run(Context* ctx, const QArgs& a, int group) {
    const size_t units = (size_t)a.N * a.K / (BITS == 4 ? 32 : 16);
    const int threads = 256;
    const size_t blocks = std::min<size_t>((units + threads - 1) / threads, (size_t)ctx->sm_count * 32);
    lux_qdequant<BITS, S, OUT, INTEGER><<<(unsigned)std::max<size_t>(blocks, 1), threads, 0, ctx->stream>>>(
        a.w, (const S*)a.scales, a.zeros, (OUT*)a.y, a.N, a.K, group);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

LuxBackendError launch_qdequant(Context* ctx, const QArgs& a, int bits) {
    const int group = a.K / a.G;
    cudaError_t e = cudaErrorInvalidValue;
    if (bits == 4 && a.scale_dtype == LUX_QDTYPE_F16) {
        if (a.y_dtype == LUX_QDTYPE_F32)       e = run<4, __half, float, false>(ctx, a, group);
        else if (a.y_dtype == LUX_QDTYPE_F16)  e = run<4, __half, __half, false>(ctx, a, group);
        else                                   e = run<4, __half, __nv_bfloat16, false>(ctx, a, group);
    } else if (bits == 8 && a.scale_dtype == LUX_QDTYPE_F32) {
        if (a.y_dtype == LUX_QDTYPE_F32)       e = run<8, float, float, false>(ctx, a, group);
        else if (a.y_dtype == LUX_QDTYPE_F16)  e = run<8, float, __half, false>(ctx, a, group);
        else                                   e = run<8, float, __nv_bfloat16, false>(ctx, a, group);
    } else {
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    return map_cuda(e, "lux_qdequant");
}

LuxBackendError launch_qunpack(Context* ctx, const QArgs& a, int bits) {
    const int group = a.K / a.G;
    cudaError_t e = bits == 4 ? run<4, __half, int8_t, true>(ctx, a, group)
                              : run<8, float, int8_t, true>(ctx, a, group);
    return map_cuda(e, "lux_qunpack");
}

const void* kernel_addr_qdequant_i4() { return (const void*)lux_qdequant<4, __half, float, false>; }
const void* kernel_addr_qdequant_i8() { return (const void*)lux_qdequant<8, float, float, false>; }

}  // namespace luxcuda
