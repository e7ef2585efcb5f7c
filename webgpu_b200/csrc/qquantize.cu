// lux_qquantize -- the quantize side of the group-quantized format: an f32 (or 16-bit) matrix
// [N, K] becomes the packed integers, the scale table and the zero-point table that the matmul
// kernels read.  One pass over the input, HBM-bound (4 bytes read and 0.5-1 byte written per
// element); the reference does it in two dispatches,
//
//   compute_group_scales       luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:157-232
//   quantize_nax_int4_sym      :236-259
//   quantize_nax_int4_asym     :288-310 (with pack_nax_int4_asym_x8, :115-122)
//   quantize_nax_int8_group    :336-362 (symmetric branch; pack_nax_int8_x4, :135-140)
//
// whose arithmetic is reproduced operation by operation (IEEE division, round-half-to-even,
// saturating float -> int conversion, min / max seeded with +-1e30, the zero-point computed before
// the "scale == 0 -> 1" guard), so that packed bytes, scales and zero-points come out bit-identical.
// That includes the asymmetric int4 shader's own behaviour: it stores clamp(round(v / scale), 0, 15),
// the zero-point is subtracted and added back around a second clamp and never shifts the value, so
// negative inputs are stored as 0.  LUX_QQUANT_FLAG_SHIFTED selects the usual
// clamp(round(v / scale) + zp, 0, 15) instead (an extension, not the reference's arithmetic).
//
// A warp works on 256 consecutive elements of a row at a time, 8 per lane: two int4 groups of 128 (16 lanes
// each) or eight int8 groups of 32 (4 lanes each).  Group minimum and maximum by shuffles inside the
// group's lanes; one 4-byte (int4) or 8-byte (int8) store per lane, coalesced over the warp; the two
// int4 zero-points of a warp share one byte of the zero-point table (low nibble first).
//
// This kernel WRITES buffers that a later matmul binds as weights.  It is a plain launch (no
// programmatic-launch trigger), and the entry point marks the context so that the next matmul is
// launched fully ordered behind it.
#include "common.cuh"

namespace luxcuda {

namespace {

struct QuantParams {
    const void* x;          // [N, K] f32 / f16 / bf16
    uint8_t* w;             // int4: [N, K/2]; int8: [N, K]
    void* scales;           // [N, G] f32 or f16
    uint8_t* zeros;         // int4 asymmetric: [N, ZS]; else null
    int N, K, G, ZS;
    int x_dtype, scale_dtype;
    int shifted;            // LUX_QQUANT_FLAG_SHIFTED
    int chunks_per_row;     // ceil(K / 256)
};

__device__ __forceinline__ void load8(const QuantParams& p, size_t idx, float (&v)[8]) {
    if (p.x_dtype == LUX_QDTYPE_F32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + idx));
        const float4 b = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + idx) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) + idx));
        const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (p.x_dtype == LUX_QDTYPE_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
            } else {
                v[2 * i] = __uint_as_float(u[i] << 16);
                v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
            }
        }
    }
}

// BITS = 4: groups of 128 (16 lanes); BITS = 8: groups of 32 (4 lanes), symmetric only.
// A warp takes QCH consecutive 256-element chunks of a row and requests all of them before it
// reduces the first: 4 KB in flight per warp, so that a streaming kernel with this little
// arithmetic keeps HBM busy.
constexpr int QCH = 4;

template <int BITS, bool SYM>
__global__ void __launch_bounds__(256) lux_qquantize(const QuantParams p) {
    constexpr int GL = BITS == 4 ? 16 : 4;                  // lanes per group
    const int lane = threadIdx.x & 31;
    const size_t wid = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int wpr = (p.chunks_per_row + QCH - 1) / QCH;     // warps per row
    const size_t n = wid / (size_t)wpr;
    if (n >= (size_t)p.N) return;
    const int c0 = (int)(wid - n * (size_t)wpr) * QCH;
    float v[QCH][8];
    bool live[QCH];
#pragma unroll
    for (int ch = 0; ch < QCH; ch++) {
        const int k0 = (c0 + ch) * 256 + lane * 8;
        live[ch] = k0 < p.K;                                 // K is a multiple of the group size, so of 8
        if (live[ch]) load8(p, n * (size_t)p.K + k0, v[ch]);
    }
#pragma unroll
    for (int ch = 0; ch < QCH; ch++) {
        const int c = c0 + ch;
        const int k0 = c * 256 + lane * 8;
        if (c >= p.chunks_per_row) break;                    // warp-uniform
        float mx = -1e30f, mn = 1e30f;                       // the shader's seeds (:169-170)
        if (live[ch]) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                mx = fmaxf(mx, v[ch][i]);
                mn = fminf(mn, v[ch][i]);
            }
        }
#pragma unroll
        for (int o = GL / 2; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        }
        float scale;
        int zp = 0;
        if (SYM) {
            const float amax = fmaxf(fabsf(mx), fabsf(mn));
            scale = __fdiv_rn(amax, BITS == 4 ? 7.0f : 127.0f);
        } else {
            scale = __fdiv_rn(mx - mn, 15.0f);
            zp = min(max(__float2int_rz(rintf(__fdiv_rn(-mn, scale))), 0), 15);   // before the guard, as in the shader
        }
        if (scale == 0.0f) scale = 1.0f;
        // compact table: an f16 table stores the rounded scale, and the values are quantized with the
        // number the table holds (what dequantize will multiply by)
        const __half s16 = __float2half_rn(scale);
        if (p.scale_dtype == LUX_QDTYPE_F16) scale = __half2float(s16);
        const int g = k0 / (BITS == 4 ? 128 : 32);
        if (live[ch] && (lane % GL) == 0) {
            if (p.scale_dtype == LUX_QDTYPE_F16) reinterpret_cast<__half*>(p.scales)[n * (size_t)p.G + g] = s16;
            else reinterpret_cast<float*>(p.scales)[n * (size_t)p.G + g] = scale;
        }
        if (BITS == 4 && !SYM) {
            const int zp_hi = __shfl_sync(0xffffffffu, live[ch] ? zp : 0, 16);
            if (lane == 0 && live[ch]) p.zeros[n * (size_t)p.ZS + c] = (uint8_t)(zp | (zp_hi << 4));
        }
        if (!live[ch]) continue;
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = __float2int_rz(rintf(__fdiv_rn(v[ch][i], scale)));   // saturating; NaN -> 0
        if (BITS == 4) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int nib;
                if (SYM) nib = min(max(q[i], -8), 7) + 8;
                else if (p.shifted) nib = min(max(min(max(q[i], -32), 32) + zp, 0), 15);   // pre-clamped: a saturated q must not wrap
                else nib = min(max(q[i], 0), 15);                         // (clamp(q, 0, 15) - zp) + zp, clamped again
                word |= (uint32_t)nib << (4 * i);
            }
            reinterpret_cast<uint32_t*>(p.w)[(n * (size_t)p.K + k0) >> 3] = word;
        } else {
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo |= ((uint32_t)min(max(q[i], -128), 127) & 0xFFu) << (8 * i);
                hi |= ((uint32_t)min(max(q[4 + i], -128), 127) & 0xFFu) << (8 * i);
            }
            reinterpret_cast<uint2*>(p.w)[(n * (size_t)p.K + k0) >> 3] = make_uint2(lo, hi);
        }
    }
}

}  // namespace

const void* kernel_addr_qquantize_i4() { return (const void*)lux_qquantize<4, false>; }
const void* kernel_addr_qquantize_i8() { return (const void*)lux_qquantize<8, true>; }

}  // namespace luxcuda

using namespace luxcuda;

extern "C" LuxBackendError lux_cuda_qquantize(LuxBackendContext* context, const LuxQMatmulDesc* d, LuxBackendBuffer* x,
                                              LuxBackendBuffer* w_out, LuxBackendBuffer* scales_out,
                                              LuxBackendBuffer* zeros_out) {
    Context* ctx = as_ctx(context);
    Buffer *bx = as_buf(x), *bw = as_buf(w_out), *bs = as_buf(scales_out), *bz = as_buf(zeros_out);
    if (!ctx || !d || d->struct_size < sizeof(LuxQMatmulDesc) || !bx || !bw || !bs) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->N == 0 || d->K == 0 || (d->bits != 4 && d->bits != 8)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->x_dtype > LUX_QDTYPE_BF16 || d->scale_dtype > LUX_QDTYPE_BF16) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    // the layouts the matmul kernels read: int4 in groups of 128 (f16 or f32 scales, with or without
    // zero-points), int8 in groups of 32 with f32 scales and no zero-points
    if (d->bits == 4 && (d->group_size != 128 || d->scale_dtype == LUX_QDTYPE_BF16)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (d->bits == 8 && (d->group_size != 32 || d->scale_dtype != LUX_QDTYPE_F32 || bz)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (d->K % d->group_size) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t N = d->N, K = d->K, G = K / d->group_size, ZS = (G + 1) / 2;
    const size_t xs = d->x_dtype == LUX_QDTYPE_F32 ? 4 : 2, ss = d->scale_dtype == LUX_QDTYPE_F32 ? 4 : 2;
    if (bx->size < N * K * xs || bw->size < N * K * d->bits / 8 || bs->size < N * G * ss) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bz && bz->size < N * ZS) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!aligned16(bx->ptr) || !aligned16(bw->ptr) || !aligned16(bs->ptr)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (N * ((K + 255) / 256) > ((size_t)1 << 33)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;

    QuantParams p{};
    p.x = bx->ptr;
    p.w = (uint8_t*)bw->ptr;
    p.scales = bs->ptr;
    p.zeros = bz ? (uint8_t*)bz->ptr : nullptr;
    p.N = (int)N; p.K = (int)K; p.G = (int)G; p.ZS = (int)ZS;
    p.x_dtype = (int)d->x_dtype;
    p.scale_dtype = (int)d->scale_dtype;
    p.shifted = (d->flags & LUX_QQUANT_FLAG_SHIFTED) ? 1 : 0;
    p.chunks_per_row = (int)((K + 255) / 256);
    const size_t warps = N * (size_t)((p.chunks_per_row + QCH - 1) / QCH);
    const unsigned grid = (unsigned)((warps + 7) / 8);
    cudaSetDevice(ctx->device);
    if (d->bits == 8) lux_qquantize<8, true><<<grid, 256, 0, ctx->stream>>>(p);
    else if (bz) lux_qquantize<4, false><<<grid, 256, 0, ctx->stream>>>(p);
    else lux_qquantize<4, true><<<grid, 256, 0, ctx->stream>>>(p);
    count_launch("lux_qquantize");
    ctx->writer_pending = true;          // cleared by the wait in finish_op unless NO_SYNC
    return finish_op(ctx, (d->flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, "lux_cuda_qquantize");
}
