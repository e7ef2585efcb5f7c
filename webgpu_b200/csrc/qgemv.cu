// Streaming (HBM-bound) quantized GEMV / skinny GEMM kernels for sm_100a.
//
//   lux_qgemv_i8_g32_f32     int8 symmetric, one f32 scale per 32 K, f32 x and y
//   lux_qskinny_i4_g128      int4 asymmetric/symmetric, f16 scale + 4-bit zero-point per
//                            128 K, f16 x and y, batch M <= 32, optional SwiGLU epilogue
//
// Both replace matmul_nax_grouped (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:
// 568-626), which reads one packed u32 per weight ELEMENT, unpacks all eight nibbles to
// keep one, and fetches a 16-byte scale struct per element.  Here every packed byte is
// read exactly once with 128-bit loads, nibbles/bytes are turned into f16 in registers
// with two-operation bit tricks, the integer subtract (q - zp) happens exactly in f16
// before the multiply, products are formed exactly and accumulated in f32 by
// mma.sync.m16n8k16 (the weight tile is the 16-row operand, the batch the 8-column
// one), and the per-group scale is applied to the f32 group sum.  The contraction is
// the reference's sum over k in a different order; results agree to f32 rounding.
//
// Thread mapping inside a warp (g = lane/4, t = lane%4), fixed by the mma fragment
// layout: the lane owns weight rows (n0+g) and (n0+g+8) and K positions that depend on
// t; the four lanes of one g cover one contiguous 64-byte piece of a row per step.
#include "common.cuh"

#include <algorithm>

namespace luxcuda {

namespace {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));   // (a & mask) | orv
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + __expf(-x)); }

// =====================================================================================
// int4, group 128, f16
// =====================================================================================
//
// Per step a warp consumes one quantization group (128 K) of a 16-row tile: lane (g,t)
// loads 16 bytes = K [32t, 32t+32) of the group for each of its two rows.  A packed
// word w holds nibbles n0..n7 (n_i = (w >> 4i) & 15, quantized_nax.wgsl:125-132):
//     (w & 0x000f000f) | 0x64006400  = f16x2 (1024 + n0, 1024 + n4)
//     (w & 0x00f000f0) | 0x54005400  = f16x2 (  64 + n1,   64 + n5)
// and the same on w >> 8 gives (n2, n6), (n3, n7).  Subtracting (1024 + zp) resp.
// (64 + zp) yields the integers (n - zp) exactly.  The pairs are not adjacent in K, so
// x is staged in shared memory in the matching order once per CTA.
//
// x staging layout, per group of 128 K: 16 chunks of 8 halves; chunk (j*4 + t) holds
// x[32t + 8j + {0,4,1,5,2,6,3,7}].  Lane (m=g, t) reads chunk (j*4+t) for j = 0..3.
// Rows are padded by 64 bytes so that two batch rows fall into different bank halves.

constexpr int I4_UNROLL = 4;         // groups in flight per warp: 8 x 16 B loads per lane

struct SkinnyParams {
    const __half* x;        // [M, K]
    const uint8_t* w;       // [Nw, K/2]
    const __half* scales;   // [Nw, G]
    const uint8_t* zeros;   // [Nw, ZS] or null
    __half* y;              // [M, Nout]
    int M, Nout, K, G, ZS;
    int up_row_offset;      // SWIGLU: weight row of `up` = weight row of `gate` + this
    int kc_groups;          // groups per x chunk staged in shared memory
    int xstride;            // bytes between batch rows in shared memory
};

template <int MT, int RT, bool SWIGLU>
__global__ void __launch_bounds__(256) lux_qskinny_i4_g128(const SkinnyParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int nwarps = nthreads >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int NACC = SWIGLU ? 2 : 1;

    unsigned char* xs = smem;                                   // staged x chunk
    // reduction buffer lives after the x chunk
    float4* red = reinterpret_cast<float4*>(smem + (size_t)p.M * p.xstride);

    float res[RT][NACC][MT][4];
#pragma unroll
    for (int r = 0; r < RT; r++)
#pragma unroll
        for (int a = 0; a < NACC; a++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) res[r][a][mt][i] = 0.0f;

    const int tile0 = blockIdx.x * RT;
    const size_t row_bytes = (size_t)p.K >> 1;

    // Ask L2 for this CTA's packed rows right away: the DRAM fetch then overlaps the staging
    // of x below, and the streaming loads further down find their lines in L2.
    {
        const int rows = RT * 16 * NACC;
        const int lines_per_row = (int)(row_bytes >> 7);               // 128-byte lines (K % 256 may leave a tail)
        for (int i = tid; i < rows * lines_per_row; i += nthreads) {
            const int rr = i / lines_per_row, ln = i - rr * lines_per_row;
            const int a = rr / (RT * 16), r = rr - a * (RT * 16);
            const int row = min(tile0 * 16 + r, p.Nout - 1) + a * p.up_row_offset;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + (size_t)row * row_bytes + (size_t)ln * 128));
        }
    }

    for (int c0 = 0; c0 < p.G; c0 += p.kc_groups) {
        const int c1 = min(c0 + p.kc_groups, p.G);
        // ---- stage x[:, c0*128 : c1*128] in fragment order --------------------------
        __syncthreads();
        {
            const int chunks_per_row = (c1 - c0) * 16;           // 16-byte chunks
            const int total = p.M * chunks_per_row;
            for (int i = tid; i < total; i += nthreads) {
                int m = i / chunks_per_row, c = i - m * chunks_per_row;
                int grp = c >> 4, cc = c & 15;                   // source chunk cc = 4t + j
                int tt = cc >> 2, j = cc & 3;
                uint4 s = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + (size_t)(c0 + grp) * 128 + cc * 8);
                uint4 d;
                d.x = prmt(s.x, s.z, 0x5410);                    // (i0, i4)
                d.y = prmt(s.x, s.z, 0x7632);                    // (i1, i5)
                d.z = prmt(s.y, s.w, 0x5410);                    // (i2, i6)
                d.w = prmt(s.y, s.w, 0x7632);                    // (i3, i7)
                *reinterpret_cast<uint4*>(xs + (size_t)m * p.xstride + grp * 256 + (j * 4 + tt) * 16) = d;
            }
        }
        __syncthreads();

#pragma unroll
        for (int r = 0; r < RT; r++) {
            const int n0 = (tile0 + r) * 16;
            if (n0 >= p.Nout) break;
#pragma unroll
            for (int a = 0; a < NACC; a++) {
                const int ra = min(n0 + g, p.Nout - 1) + a * p.up_row_offset;
                const int rb = min(n0 + g + 8, p.Nout - 1) + a * p.up_row_offset;
                const uint4* wa = reinterpret_cast<const uint4*>(p.w + (size_t)ra * row_bytes) + t;
                const uint4* wb = reinterpret_cast<const uint4*>(p.w + (size_t)rb * row_bytes) + t;
                const __half* sa = p.scales + (size_t)ra * p.G;
                const __half* sb = p.scales + (size_t)rb * p.G;
                const uint8_t* za = p.zeros ? p.zeros + (size_t)ra * p.ZS : nullptr;
                const uint8_t* zb = p.zeros ? p.zeros + (size_t)rb * p.ZS : nullptr;

                for (int gb = c0 + warp; gb < c1; gb += nwarps * I4_UNROLL) {
                    uint4 qa[I4_UNROLL], qb[I4_UNROLL];
                    float fsa[I4_UNROLL], fsb[I4_UNROLL];
                    uint32_t zpa[I4_UNROLL], zpb[I4_UNROLL];
#pragma unroll
                    for (int u = 0; u < I4_UNROLL; u++) {
                        const int gi = gb + u * nwarps;
                        if (gi < c1) {
                            qa[u] = ldg_stream(wa + gi * 4);
                            qb[u] = ldg_stream(wb + gi * 4);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < I4_UNROLL; u++) {
                        const int gi = gb + u * nwarps;
                        if (gi < c1) {
                            fsa[u] = __half2float(__ldg(sa + gi));
                            fsb[u] = __half2float(__ldg(sb + gi));
                            if (za) {
                                zpa[u] = (__ldg(za + (gi >> 1)) >> ((gi & 1) * 4)) & 0xFu;
                                zpb[u] = (__ldg(zb + (gi >> 1)) >> ((gi & 1) * 4)) & 0xFu;
                            } else {
                                zpa[u] = 8u; zpb[u] = 8u;       // symmetric: stored value - 8
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < I4_UNROLL; u++) {
                        const int gi = gb + u * nwarps;
                        if (gi >= c1) break;
                        // (1024 + zp) and (64 + zp) as f16x2 bit patterns
                        const uint32_t za_lo = (0x6400u | zpa[u]) * 0x00010001u;
                        const uint32_t za_hi = (0x5400u | (zpa[u] << 4)) * 0x00010001u;
                        const uint32_t zb_lo = (0x6400u | zpb[u]) * 0x00010001u;
                        const uint32_t zb_hi = (0x5400u | (zpb[u] << 4)) * 0x00010001u;
                        const uint32_t wqa[4] = {qa[u].x, qa[u].y, qa[u].z, qa[u].w};
                        const uint32_t wqb[4] = {qb[u].x, qb[u].y, qb[u].z, qb[u].w};

                        float acc[MT][4];
#pragma unroll
                        for (int mt = 0; mt < MT; mt++)
#pragma unroll
                            for (int i = 0; i < 4; i++) acc[mt][i] = 0.0f;

                        const unsigned char* xg = xs + (gi - c0) * 256 + t * 16;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint32_t va = wqa[j], vb = wqb[j];
                            const uint32_t a0 = hsub2_u32(lop3_and_or(va, 0x000f000fu, 0x64006400u), za_lo);
                            const uint32_t a1 = hsub2_u32(lop3_and_or(vb, 0x000f000fu, 0x64006400u), zb_lo);
                            const uint32_t a2 = hsub2_u32(lop3_and_or(va, 0x00f000f0u, 0x54005400u), za_hi);
                            const uint32_t a3 = hsub2_u32(lop3_and_or(vb, 0x00f000f0u, 0x54005400u), zb_hi);
                            va >>= 8; vb >>= 8;
                            const uint32_t a4 = hsub2_u32(lop3_and_or(va, 0x000f000fu, 0x64006400u), za_lo);
                            const uint32_t a5 = hsub2_u32(lop3_and_or(vb, 0x000f000fu, 0x64006400u), zb_lo);
                            const uint32_t a6 = hsub2_u32(lop3_and_or(va, 0x00f000f0u, 0x54005400u), za_hi);
                            const uint32_t a7 = hsub2_u32(lop3_and_or(vb, 0x00f000f0u, 0x54005400u), zb_hi);
#pragma unroll
                            for (int mt = 0; mt < MT; mt++) {
                                const int m = min(mt * 8 + g, p.M - 1);
                                const uint4 xv = *reinterpret_cast<const uint4*>(xg + (size_t)m * p.xstride + j * 64);
                                mma16816(acc[mt], a0, a1, a2, a3, xv.x, xv.y, acc[mt]);
                                mma16816(acc[mt], a4, a5, a6, a7, xv.z, xv.w, acc[mt]);
                            }
                        }
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            res[r][a][mt][0] = fmaf(fsa[u], acc[mt][0], res[r][a][mt][0]);
                            res[r][a][mt][1] = fmaf(fsa[u], acc[mt][1], res[r][a][mt][1]);
                            res[r][a][mt][2] = fmaf(fsb[u], acc[mt][2], res[r][a][mt][2]);
                            res[r][a][mt][3] = fmaf(fsb[u], acc[mt][3], res[r][a][mt][3]);
                        }
                    }
                }
            }
        }
    }

    // ---- cross-warp reduction and store ---------------------------------------------
    // red[(warp * RT*NACC*MT + slot) * 32 + lane] : one float4 per lane per slot
    constexpr int SLOTS = RT * NACC * MT;
#pragma unroll
    for (int r = 0; r < RT; r++)
#pragma unroll
        for (int a = 0; a < NACC; a++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const int slot = (r * NACC + a) * MT + mt;
                red[(warp * SLOTS + slot) * 32 + lane] =
                    make_float4(res[r][a][mt][0], res[r][a][mt][1], res[r][a][mt][2], res[r][a][mt][3]);
            }
    __syncthreads();
    for (int o = tid; o < RT * MT * 32; o += nthreads) {
        const int ln = o & 31, rm = o >> 5;
        const int r = rm / MT, mt = rm - r * MT;
        float4 sum[NACC];
#pragma unroll
        for (int a = 0; a < NACC; a++) {
            const int slot = (r * NACC + a) * MT + mt;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int w = 0; w < nwarps; w++) {
                const float4 v = red[(w * SLOTS + slot) * 32 + ln];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            sum[a] = s;
        }
        float4 o4 = sum[0];
        if (SWIGLU) {
            o4.x = silu_f32(sum[0].x) * sum[NACC - 1].x;
            o4.y = silu_f32(sum[0].y) * sum[NACC - 1].y;
            o4.z = silu_f32(sum[0].z) * sum[NACC - 1].z;
            o4.w = silu_f32(sum[0].w) * sum[NACC - 1].w;
        }
        const int gg = ln >> 2, tt = ln & 3;
        const int n_a = (tile0 + r) * 16 + gg, n_b = n_a + 8;
        const int m0 = mt * 8 + tt * 2, m1 = m0 + 1;
        if (n_a < p.Nout) {
            if (m0 < p.M) p.y[(size_t)m0 * p.Nout + n_a] = __float2half_rn(o4.x);
            if (m1 < p.M) p.y[(size_t)m1 * p.Nout + n_a] = __float2half_rn(o4.y);
        }
        if (n_b < p.Nout) {
            if (m0 < p.M) p.y[(size_t)m0 * p.Nout + n_b] = __float2half_rn(o4.z);
            if (m1 < p.M) p.y[(size_t)m1 * p.Nout + n_b] = __float2half_rn(o4.w);
        }
    }
}

// =====================================================================================
// int8, group 32, f32
// =====================================================================================
//
// Per step a warp consumes 64 K (two groups) of a 16-row tile: lane (g,t) loads 16
// bytes = K [16t, 16t+16) for each of its two rows, so lanes t=0,1 hold the first
// group and t=2,3 the second.  Bytes become f16 exactly: b ^ 0x80 is b + 128 in 0..255,
// prmt places it under 0x64 giving 1024 + 128 + b, and subtracting 1152 leaves b.
// x is f32: it is split once per CTA into x_hi = f16(x) and x_lo = f16(x - x_hi), both
// multiplied exactly by the tensor core and summed in f32, which carries ~22 bits of x.
// The 8 batch columns of the mma are used to keep the two groups (and hi/lo) apart:
//     column 0: x_hi on the first group's K, 0 elsewhere   column 1: x_hi, second group
//     column 2: x_lo on the first group's K                column 3: x_lo, second group
// so one mma yields both group sums, each scaled by its own f32 scale afterwards.

constexpr int I8_UNROLL = 4;

struct GemvI8Params {
    const float* x;         // [K] (one batch row per blockIdx.y)
    const int8_t* w;        // [N, K]
    const float* scales;    // [N, G]
    float* y;               // [N]
    int N, K, G;
    size_t x_stride, y_stride;
};

__global__ void __launch_bounds__(512) lux_qgemv_i8_g32_f32(const GemvI8Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __half* xhi = reinterpret_cast<__half*>(smem);
    __half* xlo = xhi + p.K;
    float* red = reinterpret_cast<float*>(xlo + p.K);           // [nwarps][16]
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const int g = lane >> 2, t = lane & 3;
    const float* x = p.x + (size_t)blockIdx.y * p.x_stride;
    float* y = p.y + (size_t)blockIdx.y * p.y_stride;

    for (int k = tid * 4; k < p.K; k += nthreads * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + k);
        const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y);
        const __half h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
        *reinterpret_cast<__half2*>(xhi + k) = __halves2half2(h0, h1);
        *reinterpret_cast<__half2*>(xhi + k + 2) = __halves2half2(h2, h3);
        *reinterpret_cast<__half2*>(xlo + k) = __halves2half2(__float2half_rn(v.x - __half2float(h0)),
                                                             __float2half_rn(v.y - __half2float(h1)));
        *reinterpret_cast<__half2*>(xlo + k + 2) = __halves2half2(__float2half_rn(v.z - __half2float(h2)),
                                                                 __float2half_rn(v.w - __half2float(h3)));
    }
    __syncthreads();

    const int n0 = blockIdx.x * 16;
    const int ra = min(n0 + g, p.N - 1), rb = min(n0 + g + 8, p.N - 1);
    const uint4* wa = reinterpret_cast<const uint4*>(p.w + (size_t)ra * p.K) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(p.w + (size_t)rb * p.K) + t;
    const float2* sa = reinterpret_cast<const float2*>(p.scales + (size_t)ra * p.G);
    const float2* sb = reinterpret_cast<const float2*>(p.scales + (size_t)rb * p.G);
    // B-fragment source for this lane's batch column c = g (see the table above)
    const bool b_live = (g < 4) && ((t >> 1) == (g & 1));
    const __half* xsrc = (g < 2) ? xhi : xlo;

    const int steps = p.K >> 6;                                  // 64 K per step
    float res_a = 0.0f, res_b = 0.0f;
    const uint32_t bias = 0x64806480u;                           // f16x2 (1152, 1152)

    for (int sb0 = warp; sb0 < steps; sb0 += nwarps * I8_UNROLL) {
        uint4 qa[I8_UNROLL], qb[I8_UNROLL];
        float2 fa[I8_UNROLL], fb[I8_UNROLL];
#pragma unroll
        for (int u = 0; u < I8_UNROLL; u++) {
            const int s = sb0 + u * nwarps;
            if (s < steps) {
                qa[u] = ldg_stream(wa + s * 4);
                qb[u] = ldg_stream(wb + s * 4);
            }
        }
#pragma unroll
        for (int u = 0; u < I8_UNROLL; u++) {
            const int s = sb0 + u * nwarps;
            if (s < steps) {
                fa[u] = __ldg(sa + s);
                fb[u] = __ldg(sb + s);
            }
        }
#pragma unroll
        for (int u = 0; u < I8_UNROLL; u++) {
            const int s = sb0 + u * nwarps;
            if (s >= steps) break;
            uint4 xb0 = make_uint4(0, 0, 0, 0), xb1 = make_uint4(0, 0, 0, 0);
            if (b_live) {
                const uint4* xp = reinterpret_cast<const uint4*>(xsrc + s * 64 + t * 16);
                xb0 = xp[0];
                xb1 = xp[1];
            }
            const uint32_t xw[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
            const uint32_t wqa[4] = {qa[u].x, qa[u].y, qa[u].z, qa[u].w};
            const uint32_t wqb[4] = {qb[u].x, qb[u].y, qb[u].z, qb[u].w};
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t va = wqa[j] ^ 0x80808080u, vb = wqb[j] ^ 0x80808080u;
                const uint32_t a0 = hsub2_u32(prmt(va, 0x64646464u, 0x4140), bias);   // row a, bytes 0,1
                const uint32_t a1 = hsub2_u32(prmt(vb, 0x64646464u, 0x4140), bias);   // row b, bytes 0,1
                const uint32_t a2 = hsub2_u32(prmt(va, 0x64646464u, 0x4342), bias);   // row a, bytes 2,3
                const uint32_t a3 = hsub2_u32(prmt(vb, 0x64646464u, 0x4342), bias);   // row b, bytes 2,3
                mma16816(acc, a0, a1, a2, a3, xw[2 * j], xw[2 * j + 1], acc);
            }
            // columns (2t, 2t+1): lanes t=0 hold (hi,g0),(hi,g1); t=1 hold (lo,g0),(lo,g1);
            // t=2,3 hold zeros.  quantized_nax.wgsl:378: value = f32(q) * scale.
            res_a = fmaf(fa[u].x, acc[0], res_a);
            res_a = fmaf(fa[u].y, acc[1], res_a);
            res_b = fmaf(fb[u].x, acc[2], res_b);
            res_b = fmaf(fb[u].y, acc[3], res_b);
        }
    }
    // hi + lo parts sit in lanes t=0 and t=1
    res_a += __shfl_xor_sync(0xffffffffu, res_a, 1);
    res_b += __shfl_xor_sync(0xffffffffu, res_b, 1);
    if (t == 0) {
        red[warp * 16 + g] = res_a;
        red[warp * 16 + g + 8] = res_b;
    }
    __syncthreads();
    if (tid < 16) {
        float s = 0.0f;
        for (int w = 0; w < nwarps; w++) s += red[w * 16 + tid];
        if (n0 + tid < p.N) y[n0 + tid] = s;
    }
}

}  // namespace

// -------------------------------------------------------------------------------------
// Host-side launchers
// -------------------------------------------------------------------------------------

template <int MT, int RT, bool SW>
static cudaError_t launch_skinny_inst(const SkinnyParams& p, int grid, int threads, size_t smem, cudaStream_t st) {
    auto kfn = lux_qskinny_i4_g128<MT, RT, SW>;
    // Raise the dynamic shared-memory limit once per device, not on every launch.
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    kfn<<<grid, threads, smem, st>>>(p);
    return cudaGetLastError();
}

template <int MT, bool SW>
static cudaError_t launch_skinny_rt(int rt, const SkinnyParams& p, int grid, int threads, size_t smem, cudaStream_t st) {
    switch (rt) {
        case 1: return launch_skinny_inst<MT, 1, SW>(p, grid, threads, smem, st);
        case 2: return launch_skinny_inst<MT, 2, SW>(p, grid, threads, smem, st);
        default: return launch_skinny_inst<MT, 4, SW>(p, grid, threads, smem, st);
    }
}

LuxBackendError launch_qskinny_i4(Context* ctx, const QArgs& a) {
    if (a.M < 1 || a.M > 32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    SkinnyParams p{};
    p.x = (const __half*)a.x;
    p.w = a.w;
    p.scales = (const __half*)a.scales;
    p.zeros = a.zeros;
    p.y = (__half*)a.y;
    p.M = a.M;
    p.K = a.K;
    p.G = a.G;
    p.ZS = (a.G + 1) / 2;
    p.Nout = a.swiglu ? a.N / 2 : a.N;
    p.up_row_offset = a.swiglu ? a.N / 2 : 0;

    const int MT = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    const int tiles = (p.Nout + 15) / 16;
    const int sms = ctx->sm_count;

    // Warps per CTA split K; enough of them that every SM has ~16+ warps of loads in
    // flight even when there are few row tiles, but never more warps than groups.
    int wpc = g_tune.gemv_i4_warps;
    if (wpc <= 0) wpc = (tiles * 2 >= sms * 5) ? 4 : 8;
    wpc = std::max(1, std::min({wpc, 8, a.G}));
    // x chunk: keep the staged activations within ~64 KB so several CTAs fit per SM.
    const int budget = 64 * 1024;
    int kc_groups = a.G;
    while (kc_groups > wpc && (size_t)a.M * ((size_t)kc_groups * 256 + 64) > (size_t)budget)
        kc_groups = (kc_groups + 1) / 2;
    kc_groups = std::max(kc_groups, 1);
    p.kc_groups = kc_groups;
    p.xstride = kc_groups * 256 + 64;
    // Row tiles per CTA: share one x staging between tiles when the grid would
    // otherwise exceed what can be resident at once, or when x is re-staged per chunk.
    int rt = g_tune.gemv_i4_row_tiles;
    if (rt <= 0) {
        rt = 1;
        const int resident = sms * (MT >= 2 ? 4 : 6);
        while (rt < 4 && (tiles + rt - 1) / rt > resident) rt *= 2;
        if (a.M > 8 && rt < 4) rt = 4;
        if (a.swiglu && MT == 4) rt = std::min(rt, 2);          // register budget
    }
    rt = rt >= 4 ? 4 : (rt >= 2 ? 2 : 1);
    const int grid = (tiles + rt - 1) / rt;
    const int threads = wpc * 32;
    const int nacc = a.swiglu ? 2 : 1;
    const size_t smem = (size_t)a.M * p.xstride + (size_t)wpc * rt * nacc * MT * 32 * sizeof(float4);
    if (smem > 200 * 1024) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    cudaError_t e;
    if (a.swiglu) {
        e = MT == 1 ? launch_skinny_rt<1, true>(rt, p, grid, threads, smem, ctx->stream)
          : MT == 2 ? launch_skinny_rt<2, true>(rt, p, grid, threads, smem, ctx->stream)
                    : launch_skinny_rt<4, true>(rt, p, grid, threads, smem, ctx->stream);
    } else {
        e = MT == 1 ? launch_skinny_rt<1, false>(rt, p, grid, threads, smem, ctx->stream)
          : MT == 2 ? launch_skinny_rt<2, false>(rt, p, grid, threads, smem, ctx->stream)
                    : launch_skinny_rt<4, false>(rt, p, grid, threads, smem, ctx->stream);
    }
    count_launch(a.swiglu ? "lux_qskinny_i4_g128_swiglu" : "lux_qskinny_i4_g128");
    return map_cuda(e, "lux_qskinny_i4_g128");
}

LuxBackendError launch_qgemv_i8(Context* ctx, const QArgs& a) {
    if (a.K % 64) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    GemvI8Params p{};
    p.x = (const float*)a.x;
    p.w = (const int8_t*)a.w;
    p.scales = (const float*)a.scales;
    p.y = (float*)a.y;
    p.N = a.N;
    p.K = a.K;
    p.G = a.G;
    p.x_stride = a.K;
    p.y_stride = a.N;
    const int steps = a.K / 64;
    int wpc = g_tune.gemv_i8_warps;
    if (wpc <= 0) wpc = 8;
    wpc = std::max(1, std::min({wpc, 16, steps}));
    const size_t smem = (size_t)a.K * 4 + (size_t)wpc * 16 * sizeof(float);
    if (smem > 200 * 1024) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(lux_qgemv_i8_g32_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return map_cuda(e, "cudaFuncSetAttribute");
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    dim3 grid((a.N + 15) / 16, a.M);
    lux_qgemv_i8_g32_f32<<<grid, wpc * 32, smem, ctx->stream>>>(p);
    count_launch("lux_qgemv_i8_g32_f32");
    return map_cuda(cudaGetLastError(), "lux_qgemv_i8_g32_f32");
}

// Kernel-table hooks (kernel_table.cu): addresses of representative instantiations.
const void* kernel_addr_qskinny_i4() { return (const void*)lux_qskinny_i4_g128<1, 1, false>; }
const void* kernel_addr_qskinny_i4_swiglu() { return (const void*)lux_qskinny_i4_g128<1, 1, true>; }
const void* kernel_addr_qgemv_i8() { return (const void*)lux_qgemv_i8_g32_f32; }

}  // namespace luxcuda
