// lux_qgemv_i4_g128_stream -- int4 g128 decode GEMV (batch M <= 16) as a persistent,
// bulk-copy-fed streaming kernel for sm_100a.
//
// A decode GEMV moves tens of megabytes and lasts a few microseconds, i.e. a handful of
// DRAM latencies: what matters is that every SM has its whole share of the weight matrix
// in flight from the first nanosecond and never waits on a dependent load.  So:
//
//   * one CTA per SM, owning a contiguous range of 16-row weight tiles;
//   * a producer warp streams the packed rows of those tiles into a shared-memory ring
//     with cp.async.bulk (one copy per row piece, completion on an mbarrier): ~200 KB per
//     SM is in flight at once, independent of registers or occupancy;
//   * eight consumer warps split each stage along K, unpack nibbles to f16 with
//     lop3 + one exact subtract (q - zp), multiply-accumulate on mma.sync.m16n8k16 with
//     f32 accumulation, apply the f16 group scale to the f32 group sum, and reduce across
//     warps through shared memory once per tile;
//   * scales and zero-points for the NEXT stage are prefetched into registers while the
//     current stage is computed, so no load sits on the critical path.
//
// Arithmetic is the same as lux_qskinny_i4_g128 (and as the reference's
// matmul_nax_grouped, kernels/wgsl/gpu/quantized_nax.wgsl:568-626, in a different
// summation order).  Every mbarrier wait is bounded; a wait that gives up sets a status
// word and the CTA drains and exits.
#include "common.cuh"

#include <algorithm>

namespace luxcuda {

namespace {

constexpr int CW = 8;                          // consumer warps
constexpr int STREAM_THREADS = (CW + 1) * 32;  // + one producer warp
constexpr uint32_t WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 31u) == 31u && *abort_flag) return false;
    }
    *abort_flag = 1u;
    return false;
}
// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a
// multiple of 16.  The weights are read exactly once, so they are marked evict-first in L2.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
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
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + __expf(-x)); }

struct StreamParams {
    const __half* x;        // [M, K]
    const uint8_t* w;       // [Nw, K/2]
    const __half* scales;   // [Nw, G]
    const uint8_t* zeros;   // [Nw, ZS] or null
    __half* y;              // [M, Nout]
    uint32_t* status;
    int M, Nout, K, G, ZS;
    int up_row_offset;
    int tiles;              // ceil(Nout / 16)
    int stages;             // ring depth
    int cg;                 // groups per stage (multiple of CW, <= 4*CW)
    int xstride;            // bytes between batch rows of the staged x
    int row_pitch;          // bytes between weight rows inside a stage (cg*64 + 64)
};

// Shared memory: [x staged: M * xstride][ring: stages * 16 * row_pitch][reduction: 2 buffers]
// [barriers: full[stages], empty[stages]][abort flag]
template <int MT, bool SWIGLU>
__global__ void __launch_bounds__(STREAM_THREADS, 1) lux_qgemv_i4_g128_stream(const StreamParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NACC = SWIGLU ? 2 : 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.stages;
    const int stage_bytes = 16 * p.row_pitch;

    unsigned char* xs = smem;
    unsigned char* ring = xs + (size_t)p.M * p.xstride;
    float4* red = reinterpret_cast<float4*>(ring + (size_t)S * stage_bytes);       // [2][CW][NACC*MT][32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * CW * NACC * MT * 32);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 4);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(S + s); };
    auto red_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + b); };
    auto red_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 2 + b); };

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(red_full(b), CW);
            mbar_init(red_empty(b), 1);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // contiguous, balanced range of tiles for this CTA
    const int tile_lo = (int)(((long long)blockIdx.x * p.tiles) / gridDim.x);
    const int tile_hi = (int)(((long long)(blockIdx.x + 1) * p.tiles) / gridDim.x);
    const int nchunks = (p.G + p.cg - 1) / p.cg;
    const size_t row_bytes = (size_t)p.K >> 1;

    if (warp == CW) {
        // ================================ producer ======================================
        const uint64_t policy = l2_evict_first_policy();
        int it = 0;
        bool ok = true;
        for (int tile = tile_lo; tile < tile_hi && ok; tile++) {
            for (int a = 0; a < NACC && ok; a++) {
                for (int c = 0; c < nchunks; c++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (uint32_t)(it / S) & 1u;
                    const int gi0 = c * p.cg;
                    const int cgs = min(p.cg, p.G - gi0);
                    ok = __all_sync(0xffffffffu, mbar_wait(empty(s), ph ^ 1u, abort_flag));
                    if (!ok) break;
                    if (lane == 0) mbar_expect_tx(full(s), (uint32_t)(16 * cgs * 64));
                    __syncwarp();
                    if (lane < 16) {
                        const int row = min(tile * 16 + lane, p.Nout - 1) + a * p.up_row_offset;
                        bulk_g2s(smem_u32(ring + (size_t)s * stage_bytes + lane * p.row_pitch),
                                 p.w + (size_t)row * row_bytes + (size_t)gi0 * 64, (uint32_t)(cgs * 64), full(s), policy);
                    }
                }
            }
        }
    } else {
        // ================================ consumers =====================================
        // Stage x once, in mma-fragment order (see lux_qskinny_i4_g128): per group of 128 K,
        // chunk (j*4 + t) holds x[32t + 8j + {0,4,1,5,2,6,3,7}].
        {
            const int chunks_per_row = p.G * 16;
            const int total = p.M * chunks_per_row;
            for (int i = tid; i < total; i += CW * 32) {
                const int m = i / chunks_per_row, c = i - m * chunks_per_row;
                const int grp = c >> 4, cc = c & 15, tt = cc >> 2, j = cc & 3;
                const uint4 s4 = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + (size_t)grp * 128 + cc * 8);
                uint4 d;
                d.x = prmt(s4.x, s4.z, 0x5410);
                d.y = prmt(s4.x, s4.z, 0x7632);
                d.z = prmt(s4.y, s4.w, 0x5410);
                d.w = prmt(s4.y, s4.w, 0x7632);
                *reinterpret_cast<uint4*>(xs + (size_t)m * p.xstride + grp * 256 + (j * 4 + tt) * 16) = d;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");

        const int gpw = p.cg / CW;                 // groups per warp per stage (1, 2 or 4), contiguous
        float res[NACC][MT][4];
#pragma unroll
        for (int a = 0; a < NACC; a++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) res[a][mt][i] = 0.0f;

        // scale / zero-point prefetch for one stage: this lane's two rows, up to 4 groups
        struct Meta { float sa[4], sb[4]; uint32_t za[4], zb[4]; };
        auto load_meta = [&](int tile, int a, int c, Meta& mt_) {
            const int ra = min(tile * 16 + g, p.Nout - 1) + a * p.up_row_offset;
            const int rb = min(tile * 16 + g + 8, p.Nout - 1) + a * p.up_row_offset;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int gi = c * p.cg + warp * gpw + u;
                const bool live = u < gpw && gi < p.G;
                const int gic = live ? gi : 0;
                mt_.sa[u] = live ? __half2float(__ldg(p.scales + (size_t)ra * p.G + gic)) : 0.0f;
                mt_.sb[u] = live ? __half2float(__ldg(p.scales + (size_t)rb * p.G + gic)) : 0.0f;
                if (p.zeros) {
                    mt_.za[u] = (__ldg(p.zeros + (size_t)ra * p.ZS + (gic >> 1)) >> ((gic & 1) * 4)) & 0xFu;
                    mt_.zb[u] = (__ldg(p.zeros + (size_t)rb * p.ZS + (gic >> 1)) >> ((gic & 1) * 4)) & 0xFu;
                } else {
                    mt_.za[u] = 8u;
                    mt_.zb[u] = 8u;
                }
            }
        };

        Meta cur, nxt;
        bool ok = true;
        if (tile_lo < tile_hi) load_meta(tile_lo, 0, 0, cur);
        int it = 0;
        for (int tile = tile_lo; tile < tile_hi && ok; tile++) {
#pragma unroll
            for (int a = 0; a < NACC; a++) {
                for (int c = 0; c < nchunks && ok; c++, it++) {
                    // prefetch the next stage's scales while this one is waited for / computed
                    {
                        int nc = c + 1, na = a, ntile = tile;
                        if (nc == nchunks) { nc = 0; na = a + 1; }
                        if (na == NACC) { na = 0; ntile = tile + 1; }
                        if (ntile < tile_hi) load_meta(ntile, na, nc, nxt);
                    }
                    const int s = it % S;
                    const uint32_t ph = (uint32_t)(it / S) & 1u;
                    ok = __all_sync(0xffffffffu, mbar_wait(full(s), ph, abort_flag));
                    if (!ok) break;
                    const unsigned char* st = ring + (size_t)s * stage_bytes;
                    const int gi0 = c * p.cg;
                    const int cgs = min(p.cg, p.G - gi0);

                    float acc[4][MT][4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
#pragma unroll
                        for (int mt = 0; mt < MT; mt++)
#pragma unroll
                            for (int i = 0; i < 4; i++) acc[u][mt][i] = 0.0f;

#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int gl = warp * gpw + u;                 // group inside the stage
                        if (u < gpw && gl < cgs) {
                            const uint4 qa = *reinterpret_cast<const uint4*>(st + g * p.row_pitch + gl * 64 + t * 16);
                            const uint4 qb = *reinterpret_cast<const uint4*>(st + (g + 8) * p.row_pitch + gl * 64 + t * 16);
                            const uint32_t za_lo = (0x6400u | cur.za[u]) * 0x00010001u;
                            const uint32_t za_hi = (0x5400u | (cur.za[u] << 4)) * 0x00010001u;
                            const uint32_t zb_lo = (0x6400u | cur.zb[u]) * 0x00010001u;
                            const uint32_t zb_hi = (0x5400u | (cur.zb[u] << 4)) * 0x00010001u;
                            const uint32_t wqa[4] = {qa.x, qa.y, qa.z, qa.w};
                            const uint32_t wqb[4] = {qb.x, qb.y, qb.z, qb.w};
                            const unsigned char* xg = xs + (gi0 + gl) * 256 + t * 16;
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
                                    mma16816(acc[u][mt], a0, a1, a2, a3, xv.x, xv.y);
                                    mma16816(acc[u][mt], a4, a5, a6, a7, xv.z, xv.w);
                                }
                            }
                        }
                    }
                    // this warp is done reading the stage: hand it back to the producer
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty(s));
#pragma unroll
                    for (int u = 0; u < 4; u++)
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            res[a][mt][0] = fmaf(cur.sa[u], acc[u][mt][0], res[a][mt][0]);
                            res[a][mt][1] = fmaf(cur.sa[u], acc[u][mt][1], res[a][mt][1]);
                            res[a][mt][2] = fmaf(cur.sb[u], acc[u][mt][2], res[a][mt][2]);
                            res[a][mt][3] = fmaf(cur.sb[u], acc[u][mt][3], res[a][mt][3]);
                        }
                    cur = nxt;
                }
            }
            if (!ok) break;
            // ---- tile finished: reduce the CW partial sums, one reducer warp per tile.
            // Two buffers, handed over with mbarriers (bounded waits, like every other wait
            // here): writers wait until the buffer's previous reducer has released it.
            const int ti = tile - tile_lo;
            const int buf = ti & 1;
            const uint32_t use = (uint32_t)(ti >> 1);
            float4* rb = red + (size_t)buf * CW * NACC * MT * 32;
            ok = __all_sync(0xffffffffu, mbar_wait(red_empty(buf), (use & 1u) ^ 1u, abort_flag));
            if (!ok) break;
#pragma unroll
            for (int a = 0; a < NACC; a++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    rb[(warp * NACC * MT + a * MT + mt) * 32 + lane] =
                        make_float4(res[a][mt][0], res[a][mt][1], res[a][mt][2], res[a][mt][3]);
#pragma unroll
                    for (int i = 0; i < 4; i++) res[a][mt][i] = 0.0f;
                }
            __syncwarp();
            if (lane == 0) mbar_arrive(red_full(buf));
            if (warp == (ti % CW)) {
                ok = __all_sync(0xffffffffu, mbar_wait(red_full(buf), use & 1u, abort_flag));
                if (!ok) break;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    float4 sum[NACC];
#pragma unroll
                    for (int a = 0; a < NACC; a++) {
                        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int w = 0; w < CW; w++) {
                            const float4 v = rb[(w * NACC * MT + a * MT + mt) * 32 + lane];
                            s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
                        }
                        sum[a] = s4;
                    }
                    float4 o4 = sum[0];
                    if (SWIGLU) {
                        o4.x = silu_f32(sum[0].x) * sum[NACC - 1].x;
                        o4.y = silu_f32(sum[0].y) * sum[NACC - 1].y;
                        o4.z = silu_f32(sum[0].z) * sum[NACC - 1].z;
                        o4.w = silu_f32(sum[0].w) * sum[NACC - 1].w;
                    }
                    const int n_a = tile * 16 + g, n_b = n_a + 8;
                    const int m0 = mt * 8 + t * 2, m1 = m0 + 1;
                    if (n_a < p.Nout) {
                        if (m0 < p.M) p.y[(size_t)m0 * p.Nout + n_a] = __float2half_rn(o4.x);
                        if (m1 < p.M) p.y[(size_t)m1 * p.Nout + n_a] = __float2half_rn(o4.y);
                    }
                    if (n_b < p.Nout) {
                        if (m0 < p.M) p.y[(size_t)m0 * p.Nout + n_b] = __float2half_rn(o4.z);
                        if (m1 < p.M) p.y[(size_t)m1 * p.Nout + n_b] = __float2half_rn(o4.w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(red_empty(buf));
            }
        }
    }

    __syncthreads();
    if (*abort_flag) {
        // A bounded wait gave up: report it and give copies still in flight time to land in
        // this CTA's shared memory before it is released.
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C050002u);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
}

template <int MT, bool SW>
cudaError_t launch_stream_inst(const StreamParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i4_g128_stream<MT, SW>;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    kfn<<<grid, STREAM_THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

}  // namespace

// Returns NOT_SUPPORTED when the shape does not suit the ring kernel (the caller then
// uses lux_qskinny_i4_g128).
LuxBackendError launch_qgemv_i4_stream(Context* ctx, const QArgs& a) {
    if (a.M < 1 || a.M > 16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (a.G < CW) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int MT = a.M <= 8 ? 1 : 2;
    const int nacc = a.swiglu ? 2 : 1;
    StreamParams p{};
    p.x = (const __half*)a.x;
    p.w = a.w;
    p.scales = (const __half*)a.scales;
    p.zeros = a.zeros;
    p.y = (__half*)a.y;
    p.status = ctx->d_status;
    p.M = a.M;
    p.K = a.K;
    p.G = a.G;
    p.ZS = (a.G + 1) / 2;
    p.Nout = a.swiglu ? a.N / 2 : a.N;
    p.up_row_offset = a.swiglu ? a.N / 2 : 0;
    p.tiles = (p.Nout + 15) / 16;
    p.xstride = a.G * 256 + 64;

    const size_t smem_max = 227 * 1024;
    const size_t x_bytes = (size_t)a.M * p.xstride;
    const size_t red_bytes = (size_t)2 * CW * nacc * MT * 32 * sizeof(float4);
    int cg = g_tune.gemv_stream_cg > 0 ? g_tune.gemv_stream_cg * CW : 4 * CW;   // groups per stage
    cg = std::min(cg, 4 * CW);
    while (cg > CW && cg > a.G) cg -= CW;
    int stages = 0;
    for (;; cg -= CW) {
        const size_t stage_bytes = (size_t)16 * (cg * 64 + 64);
        const size_t fixed = x_bytes + red_bytes + 2048;
        stages = fixed < smem_max ? (int)((smem_max - fixed) / (stage_bytes + 16)) : 0;
        if (stages >= 4 || cg == CW) break;
    }
    if (stages < 3) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int nchunks = (a.G + cg - 1) / cg;
    const int grid = std::min(ctx->sm_count, p.tiles);
    const int max_items = ((p.tiles + grid - 1) / grid) * nacc * nchunks;
    stages = std::min({stages, max_items, g_tune.gemv_stream_stages > 0 ? g_tune.gemv_stream_stages : 64});
    stages = std::max(stages, 1);
    p.cg = cg;
    p.stages = stages;
    p.row_pitch = cg * 64 + 64;
    const size_t smem = x_bytes + (size_t)stages * 16 * p.row_pitch + red_bytes + (size_t)stages * 16 + 32 + 64;

    cudaError_t e;
    if (a.swiglu) e = MT == 1 ? launch_stream_inst<1, true>(p, grid, smem, ctx->stream)
                              : launch_stream_inst<2, true>(p, grid, smem, ctx->stream);
    else          e = MT == 1 ? launch_stream_inst<1, false>(p, grid, smem, ctx->stream)
                              : launch_stream_inst<2, false>(p, grid, smem, ctx->stream);
    count_launch();
    return map_cuda(e, "lux_qgemv_i4_g128_stream");
}

const void* kernel_addr_qgemv_i4_stream() { return (const void*)lux_qgemv_i4_g128_stream<1, false>; }

}  // namespace luxcuda
