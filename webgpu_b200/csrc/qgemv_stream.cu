// lux_qgemv_i4_g128_stream -- int4 g128 decode GEMV (batch M <= 16) as a persistent,
// bulk-copy-fed streaming kernel for sm_100a.
//
// A decode GEMV moves tens of megabytes and lasts a few microseconds, i.e. a handful of
// DRAM latencies: what matters is that every SM has its whole share of the weight matrix
// in flight from the first nanosecond and never waits on a dependent load.  So:
//
//   * one CTA per SM, owning a contiguous range of 16-row weight tiles;
//   * a producer thread streams those tiles into a shared-memory ring with ONE tiled TMA
//     load per stage (completion on an mbarrier): ~200 KB per SM is in flight at once,
//     independent of registers or occupancy.  The tensor map views the packed matrix as
//     [128-byte line][row][byte] so that a stage lands as [line][row][128 B] with the
//     hardware 128-byte swizzle keyed by the ROW: the eight rows a quarter-warp reads at
//     the same K offset fall into different banks;
//   * eight consumer warps split each stage along K, unpack nibbles to f16 with
//     lop3 + one exact subtract (q - zp), multiply-accumulate on mma.sync.m16n8k16 with
//     f32 accumulation, apply the f16 group scale to the f32 group sum, and reduce across
//     warps through shared memory once per tile;
//   * the scales and zero-points of a tile travel the same way (two more bulk copies per
//     tile into a small ring of their own), so the consumers never issue a global load:
//     nothing but shared-memory reads sits on the critical path.
//
// Arithmetic is the same as lux_qskinny_i4_g128 (and as the reference's
// matmul_nax_grouped, kernels/wgsl/gpu/quantized_nax.wgsl:568-626, in a different
// summation order).  Every mbarrier wait is bounded; a wait that gives up sets a status
// word and the CTA drains and exits.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>

namespace luxcuda {

namespace {

constexpr int META_SLOTS = 8;                  // ring of per-tile scale / zero-point blocks
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
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy) : "memory");
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
    int cg;                 // groups per stage (multiple of the consumer warp count, even)
    int meta_bytes;         // bytes of one scale/zero-point slot
    int zeros_off;          // offset of the zero-points inside a slot
    int xstride;            // bytes between batch rows of the staged x
};

// Fragment row g (0..7) of the mma reads weight row rho(g) of the tile (and g+8 reads
// rho(g)+8).  rho puts the two rows that share a quarter-warp four apart, so the 128-byte
// swizzle (16-byte chunk index XOR row%8) sends them to different bank halves.
__device__ __forceinline__ int rho(int g) { return (g >> 1) | ((g & 1) << 2); }

// Shared memory (1024-byte aligned base): [ring: stages * cg * 1024][x staged: M * xstride]
// [meta ring][reduction: 2 buffers][barriers][abort flag].  A stage holds cg/2 lines of
// [16 rows][128 B].  CW = consumer warps (+ one producer warp).
template <int MT, bool SWIGLU, int CW>
__global__ void __launch_bounds__((CW + 1) * 32, 1)
lux_qgemv_i4_g128_stream(const __grid_constant__ CUtensorMap map_w, const StreamParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int NACC = SWIGLU ? 2 : 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.stages;
    const int stage_bytes = p.cg * 1024;               // cg/2 lines x 16 rows x 128 B

    unsigned char* ring = smem;
    unsigned char* xs = ring + (size_t)S * stage_bytes;
    unsigned char* meta = xs + (size_t)p.M * p.xstride;
    float4* red = reinterpret_cast<float4*>(meta + (size_t)META_SLOTS * p.meta_bytes);   // [2][CW][NACC*MT][32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * CW * NACC * MT * 32);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 4 + 2 * META_SLOTS);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(S + s); };
    auto red_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + b); };
    auto red_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 2 + b); };
    auto meta_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 4 + b); };
    auto meta_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 4 + META_SLOTS + b); };

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(red_full(b), CW);
            mbar_init(red_empty(b), 1);
        }
        for (int b = 0; b < META_SLOTS; b++) {
            mbar_init(meta_full(b), 1);
            mbar_init(meta_empty(b), CW);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // contiguous, balanced range of tiles for this CTA
    const int tile_lo = (int)(((long long)blockIdx.x * p.tiles) / gridDim.x);
    const int tile_hi = (int)(((long long)(blockIdx.x + 1) * p.tiles) / gridDim.x);
    const int nchunks = (p.G + p.cg - 1) / p.cg;

    if (warp == CW) {
        // ================================ producer ======================================
        const uint64_t policy = l2_evict_first_policy();
        int s = 0, ms = 0;
        uint32_t ph = 0, mph = 0;                    // ring phases, advanced on wrap-around
        bool ok = true;
        for (int tile = tile_lo; tile < tile_hi && ok; tile++) {
            for (int a = 0; a < NACC && ok; a++) {
                const int row0 = tile * 16 + a * p.up_row_offset;
                // scales [16, G] and zero-points [16, ZS] of this tile: two contiguous blocks
                ok = __all_sync(0xffffffffu, mbar_wait(meta_empty(ms), mph ^ 1u, abort_flag));
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t sb = (uint32_t)(32 * p.G), zb = p.zeros ? (uint32_t)(16 * p.ZS) : 0u;
                    mbar_expect_tx(meta_full(ms), sb + zb);
                    unsigned char* slot = meta + (size_t)ms * p.meta_bytes;
                    bulk_g2s(smem_u32(slot), p.scales + (size_t)row0 * p.G, sb, meta_full(ms), policy);
                    if (p.zeros)
                        bulk_g2s(smem_u32(slot + p.zeros_off), p.zeros + (size_t)row0 * p.ZS, zb, meta_full(ms), policy);
                }
                if (++ms == META_SLOTS) { ms = 0; mph ^= 1u; }
                for (int c = 0; c < nchunks; c++) {
                    ok = __all_sync(0xffffffffu, mbar_wait(empty(s), ph ^ 1u, abort_flag));
                    if (!ok) break;
                    if (lane == 0) {
                        // one box: bytes [0,128) x rows [row0, row0+16) x lines [c*cg/2, +cg/2);
                        // lines past the end of a row are zero-filled and still counted
                        mbar_expect_tx(full(s), (uint32_t)stage_bytes);
                        tma_load_3d(smem_u32(ring + (size_t)s * stage_bytes), &map_w, 0, row0, c * (p.cg >> 1), full(s), policy);
                    }
                    if (++s == S) { s = 0; ph ^= 1u; }
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

        bool ok = true;
        int s = 0, ms = 0;
        uint32_t ph = 0, mph = 0;
        const int rg = rho(g);                       // tile row this lane's fragment row g reads
        for (int tile = tile_lo; tile < tile_hi && ok; tile++) {
#pragma unroll
            for (int a = 0; a < NACC; a++) {
                if (!ok) break;
                // this tile's scales / zero-points have landed?
                ok = __all_sync(0xffffffffu, mbar_wait(meta_full(ms), mph, abort_flag));
                if (!ok) break;
                const unsigned char* slot = meta + (size_t)ms * p.meta_bytes;
                const __half* ms_a = reinterpret_cast<const __half*>(slot) + (size_t)rg * p.G;
                const __half* ms_b = ms_a + (size_t)8 * p.G;
                const unsigned char* mz_a = slot + p.zeros_off + (size_t)rg * p.ZS;
                const unsigned char* mz_b = mz_a + (size_t)8 * p.ZS;
                for (int c = 0; c < nchunks && ok; c++) {
                    ok = __all_sync(0xffffffffu, mbar_wait(full(s), ph, abort_flag));
                    if (!ok) break;
                    const unsigned char* st = ring + (size_t)s * stage_bytes;
                    const int gi0 = c * p.cg;
                    const int cgs = min(p.cg, p.G - gi0);          // groups of this stage inside the row

                    float acc[4][MT][4];
                    float sc_a[4], sc_b[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
#pragma unroll
                        for (int mt = 0; mt < MT; mt++)
#pragma unroll
                            for (int i = 0; i < 4; i++) acc[u][mt][i] = 0.0f;

#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int gl = warp * gpw + u;                 // group inside the stage
                        sc_a[u] = 0.0f;
                        sc_b[u] = 0.0f;
                        if (u < gpw && gl < cgs) {
                            const int gi = gi0 + gl;
                            // line gl/2, row rg, logical 16-byte chunk (gl%2)*4 + t, swizzled by row%8
                            const unsigned char* ln = st + (gl >> 1) * 2048 + rg * 128 + (((((gl & 1) << 2) | t) ^ rg) << 4);
                            const uint4 qa = *reinterpret_cast<const uint4*>(ln);
                            const uint4 qb = *reinterpret_cast<const uint4*>(ln + 1024);
                            sc_a[u] = __half2float(ms_a[gi]);
                            sc_b[u] = __half2float(ms_b[gi]);
                            uint32_t zpa = 8u, zpb = 8u;                // symmetric: stored value - 8
                            if (p.zeros) {
                                zpa = ((uint32_t)mz_a[gi >> 1] >> ((gi & 1) * 4)) & 0xFu;
                                zpb = ((uint32_t)mz_b[gi >> 1] >> ((gi & 1) * 4)) & 0xFu;
                            }
                            const uint32_t za_lo = (0x6400u | zpa) * 0x00010001u;
                            const uint32_t za_hi = (0x5400u | (zpa << 4)) * 0x00010001u;
                            const uint32_t zb_lo = (0x6400u | zpb) * 0x00010001u;
                            const uint32_t zb_hi = (0x5400u | (zpb << 4)) * 0x00010001u;
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
                    if (++s == S) { s = 0; ph ^= 1u; }
#pragma unroll
                    for (int u = 0; u < 4; u++)
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            res[a][mt][0] = fmaf(sc_a[u], acc[u][mt][0], res[a][mt][0]);
                            res[a][mt][1] = fmaf(sc_a[u], acc[u][mt][1], res[a][mt][1]);
                            res[a][mt][2] = fmaf(sc_b[u], acc[u][mt][2], res[a][mt][2]);
                            res[a][mt][3] = fmaf(sc_b[u], acc[u][mt][3], res[a][mt][3]);
                        }
                }
                // done with this tile's scale block
                __syncwarp();
                if (lane == 0) mbar_arrive(meta_empty(ms));
                if (++ms == META_SLOTS) { ms = 0; mph ^= 1u; }
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
                    const int n_a = tile * 16 + rg, n_b = n_a + 8;
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

template <int MT, bool SW, int CW>
cudaError_t launch_stream_inst(const CUtensorMap& map, const StreamParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i4_g128_stream<MT, SW, CW>;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    kfn<<<grid, (CW + 1) * 32, smem, st>>>(map, p);
    return cudaGetLastError();
}

template <int CW>
LuxBackendError launch_stream_cw(Context* ctx, const QArgs& a) {
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
    p.tiles = p.Nout / 16;
    p.xstride = a.G * 256 + 64;
    p.zeros_off = (32 * a.G + 15) / 16 * 16;
    p.meta_bytes = p.zeros_off + (16 * p.ZS + 15) / 16 * 16;

    const size_t smem_max = 227 * 1024;
    const size_t x_bytes = (size_t)a.M * p.xstride;
    const size_t red_bytes = (size_t)2 * CW * nacc * MT * 32 * sizeof(float4);
    const size_t fixed = 1024 + x_bytes + red_bytes + (size_t)META_SLOTS * p.meta_bytes + 1024;
    int cg = g_tune.gemv_stream_cg > 0 ? g_tune.gemv_stream_cg * CW : 32;      // groups per stage
    cg = std::max(CW, std::min(cg, 32) / CW * CW);
    while (cg > CW && cg > a.G) cg -= CW;
    int stages = 0;
    for (;; cg -= CW) {
        const size_t stage_bytes = (size_t)cg * 1024;
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
    const size_t smem = 1024 + (size_t)stages * cg * 1024 + x_bytes + (size_t)META_SLOTS * p.meta_bytes + red_bytes +
                       (size_t)(2 * stages + 4 + 2 * META_SLOTS) * 8 + 64;

    // Packed weights viewed as [line of 128 B][row][byte]: a box of (128 B, 16 rows, cg/2
    // lines) lands in shared memory as [line][row][128 B], swizzled by the row index.
    alignas(64) CUtensorMap map;
    const uint64_t dims[3] = {128, (uint64_t)a.N, (uint64_t)a.K / 256};
    const uint64_t strides[2] = {(uint64_t)a.K / 2, 128};
    const uint32_t box[3] = {128, 16, (uint32_t)cg / 2};
    if (!encode_tensor_map_u8(&map, 3, a.w, dims, strides, box, true)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    cudaError_t e;
    if (a.swiglu) e = MT == 1 ? launch_stream_inst<1, true, CW>(map, p, grid, smem, ctx->stream)
                              : launch_stream_inst<2, true, CW>(map, p, grid, smem, ctx->stream);
    else          e = MT == 1 ? launch_stream_inst<1, false, CW>(map, p, grid, smem, ctx->stream)
                              : launch_stream_inst<2, false, CW>(map, p, grid, smem, ctx->stream);
    count_launch();
    return map_cuda(e, "lux_qgemv_i4_g128_stream");
}

}  // namespace

// Returns NOT_SUPPORTED when the shape does not suit the ring kernel (the caller then
// uses lux_qskinny_i4_g128): batch above 16, fewer than 8 or an odd number of groups per
// row (a 128-byte line of packed weights holds two groups), an output size
// that is not a multiple of the 16-row tile (the per-tile scale block must be one aligned,
// contiguous copy), or activations too large to stage beside a useful ring.
LuxBackendError launch_qgemv_i4_stream(Context* ctx, const QArgs& a) {
    const int nout = a.swiglu ? a.N / 2 : a.N;
    if (a.M < 1 || a.M > 16 || a.G < 8 || (a.G & 1) || nout % 16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    int cw = g_tune.gemv_stream_warps > 0 ? g_tune.gemv_stream_warps : 16;
    if (a.G < 16) cw = 8;
    return cw >= 16 ? launch_stream_cw<16>(ctx, a) : launch_stream_cw<8>(ctx, a);
}

const void* kernel_addr_qgemv_i4_stream() { return (const void*)lux_qgemv_i4_g128_stream<1, false, 16>; }

}  // namespace luxcuda
