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
//   * 8 or 16 consumer warps split each stage along K, turn nibbles into exact f16 values
//     with one lop3 per pair, multiply-accumulate on mma.sync.m16n8k16 with f32
//     accumulation, subtract the zero-point term per group ((1024 + zp) * sum of x, see the
//     kernel comment), apply the f16 group scale to the f32 group sum, and reduce across
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
#include <type_traits>

namespace luxcuda {

namespace {

constexpr int META_SLOTS = 8;                  // ring of per-tile scale / zero-point blocks
// one try_wait may suspend for a few microseconds; 2^15 of them bound a wait to ~0.1 s
constexpr uint32_t WAIT_LIMIT = 1u << 15;

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
// Warp-level wait: lane 0 polls (32 lanes polling the same barrier word are served one by
// one), the outcome is broadcast, and __syncwarp orders the other lanes' later reads after
// lane 0's acquire.  Must be called by a converged warp.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag);
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
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
    int tiles_base, tiles_rem;   // CTA b owns tiles [b*base + min(b, rem), +base + (b < rem))
    int stages;             // ring depth
    int cg;                 // groups per stage (= consumer warps * groups per warp, even)
    int nchunks;            // stages per (tile, gate/up) = ceil(G / cg)
    int meta_bytes;         // bytes of one scale/zero-point slot
    int zeros_off;          // offset of the zero-points inside a slot
    int xstride;            // bytes between batch rows of the staged x
    int tb;                 // tiles per reduction batch
    int tmax;               // lanes t < tmax hold live batch columns (ceil(min(M, 8) / 2))
};

// Fragment row g (0..7) of the mma reads weight row rho(g) of the tile (and g+8 reads
// rho(g)+8).  rho puts the two rows that share a quarter-warp four apart, so the 128-byte
// swizzle (16-byte chunk index XOR row%8) sends them to different bank halves.
__device__ __forceinline__ int rho(int g) { return (g >> 1) | ((g & 1) << 2); }
__device__ __forceinline__ int rho_inv(int r) { return ((r & 3) << 1) | (r >> 2); }

// Shared memory (1024-byte aligned base):
//   [ring: stages * cg * 1024]   a stage holds cg/2 lines of [16 rows][128 B], swizzled
//   [x staged: M * xstride]      f16 activations in mma-fragment order
//   [xsum: G * 8*MT * 8]         per (group, batch row): {sum x, 960 * sum of odd-k x} f32
//   [meta ring: 8 slots]         per-tile scales [16][G] f16 + zero-points [16][ZS]
//   [partials: tb tiles x CW warps x (gate/up) x MT x 8*tmax float4]
//   [barriers][abort flag]
// CW = consumer warps (+ one producer warp), GPW = groups per warp per stage.
//
// Zero-points are folded out of the inner loop: the mma multiplies x by the RAW nibble
// patterns (1024 + n for even k, 64 + n for odd k, exact in f16) and the group sum is
// corrected afterwards,
//   sum_k (n_k - zp) x_k = acc - (1024 + zp) * sum_k x_k + 960 * sum_{k odd} x_k,
// which is the same integer-subtract-then-multiply value up to f32 rounding.
//
// Each warp owns a K slice of every stage, so a tile's result is the sum of CW partial
// vectors.  Warps drop their partials into shared memory without waiting for anybody and
// the CTA reduces a whole batch of tiles at once (one bounded hand-over per batch).
template <int MT, bool SWIGLU, int CW, int GPW>
__global__ void __launch_bounds__((CW + 1) * 32, 1)
lux_qgemv_i4_g128_stream(const __grid_constant__ CUtensorMap map_w, const StreamParams p) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by OFFSET from the __shared__ symbol, so that every access below
    // stays a 32-bit shared-memory access (a round trip through an integer would turn them
    // into generic 64-bit ones).
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int NACC = SWIGLU ? 2 : 1;
    constexpr int MPAD = 8 * MT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    const int stage_bytes = p.cg * 1024;               // cg/2 lines x 16 rows x 128 B
    const int slot4 = 8 * p.tmax;                      // float4 per (tile, warp, gate/up, mt)

    unsigned char* ring = smem;
    unsigned char* xs = ring + (size_t)S * stage_bytes;
    float2* xsum = reinterpret_cast<float2*>(xs + (size_t)p.M * p.xstride);
    unsigned char* meta = reinterpret_cast<unsigned char*>(xsum + (size_t)p.G * MPAD);
    float4* part = reinterpret_cast<float4*>(meta + (size_t)META_SLOTS * p.meta_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(part + (size_t)p.tb * CW * NACC * MT * slot4);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 2 + 2 * META_SLOTS);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(S + s); };
    const uint32_t batch_full = bar0 + 8u * (uint32_t)(2 * S);
    const uint32_t batch_empty = bar0 + 8u * (uint32_t)(2 * S + 1);
    auto meta_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 2 + b); };
    auto meta_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * S + 2 + META_SLOTS + b); };

    // contiguous, balanced range of tiles for this CTA (split computed on the host)
    const int b = (int)blockIdx.x;
    const int tile_lo = b * p.tiles_base + min(b, p.tiles_rem);
    const int tile_hi = tile_lo + p.tiles_base + (b < p.tiles_rem ? 1 : 0);
    const int nchunks = p.nchunks;

    if (warp == CW) {
        // ================================ producer (one thread) =========================
        // Lane 0 does all the work; the CTA-wide barrier in the middle is executed by the
        // whole warp together (bar.sync needs a converged warp).
        const uint64_t policy = l2_evict_first_policy();
        const uint32_t sb = (uint32_t)(32 * p.G), zb = p.zeros ? (uint32_t)(16 * p.ZS) : 0u;
        const int lines = p.cg >> 1;
        int s = 0, ms = 0, tile = tile_lo, a = 0, c = 0;
        uint32_t ph = 0, mph = 0;
        const int total = (tile_hi - tile_lo) * NACC * nchunks;
        const int pre = min(total, min(S, META_SLOTS));
        // Issues the next stage (and, with a tile's first stage, its scale block).  The
        // first ring-full of stages needs no wait: every barrier is still in its first phase.
        auto produce = [&](bool may_wait) -> bool {
            const int row0 = tile * 16 + a * p.up_row_offset;
            if (may_wait && !mbar_wait(empty(s), ph ^ 1u, abort_flag)) return false;
            // one box: bytes [0,128) x rows [row0, row0+16) x lines [c*lines, +lines);
            // lines past the end of a row are zero-filled and still counted
            mbar_expect_tx(full(s), (uint32_t)stage_bytes);
            tma_load_3d(smem_u32(ring + (size_t)s * stage_bytes), &map_w, 0, row0, c * lines, full(s), policy);
            if (++s == S) { s = 0; ph ^= 1u; }
            if (c == 0) {
                // scales [16, G] and zero-points [16, ZS] of this tile: two contiguous blocks
                if (may_wait && !mbar_wait(meta_empty(ms), mph ^ 1u, abort_flag)) return false;
                unsigned char* slot = meta + (size_t)ms * p.meta_bytes;
                mbar_expect_tx(meta_full(ms), sb + zb);
                bulk_g2s(smem_u32(slot), p.scales + (size_t)row0 * p.G, sb, meta_full(ms), policy);
                if (p.zeros)
                    bulk_g2s(smem_u32(slot + p.zeros_off), p.zeros + (size_t)row0 * p.ZS, zb, meta_full(ms), policy);
                if (++ms == META_SLOTS) { ms = 0; mph ^= 1u; }
            }
            if (++c == nchunks) { c = 0; if (++a == NACC) { a = 0; ++tile; } }
            return true;
        };
        // barrier i of the block [full | empty | batch_full, batch_empty | meta_full | meta_empty]
        // is initialised by lane i (mod 32): counts 1 for the copy barriers, CW for the rest
        if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int i = lane; i < 2 * S + 2 + 2 * META_SLOTS; i += 32) {
            const bool by_copy = i < S || (i >= 2 * S + 2 && i < 2 * S + 2 + META_SLOTS);
            mbar_init(bar0 + 8u * (uint32_t)i, by_copy ? 1u : (uint32_t)CW);
        }
        if (lane == 0) *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        asm volatile("bar.sync 0;" ::: "memory");           // barriers are live for everybody
        if (lane == 0) {
            for (int it = 0; it < pre; it++) produce(false);   // first ring-full: nothing to wait for
            for (int it = pre; it < total; it++)
                if (!produce(true)) break;
        }
        __syncwarp();
    } else {
        // ================================ consumers =====================================
        const int g = lane >> 2, t = lane & 3;
        asm volatile("bar.sync 0;" ::: "memory");         // barriers initialised; the producer starts streaming
        // Stage x once, in mma-fragment order (see lux_qskinny_i4_g128): per group of 128 K,
        // chunk (j*4 + t) holds x[32t + 8j + {0,4,1,5,2,6,3,7}].  The same pass forms, per
        // (batch row, group), sum x and 960 * (sum of x at odd k) in f32: the 16 chunks of a
        // group sit in 16 consecutive lanes.
        for (int i = tid; i < p.G * MPAD; i += CW * 32)
            if ((i % MPAD) >= p.M) xsum[i] = make_float2(0.f, 0.f);
        for (int m = 0; m < p.M; m++) {
            const __half* xrow = p.x + (size_t)m * p.K;
            unsigned char* xdst = xs + (size_t)m * p.xstride;
            for (int c = tid; c < p.G * 16; c += CW * 32) {
                const int grp = c >> 4, cc = c & 15, tt = cc >> 2, j = cc & 3;
                const uint4 s4 = *reinterpret_cast<const uint4*>(xrow + c * 8);
                uint4 d;
                d.x = prmt(s4.x, s4.z, 0x5410);
                d.y = prmt(s4.x, s4.z, 0x7632);
                d.z = prmt(s4.y, s4.w, 0x5410);
                d.w = prmt(s4.y, s4.w, 0x7632);
                *reinterpret_cast<uint4*>(xdst + grp * 256 + (j * 4 + tt) * 16) = d;
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&s4.z));
                const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&s4.w));
                float se = (f0.x + f1.x) + (f2.x + f3.x), so = (f0.y + f1.y) + (f2.y + f3.y);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
                    se += __shfl_xor_sync(0xffffffffu, se, o);
                    so += __shfl_xor_sync(0xffffffffu, so, o);
                }
                if (cc == 0) xsum[grp * MPAD + m] = make_float2(se + so, 960.0f * so);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");

        float res[NACC][MT][4];
        bool ok = true;
        int s = 0, ms = 0;
        uint32_t ph = 0, mph = 0, bph = 0;
        const int rg = rho(g);                       // tile row this lane's fragment row g reads
        const int w_off = rg * 128;                  // row inside a line
        // batch column (mt*8 + g) of the mma's 8-column operand: lanes whose column is past
        // the batch feed zeros and skip the shared-memory read
        int xm_off[MT];
        bool xm_live[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            xm_live[mt] = mt * 8 + g < p.M;
            xm_off[mt] = min(mt * 8 + g, p.M - 1) * p.xstride + t * 16;
        }

        for (int tile0 = tile_lo; tile0 < tile_hi && ok; tile0 += p.tb) {
            const int tile1 = min(tile0 + p.tb, tile_hi);
            if (tile0 != tile_lo) {
                // the previous batch's partials must have been consumed before they are overwritten
                ok = warp_wait(batch_empty, bph ^ 1u, abort_flag, lane);
                if (!ok) break;
            }
            for (int tile = tile0; tile < tile1 && ok; tile++) {
#pragma unroll
                for (int a = 0; a < NACC; a++) {
                    if (!ok) break;
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) res[a][mt][i] = 0.0f;
                    const unsigned char* slot = meta + (size_t)ms * p.meta_bytes;
                    const __half* ms_a = reinterpret_cast<const __half*>(slot) + (size_t)rg * p.G;
                    const __half* ms_b = ms_a + (size_t)8 * p.G;
                    const unsigned char* mz_a = slot + p.zeros_off + (size_t)rg * p.ZS;
                    const unsigned char* mz_b = mz_a + (size_t)8 * p.ZS;
                    for (int c = 0; c < nchunks && ok; c++) {
                        ok = warp_wait(full(s), ph, abort_flag, lane);
                        if (!ok) break;
                        if (c == 0) {
                            // this tile's scales / zero-points (issued right after its first stage)
                            ok = warp_wait(meta_full(ms), mph, abort_flag, lane);
                            if (!ok) break;
                        }
                        const unsigned char* st = ring + (size_t)s * stage_bytes;
                        const int gi0 = c * p.cg;
                        const int cgs = min(p.cg, p.G - gi0);      // groups of this stage inside the row

                        // everything the per-group correction needs, fetched before the mma work
                        float sa[GPW], sb_[GPW], ca[GPW], cb[GPW];
                        float4 xq[GPW][MT];
#pragma unroll
                        for (int u = 0; u < GPW; u++) {
                            const int gi = min(gi0 + warp * GPW + u, p.G - 1);
                            sa[u] = __half2float(ms_a[gi]);
                            sb_[u] = __half2float(ms_b[gi]);
                            uint32_t zpa = 8u, zpb = 8u;            // symmetric: stored value - 8
                            if (p.zeros) {
                                zpa = ((uint32_t)mz_a[gi >> 1] >> ((gi & 1) * 4)) & 0xFu;
                                zpb = ((uint32_t)mz_b[gi >> 1] >> ((gi & 1) * 4)) & 0xFu;
                            }
                            ca[u] = -__uint_as_float(0x44800000u | (zpa << 13));    // -(1024 + zp), exact
                            cb[u] = -__uint_as_float(0x44800000u | (zpb << 13));
#pragma unroll
                            for (int mt = 0; mt < MT; mt++)
                                xq[u][mt] = *reinterpret_cast<const float4*>(xsum + gi * MPAD + mt * 8 + 2 * t);
                        }

                        float acc[GPW][MT][4];
#pragma unroll
                        for (int u = 0; u < GPW; u++)
#pragma unroll
                            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                                for (int i = 0; i < 4; i++) acc[u][mt][i] = 0.0f;

#pragma unroll
                        for (int u = 0; u < GPW; u++) {
                            const int gl = warp * GPW + u;             // group inside the stage
                            if (gl < cgs) {
                                // line gl/2, row rg, logical 16-byte chunk (gl%2)*4 + t, swizzled by row%8
                                const unsigned char* ln = st + (gl >> 1) * 2048 + w_off + (((((gl & 1) << 2) | t) ^ rg) << 4);
                                const uint4 qa = *reinterpret_cast<const uint4*>(ln);
                                const uint4 qb = *reinterpret_cast<const uint4*>(ln + 1024);
                                const uint32_t wqa[4] = {qa.x, qa.y, qa.z, qa.w};
                                const uint32_t wqb[4] = {qb.x, qb.y, qb.z, qb.w};
                                const unsigned char* xg = xs + (gi0 + gl) * 256;
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    uint32_t va = wqa[j], vb = wqb[j];
                                    const uint32_t a0 = lop3_and_or(va, 0x000f000fu, 0x64006400u);   // 1024 + (n0, n4)
                                    const uint32_t a1 = lop3_and_or(vb, 0x000f000fu, 0x64006400u);
                                    const uint32_t a2 = lop3_and_or(va, 0x00f000f0u, 0x54005400u);   //   64 + (n1, n5)
                                    const uint32_t a3 = lop3_and_or(vb, 0x00f000f0u, 0x54005400u);
                                    va >>= 8; vb >>= 8;
                                    const uint32_t a4 = lop3_and_or(va, 0x000f000fu, 0x64006400u);   // 1024 + (n2, n6)
                                    const uint32_t a5 = lop3_and_or(vb, 0x000f000fu, 0x64006400u);
                                    const uint32_t a6 = lop3_and_or(va, 0x00f000f0u, 0x54005400u);   //   64 + (n3, n7)
                                    const uint32_t a7 = lop3_and_or(vb, 0x00f000f0u, 0x54005400u);
#pragma unroll
                                    for (int mt = 0; mt < MT; mt++) {
                                        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                                        if (xm_live[mt]) xv = *reinterpret_cast<const uint4*>(xg + xm_off[mt] + j * 64);
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
                        // fold the zero-points back in and apply the group scales (f32)
#pragma unroll
                        for (int u = 0; u < GPW; u++) {
                            if (warp * GPW + u < cgs) {
#pragma unroll
                                for (int mt = 0; mt < MT; mt++) {
                                    res[a][mt][0] = fmaf(sa[u], fmaf(ca[u], xq[u][mt].x, acc[u][mt][0] + xq[u][mt].y), res[a][mt][0]);
                                    res[a][mt][1] = fmaf(sa[u], fmaf(ca[u], xq[u][mt].z, acc[u][mt][1] + xq[u][mt].w), res[a][mt][1]);
                                    res[a][mt][2] = fmaf(sb_[u], fmaf(cb[u], xq[u][mt].x, acc[u][mt][2] + xq[u][mt].y), res[a][mt][2]);
                                    res[a][mt][3] = fmaf(sb_[u], fmaf(cb[u], xq[u][mt].z, acc[u][mt][3] + xq[u][mt].w), res[a][mt][3]);
                                }
                            }
                        }
                    }
                    // done with this tile's scale block
                    __syncwarp();
                    if (lane == 0) mbar_arrive(meta_empty(ms));
                    if (++ms == META_SLOTS) { ms = 0; mph ^= 1u; }
                    // drop this warp's partial sums for the tile; nobody is waited for
                    if (t < p.tmax) {
#pragma unroll
                        for (int mt = 0; mt < MT; mt++)
                            part[((((size_t)(tile - tile0) * CW + warp) * NACC + a) * MT + mt) * slot4 + g * p.tmax + t] =
                                make_float4(res[a][mt][0], res[a][mt][1], res[a][mt][2], res[a][mt][3]);
                    }
                }
            }
            if (!ok) break;
            // ---- batch finished: every warp's partials are in; reduce them together ---------
            __syncwarp();
            if (lane == 0) mbar_arrive(batch_full);
            ok = warp_wait(batch_full, bph, abort_flag, lane);
            if (!ok) break;
            const int nout = (tile1 - tile0) * 16 * MPAD;           // (tile, row, batch column)
            for (int o = tid; o < nout; o += CW * 32) {
                const int m = o % MPAD, r = (o / MPAD) & 15, tb = o / (16 * MPAD);
                if (m >= p.M) continue;
                const int mt = m >> 3, tt = (m & 7) >> 1;
                const int comp = ((r >> 3) << 1) | (m & 1);          // float4 component: row half, column parity
                const int lane_slot = rho_inv(r & 7) * p.tmax + tt;
                float sum[NACC];
#pragma unroll
                for (int a = 0; a < NACC; a++) {
                    const float* v0 = reinterpret_cast<const float*>(
                        part + (((size_t)tb * CW * NACC + a) * MT + mt) * slot4 + lane_slot) + comp;
                    const size_t wstride = (size_t)NACC * MT * slot4 * 4;       // floats between warps
                    float vals[CW];
#pragma unroll
                    for (int w = 0; w < CW; w++) vals[w] = v0[w * wstride];
                    float acc1 = 0.0f;
#pragma unroll
                    for (int w = 0; w < CW; w++) acc1 += vals[w];                // fixed order: deterministic
                    sum[a] = acc1;
                }
                const float out = SWIGLU ? silu_f32(sum[0]) * sum[NACC - 1] : sum[0];
                p.y[(size_t)m * p.Nout + (tile0 + tb) * 16 + r] = __float2half_rn(out);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(batch_empty);
            bph ^= 1u;
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

template <int MT, bool SW, int CW, int GPW>
cudaError_t launch_stream_inst(const CUtensorMap& map, const StreamParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i4_g128_stream<MT, SW, CW, GPW>;
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
    const int tiles = p.Nout / 16;
    p.xstride = a.G * 256 + 64;
    p.zeros_off = (32 * a.G + 15) / 16 * 16;
    p.meta_bytes = p.zeros_off + (16 * p.ZS + 15) / 16 * 16;

    const size_t smem_max = 227 * 1024;
    const size_t x_bytes = (size_t)a.M * p.xstride;
    // partial sums: 8*tmax float4 per (tile, warp, gate/up, mt); batch as many tiles as fit in
    // ~16 KB, at most the tiles one CTA owns
    const int grid0 = std::min(ctx->sm_count, tiles);
    const int tiles_per_cta = (tiles + grid0 - 1) / grid0;
    p.tmax = (std::min(a.M, 8) + 1) / 2;
    const size_t part_tile = (size_t)CW * nacc * MT * 8 * p.tmax * sizeof(float4);
    p.tb = (int)std::max<size_t>(1, std::min<size_t>((size_t)tiles_per_cta, (16 * 1024) / part_tile));
    const size_t red_bytes = (size_t)p.tb * part_tile;
    const size_t xsum_bytes = (size_t)a.G * 8 * MT * sizeof(float2);
    const size_t fixed = 1024 + x_bytes + xsum_bytes + red_bytes + (size_t)META_SLOTS * p.meta_bytes + 1024;
    int cg = g_tune.gemv_stream_cg > 0 ? g_tune.gemv_stream_cg * CW : 32;      // groups per stage
    cg = std::max(CW, std::min(cg, 32) / CW * CW);
    if (cg == 3 * CW) cg = 2 * CW;                 // groups per warp is 1, 2 or 4
    while (cg > CW && cg > a.G) cg /= 2;
    int stages = 0;
    for (;; cg /= 2) {
        const size_t stage_bytes = (size_t)cg * 1024;
        stages = fixed < smem_max ? (int)((smem_max - fixed) / (stage_bytes + 16)) : 0;
        if (stages >= 4 || cg == CW) break;
    }
    if (stages < 3) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int nchunks = (a.G + cg - 1) / cg;
    const int grid = std::min(ctx->sm_count, tiles);
    const int max_items = ((tiles + grid - 1) / grid) * nacc * nchunks;
    p.tiles_base = tiles / grid;
    p.tiles_rem = tiles % grid;
    p.nchunks = nchunks;
    stages = std::min({stages, max_items, g_tune.gemv_stream_stages > 0 ? g_tune.gemv_stream_stages : 64});
    stages = std::max(stages, 1);
    p.cg = cg;
    p.stages = stages;
    const size_t smem = 1024 + (size_t)stages * cg * 1024 + x_bytes + xsum_bytes + (size_t)META_SLOTS * p.meta_bytes + red_bytes +
                       (size_t)(2 * stages + 2 + 2 * META_SLOTS) * 8 + 64;

    // Packed weights viewed as [line of 128 B][row][byte]: a box of (128 B, 16 rows, cg/2
    // lines) lands in shared memory as [line][row][128 B], swizzled by the row index.
    alignas(64) CUtensorMap map;
    const uint64_t dims[3] = {128, (uint64_t)a.N, (uint64_t)a.K / 256};
    const uint64_t strides[2] = {(uint64_t)a.K / 2, 128};
    const uint32_t box[3] = {128, 16, (uint32_t)cg / 2};
    if (!encode_tensor_map_u8(&map, 3, a.w, dims, strides, box, true)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    cudaError_t e = cudaErrorInvalidValue;
    auto go = [&](auto gpw_tag) {
        constexpr int GPW = decltype(gpw_tag)::value;
        if (a.swiglu) return MT == 1 ? launch_stream_inst<1, true, CW, GPW>(map, p, grid, smem, ctx->stream)
                                     : launch_stream_inst<2, true, CW, GPW>(map, p, grid, smem, ctx->stream);
        return MT == 1 ? launch_stream_inst<1, false, CW, GPW>(map, p, grid, smem, ctx->stream)
                       : launch_stream_inst<2, false, CW, GPW>(map, p, grid, smem, ctx->stream);
    };
    switch (cg / CW) {
        case 1: e = go(std::integral_constant<int, 1>{}); break;
        case 2: e = go(std::integral_constant<int, 2>{}); break;
        case 4: if constexpr (CW == 8) e = go(std::integral_constant<int, 4>{}); break;
        default: break;
    }
    count_launch("lux_qgemv_i4_g128_stream");
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


const void* kernel_addr_qgemv_i4_stream() { return (const void*)lux_qgemv_i4_g128_stream<1, false, 16, 2>; }

}  // namespace luxcuda
