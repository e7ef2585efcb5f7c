// lux_qgemv_i4_g128_units -- int4 g128 decode GEMV (batch M <= 16), warp-autonomous version.
//
// Measurements of the other int4 kernels on B200 showed that neither HBM nor the unpack + mma
// arithmetic limits them: the time goes into the short serial sections between pieces of
// work (barrier waits, scale look-ups, hand-offs), which run at tens of cycles per
// instruction when sixteen warps reach them together, into issuing many small TMA copies
// (~130 cycles each, one at a time per SM), and into memory sitting idle whenever less than
// the bandwidth-delay product (~60 KB per SM) is in flight.  This kernel has no barrier
// and no cross-thread hand-off inside its loop:
//
//   * one persistent CTA per SM owns a contiguous range of 16-row tiles; a tile is cut along
//     K into U units of KS groups, and every (tile, gate/up, unit) is handled by ONE warp
//     from start to finish;
//   * the warp streams its units in chunks of CG groups (2 or 4) through a PRIVATE FIFO in
//     shared memory filled with per-lane 16-byte cp.async copies.  Each lane copies exactly
//     the bytes it will later read back itself (its 32 nibbles of rows g and g+8 of every
//     group), so cp.async.wait_group is the only synchronisation, the layout is free of bank
//     conflicts by construction, and the FIFOs together hold ~190 KB per SM in flight --
//     for a 4096 x 14336 layer that is the SM's whole share, requested in the first microsecond;
//   * x is staged once per CTA in shared memory in mma-fragment order together with its
//     per-group sums; the CTA's scales and zero-points are staged once too, so the loop makes
//     no dependent global load.  These are requested BEFORE the weights: requests are served
//     roughly in order, and an x request queued behind 190 KB of weights arrives 4 us late.  The zero-point is folded out of the inner loop exactly as in
//     the ring kernel (sum (n - zp) x = acc - (1024 + zp) sum x + 960 sum_{odd k} x);
//   * a unit's partial result goes to its own slot in shared memory; after the last unit the
//     CTA meets once (__syncthreads) and adds the U partials of every output in a fixed order.
//
// Two arithmetic variants share this structure:
//
//   lux_qgemv_i4_g128_units     (batch 1..16)  nibbles -> f16 with the lop3 magic-number trick,
//       mma.m16n8k16.f16 with f32 accumulation: the arithmetic of lux_qskinny_i4_g128.
//   lux_qgemv_i4_g128_units_fx  (batch 1..2)   the integer pipe of an SM sub-core issues one
//       lop3 per TWO cycles, and at 5 integer ops per 8 nibbles the unpack above -- not HBM, not
//       the tensor pipe -- bounds the f16 variant.  This one spends ONE op per 8 nibbles: a
//       weight word's bytes are R = lo + 16 hi, and w & 0xf0f0f0f0 gives H = 16 hi; both are
//       valid u8 operands of mma.m16n8k32.u8.s8 (half as many mma as f16), and
//       lo Xe + hi Xo = R Xe + H (Zo - Xe) when the odd-k activation is held as Xo = 16 Zo.
//       The activations are converted once per CTA to block fixed point: per group of 128,
//       X = rint(x 2^(30-E)) for even k and 16 rint(x 2^(26-E)) for odd k, with 2^E just above
//       the group's largest |x|.  An f16 has 11 significant bits, so every value down to 2^-19
//       (even k) resp. 2^-15 (odd k) of the group's largest magnitude is represented EXACTLY; a
//       smaller one is rounded with an absolute error of at most 2^(E-31) resp. 2^(E-27), i.e.
//       2^-27 of the group's largest magnitude -- below the 2^-24 relative rounding of the f32
//       products the reference forms (kernels/wgsl/gpu/quantized_nax.wgsl:615-618).  Xe and
//       W = Zo - Xe are split into four signed bytes I = d0 + 256 d1 + 65536 d2 + 2^24 d3 that
//       ride in four of the eight B columns (all eight at batch 2).  The int32 accumulators are
//       exact; sum (n - zp) X is completed exactly in f32 per plane, scaled by 2^(E-30) 256^plane
//       and the group's f16 scale, and the planes are added at the end of a unit.
//
// Both compute matmul_nax_grouped (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:568-626)
// in a different summation order.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstring>

namespace luxcuda {

namespace {

constexpr int UW = 16;                          // warps per CTA
constexpr int MAX_STAGES = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
// 16-byte asynchronous copy global -> shared, bypassing L1 (the data is read once)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// wait until at most n of this thread's most recent copy groups are still pending
__device__ __forceinline__ void cp_async_wait(int n) {
#define LUX_WAIT_CASE(N) case N: asm volatile("cp.async.wait_group " #N ";" ::: "memory"); break;
    switch (n) {
        LUX_WAIT_CASE(0) LUX_WAIT_CASE(1) LUX_WAIT_CASE(2) LUX_WAIT_CASE(3) LUX_WAIT_CASE(4) LUX_WAIT_CASE(5)
        LUX_WAIT_CASE(6) LUX_WAIT_CASE(7) LUX_WAIT_CASE(8) LUX_WAIT_CASE(9) LUX_WAIT_CASE(10) LUX_WAIT_CASE(11)
        LUX_WAIT_CASE(12) LUX_WAIT_CASE(13) LUX_WAIT_CASE(14) LUX_WAIT_CASE(15) LUX_WAIT_CASE(16) LUX_WAIT_CASE(17)
        LUX_WAIT_CASE(18) LUX_WAIT_CASE(19) LUX_WAIT_CASE(20) LUX_WAIT_CASE(21) LUX_WAIT_CASE(22) LUX_WAIT_CASE(23)
        LUX_WAIT_CASE(24) LUX_WAIT_CASE(25) LUX_WAIT_CASE(26) LUX_WAIT_CASE(27) LUX_WAIT_CASE(28)
        // waiting for more than was asked is always safe
        default: asm volatile("cp.async.wait_group 28;" ::: "memory"); break;
    }
#undef LUX_WAIT_CASE
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(s32) += A(u8, 16x32) * B(s8, 32x8)
__device__ __forceinline__ void mma16832_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + __expf(-x)); }


struct UnitsParams {
    const __half* x;        // [M, K]
    const uint8_t* w;       // [Nw, K/2]
    const __half* scales;   // [Nw, G]
    const uint8_t* zeros;   // [Nw, ZS] or null
    __half* y;              // [M, Nout]
    int M, Nout, K, G, ZS;
    int up_row_offset;
    int tiles_base, tiles_rem;   // CTA b owns tiles [b*base + min(b, rem), +base + (b < rem))
    int U, KS;              // units per (tile, gate/up) and groups per unit (U * KS == G, KS % CG == 0)
    int S;                  // FIFO depth in chunks (per warp)
    int S0;                 // chunks requested before the loop starts (the rest ramp up inside it)
    int xstride;            // bytes between batch rows of the staged x
    int tmax;               // lanes t < tmax hold live batch columns
    int units_cap;          // partial-sum slots available per CTA
    int rows_cap;           // weight rows (gate + up) whose scales / zero-points are staged per CTA
    uint32_t* status;       // device status word for a wait that gave up (may be null)
    uint32_t inv_upt, inv_U; // ceil(2^32 / (units per tile)), ceil(2^32 / U): division-free unit table
    int planes;             // fixed-point variant: signed byte planes of the activations, 4 or 3
    int bf16;               // fixed-point variant: x and y are bf16 instead of f16
    PushTarget push;        // world > 1: the outputs go to the peers' all-reduce windows instead of y
};

// Shared memory: [x staged: M * xstride][xsum: G * 8*MT * 8][scales: rows_cap * G f16]
// [zero-points: rows_cap * ZS bytes, padded to 16][partials: units_cap x MT x 8*tmax float4]
// [unit table: units_cap x int4][FIFOs: UW x S x CG KB]
template <int MT, bool SWIGLU, bool M1, int CG>
__global__ void __launch_bounds__(UW * 32, 1) lux_qgemv_i4_g128_units(const UnitsParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NACC = SWIGLU ? 2 : 1;
    constexpr int MPAD = 8 * MT;
    constexpr int CHUNK = CG * 1024;                    // bytes: 16 rows x CG groups x 64
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int slot4 = MT * 8 * p.tmax;                  // float4 per unit

    unsigned char* xs = smem;
    float2* xsum = reinterpret_cast<float2*>(xs + (size_t)p.M * p.xstride);
    __half* ssm = reinterpret_cast<__half*>(xsum + (size_t)p.G * MPAD);
    unsigned char* zsm = reinterpret_cast<unsigned char*>(ssm + (size_t)p.rows_cap * p.G);
    float4* part = reinterpret_cast<float4*>(zsm + (((size_t)p.rows_cap * p.ZS + 15) & ~(size_t)15));
    int4* utab = reinterpret_cast<int4*>(part + (size_t)p.units_cap * slot4);
    unsigned char* fifo = reinterpret_cast<unsigned char*>(utab + p.units_cap) + (size_t)warp * p.S * CHUNK;
    const uint32_t fifo_lane = smem_u32(fifo) + lane * 16;

    // contiguous, balanced range of tiles for this CTA (split computed on the host)
    const int b = (int)blockIdx.x;
    const int tile_lo = b * p.tiles_base + min(b, p.tiles_rem);
    const int ntiles = p.tiles_base + (b < p.tiles_rem ? 1 : 0);
    const int upt = NACC * p.U;                          // units per tile
    const int nunits = ntiles * upt;
    const int NC = p.KS / CG;                            // chunks per unit
    // this warp's units: warp, warp + UW, ...  -> flat chunk sequence q = 0 .. my_chunks-1
    const int my_units = nunits > warp ? (nunits - warp + UW - 1) / UW : 0;
    const int my_chunks = my_units * NC;
    const size_t row_bytes = (size_t)p.K >> 1;
    const int rows_half = ntiles * 16;                   // staged rows per gate / up half

    // Unit table: {first weight row, first group, first staged row} of every unit of this
    // CTA, so that the hot loop never divides.  Entry ul is written by the warp that owns it.
    for (int ul = warp + lane * UW; ul < nunits; ul += 32 * UW) {
        const int tl = ul / upt, rem = ul - tl * upt;
        const int a = rem / p.U, k = rem - a * p.U;
        utab[ul] = make_int4((tile_lo + tl) * 16 + a * p.up_row_offset, k * p.KS, a * rows_half + tl * 16, 0);
    }
    __syncwarp();

    // ---- copy group 0, requested before any weight so that it is served first: x, scattered
    // 16 bytes at a time to the positions of the mma-fragment order (chunk (t, j) of a group
    // goes to slot (j, t)), and this CTA's scales and zero-points (contiguous rows per half)
    {
        const uint32_t xs_s = smem_u32(xs);
        for (int m = 0; m < p.M; m++) {
            const __half* xrow = p.x + (size_t)m * p.K;
            for (int c = tid; c < p.G * 16; c += UW * 32) {
                const int grp = c >> 4, cc = c & 15, tt = cc >> 2, j = cc & 3;
                cp_async16(xs_s + m * p.xstride + grp * 256 + (j * 4 + tt) * 16, xrow + c * 8);
            }
        }
        const int sc16 = rows_half * p.G / 8;            // 16-byte pieces of scales per half
        const int zp16 = rows_half * p.ZS / 16;
        for (int a = 0; a < NACC; a++) {
            const size_t row0 = (size_t)tile_lo * 16 + (size_t)a * p.up_row_offset;
            const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(p.scales + row0 * p.G);
            const uint32_t sdst = smem_u32(ssm + (size_t)a * rows_half * p.G);
            for (int i = tid; i < sc16; i += UW * 32) cp_async16(sdst + i * 16, ssrc + (size_t)i * 16);
            if (p.zeros) {
                const unsigned char* zsrc = p.zeros + row0 * p.ZS;
                const uint32_t zdst = smem_u32(zsm + (size_t)a * rows_half * p.ZS);
                for (int i = tid; i < zp16; i += UW * 32) cp_async16(zdst + i * 16, zsrc + (size_t)i * 16);
            }
        }
        if (!p.zeros)                                     // symmetric: every zero-point is 8
            for (int i = tid; i < (NACC * rows_half * p.ZS + 3) / 4; i += UW * 32)
                reinterpret_cast<uint32_t*>(zsm)[i] = 0x88888888u;
        cp_async_commit();
    }

    // A cursor walks this warp's chunks in order: unit index ui (0,1,..), chunk ci inside it.
    struct Cursor { int ui, ci; };
    auto advance = [&](Cursor& c) { if (++c.ci == NC) { c.ci = 0; ++c.ui; } };
    // request one chunk into FIFO slot `slot`: lane (g, t) copies bytes [t*16, +16) of rows g and
    // g+8 of each group -- piece k of the slot is one 16-byte column of 32 lanes
    auto issue_chunk = [&](const Cursor& c, int slot) {
        const int4 u = utab[warp + c.ui * UW];
        const int gi0 = u.y + c.ci * CG;
        const unsigned char* pa = p.w + (size_t)(u.x + g) * row_bytes + (size_t)gi0 * 64 + t * 16;
        const unsigned char* pb = pa + 8 * row_bytes;
        const uint32_t dst = fifo_lane + slot * CHUNK;
#pragma unroll
        for (int k = 0; k < CG; k++) {
            cp_async16(dst + (2 * k) * 512, pa + k * 64);
            cp_async16(dst + (2 * k + 1) * 512, pb + k * 64);
        }
    };

    // every warp's group-0 requests go out before any warp's weight requests
    __syncthreads();
    // Start the FIFO with S0 chunks; it ramps up to S inside the loop.  (A warp whose copy
    // requests exceed what the SM can keep in flight stalls on the request itself, so asking
    // for everything here would keep every warp from computing until most of it had landed.)
    // One copy group per chunk: chunk q has landed when at most issued-1-q groups are pending.
    Cursor cload{0, 0}, ccur{0, 0};
    int issued = 0, islot = 0;
    for (int s0 = 0; s0 < p.S0 && issued < my_chunks; s0++) {
        issue_chunk(cload, islot);
        cp_async_commit();
        advance(cload);
        issued++;
        if (++islot == p.S) islot = 0;
    }

    // ---- group 0 has landed: every thread puts the 16-byte pieces of x it copied into
    // fragment order in place (the same walk as above), and the per-group sums are formed ------
    for (int i = tid; i < p.G * MPAD; i += UW * 32)
        if ((i % MPAD) >= p.M) xsum[i] = make_float2(0.f, 0.f);
    cp_async_wait(issued);
    for (int m = 0; m < p.M; m++) {
        unsigned char* xdst = xs + (size_t)m * p.xstride;
        for (int c = tid; c < p.G * 16; c += UW * 32) {
            const int grp = c >> 4, cc = c & 15, tt = cc >> 2, j = cc & 3;
            uint4* slot16 = reinterpret_cast<uint4*>(xdst + grp * 256 + (j * 4 + tt) * 16);
            const uint4 s4 = *slot16;
            uint4 d;
            d.x = prmt(s4.x, s4.z, 0x5410);
            d.y = prmt(s4.x, s4.z, 0x7632);
            d.z = prmt(s4.y, s4.w, 0x5410);
            d.w = prmt(s4.y, s4.w, 0x7632);
            *slot16 = d;
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
    __syncthreads();

    int xm_off[MT];
    bool xm_live[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        xm_live[mt] = mt * 8 + g < p.M;
        xm_off[mt] = min(mt * 8 + g, p.M - 1) * p.xstride + t * 16;
    }
    float res[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) res[mt][i] = 0.0f;

    int slot = 0;
    for (int q = 0; q < my_chunks; q++) {
        cp_async_wait(issued - 1 - q);
        uint4 wq[2 * CG];
        {
            const unsigned char* src = fifo + slot * CHUNK + lane * 16;
#pragma unroll
            for (int k = 0; k < 2 * CG; k++) wq[k] = *reinterpret_cast<const uint4*>(src + k * 512);
        }
        if (++slot == p.S) slot = 0;
        // chunk q's slot is free again (this lane has read back everything it copied): request
        // up to two more chunks while the FIFO has room
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (issued < my_chunks && issued - (q + 1) < p.S) {
                issue_chunk(cload, islot);
                cp_async_commit();
                advance(cload);
                issued++;
                if (++islot == p.S) islot = 0;
            }
        }

        const int4 u4 = utab[warp + ccur.ui * UW];
        const int gi0 = u4.y + ccur.ci * CG;
        float acc[CG][MT][4];
#pragma unroll
        for (int u = 0; u < CG; u++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[u][mt][i] = 0.0f;
#pragma unroll
        for (int u = 0; u < CG; u++) {
            const uint32_t wqa[4] = {wq[2 * u].x, wq[2 * u].y, wq[2 * u].z, wq[2 * u].w};
            const uint32_t wqb[4] = {wq[2 * u + 1].x, wq[2 * u + 1].y, wq[2 * u + 1].z, wq[2 * u + 1].w};
            const unsigned char* xg = xs + (gi0 + u) * 256;
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
        // scales and zero-points of rows g / g+8 for the CG groups, from the staged copy
        const int mra = u4.z + g, mrb = mra + 8;
        float fsa[CG], fsb[CG];
        uint32_t za, zb;
        if (CG == 4) {
            const uint2 sa = *reinterpret_cast<const uint2*>(ssm + (size_t)mra * p.G + gi0);
            const uint2 sb = *reinterpret_cast<const uint2*>(ssm + (size_t)mrb * p.G + gi0);
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(&sa.x));
            const float2 a23 = __half22float2(*reinterpret_cast<const __half2*>(&sa.y));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&sb.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&sb.y));
            fsa[0] = a01.x; fsa[1] = a01.y; fsa[CG - 2] = a23.x; fsa[CG - 1] = a23.y;
            fsb[0] = b01.x; fsb[1] = b01.y; fsb[CG - 2] = b23.x; fsb[CG - 1] = b23.y;
            za = *reinterpret_cast<const unsigned short*>(zsm + (size_t)mra * p.ZS + (gi0 >> 1));
            zb = *reinterpret_cast<const unsigned short*>(zsm + (size_t)mrb * p.ZS + (gi0 >> 1));
        } else {
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(ssm + (size_t)mra * p.G + gi0));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(ssm + (size_t)mrb * p.G + gi0));
            fsa[0] = a01.x; fsa[1] = a01.y;
            fsb[0] = b01.x; fsb[1] = b01.y;
            za = zsm[(size_t)mra * p.ZS + (gi0 >> 1)];
            zb = zsm[(size_t)mrb * p.ZS + (gi0 >> 1)];
        }
#pragma unroll
        for (int u = 0; u < CG; u++) {
            const uint32_t zpa = (za >> (4 * u)) & 0xFu, zpb = (zb >> (4 * u)) & 0xFu;
            const float ca = -__uint_as_float(0x44800000u | (zpa << 13));       // -(1024 + zp), exact
            const float cb = -__uint_as_float(0x44800000u | (zpb << 13));
            if (M1) {
                // batch 1: only column 0 (accumulators 0 and 2 of lanes t = 0) is live
                const float2 xq = xsum[(gi0 + u) * MPAD];
                res[0][0] = fmaf(fsa[u], fmaf(ca, xq.x, acc[u][0][0] + xq.y), res[0][0]);
                res[0][2] = fmaf(fsb[u], fmaf(cb, xq.x, acc[u][0][2] + xq.y), res[0][2]);
            } else {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const float4 xq = *reinterpret_cast<const float4*>(xsum + (gi0 + u) * MPAD + mt * 8 + 2 * t);
                    res[mt][0] = fmaf(fsa[u], fmaf(ca, xq.x, acc[u][mt][0] + xq.y), res[mt][0]);
                    res[mt][1] = fmaf(fsa[u], fmaf(ca, xq.z, acc[u][mt][1] + xq.w), res[mt][1]);
                    res[mt][2] = fmaf(fsb[u], fmaf(cb, xq.x, acc[u][mt][2] + xq.y), res[mt][2]);
                    res[mt][3] = fmaf(fsb[u], fmaf(cb, xq.z, acc[u][mt][3] + xq.w), res[mt][3]);
                }
            }
        }
        // end of a unit: drop its partial sums into its slot
        if (ccur.ci == NC - 1) {
            const int ul = warp + ccur.ui * UW;
            if (t < p.tmax) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    part[(size_t)ul * slot4 + mt * 8 * p.tmax + g * p.tmax + t] =
                        make_float4(res[mt][0], res[mt][1], res[mt][2], res[mt][3]);
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) res[mt][i] = 0.0f;
        }
        advance(ccur);
    }

    // ---- every unit of the CTA is done: add the U partials of each output -------------------
    __syncthreads();
    const int nout = ntiles * 16 * MPAD;                     // (tile, row, batch column)
    for (int o = tid; o < nout; o += UW * 32) {
        const int m = o % MPAD, r = (o / MPAD) & 15, tl = o / (16 * MPAD);
        if (m >= p.M) continue;
        const int mt = m >> 3, tt = (m & 7) >> 1;
        const int comp = ((r >> 3) << 1) | (m & 1);           // float4 component: row half, column parity
        const int lane_slot = mt * 8 * p.tmax + (r & 7) * p.tmax + tt;
        float sum[NACC];
#pragma unroll
        for (int a = 0; a < NACC; a++) {
            const float* v0 = reinterpret_cast<const float*>(part + (size_t)((tl * NACC + a) * p.U) * slot4 + lane_slot) + comp;
            float acc1 = 0.0f;
            for (int k = 0; k < p.U; k++) acc1 += v0[(size_t)k * slot4 * 4];         // fixed order: deterministic
            sum[a] = acc1;
        }
        const float out = SWIGLU ? silu_f32(sum[0]) * sum[NACC - 1] : sum[0];
        p.y[(size_t)m * p.Nout + (tile_lo + tl) * 16 + r] = __float2half_rn(out);
    }
}

// ---- block-fixed-point variant, batch MM = 1, 2 or 4 (three rows run as four) -------------------------
// Here the FIFOs are filled by TMA instead of cp.async: per-lane copies stall the REQUESTING warp
// once the SM's load queue is full, which kept the compute warps from computing while the
// memory pipe was busy.  One elected lane per warp asks for a whole chunk (one 3-D box:
// 128 bytes x 16 rows x CG/2 lines, 128-byte swizzle) that completes on a per-slot mbarrier
// of its own warp; nothing is shared between warps.  Every barrier wait is bounded; a wait that
// gives up sets a flag, every warp leaves its loop, and the status word reports it.
//
// Shared memory: [FIFOs: UW x S x CG KB, 1024-byte aligned]
// [xq: G x NT column tiles x (planes x MMT) x 128 signed bytes, each 128 in B-fragment order; a column tile
//  is the 8-column B operand of one MMA and holds MMT = min(MM, 2) batch rows, NT = MM / MMT tiles]
// [xmeta: G x NT x 8 columns x {coef, digit sum}; column = plane (MM = 1) or 2 plane + (m & 1)]
// [scales][zero-points][partials: units_cap x 16 rows x MM float][unit table][barriers][flag]
//
// B-fragment order of one (group, plane, batch row): lane column t' = k >> 5 owns 32 bytes; inside,
// byte ((h*2 + jp)*2 + b)*4 + i holds k = 32t' + 16jp + 8b + 2i + h.  With the weights of lane
// (g, t) being words j = 0..3 = nibbles k = 32t + 8j + (0..7) of its two rows, the mma for
// (parity h, word pair jp) takes a0/a1 = word 2jp of the two rows masked to parity h, a2/a3 =
// word 2jp+1, and b0/b1 = bytes [(h*2+jp)*8, +8) of the lane's 32.
//
// Fragment row g reads tile row rho(g) = (g >> 1) | ((g & 1) << 2) (and rho(g) + 8): with the
// swizzle keyed by row % 8, a quarter-warp's two rows then land in different bank groups.
constexpr uint32_t WAIT_LIMIT = 1u << 15;      // one try_wait may suspend for microseconds: ~0.1 s in all

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// lane 0 polls, the outcome is broadcast; must be called by a converged warp
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag);
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ int rho(int g) { return (g >> 1) | ((g & 1) << 2); }

// Accumulator chains per group of four MMAs (1, 2 or 4).  One chain of four dependent mma.sync is the
// fastest: with four independent accumulators (added as floats afterwards) config 2 went from 7.45 to
// 8.3 us and a batch of four on config 4's gate_up from 19.1 to 19.9 us, so the chain's latency is not
// what the loop waits for; its time follows the NUMBER of mma.sync and of the operations around them.
constexpr int FXCH = 1;

template <int MM, bool SWIGLU, int CG, int UWT>
__global__ void __launch_bounds__(UWT * 32, UWT == 8 ? 2 : 1)
lux_qgemv_i4_g128_units_fx(const __grid_constant__ CUtensorMap map_w, const UnitsParams p) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by OFFSET from the __shared__ symbol (keeps 32-bit shared addressing)
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int NACC = SWIGLU ? 2 : 1;
    constexpr int CHUNK = CG * 1024;
    constexpr int UW = UWT;                             // warps per CTA (shadows the file-wide 16)
    constexpr int MMT = MM < 2 ? MM : 2;                // batch rows per column tile
    constexpr int NT = MM / MMT;                        // column tiles (MMAs per weight fragment pair)
    const int XT = p.planes * MMT * 128;                // bytes of xq per (group, column tile)
    const int XG = XT * NT;                             // bytes of xq per group
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    unsigned char* fifo = smem + (size_t)warp * p.S * CHUNK;
    unsigned char* xq = smem + (size_t)UW * p.S * CHUNK;
    float4* xmeta = reinterpret_cast<float4*>(xq + (size_t)p.G * XG);
    __half* ssm = reinterpret_cast<__half*>(xmeta + (size_t)p.G * 4 * NT);
    unsigned char* zsm = reinterpret_cast<unsigned char*>(ssm + (size_t)p.rows_cap * p.G);
    float* part = reinterpret_cast<float*>(zsm + (((size_t)p.rows_cap * p.ZS + 15) & ~(size_t)15));
    int4* utab = reinterpret_cast<int4*>(part + (size_t)p.units_cap * 16 * MM);
    uint64_t* bars = reinterpret_cast<uint64_t*>(utab + p.units_cap);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + UW * MAX_STAGES);
    const uint32_t bar0 = smem_u32(bars + warp * MAX_STAGES);          // this warp's barriers

    const int b = (int)blockIdx.x;
    const int tile_lo = b * p.tiles_base + min(b, p.tiles_rem);
    const int ntiles = p.tiles_base + (b < p.tiles_rem ? 1 : 0);
    const int upt = NACC * p.U;
    const int nunits = ntiles * upt;
    const int NC = p.KS / CG;
    const int my_units = nunits > warp ? (nunits - warp + UW - 1) / UW : 0;
    const int my_chunks = my_units * NC;
    const int rows_half = ntiles * 16;

    pdl_launch_dependents();
    const int npieces = p.M * p.G * 16;                  // 16-byte pieces of x, (m, group, 16th)

    // ---- barriers and the first weight request: the very first thing every warp does ----------
    // exact division of a small number by a small constant: multiply by ceil(2^32 / d)
    auto div_small = [](uint32_t n, uint32_t d, uint32_t inv) { return d == 1u ? n : __umulhi(n, inv); };
    uint64_t policy = 0;
    int issued = 0;
    if (lane == 0) {
        if (warp == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            *abort_flag = 0u;
        }
        for (int s0 = 0; s0 < p.S; s0++) mbar_init(bar0 + 8u * (uint32_t)s0, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        if (my_chunks > 0) {
            // this warp's first unit is unit `warp` of the CTA: its first chunk goes out before the
            // unit table exists
            const int tl = (int)div_small((uint32_t)warp, (uint32_t)upt, p.inv_upt), rem = warp - tl * upt;
            const int a = (int)div_small((uint32_t)rem, (uint32_t)p.U, p.inv_U), k = rem - a * p.U;
            mbar_expect_tx(bar0, (uint32_t)CHUNK);
            tma_load_3d(smem_u32(fifo), &map_w, 0, (tile_lo + tl) * 16 + a * p.up_row_offset, (k * p.KS) >> 1, bar0, policy);
            issued = 1;
        }
    }
    for (int ul = warp + lane * UW; ul < nunits; ul += 32 * UW) {
        const int tl = (int)div_small((uint32_t)ul, (uint32_t)upt, p.inv_upt), rem = ul - tl * upt;
        const int a = (int)div_small((uint32_t)rem, (uint32_t)p.U, p.inv_U), k = rem - a * p.U;
        utab[ul] = make_int4((tile_lo + tl) * 16 + a * p.up_row_offset, k * p.KS, a * rows_half + tl * 16, 0);
    }
    __syncwarp();

    // A cursor walks this warp's chunks in order: unit index ui (0, 1, ..), chunk ci inside it.
    struct Cursor { int ui, ci; };
    auto advance = [&](Cursor& c) { if (++c.ci == NC) { c.ci = 0; ++c.ui; } };
    Cursor cload{0, 0}, ccur{0, 0};
    if (issued) advance(cload);                           // lane 0: the first chunk is already on its way
    // lane 0 only: ask for the next chunk into FIFO slot `slot` (the slot's barrier is armed first)
    auto issue_chunk = [&](int slot) {
        const int4 u = utab[warp + cload.ui * UW];
        const uint32_t bar = bar0 + 8u * (uint32_t)slot;
        mbar_expect_tx(bar, (uint32_t)CHUNK);
        tma_load_3d(smem_u32(fifo + (size_t)slot * CHUNK), &map_w, 0, u.x, (u.y + cload.ci * CG) >> 1, bar, policy);
        advance(cload);
        issued++;
    };

    // ---- this CTA's scales and zero-points (one cp.async group), requested before the bulk of
    // the weights: small copies queued behind the weight stream would arrive microseconds later -
    {
        const int sc16 = rows_half * p.G / 8;
        const int zp16 = rows_half * p.ZS / 16;
        for (int a = 0; a < NACC; a++) {
            const size_t row0 = (size_t)tile_lo * 16 + (size_t)a * p.up_row_offset;
            const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(p.scales + row0 * p.G);
            const uint32_t sdst = smem_u32(ssm + (size_t)a * rows_half * p.G);
            for (int i = tid; i < sc16; i += UW * 32) cp_async16(sdst + i * 16, ssrc + (size_t)i * 16);
            if (p.zeros) {
                const unsigned char* zsrc = p.zeros + row0 * p.ZS;
                const uint32_t zdst = smem_u32(zsm + (size_t)a * rows_half * p.ZS);
                for (int i = tid; i < zp16; i += UW * 32) cp_async16(zdst + i * 16, zsrc + (size_t)i * 16);
            }
        }
        cp_async_commit();
    }
    if (!p.zeros)                                         // symmetric: every zero-point is 8
        for (int i = tid; i < (NACC * rows_half * p.ZS + 3) / 4; i += UW * 32)
            reinterpret_cast<uint32_t*>(zsm)[i] = 0x88888888u;

    // Everything above read static model state only; x may come from the previous kernel.
    pdl_wait();

    // ---- x -> block fixed point, four signed byte planes in B-fragment order -----------------
    // a thread's pieces are requested together (one round trip to L2 per MM pieces, not one each)
    auto convert = [&](int c, const uint4 s4) {
        const int m = MM == 1 ? 0 : c / (p.G * 16), cg16 = c - m * p.G * 16;
        const int grp = cg16 >> 4, l16 = cg16 & 15;
        float v[8];
        if (p.bf16) {
            // a bf16 is the upper half of the f32 of the same value
            v[0] = __uint_as_float(s4.x << 16); v[1] = __uint_as_float(s4.x & 0xffff0000u);
            v[2] = __uint_as_float(s4.y << 16); v[3] = __uint_as_float(s4.y & 0xffff0000u);
            v[4] = __uint_as_float(s4.z << 16); v[5] = __uint_as_float(s4.z & 0xffff0000u);
            v[6] = __uint_as_float(s4.w << 16); v[7] = __uint_as_float(s4.w & 0xffff0000u);
        } else {
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&s4.z));
            const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&s4.w));
            v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
        }
        // largest |x| of the group as a 16-bit pattern (monotonic for non-negative values in f16 and
        // in bf16 alike; inf and NaN, exponent field all ones, compare above every finite value)
        uint32_t mb = __vmaxu2(__vmaxu2(s4.x & 0x7fff7fffu, s4.y & 0x7fff7fffu),
                               __vmaxu2(s4.z & 0x7fff7fffu, s4.w & 0x7fff7fffu));
        mb = max(mb & 0xffffu, mb >> 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
        const bool bad = mb >= (p.bf16 ? 0x7F80u : 0x7C00u);
        const float amax = p.bf16 ? __uint_as_float(mb << 16) : __half2float(__ushort_as_half((unsigned short)mb));
        // amax = f * 2^E with f in [0.5, 1): biased exponent eb = E + 126.  x * 2^(30-E) is exact.
        // (bf16 reaches exponents f16 does not: below 2^-86 the block exponent stops following the
        // group, so that both powers of two below stay normal; such a group keeps fewer bits.)
        const unsigned eb = max(__float_as_uint(amax) >> 23, 40u);
        // four planes: 30 bits below the block exponent; three (rows too long for four): 22
        const unsigned sh = p.planes == 4 ? 30u : 22u;
        const float up = (mb != 0u && !bad) ? __uint_as_float((253u + sh - eb) << 23) : 0.0f;   // 2^(sh-E)
        float down = mb != 0u ? __uint_as_float((eb + 1u - sh) << 23) : 0.0f;                  // 2^(E-sh)
        if (bad) down = __uint_as_float(0x7FC00000u);    // inf / NaN in the group: the outputs are NaN
        // Even k: X = rint(x 2^(30-E)).  Odd k: Z = rint(x 2^(26-E)) and X = 16 Z, so that the
        // high nibble's product n X equals (16 n) Z: the weights' bytes then need one mask, not two.
        // With R = lo + 16 hi the raw byte and H = 16 hi the masked one,
        //   lo Xe + hi Xo = R Xe + H (Zo - Xe),
        // so the B operand holds the digits of Xe against R and of W = Zo - Xe against H.
        // I + 0x80808080 has bytes d0+128 .. d3+128 (I = d0 + 256 d1 + 65536 d2 + 2^24 d3, digits in
        // [-128, 127]; |I| < 2^30 + 2^26 fits); flipping the top bit of each turns them into the
        // digits as signed bytes.
        uint32_t e[8], xo[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int xe = __float2int_rn(v[2 * i] * up);
            const int zo = __float2int_rn(v[2 * i + 1] * (up * 0.0625f));
            e[2 * i] = ((uint32_t)xe + 0x80808080u) ^ 0x80808080u;
            e[2 * i + 1] = ((uint32_t)(zo - xe) + 0x80808080u) ^ 0x80808080u;
            xo[i] = ((uint32_t)(16 * zo) + 0x80808080u) ^ 0x80808080u;   // digits of the odd k's true X, for the sums
        }
        // byte transpose: word h of plane pl holds, for i = 0..3, the digit of Xe (h = 0) or W (h = 1)
        // of the byte with nibbles k = 2i, 2i+1
        uint32_t pw[4][2], po[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a01 = prmt(e[h], e[2 + h], 0x5140), a23 = prmt(e[4 + h], e[6 + h], 0x5140);
            const uint32_t c01 = prmt(e[h], e[2 + h], 0x7362), c23 = prmt(e[4 + h], e[6 + h], 0x7362);
            pw[0][h] = prmt(a01, a23, 0x5410);
            pw[1][h] = prmt(a01, a23, 0x7632);
            pw[2][h] = prmt(c01, c23, 0x5410);
            pw[3][h] = prmt(c01, c23, 0x7632);
        }
        {
            const uint32_t a01 = prmt(xo[0], xo[1], 0x5140), a23 = prmt(xo[2], xo[3], 0x5140);
            const uint32_t c01 = prmt(xo[0], xo[1], 0x7362), c23 = prmt(xo[2], xo[3], 0x7362);
            po[0] = prmt(a01, a23, 0x5410);
            po[1] = prmt(a01, a23, 0x7632);
            po[2] = prmt(c01, c23, 0x5410);
            po[3] = prmt(c01, c23, 0x7632);
        }
        // this thread's 8 k are 32t' + 16jp + 8b + (2i + h)
        const int tq = l16 >> 2, jp = (l16 >> 1) & 1, bb = l16 & 1;
#pragma unroll
        for (int pl = 0; pl < 4; pl++) {
            if (pl == 3 && p.planes == 3) break;             // the fourth digit of a 23-bit number is 0
            unsigned char* dst = xq + (size_t)grp * XG + (m / MMT) * XT + (pl * MMT + (m % MMT)) * 128 + tq * 32;
            *reinterpret_cast<uint32_t*>(dst + ((0 * 2 + jp) * 2 + bb) * 4) = pw[pl][0];
            *reinterpret_cast<uint32_t*>(dst + ((1 * 2 + jp) * 2 + bb) * 4) = pw[pl][1];
        }
        // sums over the group of the true X's digits per plane (for the zero-point term); two planes
        // share one register through the reduction (|sum| <= 128 * 128 fits 16 bits)
        int ds[4];
#pragma unroll
        for (int pl = 0; pl < 4; pl++)
            ds[pl] = __dp4a((int)pw[pl][0], 0x01010101, __dp4a((int)po[pl], 0x01010101, 0));
        int d01 = ds[0] + ds[1] * 65536, d23 = ds[2] + ds[3] * 65536;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            d01 += __shfl_xor_sync(0xffffffffu, d01, o);
            d23 += __shfl_xor_sync(0xffffffffu, d23, o);
        }
        if (l16 == 0) {
            const int s0 = (int)(short)(d01 & 0xffff), s1 = (d01 - s0) >> 16;
            const int s2 = (int)(short)(d23 & 0xffff), s3 = (d23 - s2) >> 16;
            // Lane t of a consumer reads one float4 = {coef, digit sum} of its columns 2t and 2t+1.
            // Every float of the group's four entries is written here exactly once; columns
            // without a plane behind them get coefficient 0 (their accumulators hold garbage).
            float4* xm = xmeta + (grp * NT + m / MMT) * 4;
            if (MM == 1) {
                xm[0] = make_float4(down, (float)s0, down * 256.0f, (float)s1);
                xm[1] = make_float4(down * 65536.0f, (float)s2, p.planes == 4 ? down * 16777216.0f : 0.f, (float)s3);
                xm[2] = make_float4(0.f, 0.f, 0.f, 0.f);
                xm[3] = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                float2* x2 = reinterpret_cast<float2*>(xm) + (m % MMT);  // .xy for the tile's first row, .zw for its second
                x2[0] = make_float2(down, (float)s0);
                x2[2] = make_float2(down * 256.0f, (float)s1);
                x2[4] = make_float2(down * 65536.0f, (float)s2);
                x2[6] = make_float2(p.planes == 4 ? down * 16777216.0f : 0.f, (float)s3);
            }
        }
    };
    for (int c0 = tid; c0 < npieces; c0 += UW * 32 * MM) {
        uint4 s4v[MM];
#pragma unroll
        for (int i = 0; i < MM; i++) {
            const int c = c0 + i * UW * 32;
            if (c < npieces) s4v[i] = __ldg(reinterpret_cast<const uint4*>(p.x) + c);
        }
#pragma unroll
        for (int i = 0; i < MM; i++) {
            const int c = c0 + i * UW * 32;
            if (c < npieces) convert(c, s4v[i]);          // warp-uniform: npieces is a multiple of 32
        }
    }
    // fill the rest of the FIFO (the async engine queues the requests: nothing stalls here; asked
    // for before the conversion they only delay the first chunk and the tables: measured slower)
    if (lane == 0)
        for (int s0 = 1; s0 < p.S && issued < my_chunks; s0++) issue_chunk(s0);
    cp_async_wait(0);                                    // the scales and zero-points have landed
    __syncthreads();

    // lanes of column g >= 4*MM multiply garbage that nobody reads: point them at a valid column
    const int col = min(g, p.planes * MMT - 1);
    const int xcol_off = col * 128 + t * 32;
    const int rg = rho(g);                               // tile row behind fragment row g
    float res[NT][2][2];                                 // [column tile][row half][column 2t / 2t+1 of the lane]
#pragma unroll
    for (int nt = 0; nt < NT; nt++) res[nt][0][0] = res[nt][0][1] = res[nt][1][0] = res[nt][1][1] = 0.0f;
    constexpr int MAGIC = 0x4B400000;                    // float 1.5 * 2^23: MAGIC + i reads as 12582912 + i

    int slot = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int q = 0; q < my_chunks; q++) {
        ok = warp_wait(bar0 + 8u * (uint32_t)slot, ph, abort_flag, lane);
        if (!ok) break;
        uint4 wq[2 * CG];
        {
            const unsigned char* st = fifo + (size_t)slot * CHUNK + rg * 128;
#pragma unroll
            for (int u = 0; u < CG; u++) {
                // line u/2, rows rg and rg+8, logical 16-byte piece (u%2)*4 + t, swizzled by row%8
                const unsigned char* ln = st + (u >> 1) * 2048 + (((((u & 1) << 2) | t) ^ rg) << 4);
                wq[2 * u] = *reinterpret_cast<const uint4*>(ln);
                wq[2 * u + 1] = *reinterpret_cast<const uint4*>(ln + 1024);
            }
        }
        // every lane has read the slot: hand it back to the async engine for the next chunk
        __syncwarp();
        if (lane == 0 && issued < my_chunks) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_chunk(slot);
        }
        if (++slot == p.S) { slot = 0; ph ^= 1u; }

        const int4 u4 = utab[warp + ccur.ui * UW];
        const int gi0 = u4.y + ccur.ci * CG;
        const int mra = u4.z + rg, mrb = mra + 8;
        float fsa[CG], fsb[CG];
        uint32_t za, zb;
        if (CG == 4) {
            const uint2 sa = *reinterpret_cast<const uint2*>(ssm + (size_t)mra * p.G + gi0);
            const uint2 sb = *reinterpret_cast<const uint2*>(ssm + (size_t)mrb * p.G + gi0);
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(&sa.x));
            const float2 a23 = __half22float2(*reinterpret_cast<const __half2*>(&sa.y));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&sb.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&sb.y));
            fsa[0] = a01.x; fsa[1] = a01.y; fsa[CG - 2] = a23.x; fsa[CG - 1] = a23.y;
            fsb[0] = b01.x; fsb[1] = b01.y; fsb[CG - 2] = b23.x; fsb[CG - 1] = b23.y;
            za = *reinterpret_cast<const unsigned short*>(zsm + (size_t)mra * p.ZS + (gi0 >> 1));
            zb = *reinterpret_cast<const unsigned short*>(zsm + (size_t)mrb * p.ZS + (gi0 >> 1));
        } else {
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(ssm + (size_t)mra * p.G + gi0));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(ssm + (size_t)mrb * p.G + gi0));
            fsa[0] = a01.x; fsa[1] = a01.y;
            fsb[0] = b01.x; fsb[1] = b01.y;
            za = zsm[(size_t)mra * p.ZS + (gi0 >> 1)];
            zb = zsm[(size_t)mrb * p.ZS + (gi0 >> 1)];
        }
#pragma unroll
        for (int u = 0; u < CG; u++) {
            const uint4 qa = wq[2 * u], qb = wq[2 * u + 1];
            constexpr uint32_t MH = 0xf0f0f0f0u;
            const uint32_t ha0 = qa.x & MH, hb0 = qb.x & MH, ha1 = qa.y & MH, hb1 = qb.y & MH;
            const uint32_t ha2 = qa.z & MH, hb2 = qb.z & MH, ha3 = qa.w & MH, hb3 = qb.w & MH;
            // -zp as a float: 12582912 - (12582912 + zp)
            const float nza = 12582912.0f - __uint_as_float(0x4B400000u | ((za >> (4 * u)) & 0xFu));
            const float nzb = 12582912.0f - __uint_as_float(0x4B400000u | ((zb >> (4 * u)) & 0xFu));
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const unsigned char* xg = xq + (size_t)(gi0 + u) * XG + nt * XT + xcol_off;
                const uint4 xlo = *reinterpret_cast<const uint4*>(xg);          // even k: word pairs 0, 1
                const uint4 xhi = *reinterpret_cast<const uint4*>(xg + 16);     // odd k
                // every accumulator starts at MAGIC, so that it reads as a float without a conversion
                int acc[FXCH][4];
#pragma unroll
                for (int ch = 0; ch < FXCH; ch++) acc[ch][0] = acc[ch][1] = acc[ch][2] = acc[ch][3] = MAGIC;
                mma16832_u8s8(acc[0], qa.x, qb.x, qa.y, qb.y, xlo.x, xlo.y);               // R  x Xe
                mma16832_u8s8(acc[1 % FXCH], ha0, hb0, ha1, hb1, xhi.x, xhi.y);           // H  x (Zo - Xe)
                mma16832_u8s8(acc[2 % FXCH], qa.z, qb.z, qa.w, qb.w, xlo.z, xlo.w);
                mma16832_u8s8(acc[3 % FXCH], ha2, hb2, ha3, hb3, xhi.z, xhi.w);
                // columns 2t, 2t+1 of this lane: coefficient 2^(E-22) 256^plane and digit sum
                const float4 xm = xmeta[((gi0 + u) * NT + nt) * 4 + t];
                // integer sum (n - zp) X of the column = acc - zp * digit-sum, all exact in f32:
                // |acc| < 2^22 (64 bytes x 255 x 128 + 64 x 240 x 128), |zp * sum| < 2^18
                float fa[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    fa[e] = __int_as_float(acc[0][e]) - 12582912.0f;
#pragma unroll
                    for (int ch = 1; ch < FXCH; ch++) fa[e] += __int_as_float(acc[ch][e]) - 12582912.0f;
                }
                float v[2][2];                               // [row half][column]
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const float ds = j ? xm.w : xm.y;
                    v[0][j] = fmaf(nza, ds, fa[j]);
                    v[1][j] = fmaf(nzb, ds, fa[2 + j]);
                }
                if (MM == 1) {
                    // both columns are planes of batch row 0: combine them before the scale
                    res[nt][0][0] = fmaf(fsa[u], fmaf(xm.z, v[0][1], xm.x * v[0][0]), res[nt][0][0]);
                    res[nt][1][0] = fmaf(fsb[u], fmaf(xm.z, v[1][1], xm.x * v[1][0]), res[nt][1][0]);
                } else {
                    res[nt][0][0] = fmaf(fsa[u] * xm.x, v[0][0], res[nt][0][0]);
                    res[nt][0][1] = fmaf(fsa[u] * xm.z, v[0][1], res[nt][0][1]);
                    res[nt][1][0] = fmaf(fsb[u] * xm.x, v[1][0], res[nt][1][0]);
                    res[nt][1][1] = fmaf(fsb[u] * xm.z, v[1][1], res[nt][1][1]);
                }
            }
        }
        // end of a unit: add the planes (lanes t) and drop the partial sums into the unit's slot
        if (ccur.ci == NC - 1) {
            const int ul = warp + ccur.ui * UW;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int m = 0; m < MMT; m++) {
                        res[nt][h][m] += __shfl_xor_sync(0xffffffffu, res[nt][h][m], 1);
                        res[nt][h][m] += __shfl_xor_sync(0xffffffffu, res[nt][h][m], 2);
                    }
            if (t == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int m = 0; m < MMT; m++) {
                        part[((size_t)ul * 16 + rg) * MM + nt * MMT + m] = res[nt][0][m];
                        part[((size_t)ul * 16 + rg + 8) * MM + nt * MMT + m] = res[nt][1][m];
                    }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) res[nt][0][0] = res[nt][0][1] = res[nt][1][0] = res[nt][1][1] = 0.0f;
        }
        advance(ccur);
    }

    __syncthreads();
    if (*abort_flag) {
        // A bounded wait gave up: report it and give copies still in flight time to land in
        // this CTA's shared memory before it is released.
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C050003u);
        if (tid == 0 && !SWIGLU && p.push.world > 1) atomicExch(p.push.ctl + PEER_CTL_FAILED, 1u);   // this rank pushes nothing
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
        return;
    }
    if (!SWIGLU && p.push.world > 1) {
        // Fused compute + collective: this kernel IS the all-reduce.  Every pair of outputs goes
        // straight from the tensor-core partial sums into slot [parity][my rank] of EVERY rank's
        // window as one self-validating 8-byte word {two f16, epoch} (plain stores to peer memory);
        // the same thread then waits for the same word of every source rank in its OWN window, adds
        // them in rank order in f32 (its own contribution as the f16 pair it pushed, so that all
        // ranks hold identical bits) and writes y.  No second kernel, no launch boundary: a CTA's
        // peers have pushed these rows by the time its own tiles are done, give or take the skew
        // between the GPUs.  The wait is bounded by a deadline (allreduce_push.cu describes the
        // protocol, the failure rule and the control words); the last CTA advances the epoch.
        const uint32_t epoch = peer_ctl_load(p.push.ctl + PEER_CTL_EPOCH) + 1u;
        bool failed = peer_ctl_load(p.push.ctl + PEER_CTL_FAILED) != 0u;
        const size_t slot_sz = 2 * p.push.max_bytes;
        const size_t par_off = (size_t)(epoch & 1u) * p.push.world * slot_sz;
        const size_t my_slot = par_off + (size_t)p.push.rank * slot_sz;
        const unsigned char* mine = p.push.peer[p.push.rank] + par_off;
        const int npairs = ntiles * 8 * MM;
        const unsigned long long t0 = peer_timer_ns();
        for (int o = tid; o < npairs && !failed; o += UW * 32) {
            const int m = o % MM, r2 = (o / MM) & 7, tl = o / (8 * MM);
            if (m >= p.M) continue;                               // the padding row of a three-row batch
            const float* v0 = part + ((size_t)(tl * p.U) * 16 + 2 * r2) * MM + m;
            float s0 = 0.0f, s1 = 0.0f;
            for (int k = 0; k < p.U; k++) {                       // fixed order: deterministic
                s0 += v0[(size_t)k * 16 * MM];
                s1 += v0[(size_t)k * 16 * MM + MM];
            }
            const __half2 h2 = __floats2half2_rn(s0, s1);
            const uint32_t pk = *reinterpret_cast<const uint32_t*>(&h2);
            const size_t col = (size_t)(tile_lo + tl) * 16 + 2 * r2;
            const size_t word = ((size_t)m * p.Nout + col) >> 1;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                if (r < p.push.world) {
                    uint2* dst = reinterpret_cast<uint2*>(p.push.peer[r] + my_slot) + word;
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(pk), "r"(epoch) : "memory");
                }
            }
            if (!p.push.reduce_here) continue;                    // a reduce-only all-reduce kernel follows
            uint32_t got[8];
            for (uint32_t it = 1;; ++it) {
                bool all = true;
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    if (r < p.push.world) {
                        uint32_t ep;
                        const uint2* src = reinterpret_cast<const uint2*>(mine + (size_t)r * slot_sz) + word;
                        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(got[r]), "=r"(ep) : "l"(src) : "memory");
                        all = all && ep == epoch;
                    }
                }
                if (all) break;
                if ((it & 15u) == 0u && peer_timer_ns() - t0 > p.push.wait_ns) { failed = true; break; }
            }
            if (failed) break;
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                if (r < p.push.world) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&got[r]));
                    a0 += f.x;
                    a1 += f.y;
                }
            }
            *reinterpret_cast<__half2*>(p.y + (size_t)m * p.Nout + col) = __floats2half2_rn(a0, a1);
        }
        const int any_failed = __syncthreads_or(failed ? 1 : 0);
        if (tid == 0 && p.push.reduce_here) peer_ctl_finish(p.push.ctl, PEER_CTL_DONE_FUSED, gridDim.x, epoch, any_failed != 0, p.status);
        return;
    }
    const int nout = ntiles * 16 * MM;
    for (int o = tid; o < nout; o += UW * 32) {
        const int m = o % MM, r = (o / MM) & 15, tl = o / (16 * MM);
        if (m >= p.M) continue;                                   // the padding row of a three-row batch
        float sum[NACC];
#pragma unroll
        for (int a = 0; a < NACC; a++) {
            const float* v0 = part + ((size_t)((tl * NACC + a) * p.U) * 16 + r) * MM + m;
            float acc1 = 0.0f;
            for (int k = 0; k < p.U; k++) acc1 += v0[(size_t)k * 16 * MM];        // fixed order: deterministic
            sum[a] = acc1;
        }
        const float out = SWIGLU ? silu_f32(sum[0]) * sum[NACC - 1] : sum[0];
        const size_t at = (size_t)m * p.Nout + (tile_lo + tl) * 16 + r;
        if (p.bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[at] = __float2bfloat16_rn(out);
        else p.y[at] = __float2half_rn(out);
    }
}

template <int MT, bool SW, bool M1, int CG>
cudaError_t launch_units_inst(const UnitsParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i4_g128_units<MT, SW, M1, CG>;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    kfn<<<grid, UW * 32, smem, st>>>(p);
    return cudaGetLastError();
}

template <int MM, bool SW, int CG, int UWT>
cudaError_t launch_units_fx_inst(bool pdl, const CUtensorMap& map, const UnitsParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i4_g128_units_fx<MM, SW, CG, UWT>;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    return launch_pdl(pdl, kfn, dim3((unsigned)grid), dim3(UWT * 32), smem, st, 1, map, p);
}

template <int MM, bool SW>
cudaError_t launch_units_fx_cg(bool pdl, int cg, int uw, const CUtensorMap& map, const UnitsParams& p, int grid, size_t smem,
                               cudaStream_t st) {
    if (uw == 8)
        return cg == 4 ? launch_units_fx_inst<MM, SW, 4, 8>(pdl, map, p, grid, smem, st)
                       : launch_units_fx_inst<MM, SW, 2, 8>(pdl, map, p, grid, smem, st);
    return cg == 4 ? launch_units_fx_inst<MM, SW, 4, 16>(pdl, map, p, grid, smem, st)
                   : launch_units_fx_inst<MM, SW, 2, 16>(pdl, map, p, grid, smem, st);
}

template <int MT, bool SW, bool M1>
cudaError_t launch_units_cg(int cg, const UnitsParams& p, int grid, size_t smem, cudaStream_t st) {
    return cg == 4 ? launch_units_inst<MT, SW, M1, 4>(p, grid, smem, st)
                   : launch_units_inst<MT, SW, M1, 2>(p, grid, smem, st);
}

}  // namespace

// Returns NOT_SUPPORTED when the shape does not suit this kernel (the caller then uses one of
// the other int4 kernels): batch above 16, an odd number of groups, an output size that is
// not a multiple of the 16-row tile, a zero-point row that is not a whole number of 16-byte
// pieces per tile, or activations / scale tables too large to stage in shared memory next
// to at least one chunk (fixed-point variant) or two chunks (f16 variant) of FIFO per warp.
LuxBackendError launch_qgemv_i4_units(Context* ctx, const QArgs& a) {
    const int nout = a.swiglu ? a.N / 2 : a.N;
    if (a.M < 1 || a.M > 16 || a.G < 2 || (a.G & 1) || nout % 16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int MT = a.M <= 8 ? 1 : 2;
    const int nacc = a.swiglu ? 2 : 1;
    const int tiles = nout / 16;
    // the staged tables are copied in 16-byte pieces per (CTA, gate/up half): 16 rows of scales
    // are 32*G bytes (always whole pieces); 16 rows of zero-points are 16*ZS bytes (always whole);
    // the sources must be 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(a.scales) & 15) || (a.zeros && (reinterpret_cast<uintptr_t>(a.zeros) & 15)) ||
        (reinterpret_cast<uintptr_t>(a.w) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15))
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (a.swiglu && (((size_t)nout * a.G * 2) & 15)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    // batch 1..4 use the block-fixed-point variant (three rows run as four) unless the tunable says
    // otherwise; a batch of 3 or 4 whose activations do not fit beside the FIFOs falls back to the f16 form
    bool fx = a.M <= 4 && g_tune.gemv_units_fx != 2;
    const bool bf16 = a.x_dtype == LUX_QDTYPE_BF16;        // only the fixed-point variant reads and writes bf16
    if (bf16 && (!fx || a.push)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int mm = a.M == 3 ? 4 : a.M;                    // batch rows the fixed-point kernel is instantiated for

    // Chunk size: 4 groups when the group count allows, else 2.
    int cg = g_tune.gemv_units_cg == 2 || g_tune.gemv_units_cg == 4 ? g_tune.gemv_units_cg : ((a.G & 3) ? 2 : 4);
    if (a.G % cg) cg = 2;
    const size_t chunk = (size_t)cg * 1024;

    // A geometry: `uw` warps per CTA, one CTA per SM.  The default is the whole SM with 16 warps.
    // gemv_units_warps = 8 selects HALF an SM (8 warps, at most 113 KB of shared memory, registers
    // for two CTAs), so that the next kernel of the stream, launched programmatically, becomes
    // resident beside this one and fills its FIFOs while this one still streams.  Measured on B200
    // (config 2): 8.5 us per GEMV against 6.9 us with 16 warps -- eight warps per SM cannot keep up
    // with the SM's share of HBM, and the overlap does not make up for it.
    struct Plan { int uw, grid, tiles_per_cta, KS, U, S; size_t fixed, smem; UnitsParams p; };
    auto make_plan = [&](int uw, size_t budget, int min_stages, int planes, Plan& pl) -> bool {
        pl.uw = uw;
        pl.grid = std::min(ctx->sm_count, tiles);
        pl.tiles_per_cta = (tiles + pl.grid - 1) / pl.grid;
        // Unit size KS (a multiple of the chunk, dividing G): the one that spreads the busiest CTA's
        // groups most evenly over its warps, each unit costing about a quarter of a group of overhead.
        int KS = 0;
        if (g_tune.gemv_units_ks > 0 && a.G % g_tune.gemv_units_ks == 0 && g_tune.gemv_units_ks % cg == 0) {
            KS = g_tune.gemv_units_ks;
        } else {
            double best = 1e30;
            for (int ks = cg; ks <= std::min(a.G, 32); ks += cg) {
                if (a.G % ks) continue;
                const int units = pl.tiles_per_cta * nacc * (a.G / ks);
                const double cost = (double)((units + uw - 1) / uw) * (ks + 0.25);
                if (cost < best - 1e-9) { best = cost; KS = ks; }
            }
        }
        if (KS == 0) return false;
        pl.KS = KS;
        pl.U = a.G / KS;
        UnitsParams& p = pl.p;
        p = UnitsParams{};
        p.x = (const __half*)a.x;
        p.w = a.w;
        p.scales = (const __half*)a.scales;
        p.zeros = a.zeros;
        p.y = (__half*)a.y;
        p.M = a.M;
        p.K = a.K;
        p.G = a.G;
        p.ZS = (a.G + 1) / 2;
        p.Nout = nout;
        p.up_row_offset = a.swiglu ? nout : 0;
        p.U = pl.U;
        p.KS = KS;
        p.xstride = a.G * 256 + 64;
        p.tmax = (std::min(a.M, 8) + 1) / 2;
        p.tiles_base = tiles / pl.grid;
        p.tiles_rem = tiles % pl.grid;
        p.units_cap = pl.tiles_per_cta * nacc * pl.U;
        p.rows_cap = pl.tiles_per_cta * 16 * nacc;
        p.planes = planes;
        const size_t x_bytes = fx ? (size_t)a.G * planes * mm * 128 + (size_t)a.G * 4 * ((mm + 1) / 2) * sizeof(float4)
                                  : (size_t)a.M * p.xstride + (size_t)a.G * 8 * MT * sizeof(float2);
        const size_t meta_bytes = (size_t)p.rows_cap * a.G * 2 + (((size_t)p.rows_cap * p.ZS + 15) & ~(size_t)15);
        const size_t part_bytes = fx ? (size_t)p.units_cap * 16 * mm * sizeof(float)
                                     : (size_t)p.units_cap * MT * 8 * p.tmax * sizeof(float4);
        // the fixed-point variant also holds its barriers and flag, and 1024 bytes of alignment slack
        pl.fixed = x_bytes + meta_bytes + part_bytes + (size_t)p.units_cap * sizeof(int4) +
                   (fx ? (size_t)uw * MAX_STAGES * 8 + 16 + 1024 : 0);
        if (pl.fixed + (size_t)min_stages * uw * chunk > budget) return false;
        const int max_chunks = (p.units_cap + uw - 1) / uw * (KS / cg);       // per warp
        int S = (int)std::min<size_t>((budget - pl.fixed) / ((size_t)uw * chunk), MAX_STAGES);
        S = std::min(S, std::max(max_chunks, 1));
        // measured on B200: the fixed-point variant is fastest two or three chunks deep (deeper FIFOs
        // only delay the first chunk and the tables at start-up; large layers do not care)
        if (g_tune.gemv_units_stages > 0) S = std::min(S, g_tune.gemv_units_stages);
        else if (fx) S = std::min(S, uw == 8 ? 3 : 2);
        pl.S = p.S = std::max(S, 1);
        p.S0 = std::min(p.S, g_tune.gemv_units_pre > 0 ? g_tune.gemv_units_pre : 1);
        pl.smem = pl.fixed + (size_t)p.S * uw * chunk;
        return true;
    };
    Plan pl;
    bool planned = false;
    // two CTAs per SM: 2 x (dynamic + 1 KB reserved) must fit the SM's 228 KB
    // Four byte planes of the activations wherever they cost no FIFO depth; rows so long that the
    // fourth plane would (28672 elements at batch 1: 114 KB of planes) keep three, i.e. 22 / 18 bits
    // below the block exponent instead of 30 / 26.  gemv_units_planes forces either.
    auto plan_planes = [&](int uw, size_t budget, int min_stages) -> bool {
        if (!fx) return make_plan(uw, budget, min_stages, 4, pl);
        Plan p3, p4;
        const bool ok3 = g_tune.gemv_units_planes != 4 && make_plan(uw, budget, min_stages, 3, p3);
        const bool ok4 = g_tune.gemv_units_planes != 3 && make_plan(uw, budget, min_stages, 4, p4);
        if (ok4 && (!ok3 || p4.S >= p3.S)) { pl = p4; return true; }
        if (ok3) { pl = p3; return true; }
        return false;
    };
    if (fx && g_tune.gemv_units_warps == 8) planned = plan_planes(8, (size_t)113 * 1024, 2);
    if (!planned && (!fx || g_tune.gemv_units_warps != 8)) planned = plan_planes(UW, (size_t)227 * 1024, fx ? (mm == 4 ? 2 : 1) : 2);
    if (!planned && fx && a.M > 2) {
        if (g_tune.gemv_i4_kernel != 3 || bf16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;     // the caller has faster kernels for this shape
        fx = false;
        planned = plan_planes(UW, (size_t)227 * 1024, 2);
    }
    if (!planned) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    UnitsParams& p = pl.p;
    const int grid = pl.grid;
    const size_t smem = pl.smem;
    p.status = ctx->d_status;
    p.bf16 = bf16 ? 1 : 0;
    p.push = PushTarget{};
    if (a.push) {
        // only the fixed-point variant pushes, and only plain (non-SwiGLU) outputs with an even row count
        if (!fx || a.swiglu || (nout & 1)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        p.push = *a.push;
    }
    {
        const uint32_t upt = (uint32_t)(nacc * pl.U);
        p.inv_upt = upt > 1 ? (uint32_t)((((uint64_t)1 << 32) + upt - 1) / upt) : 0u;
        p.inv_U = pl.U > 1 ? (uint32_t)((((uint64_t)1 << 32) + (uint32_t)pl.U - 1) / (uint32_t)pl.U) : 0u;
    }

    cudaError_t e;
    if (fx) {
        // packed weights as a 3-D tensor {128 bytes, N rows, K/256 lines}; a chunk is one box
        // {128, 16, cg/2}, 128-byte swizzle keyed by the row
        alignas(64) CUtensorMap map;
        const uint64_t dims[3] = {128, (uint64_t)a.N, (uint64_t)a.K / 256};
        const uint64_t strides[2] = {(uint64_t)a.K / 2, 128};
        const uint32_t box[3] = {128, 16, (uint32_t)cg / 2};
        if (!encode_tensor_map_u8(&map, 3, a.w, dims, strides, box, true)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        const bool pdl = pdl_allowed(ctx, a.weights_volatile);
        if (a.M == 1)
            e = a.swiglu ? launch_units_fx_cg<1, true>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream)
                         : launch_units_fx_cg<1, false>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream);
        else if (a.M == 2)
            e = a.swiglu ? launch_units_fx_cg<2, true>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream)
                         : launch_units_fx_cg<2, false>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream);
        else
            e = a.swiglu ? launch_units_fx_cg<4, true>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream)
                         : launch_units_fx_cg<4, false>(pdl, cg, pl.uw, map, p, grid, smem, ctx->stream);
    } else if (a.M == 1) {
        e = a.swiglu ? launch_units_cg<1, true, true>(cg, p, grid, smem, ctx->stream)
                     : launch_units_cg<1, false, true>(cg, p, grid, smem, ctx->stream);
    } else if (a.swiglu) {
        e = MT == 1 ? launch_units_cg<1, true, false>(cg, p, grid, smem, ctx->stream)
                    : launch_units_cg<2, true, false>(cg, p, grid, smem, ctx->stream);
    } else {
        e = MT == 1 ? launch_units_cg<1, false, false>(cg, p, grid, smem, ctx->stream)
                    : launch_units_cg<2, false, false>(cg, p, grid, smem, ctx->stream);
    }
    count_launch(fx ? "lux_qgemv_i4_g128_units_fx" : "lux_qgemv_i4_g128_units");
    return map_cuda(e, "lux_qgemv_i4_g128_units");
}

const void* kernel_addr_qgemv_i4_units() { return (const void*)lux_qgemv_i4_g128_units<1, false, false, 4>; }
const void* kernel_addr_qgemv_i4_units_fx() { return (const void*)lux_qgemv_i4_g128_units_fx<1, false, 4, 16>; }
const void* kernel_addr_qgemv_i4_units_fx_swiglu() { return (const void*)lux_qgemv_i4_g128_units_fx<1, true, 4, 16>; }
const void* kernel_addr_qgemv_i4_units_fx_batch2() { return (const void*)lux_qgemv_i4_g128_units_fx<2, false, 4, 16>; }
const void* kernel_addr_qgemv_i4_units_fx_batch4() { return (const void*)lux_qgemv_i4_g128_units_fx<4, false, 4, 16>; }

}  // namespace luxcuda
