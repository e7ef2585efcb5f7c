// lux_qgemv_i8_g32_units_fx -- int8 g32 decode GEMV (f32 in / out, batch 1 or 2), the int8
// counterpart of lux_qgemv_i4_g128_units_fx.
//
//   y[m, n] = sum_g scale[n, g] * sum_{k in group g} w[n, k] * x[m, k]        (group = 32 K)
//
// The weights ARE signed bytes: they feed mma.sync.m16n8k32.s8.s8 straight from shared memory
// with no unpacking at all (one mma per 16 rows x one quantization group).  The activations are
// converted once per CTA to block fixed point per group of 32: X = rint(x * 2^(30-E)) with 2^E
// just above the group's largest |x|.  An f32 has 24 significant bits, so every value down to 2^-6
// of the group's largest magnitude is represented exactly and a smaller one is rounded with an
// absolute error of at most 2^(E-31), i.e. 2^-31 of the group's largest magnitude (the reference's
// f32 products round at 2^-24 relative, kernels/wgsl/gpu/quantized_nax.wgsl:615-618); groups whose
// largest magnitude is below 2^-96 count as zero.  X is split into four signed bytes
// X = d0 + 256 d1 + 65536 d2 + 2^24 d3 that ride in four of the eight B columns (all eight for
// batch 2).  The int32 accumulators are exact and start at the bit pattern of 1.5 * 2^23, so they
// read as floats without a conversion; the group sum is scaled by 2^(E-30) 256^plane and the
// group's f32 scale, and the planes are added once per unit.
//
// Structure as in the int4 kernel: one persistent CTA per SM owns a contiguous range of 16-row
// tiles; a tile is cut along K into units of KS groups and every (tile, unit) belongs to ONE
// warp; each warp has a private FIFO of 4 KB chunks (16 rows x 256 K) filled by TMA (box
// 128 bytes x 16 rows x 2 lines, 128-byte swizzle keyed by the row, no multicast) completing on
// the warp's own per-slot mbarrier; the CTA's scales are staged once by cp.async; a unit's
// partial sums go to its own slot and the CTA adds them in a fixed order after one
// __syncthreads.  Every barrier wait is bounded; a wait that gives up sets a flag, every warp
// leaves its loop, and the status word reports it.
//
// Replaces matmul_nax_grouped on dequantize_nax_int8_group weights (luxcpp/webgpu
// kernels/wgsl/gpu/quantized_nax.wgsl:364-381, 568-626) in a different summation order.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>

namespace luxcuda {

namespace {

constexpr int UW = 16;                          // warps per CTA
constexpr int MAX_STAGES = 8;
constexpr int CHUNK = 4096;                     // bytes: 16 rows x 8 groups x 32
constexpr int CGRP = 8;                         // groups per chunk
constexpr uint32_t WAIT_LIMIT = 1u << 15;       // one try_wait may suspend for microseconds: ~0.1 s in all

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
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
// D(s32) += A(s8, 16x32) * B(s8, 32x8)
__device__ __forceinline__ void mma16832_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Fragment row g reads tile row (g & 3) * 2 + (g >> 2) (and that + 8): with the swizzle keyed by
// row % 8 and 8-byte reads, the four rows of a half-warp (0, 2, 4, 6 or 1, 3, 5, 7) land in
// different bank groups.
__device__ __forceinline__ int row_of(int g) { return ((g & 3) << 1) | (g >> 2); }

struct I8UnitsParams {
    const float* x;         // [M, K]
    const int8_t* w;        // [N, K]
    const float* scales;    // [N, G]
    float* y;               // [M, N]
    uint32_t* status;       // device status word for a wait that gave up (may be null)
    int M, N, K, G;         // G = K / 32
    int tiles_base, tiles_rem;   // CTA b owns tiles [b*base + min(b, rem), +base + (b < rem))
    int U, KS;              // units per tile and groups per unit (U * KS == G, KS % 8 == 0)
    int S;                  // FIFO depth in chunks (per warp)
    int units_cap;          // partial-sum slots per CTA
    int rows_cap;           // weight rows whose scales are staged per CTA
    uint32_t inv_U;         // ceil(2^32 / U) (0 when U == 1): division-free unit table
    int planes;             // signed byte planes of the activations, 4 or 3
};

// Shared memory: [FIFOs: UW x S x 4 KB, 1024-byte aligned]
// [xq: G x (4 planes x MM) x 32 signed bytes in K order]
// [xmeta: G x 8 columns x coefficient 2^(E-30) 256^plane; column = plane (MM = 1) or 2 plane + m]
// [scales: rows_cap x G f32][partials: units_cap x 16 rows x MM float][unit table][barriers][flag]
//
// mma operand order inside a group: lane (g, t) supplies k = 8t .. 8t+7 of its two rows (a0 / a1 =
// bytes 8t..8t+3 of rows g / g+8, a2 / a3 = bytes 8t+4..8t+7) and, for the B operand, the same
// eight k of column g: both are plain contiguous 8-byte reads.
template <int MM, int UWT>
__global__ void __launch_bounds__(UWT * 32, UWT == 8 ? 2 : 1)
lux_qgemv_i8_g32_units_fx(const __grid_constant__ CUtensorMap map_w, const I8UnitsParams p) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by OFFSET from the __shared__ symbol (keeps 32-bit shared addressing)
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int UW = UWT;                             // warps per CTA (shadows the file-wide 16)
    const int XG = p.planes * MM * 32;                  // bytes of xq per group
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    unsigned char* fifo = smem + (size_t)warp * p.S * CHUNK;
    unsigned char* xq = smem + (size_t)UW * p.S * CHUNK;
    float* xmeta = reinterpret_cast<float*>(xq + (size_t)p.G * XG);
    float* ssm = xmeta + (size_t)p.G * 8;
    float* part = ssm + (size_t)p.rows_cap * p.G;
    int2* utab = reinterpret_cast<int2*>(part + (size_t)p.units_cap * 16 * MM);
    uint64_t* bars = reinterpret_cast<uint64_t*>(utab + p.units_cap);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + UW * MAX_STAGES);
    const uint32_t bar0 = smem_u32(bars + warp * MAX_STAGES);          // this warp's barriers

    const int b = (int)blockIdx.x;
    const int tile_lo = b * p.tiles_base + min(b, p.tiles_rem);
    const int ntiles = p.tiles_base + (b < p.tiles_rem ? 1 : 0);
    const int nunits = ntiles * p.U;
    const int NC = p.KS / CGRP;                          // chunks per unit
    const int my_units = nunits > warp ? (nunits - warp + UW - 1) / UW : 0;
    const int my_chunks = my_units * NC;
    const int nrows = ntiles * 16;

    pdl_launch_dependents();
    const int npieces = p.M * p.K / 8;                   // pieces of 8 floats, (m, group, quarter)
    uint4 xa, xb;

    // ---- barriers and the first weight request: the very first thing every warp does ----------
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
            // unit table exists (a line of the tensor map is 128 K = 4 groups)
            const int tl = p.U == 1 ? warp : (int)__umulhi((uint32_t)warp, p.inv_U), k = warp - tl * p.U;
            mbar_expect_tx(bar0, (uint32_t)CHUNK);
            tma_load_3d(smem_u32(fifo), &map_w, 0, (tile_lo + tl) * 16, (k * p.KS) >> 2, bar0, policy);
            issued = 1;
        }
    }
    for (int ul = warp + lane * UW; ul < nunits; ul += 32 * UW) {
        const int tl = p.U == 1 ? ul : (int)__umulhi((uint32_t)ul, p.inv_U), k = ul - tl * p.U;
        utab[ul] = make_int2(tl * 16, k * p.KS);         // {first row inside the CTA, first group}
    }
    __syncwarp();

    // A cursor walks this warp's chunks in order: unit index ui (0, 1, ..), chunk ci inside it.
    struct Cursor { int ui, ci; };
    auto advance = [&](Cursor& c) { if (++c.ci == NC) { c.ci = 0; ++c.ui; } };
    Cursor cload{0, 0}, ccur{0, 0};
    if (issued) advance(cload);                           // lane 0: the first chunk is already on its way
    // lane 0 only: ask for the next chunk into FIFO slot `slot` (the slot's barrier is armed first)
    auto issue_chunk = [&](int slot) {
        const int2 u = utab[warp + cload.ui * UW];
        const uint32_t bar = bar0 + 8u * (uint32_t)slot;
        mbar_expect_tx(bar, (uint32_t)CHUNK);
        tma_load_3d(smem_u32(fifo + (size_t)slot * CHUNK), &map_w, 0, tile_lo * 16 + u.x, (u.y + cload.ci * CGRP) >> 2, bar,
                    policy);
        advance(cload);
        issued++;
    };

    // ---- this CTA's scales (one cp.async group): rows are contiguous ---------------------------
    {
        const int n16 = nrows * p.G / 4;                 // 16-byte pieces
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.scales + (size_t)tile_lo * 16 * p.G);
        const uint32_t dst = smem_u32(ssm);
        for (int i = tid; i < n16; i += UW * 32) cp_async16(dst + i * 16, src + (size_t)i * 16);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // Everything above read static model state only; x may come from the previous kernel.
    pdl_wait();

    // ---- x -> block fixed point, four signed byte planes in K order -----------------------------
    for (int c = tid; c < npieces; c += UW * 32) {
        xa = __ldg(reinterpret_cast<const uint4*>(p.x) + 2 * c);
        xb = __ldg(reinterpret_cast<const uint4*>(p.x) + 2 * c + 1);
        const int per_row = p.K / 8;
        const int m = (MM == 2 && c >= per_row) ? 1 : 0, cr = c - m * per_row;
        const int grp = cr >> 2, l4 = cr & 3;
        const uint32_t bits[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        // largest |x| of the group as a bit pattern (monotonic for non-negative floats; inf and
        // NaN compare above every finite value)
        uint32_t mb = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) mb = max(mb, bits[i] & 0x7fffffffu);
        mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
        mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
        const bool bad = mb >= 0x7f800000u;
        // amax = f * 2^E with f in [0.5, 1): biased exponent eb = E + 126.  x * 2^(30-E) is exact
        // up to the final rounding to an integer.
        const uint32_t eb = mb >> 23;
        const bool live = eb >= 30u && !bad;             // below 2^-96: the group counts as zero
        // four planes: 30 bits below the block exponent; three (rows too long for four): 22
        const uint32_t sh = p.planes == 4 ? 30u : 22u;
        const float up = live ? __uint_as_float((253u + sh - eb) << 23) : 0.0f;     // 2^(sh-E)
        float down = live ? __uint_as_float((eb + 1u - sh) << 23) : 0.0f;           // 2^(E-sh)
        if (bad) down = __uint_as_float(0x7FC00000u);    // inf / NaN in the group: the outputs are NaN
        // I + 0x80808080 has bytes d0+128 .. d3+128 (I = d0 + 256 d1 + 65536 d2 + 2^24 d3, digits in
        // [-128, 127]; |I| <= 2^30 fits); flipping the top bit of each turns them into the digits as
        // signed bytes.
        uint32_t e[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            e[i] = ((uint32_t)__float2int_rn(__uint_as_float(bits[i]) * up) + 0x80808080u) ^ 0x80808080u;
        // byte transpose: word h of plane pl holds the digits of k = 4h .. 4h+3
        uint32_t pw[4][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a01 = prmt(e[4 * h], e[4 * h + 1], 0x5140), a23 = prmt(e[4 * h + 2], e[4 * h + 3], 0x5140);
            const uint32_t c01 = prmt(e[4 * h], e[4 * h + 1], 0x7362), c23 = prmt(e[4 * h + 2], e[4 * h + 3], 0x7362);
            pw[0][h] = prmt(a01, a23, 0x5410);
            pw[1][h] = prmt(a01, a23, 0x7632);
            pw[2][h] = prmt(c01, c23, 0x5410);
            pw[3][h] = prmt(c01, c23, 0x7632);
        }
#pragma unroll
        for (int pl = 0; pl < 4; pl++) {
            if (pl == 3 && p.planes == 3) break;             // the fourth digit of a 23-bit number is 0
            *reinterpret_cast<uint2*>(xq + (size_t)grp * XG + (pl * MM + m) * 32 + l4 * 8) = make_uint2(pw[pl][0], pw[pl][1]);
        }
        if (l4 == 0) {
            // Lane t of a consumer reads {coefficient of column 2t, of column 2t+1}.  Every float of
            // the group's eight is written exactly once; columns without a plane behind them get 0
            // (their accumulators hold garbage).
            float* xm = xmeta + grp * 8;
            if (MM == 1) {
                *reinterpret_cast<float4*>(xm) = make_float4(down, down * 256.0f, down * 65536.0f, p.planes == 4 ? down * 16777216.0f : 0.f);
                *reinterpret_cast<float4*>(xm + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                xm[m] = down;
                xm[2 + m] = down * 256.0f;
                xm[4 + m] = down * 65536.0f;
                xm[6 + m] = p.planes == 4 ? down * 16777216.0f : 0.f;
            }
        }
    }
    // fill the rest of the FIFO (the async engine queues the requests: nothing stalls here)
    if (lane == 0)
        for (int s0 = 1; s0 < p.S && issued < my_chunks; s0++) issue_chunk(s0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // the scales have landed
    __syncthreads();

    // lanes of column g >= 4*MM multiply garbage that nobody reads: point them at a valid column
    const int col = min(g, p.planes * MM - 1);
    const int xcol_off = col * 32 + t * 8;
    const int rg = row_of(g);                            // tile row behind fragment row g
    float res[2][2];                                     // [row half][column 2t / 2t+1 of the lane]
    res[0][0] = res[0][1] = res[1][0] = res[1][1] = 0.0f;
    constexpr int MAGIC = 0x4B400000;                    // float 1.5 * 2^23: MAGIC + i reads as 12582912 + i

    int slot = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int q = 0; q < my_chunks; q++) {
        ok = warp_wait(bar0 + 8u * (uint32_t)slot, ph, abort_flag, lane);
        if (!ok) break;
        uint2 wa[CGRP], wb[CGRP];
        {
            const unsigned char* st = fifo + (size_t)slot * CHUNK + rg * 128 + (t & 1) * 8;
#pragma unroll
            for (int u = 0; u < CGRP; u++) {
                // line u/4, rows rg and rg+8, logical 16-byte piece (u%4)*2 + t/2, swizzled by row%8
                const unsigned char* ln = st + (u >> 2) * 2048 + (((((u & 3) << 1) | (t >> 1)) ^ rg) << 4);
                wa[u] = *reinterpret_cast<const uint2*>(ln);
                wb[u] = *reinterpret_cast<const uint2*>(ln + 1024);
            }
        }
        // every lane has read the slot: hand it back to the async engine for the next chunk
        __syncwarp();
        if (lane == 0 && issued < my_chunks) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_chunk(slot);
        }
        if (++slot == p.S) { slot = 0; ph ^= 1u; }

        const int2 u2 = utab[warp + ccur.ui * UW];
        const int gi0 = u2.y + ccur.ci * CGRP;
        const float* sa = ssm + (size_t)(u2.x + rg) * p.G + gi0;
        const float* sb = sa + (size_t)8 * p.G;
        const float4 sa0 = *reinterpret_cast<const float4*>(sa), sa1 = *reinterpret_cast<const float4*>(sa + 4);
        const float4 sb0 = *reinterpret_cast<const float4*>(sb), sb1 = *reinterpret_cast<const float4*>(sb + 4);
        const float fsa[CGRP] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
        const float fsb[CGRP] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
#pragma unroll
        for (int u = 0; u < CGRP; u++) {
            const uint2 xv = *reinterpret_cast<const uint2*>(xq + (size_t)(gi0 + u) * XG + xcol_off);
            // the accumulator starts at MAGIC, so that it can be read as a float afterwards:
            // |sum| <= 32 x 127 x 128 < 2^22
            int acc[4] = {MAGIC, MAGIC, MAGIC, MAGIC};
            mma16832_s8s8(acc, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
            const float2 cf = *reinterpret_cast<const float2*>(xmeta + (gi0 + u) * 8 + 2 * t);
            const float va0 = __int_as_float(acc[0]) - 12582912.0f, va1 = __int_as_float(acc[1]) - 12582912.0f;
            const float vb0 = __int_as_float(acc[2]) - 12582912.0f, vb1 = __int_as_float(acc[3]) - 12582912.0f;
            if (MM == 1) {
                // both columns are planes of batch row 0: combine them before the scale
                res[0][0] = fmaf(fsa[u], fmaf(cf.y, va1, cf.x * va0), res[0][0]);
                res[1][0] = fmaf(fsb[u], fmaf(cf.y, vb1, cf.x * vb0), res[1][0]);
            } else {
                res[0][0] = fmaf(fsa[u] * cf.x, va0, res[0][0]);
                res[0][1] = fmaf(fsa[u] * cf.y, va1, res[0][1]);
                res[1][0] = fmaf(fsb[u] * cf.x, vb0, res[1][0]);
                res[1][1] = fmaf(fsb[u] * cf.y, vb1, res[1][1]);
            }
        }
        // end of a unit: add the planes (lanes t) and drop the partial sums into the unit's slot
        if (ccur.ci == NC - 1) {
            const int ul = warp + ccur.ui * UW;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int m = 0; m < MM; m++) {
                    res[h][m] += __shfl_xor_sync(0xffffffffu, res[h][m], 1);
                    res[h][m] += __shfl_xor_sync(0xffffffffu, res[h][m], 2);
                }
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < MM; m++) {
                    part[((size_t)ul * 16 + rg) * MM + m] = res[0][m];
                    part[((size_t)ul * 16 + rg + 8) * MM + m] = res[1][m];
                }
            }
            res[0][0] = res[0][1] = res[1][0] = res[1][1] = 0.0f;
        }
        advance(ccur);
    }

    __syncthreads();
    if (*abort_flag) {
        // A bounded wait gave up: report it and give copies still in flight time to land in
        // this CTA's shared memory before it is released.
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C050004u);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
        return;
    }
    // ---- every unit of the CTA is done: add the U partials of each output ----------------------
    const int nout = ntiles * 16 * MM;
    for (int o = tid; o < nout; o += UW * 32) {
        const int m = o % MM, r = (o / MM) & 15, tl = o / (16 * MM);
        const float* v0 = part + ((size_t)(tl * p.U) * 16 + r) * MM + m;
        float sum = 0.0f;
        for (int k = 0; k < p.U; k++) sum += v0[(size_t)k * 16 * MM];        // fixed order: deterministic
        p.y[(size_t)m * p.N + (tile_lo + tl) * 16 + r] = sum;
    }
}

template <int MM, int UWT>
cudaError_t launch_inst(bool pdl, const CUtensorMap& map, const I8UnitsParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemv_i8_g32_units_fx<MM, UWT>;
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

}  // namespace

// Returns NOT_SUPPORTED when the shape does not suit this kernel (the caller then uses
// lux_qgemv_i8_g32_f32): batch above 2, K not a multiple of 256 (a chunk is eight groups), an
// output size that is not a multiple of the 16-row tile, operands that are not 16-byte aligned,
// or activations / scale tables too large to stage next to one chunk of FIFO per warp.
LuxBackendError launch_qgemv_i8_units(Context* ctx, const QArgs& a) {
    if (a.M < 1 || a.M > 2 || a.K % 256 || a.N % 16 || a.G * 32 != a.K) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a.scales) & 15) || (reinterpret_cast<uintptr_t>(a.w) & 15) ||
        (reinterpret_cast<uintptr_t>(a.x) & 15))
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const int tiles = a.N / 16;
    const int grid = std::min(ctx->sm_count, tiles);
    const int tiles_per_cta = (tiles + grid - 1) / grid;

    // Geometry as in the int4 kernel: the whole SM with 16 warps; gemv_units_warps = 8 selects half an
    // SM (8 warps, at most 113 KB), measured slower there.
    struct Plan { int uw, S; size_t smem; I8UnitsParams p; };
    auto make_plan = [&](int uw, size_t budget, int min_stages, int planes, Plan& pl) -> bool {
        // Unit size KS (a multiple of the 8-group chunk, dividing G): the one that spreads the busiest
        // CTA's groups most evenly over its warps, each unit costing about one group of overhead.
        int KS = 0;
        double best = 1e30;
        for (int ks = CGRP; ks <= std::min(a.G, 256); ks += CGRP) {
            if (a.G % ks) continue;
            const int units = tiles_per_cta * (a.G / ks);
            const double cost = (double)((units + uw - 1) / uw) * (ks + 1.0);
            if (cost < best - 1e-9) { best = cost; KS = ks; }
        }
        if (g_tune.gemv_units_ks > 0 && a.G % g_tune.gemv_units_ks == 0 && g_tune.gemv_units_ks % CGRP == 0) KS = g_tune.gemv_units_ks;
        if (KS == 0) return false;
        const int U = a.G / KS;
        I8UnitsParams& p = pl.p;
        p = I8UnitsParams{};
        p.x = (const float*)a.x;
        p.w = (const int8_t*)a.w;
        p.scales = (const float*)a.scales;
        p.y = (float*)a.y;
        p.status = ctx->d_status;
        p.M = a.M;
        p.N = a.N;
        p.K = a.K;
        p.G = a.G;
        p.U = U;
        p.KS = KS;
        p.tiles_base = tiles / grid;
        p.tiles_rem = tiles % grid;
        p.units_cap = tiles_per_cta * U;
        p.rows_cap = tiles_per_cta * 16;
        p.inv_U = U > 1 ? (uint32_t)((((uint64_t)1 << 32) + (uint32_t)U - 1) / (uint32_t)U) : 0u;
        p.planes = planes;
        const size_t fixed = (size_t)a.G * planes * a.M * 32 + (size_t)a.G * 8 * sizeof(float) + (size_t)p.rows_cap * a.G * sizeof(float) +
                             (size_t)p.units_cap * 16 * a.M * sizeof(float) + (size_t)p.units_cap * sizeof(int2) +
                             (size_t)uw * MAX_STAGES * 8 + 16 + 1024;
        if (fixed + (size_t)min_stages * uw * CHUNK > budget) return false;
        const int max_chunks = (p.units_cap + uw - 1) / uw * (KS / CGRP);      // per warp
        int S = (int)std::min<size_t>((budget - fixed) / ((size_t)uw * CHUNK), MAX_STAGES);
        S = std::min(S, std::max(max_chunks, 1));
        if (g_tune.gemv_units_stages > 0) S = std::min(S, g_tune.gemv_units_stages);
        else S = std::min(S, uw == 8 ? 3 : 2);
        pl.uw = uw;
        pl.S = p.S = std::max(S, 1);
        pl.smem = fixed + (size_t)p.S * uw * CHUNK;
        return true;
    };
    Plan pl;
    bool planned = false;
    // four byte planes of the activations wherever they cost no FIFO depth, else three
    auto plan_planes = [&](int uw, size_t budget, int min_stages) -> bool {
        Plan p3, p4;
        const bool ok3 = g_tune.gemv_units_planes != 4 && make_plan(uw, budget, min_stages, 3, p3);
        const bool ok4 = g_tune.gemv_units_planes != 3 && make_plan(uw, budget, min_stages, 4, p4);
        if (ok4 && (!ok3 || p4.S >= p3.S)) { pl = p4; return true; }
        if (ok3) { pl = p3; return true; }
        return false;
    };
    if (g_tune.gemv_units_warps == 8) planned = plan_planes(8, (size_t)113 * 1024, 2);
    if (!planned && g_tune.gemv_units_warps != 8) planned = plan_planes(UW, (size_t)227 * 1024, 1);
    if (!planned) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    // int8 weights as a 3-D tensor {128 bytes, N rows, K/128 lines}; a chunk is one box {128, 16, 2},
    // 128-byte swizzle keyed by the row
    alignas(64) CUtensorMap map;
    const uint64_t dims[3] = {128, (uint64_t)a.N, (uint64_t)a.K / 128};
    const uint64_t strides[2] = {(uint64_t)a.K, 128};
    const uint32_t box[3] = {128, 16, 2};
    if (!encode_tensor_map_u8(&map, 3, a.w, dims, strides, box, true)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const bool pdl = pdl_allowed(ctx, a.weights_volatile);
    cudaError_t e;
    if (pl.uw == 8)
        e = a.M == 1 ? launch_inst<1, 8>(pdl, map, pl.p, grid, pl.smem, ctx->stream)
                     : launch_inst<2, 8>(pdl, map, pl.p, grid, pl.smem, ctx->stream);
    else
        e = a.M == 1 ? launch_inst<1, 16>(pdl, map, pl.p, grid, pl.smem, ctx->stream)
                     : launch_inst<2, 16>(pdl, map, pl.p, grid, pl.smem, ctx->stream);
    count_launch("lux_qgemv_i8_g32_units_fx");
    return map_cuda(e, "lux_qgemv_i8_g32_units_fx");
}

const void* kernel_addr_qgemv_i8_units_fx() { return (const void*)lux_qgemv_i8_g32_units_fx<1, 16>; }

}  // namespace luxcuda
