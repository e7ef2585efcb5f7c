// int4 g128 weight-only GEMM on tcgen05 with the converted WEIGHTS as the tensor-memory A
// operand: the default for every batch the tensor-core route takes (M >= 33) without SwiGLU.
//
//   y[M, N] = x[M, K] . dequant(W[N, K])^T      x, y bf16 or f16; f32 accumulate in TMEM
//
// Same contraction as matmul_nax_grouped (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:
// 568-626) and the same dequantized values as dequantize_nax_int4_asym (:312-330) narrowed once.
// The accumulator is held transposed: D[weight row, batch row], 128 weight rows on the 128 TMEM
// lanes and 256 batch rows on 256 columns, so that
//
//   * one tcgen05.mma is 128 x 256 x 16 (the shape that issues at the full tensor rate),
//   * a weight tile is converted once per 256 batch rows,
//   * the converted tile never touches shared memory: a converting thread owns one weight row
//     (= its TMEM lane), reads that row's packed bytes straight from global memory into
//     registers one quantization group ahead, and writes the converted 64-K block with one
//     tcgen05.st; shared memory only carries the x tiles (TMA, 128B swizzle) the tensor core
//     reads as the B operand.
//
// The ring works in units of 128 K (one quantization group, two 64-K swizzle blocks): up to three
// units of x in shared memory and of converted weights in TMEM.
//
//   warp 0        TMA producer of the x tiles (256 batch rows x 128 K per unit, two boxes).
//   warp 1        one wait, eight tcgen05.mma (A in TMEM, B in shared memory) and one commit per
//                 unit; the commit hands the unit back to the producer and the converters.
//   warps 2..     converters, in groups of four warps (one per TMEM lane quarter); group g takes
//                 units g, g + NG, ... of the CTA's K range.
//   warps 2..9    epilogue.
//
// Split-K: with KS = 2 (or 4) the CTAs of a cluster take the halves (quarters) of K for the same tile;
// each then leaves the accumulator columns the other one finishes in the pair's slot of a
// context-owned exchange buffer in global memory (L2-resident; no entry point allocates), one
// cluster barrier publishes both halves, and each adds what it found to its own half and writes
// it.  No multicast anywhere.  Every mbarrier wait is bounded; the cluster barriers are
// hardware barriers that every thread reaches on every path.
#include "common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <type_traits>

namespace luxcuda {

namespace {

using namespace tcptx;

// Two tile widths.  BN = 256 batch rows per CTA (= UMMA N = accumulator columns): one CTA per SM,
// all 512 TMEM columns, 3 x 64 KB of x.  BN = 64 for batches of up to 64 rows: 256 TMEM columns
// (accumulator [0, 64) + A units [64, 256)) and 3 x 16 KB of x, so that TWO CTAs share an SM.  Below
// ~128 batch rows the kernel is bound by its one MMA-issuing thread (wait + eight MMAs + commit per
// 128 K whatever N is); a second CTA per SM is a second issuing thread per SM.
constexpr int WA_BN = 256;                 // the wide tile (batch tiling of large batches uses it)
constexpr int WA_BN_SMALL = 64;
constexpr int WA_A_COLS = BK / 2;          // TMEM columns of a converted 64-K block (2 K per column)
constexpr int WA_UNIT_K = 128;             // K per ring slot: one quantization group = two 64-K blocks
constexpr int WA_UNIT_A_COLS = 2 * WA_A_COLS;
constexpr int WA_MAX_UNITS = 3;            // ring depth: 3 units of x in shared memory, 3 x 64 columns of A in TMEM
constexpr int WA_MAX_GROUPS = 3;           // converter groups <= ring depth
constexpr int WA_MAX_THREADS = (2 + 4 * WA_MAX_GROUPS) * 32;
constexpr int WA_SMALL_THREADS = (2 + 4 * 2) * 32;   // the narrow tile always runs two converter groups
// split-K exchange: the (BN / KS columns) x 128 rows x f32 block one CTA leaves for a peer
__host__ __device__ constexpr int wa_slot_bytes(int bn, int ks) { return (bn / ks) * BM * 4; }
constexpr int WA_STAGE_PITCH = 320;        // bytes per batch row of the staged output tile: 256 + 64, so that the
                                           // even and the odd lanes of a staging store use different banks


struct WaParams {
    const uint8_t* w;         // [N, K/2]
    const __half* scales;     // [N, G]
    const uint8_t* zeros;     // [N, ZS] or null
    void* y;                  // [M, N]
    uint32_t* status;
    unsigned char* splitk;    // KS == 2: one 128 KB slot per CTA pair for the exchange of partial sums
    int M, Nout, K, G, ZS;    // Nout = outputs = row pitch of y (half the weight rows with SwiGLU)
    int stages;               // ring depth in units of 128 K (x in shared memory, A in TMEM)
    int groups;               // converter groups of four warps, <= stages
    int up_row_offset;        // SwiGLU: weight row of `up` = weight row of `gate` + this (= number of outputs)
    int ncols;                // batch rows per tile = UMMA N: 256, or the batch rounded up to 16 when it is smaller
    int prefetch;             // units ahead of the register fetch at which a thread asks L2 for its row's line (0 = off)
};

// Group constants of one weight row: zero-point pair and the scale (bf16: split in two).
template <bool BF16>
__device__ __forceinline__ void group_consts(__half sh, uint32_t zp, uint32_t& zc, uint32_t& sa, uint32_t& sb) {
    if (BF16) {
        const uint32_t sbits = __float_as_uint(__half2float(sh));
        const uint32_t hi = sbits & 0xFFFF0000u;                    // top 8 significand bits
        const float lo = __half2float(sh) - __uint_as_float(hi);     // remaining 3 bits, exact
        sa = (hi >> 16) * 0x00010001u;
        sb = (__float_as_uint(lo) >> 16) * 0x00010001u;
        zc = (0x4300u | zp) | ((0x4180u | (zp << 3)) << 16);        // (128 + zp, 16 + zp)
    } else {
        sa = (uint32_t)__half_as_ushort(sh) * 0x00010001u;
        sb = 0u;
        zc = (0x6400u | zp) | ((0x5400u | (zp << 4)) << 16);        // (1024 + zp, 64 + zp)
    }
}

template <int CW> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[CW]);
template <> __device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_cols<8>(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr) : "memory");
}

template <bool BF16, int KS, bool SW, int BN>
__global__ void __launch_bounds__(BN == WA_BN_SMALL ? WA_SMALL_THREADS : WA_MAX_THREADS, BN == WA_BN_SMALL ? 2 : 1)
lux_qgemm_i4_tc_wa(const __grid_constant__ CUtensorMap map_x, const WaParams p) {
    constexpr int X_BYTES = BN * 128;                 // x tile of a stage: BN rows x 64 K x 2 bytes
    constexpr int UNIT_X_BYTES = 2 * X_BYTES;         // a ring slot: 128 K
    constexpr uint32_t TMEM_COLS = BN == WA_BN_SMALL ? 256u : 512u;   // accumulator [0, BN) + A units [BN, BN + 192)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int P = p.stages;                          // ring depth in units of 128 K
    unsigned char* x_ring = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_ring + (size_t)P * UNIT_X_BYTES);
    // bars[0..P) full, [P..2P) empty, [2P] acc_full
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int OUT_W = SW ? BM / 2 : BM;         // outputs per tile: with SwiGLU lanes 0..63 hold gate rows, 64..127 up rows
    const int n0 = blockIdx.x * OUT_W;              // first output (= first gate / weight row) of the tile
    const int m0 = blockIdx.y * BN;                 // first batch row of the tile
    const int ksplit = KS == 1 ? 0 : (int)blockIdx.z;
    const int k_len = p.K / KS;
    const int k_base = ksplit * k_len;
    const int U = k_len / WA_UNIT_K;                // units (= quantization groups) of this CTA
    const int g_base = k_base / WA_UNIT_K;

    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(P + s); };
    const uint32_t acc_full = bar0 + 8u * (uint32_t)(2 * P);

    auto load_x_unit = [&](int u, int s) {
        mbar_expect_tx(full(s), (uint32_t)(2 * p.ncols * 128));
        // byte coordinates: the map describes x as [M][2K bytes]; two 64-K boxes per unit
        const uint32_t dst = smem_u32(x_ring + (size_t)s * UNIT_X_BYTES);
        const int kbyte = (k_base + u * WA_UNIT_K) * 2;
        tma_load_2d(dst, &map_x, kbyte, m0, full(s));
        tma_load_2d(dst + X_BYTES, &map_x, kbyte + 128, m0, full(s));
    };

    // Converter state, set up before the CTA-wide barrier so that the first weight bytes are
    // already on their way while the barriers and the tensor memory are being set up.
    const int grp = (warp - 2) >> 2;
    const int quad = warp & 3;                          // TMEM lane quarter of this warp
    const int NG = p.groups;
    uint4 nq[4];                                        // next unit's 64 packed bytes of this thread's row
    __half nsh = __float2half(0.f);
    uint32_t nzb = 0x88u;                               // byte holding the next unit's zero-point nibble (raw: no use of a loaded value inside fetch)
    const uint8_t* wp = nullptr;
    const __half* sp = nullptr;
    const uint8_t* zrow = nullptr;
    auto fetch = [&](int u) {
        const uint4* src = reinterpret_cast<const uint4*>(wp + (size_t)u * (WA_UNIT_K / 2));
#pragma unroll
        for (int i = 0; i < 4; i++) nq[i] = __ldg(src + i);
        // the line two fetches ahead is asked for now, so that the register fetch finds it in L2
        if (p.prefetch && u + p.prefetch < U)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(wp + (size_t)(u + p.prefetch) * (WA_UNIT_K / 2)));
        nsh = __ldg(sp + u);
        if (zrow) nzb = (uint32_t)__ldg(zrow + ((g_base + u) >> 1));
    };
    if (warp >= 2) {
        const int r = quad * 32 + lane;                 // this thread's TMEM lane and its weight row
        const int wrow = SW ? (r < OUT_W ? n0 + r : p.up_row_offset + n0 + r - OUT_W) : n0 + r;
        wp = p.w + (size_t)wrow * (p.K / 2) + (k_base >> 1);
        sp = p.scales + (size_t)wrow * p.G + g_base;
        zrow = p.zeros ? p.zeros + (size_t)wrow * p.ZS : nullptr;
        if (grp < U) fetch(grp);
    } else if (tid == 1) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    } else if (tid == 0) {
        for (int s = 0; s < P; s++) {
            mbar_init(full(s), 5);          // the producer's expect_tx arrival + four converter warps
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // first lap of the x ring: every slot is free, nothing to wait for, and the loads need
        // neither the tensor memory nor the other warps, so they start before the CTA barrier.
        // x may come from the previous kernel of the stream (the weights fetched above are
        // static): wait for it here; the CTA barrier below orders every other thread's later
        // reads and the output stores behind this wait.
        pdl_wait();
        for (int u = 0; u < P && u < U; u++) load_x_unit(u, u);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a0 = tmem_base + (uint32_t)BN;         // first A unit

    bool ok = true;
    if (warp == 0) {
        // =============================== TMA producer of x ==============================
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 1;                  // second lap onwards: the first was issued above
            for (int u = P; u < U; u++) {
                if (!mbar_wait_relaxed(empty(s), ph ^ 1u, abort_flag)) break;
                load_x_unit(u, s);
                if (++s == P) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer =====================================
        // One wait, eight MMAs and one commit per unit: a satisfied mbarrier wait and a commit
        // cost this thread ~200 and ~100 cycles, so they are paid once per 128 K, not per 64.
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BF16, p.ncols);
            int s = 0;
            uint32_t ph = 0;
            for (int u = 0; u < U; u++) {
                ok = mbar_wait(full(s), ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(x_ring + (size_t)s * UNIT_X_BYTES));
                const uint32_t a_tmem = tmem_a0 + (uint32_t)(s * WA_UNIT_A_COLS);
#pragma unroll
                for (int k = 0; k < WA_UNIT_K / 16; k++) {
                    // 16 K = 8 TMEM columns of A; in x: +32 bytes inside the 128-byte swizzle row
                    // (+2 in the 16-byte address field), the second 64-K box X_BYTES further on
                    const uint64_t b_off = (uint64_t)((k >> 2) * (X_BYTES >> 4) + 2 * (k & 3));
                    umma_f16_ts(tmem_base, a_tmem + (uint32_t)(k * 8), b_desc + b_off, idesc, (u | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty(s));        // x unit and A unit reusable once these MMAs have read them
                if (++s == P) { s = 0; ph ^= 1u; }
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        // =============================== converters =====================================
        // Group `grp` takes units grp, grp + NG, ...; NG <= P keeps a group at most one lap of the
        // ring ahead of the commit it waits for, which is what a one-bit phase can tell apart.
        for (int u = grp; u < U && ok; u += NG) {
            uint4 cq[4];
#pragma unroll
            for (int i = 0; i < 4; i++) cq[i] = nq[i];
            uint32_t zc, sa, sb;
            group_consts<BF16>(nsh, (nzb >> (((g_base + u) & 1) * 4)) & 0xFu, zc, sa, sb);
            if (u + NG < U) fetch(u + NG);
            const int s = u % P;
            const uint32_t ph = (uint32_t)(u / P) & 1u;
            const uint32_t a_dst = tmem_a0 + ((uint32_t)(quad * 32) << 16) + (uint32_t)(s * WA_UNIT_A_COLS);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t words[8] = {cq[2 * h].x, cq[2 * h].y, cq[2 * h].z, cq[2 * h].w,
                                           cq[2 * h + 1].x, cq[2 * h + 1].y, cq[2 * h + 1].z, cq[2 * h + 1].w};
                uint32_t out[32];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint4 v = BF16 ? dequant_word_bf16(words[j], zc, sa, sb) : dequant_word_f16(words[j], zc, sa);
                    out[4 * j + 0] = v.x; out[4 * j + 1] = v.y; out[4 * j + 2] = v.z; out[4 * j + 3] = v.w;
                }
                if (h == 0) {
                    ok = warp_wait_relaxed(empty(s), ph ^ 1u, abort_flag, lane);   // A unit s free (warp-uniform outcome)
                    if (!ok) break;
                    tc_fence_after();
                }
                tmem_st32(a_dst + (uint32_t)(h * WA_A_COLS), out);
            }
            if (!ok) break;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(full(s));
        }
        if (ok && warp < 10) ok = warp_wait(acc_full, 0u, abort_flag, lane);
        if (ok) tc_fence_after();
    }
    __syncwarp();

    // =============================== epilogue ===========================================
    // Warps 2..9: quarter `quad` of the lanes (weight rows), half `eh` of the columns handled,
    // in chunks of 32 columns.  KS == 2: each CTA writes the 128 columns the peer finishes to the
    // pair's slot in global memory (it stays in L2), one cluster barrier publishes both halves, and
    // each adds what the peer left for it.  (Through distributed shared memory the same 64 KB took
    // 2 us per CTA, by remote stores and by bulk copies alike; the barrier's release waits for them.)
    // The narrowed output tile is staged in the idle ring for row-wise 16-byte stores.
    const int eh = (warp - 2) >> 2;
    const bool ep_warp = warp >= 2 && warp < 10;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int my_row = quad * 32 + lane;
    constexpr int KEEP = BN / KS;                               // columns this CTA writes
    const int keep0 = ksplit * KEEP;                            // the first of them
    constexpr int PER_WARP = KEEP / 2;                          // per epilogue warp
    constexpr int CW = PER_WARP < 32 ? PER_WARP : 32;           // columns per TMEM read (32, 16 or 8)
    constexpr int NCH = PER_WARP / CW;                          // reads per warp
    constexpr int SLOT = wa_slot_bytes(BN, KS);                 // split-K: KEEP columns x 128 rows x f32
    // an exchange block: 16 bytes (4 columns) per weight row, rows consecutive, [column quads][128 rows]:
    // a warp's store or load is one contiguous 512-byte piece
    unsigned char* stage = x_ring;                                           // [column][WA_STAGE_PITCH bytes]
    const bool odd = lane & 1;
    // lanes pair up: the even lane stages (row, row + 1) of the even columns, the odd lane of the odd ones
    unsigned char* srow = stage + (quad * 32 + (lane & ~1)) * 2;

    // CW accumulator columns of a peer's share -> the peer's block `dst`, column quad q0 onwards
    // (reads that lie entirely beyond the batch's columns are skipped, by sender and receiver alike)
    auto send_chunk = [&](int col, unsigned char* dst, int q0) {
        if (col >= p.ncols) return;
        uint32_t acc[CW];
        tmem_ld_cols<CW>(lane_addr + (uint32_t)col, acc);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < CW; i += 4)
            __stcg(reinterpret_cast<uint4*>(dst + ((q0 + (i >> 2)) * BM + my_row) * 16), make_uint4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]));
    };
    // what a peer left for CW of this CTA's columns (requested for every read of the warp before any is used)
    auto load_peer = [&](float4 (&r)[CW / 4], int c0, const unsigned char* rsrc, int q0) {
        if (keep0 + c0 >= p.ncols) return;
#pragma unroll
        for (int i = 0; i < CW / 4; i++) r[i] = __ldcg(reinterpret_cast<const float4*>(rsrc + ((q0 + i) * BM + my_row) * 16));
    };
    auto acc_add = [&](uint32_t (&acc)[CW], const float4 (&r4)[CW / 4]) {
#pragma unroll
        for (int i = 0; i < CW / 4; i++) {
            const float4 r = r4[i];
            acc[4 * i + 0] = __float_as_uint(__uint_as_float(acc[4 * i + 0]) + r.x);
            acc[4 * i + 1] = __float_as_uint(__uint_as_float(acc[4 * i + 1]) + r.y);
            acc[4 * i + 2] = __float_as_uint(__uint_as_float(acc[4 * i + 2]) + r.z);
            acc[4 * i + 3] = __float_as_uint(__uint_as_float(acc[4 * i + 3]) + r.w);
        }
    };
    // the accumulator columns keep0 + c0 .. + CW of this thread's row, plus up to three peers' sums
    auto finalize_chunk = [&](int c0, const float4 (&peer)[CW / 4], const unsigned char* more = nullptr, int q0 = 0) {
        if (keep0 + c0 >= p.ncols) return;
        uint32_t acc[CW];
        tmem_ld_cols<CW>(lane_addr + (uint32_t)(keep0 + c0), acc);
        tmem_ld_wait();
        if (KS >= 2) acc_add(acc, peer);
        if (KS == 4) {
            // sources 1 and 2 of this CTA's slot row (source 0 came in `peer`)
            float4 r1[CW / 4], r2[CW / 4];
            load_peer(r1, c0, more, q0);
            load_peer(r2, c0, more + SLOT, q0);
            acc_add(acc, r1);
            acc_add(acc, r2);
        }
        if constexpr (SW) {
            // gate and up of one output sit on different lanes (r and r + 64): the sums go to
            // shared memory as f32, [column][128 rows], and are combined in the write-out pass
            float* fcol = reinterpret_cast<float*>(stage) + my_row;
#pragma unroll
            for (int i = 0; i < CW; i++) fcol[(c0 + i) * BM] = __uint_as_float(acc[i]);
        } else {
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                const float mine = __uint_as_float(odd ? acc[i + 1] : acc[i]);
                const float give = __uint_as_float(odd ? acc[i] : acc[i + 1]);
                const float got = __shfl_xor_sync(0xffffffffu, give, 1);
                const uint32_t v = odd ? pack2<BF16>(got, mine) : pack2<BF16>(mine, got);
                *reinterpret_cast<uint32_t*>(srow + (c0 + i + (odd ? 1 : 0)) * WA_STAGE_PITCH) = v;
            }
        }
    };

    if (KS == 4) {
        // four CTAs, four quarters of K: CTA r finishes columns [KEEP r, KEEP r + KEEP); block (d, s) of
        // the tile's slot holds what the s-th CTA after d (cyclically) leaves for d.  One read per warp.
        static_assert(KS != 4 || NCH == 1, "four K splits: one TMEM read per epilogue warp");
        unsigned char* slot4 = p.splitk + (size_t)(blockIdx.x + gridDim.x * blockIdx.y) * (12 * SLOT);
        if (ep_warp && ok) {
#pragma unroll 1
            for (int dd = 1; dd < 4; dd++) {
                const int d = (ksplit + dd) & 3;                    // destination; this CTA is its source 3 - dd
                send_chunk(d * KEEP + eh * PER_WARP, slot4 + (size_t)(d * 3 + 3 - dd) * SLOT, eh * (PER_WARP / 4));
            }
        }
        cluster_sync_all();          // release / acquire at cluster scope: every block is published
        if (ep_warp && ok) {
            const unsigned char* row = slot4 + (size_t)(ksplit * 3) * SLOT;
            float4 r0[CW / 4];
            load_peer(r0, eh * PER_WARP, row, eh * (PER_WARP / 4));
            finalize_chunk(eh * PER_WARP, r0, row + SLOT, eh * (PER_WARP / 4));
        }
    } else if (KS == 2) {
        // each CTA leaves the KEEP columns the other one finishes in the pair's slot
        unsigned char* slot = p.splitk + (size_t)(blockIdx.x + gridDim.x * blockIdx.y) * (2 * SLOT);
        const int send0 = (1 - ksplit) * KEEP;
        unsigned char* theirs = slot + (size_t)(1 - ksplit) * SLOT;
        const unsigned char* mine = slot + (size_t)ksplit * SLOT;
        if (ep_warp && ok) {
#pragma unroll
            for (int ch = 0; ch < NCH; ch++)
                send_chunk(send0 + eh * PER_WARP + ch * CW, theirs, (eh * PER_WARP + ch * CW) / 4);
        }
        cluster_sync_all();          // release / acquire at cluster scope: both halves are published
        if (ep_warp && ok) {
            float4 rr[NCH][CW / 4];
#pragma unroll
            for (int ch = 0; ch < NCH; ch++) load_peer(rr[ch], eh * PER_WARP + ch * CW, mine, (eh * PER_WARP + ch * CW) / 4);
#pragma unroll
            for (int ch = 0; ch < NCH; ch++) finalize_chunk(eh * PER_WARP + ch * CW, rr[ch]);
        }
    } else if (ep_warp && ok) {
#pragma unroll 1
        for (int c0 = eh * PER_WARP; c0 < (eh + 1) * PER_WARP; c0 += CW) {
            const float4 none[CW / 4] = {};
            finalize_chunk(c0, none);
        }
    }
    if (ep_warp) {
        if (ok) tc_fence_before();
        // the eight epilogue warps (and only they) meet here on every path
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ok && SW) {
            // one batch row of the tile = 64 outputs = 128 contiguous bytes of y: 8 lanes x 16 bytes,
            // each lane combining eight (gate, up) pairs: silu(gate) * up, narrowed once
            // (steel_gemm_fused.wgsl:91-94, 452-558)
            const int sub = lane >> 3, l8 = lane & 7;
#pragma unroll 2
            for (int c = (warp - 2) * 4 + sub; c < KEEP; c += 32) {
                const int m = m0 + keep0 + c;
                if (m < p.M && keep0 + c < p.ncols) {
                    const float4* gp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(stage) + c * BM + l8 * 8);
                    const float4 g0 = gp[0], g1 = gp[1], u0 = gp[OUT_W / 4], u1 = gp[OUT_W / 4 + 1];
                    uint4 v;
                    v.x = pack2<BF16>(silu_f32(g0.x) * u0.x, silu_f32(g0.y) * u0.y);
                    v.y = pack2<BF16>(silu_f32(g0.z) * u0.z, silu_f32(g0.w) * u0.w);
                    v.z = pack2<BF16>(silu_f32(g1.x) * u1.x, silu_f32(g1.y) * u1.y);
                    v.w = pack2<BF16>(silu_f32(g1.z) * u1.z, silu_f32(g1.w) * u1.w);
                    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(p.y) + ((size_t)m * p.Nout + n0 + l8 * 8) * 2) = v;
                }
            }
        } else if (ok) {
            // one batch row of the tile = 128 weight rows = 256 contiguous bytes of y: 16 lanes x 16 bytes
            const int sub = lane >> 4, l16 = lane & 15;
#pragma unroll 4
            for (int c = (warp - 2) * 2 + sub; c < KEEP; c += 16) {
                const int m = m0 + keep0 + c;
                if (m < p.M) {
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + c * WA_STAGE_PITCH + l16 * 16);
                    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(p.y) + ((size_t)m * p.Nout + n0 + l16 * 8) * 2) = v;
                }
            }
        }
    }

    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C050002u);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <bool BF16, int KS, bool SW, int BN>
cudaError_t launch_wa(bool pdl, const CUtensorMap& mx, const WaParams& p, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemm_i4_tc_wa<BF16, KS, SW, BN>;
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev].load(std::memory_order_relaxed) < smem) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev].store(smem, std::memory_order_relaxed);
    }
    return launch_pdl(pdl, kfn, grid, dim3((unsigned)threads), smem, st, (unsigned)KS, mx, p);
}

}  // namespace

// Takes int4 GEMMs without a push epilogue whose outputs come in whole tiles (128 weight rows;
// with SwiGLU 64 outputs = 64 gate + 64 up rows); everything else stays with lux_qgemm_i4_tc.
LuxBackendError launch_qgemm_i4_tc_wa(Context* ctx, const QArgs& a) {
    const int nout = a.swiglu ? a.N / 2 : a.N;
    const int out_w = a.swiglu ? BM / 2 : BM;                   // outputs per tile
    if (a.push || nout % out_w || a.K % 128 || a.M < 1) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (a.scale_dtype != LUX_QDTYPE_F16 || a.x_dtype != a.y_dtype) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (a.x_dtype != LUX_QDTYPE_BF16 && a.x_dtype != LUX_QDTYPE_F16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15u) || (a.K / 2) % 16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    // x is fetched by TMA and y written in 16-byte pieces: a caller's oddly offset view stays with the
    // kernels that use plain loads and stores
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.y) & 15u)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    const bool bf16 = a.x_dtype == LUX_QDTYPE_BF16;

    // Split K over a cluster of two or four CTAs when whole tiles alone would leave most slots idle
    // (`slots` = CTAs resident at once).
    auto plan = [&](int bn, int slots, int& ks_out) {
        const int tiles = (nout / out_w) * ((a.M + bn - 1) / bn);
        const bool can_split = a.K % 256 == 0 && (size_t)tiles * (2 * wa_slot_bytes(bn, 2)) <= ctx->d_splitk_bytes;
        const bool can_split4 = a.K % 512 == 0 && (size_t)tiles * (12 * wa_slot_bytes(bn, 4)) <= ctx->d_splitk_bytes;
        int ks = (tiles * 4 <= slots && can_split4) ? 4 : (tiles * 2 <= slots && can_split) ? 2 : 1;
        if (g_tune.gemm_tc_splitk == 1 || (g_tune.gemm_tc_splitk == 2 && can_split) || (g_tune.gemm_tc_splitk == 4 && can_split4))
            ks = g_tune.gemm_tc_splitk;
        ks_out = ks;
        return tiles * ks;                                      // CTAs of the launch
    };
    // Batches of up to 64 rows may take the narrow tile, two CTAs per SM: worth it when the launch has
    // more CTAs than SMs (measured, config 4 at 16..64 rows: gate_up 41 -> 27 us, qkv 12.9 -> 11.0 us;
    // with 128 CTAs or fewer, `o` and `down`, the narrow tile only packs them onto half the SMs:
    // 9.2 -> 10.4 us and 19.9 -> 24.8 us).  gemm_wa_narrow = 1 / 2 forces the narrow / wide tile.
    int ks = 1, ks_narrow = 1;
    plan(WA_BN, ctx->sm_count, ks);
    bool narrow = false;
    if (a.M <= WA_BN_SMALL && g_tune.gemm_wa_narrow != 2) {
        const int ctas = plan(WA_BN_SMALL, 2 * ctx->sm_count, ks_narrow);
        narrow = ctas > ctx->sm_count || g_tune.gemm_wa_narrow == 1;
    }
    if (narrow) ks = ks_narrow;
    const int bn = narrow ? WA_BN_SMALL : WA_BN;
    const int stages = g_tune.gemm_tc_stages >= 2 && g_tune.gemm_tc_stages <= WA_MAX_UNITS ? g_tune.gemm_tc_stages : WA_MAX_UNITS;
    int groups = g_tune.gemm_tc_groups >= 2 && g_tune.gemm_tc_groups <= WA_MAX_GROUPS ? g_tune.gemm_tc_groups : 2;
    groups = narrow ? 2 : std::min(groups, stages);
    const size_t smem = 1024 + (size_t)stages * (2 * bn * 128) + 512;

    CUtensorMap mx;
    const uint64_t dims[2] = {(uint64_t)a.K * 2, (uint64_t)a.M};
    const uint64_t strides[1] = {(uint64_t)a.K * 2};
    const int ncols = a.M >= bn ? bn : (a.M + 15) / 16 * 16;
    const uint32_t box[2] = {128, (uint32_t)ncols};
    if (!encode_tensor_map_u8(&mx, 2, a.x, dims, strides, box, true)) return LUX_BACKEND_ERROR_INTERNAL;

    WaParams p{};
    p.w = a.w;
    p.scales = (const __half*)a.scales;
    p.zeros = a.zeros;
    p.y = a.y;
    p.status = ctx->d_status;
    p.splitk = (unsigned char*)ctx->d_splitk;
    p.M = a.M; p.Nout = nout; p.K = a.K; p.G = a.G; p.ZS = (a.G + 1) / 2;
    p.up_row_offset = a.swiglu ? nout : 0;
    p.stages = stages;
    p.groups = groups;
    p.ncols = ncols;
    p.prefetch = g_tune.gemm_wa_prefetch < 0 ? 0 : (g_tune.gemm_wa_prefetch > 0 ? g_tune.gemm_wa_prefetch : 2);

    dim3 grid(nout / out_w, (a.M + bn - 1) / bn, ks);
    const int threads = (2 + 4 * groups) * 32;                  // groups >= 2: the epilogue needs warps 2..9
    const bool pdl = pdl_allowed(ctx, a.weights_volatile);
    auto go = [&](auto bf_tag, auto sw_tag, auto bn_tag) {
        constexpr bool BF_ = decltype(bf_tag)::value;
        constexpr bool SW_ = decltype(sw_tag)::value;
        constexpr int BN_ = decltype(bn_tag)::value;
        return ks == 4 ? launch_wa<BF_, 4, SW_, BN_>(pdl, mx, p, grid, threads, smem, ctx->stream)
             : ks == 2 ? launch_wa<BF_, 2, SW_, BN_>(pdl, mx, p, grid, threads, smem, ctx->stream)
                       : launch_wa<BF_, 1, SW_, BN_>(pdl, mx, p, grid, threads, smem, ctx->stream);
    };
    auto go_bn = [&](auto bf_tag, auto sw_tag) {
        return narrow ? go(bf_tag, sw_tag, std::integral_constant<int, WA_BN_SMALL>{})
                      : go(bf_tag, sw_tag, std::integral_constant<int, WA_BN>{});
    };
    cudaError_t e;
    if (a.swiglu) e = bf16 ? go_bn(std::true_type{}, std::true_type{}) : go_bn(std::false_type{}, std::true_type{});
    else          e = bf16 ? go_bn(std::true_type{}, std::false_type{}) : go_bn(std::false_type{}, std::false_type{});
    count_launch(bf16 ? "lux_qgemm_i4_tc_wa_bf16" : "lux_qgemm_i4_tc_wa_f16");
    return map_cuda(e, "lux_qgemm_i4_tc_wa");
}


const void* kernel_addr_qgemm_i4_tc_wa_bf16() { return (const void*)lux_qgemm_i4_tc_wa<true, 2, false, WA_BN>; }
const void* kernel_addr_qgemm_i4_tc_wa_f16() { return (const void*)lux_qgemm_i4_tc_wa<false, 2, false, WA_BN>; }
const void* kernel_addr_qgemm_i4_tc_wa_bf16_swiglu() { return (const void*)lux_qgemm_i4_tc_wa<true, 1, true, WA_BN>; }
const void* kernel_addr_qgemm_i4_tc_wa_f16_swiglu() { return (const void*)lux_qgemm_i4_tc_wa<false, 1, true, WA_BN>; }

}  // namespace luxcuda
