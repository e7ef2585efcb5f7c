// int4 g128 weight-only GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for
// batches too large for the streaming kernel (prefill, M >= 33).
//
//   y[M, N] = x[M, K] . dequant(W[N, K])^T      x, y bf16 or f16; f32 accumulate in TMEM
//
// Replaces matmul_nax_grouped (luxcpp/webgpu kernels/wgsl/gpu/quantized_nax.wgsl:568-626:
// 16x16 tiles, scalar f32 FMAs, two barriers per 16 K).  One CTA computes a 128 (batch)
// x BN (weight rows) tile:
//
//   warp 0      TMA producer: per 64-K block loads the x tile (128 x 64, 128B-swizzled)
//               and the PACKED weight tile (BN x 32 bytes) into a shared-memory ring.
//   warps 2..9  dequantizers: read packed nibbles from the ring, form (q - zp) exactly,
//               multiply by the group scale with ONE rounding to the operand type
//               (bf16: fma(d, s_hi, d*s_lo) with s = s_hi + s_lo split so that every
//               intermediate is exact; f16: one correctly rounded multiply), and store
//               the K-major, 128B-swizzled B tile the tensor core reads.  The values are
//               the same bits lux_qdequant produces (quantized_nax.wgsl:312-330 then one
//               narrowing).
//   warp 1      issues tcgen05.mma (M=128, N=BN, K=16; four per block) into TMEM and
//               commits each stage back to the producer.
//   warps 2..9  epilogue: tcgen05.ld the f32 accumulators, optional SwiGLU
//               (steel_gemm_fused.wgsl:452-558), narrow once, 16-byte stores.
//
// Every mbarrier wait is bounded: if it gives up, the CTA records a status word, lets
// outstanding copies land, frees its TMEM and returns; the host reports DEVICE_LOST.
// No cluster launch and no multicast anywhere: the same kernel serves multi-GPU runs.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>

namespace luxcuda {

namespace {

constexpr int BM = 128;              // batch rows per CTA (UMMA M)
constexpr int BK = 64;               // K per pipeline stage: one 128-byte swizzle row
constexpr int NUM_DQ_WARPS = 8;
constexpr int NUM_THREADS = (2 + NUM_DQ_WARPS) * 32;
// one try_wait may suspend for a few microseconds; 2^15 of them bound a wait to ~0.1 s
constexpr uint32_t WAIT_LIMIT = 1u << 15;

// ---- PTX wrappers ----------------------------------------------------------------------

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
// Bounded wait.  Returns false if the phase did not complete within WAIT_LIMIT polls or
// another thread of the CTA already gave up.
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// Plain (untiled) bulk copy global -> shared: 16-byte aligned addresses, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
    return d;
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (SBO); version 1 (sm_100); LBO unused for swizzled
// K-major and set to 1.  Field positions: start[0,14) LBO[16,30) SBO[32,46)
// version[46,48) layout[61,64), all addresses in 16-byte units.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

// Instruction descriptor for kind::f16: D=f32 (bits 4-5 = 1), A/B format at bits 7-9 /
// 10-12 (0 = f16, 1 = bf16), both K-major (bits 15, 16 = 0), N>>3 at bits 17-22,
// M>>4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, int n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

// ---- dequantization of one packed word (8 nibbles) to 8 elements in K order ---------------

// bf16: pair (n_lo, n_hi) of byte i becomes bf16x2 (128 + n_lo, 16 + n_hi): the low nibble
// sits in mantissa bits 0-3 under exponent 2^7, the high nibble (after >>1) in mantissa
// bits 3-6 under exponent 2^4.  bz = (128 + zp, 16 + zp).  Then
//   d = pair - bz (exact), c = d * s_lo (exact: 4 x 3 bits), r = fma(d, s_hi, c) (one rounding)
// which is bf16_rne(f32(q - zp) * f32(scale)).
__device__ __forceinline__ uint4 dequant_word_bf16(uint32_t w, uint32_t bz, uint32_t s_hi2, uint32_t s_lo2) {
    const uint32_t u = w >> 1;
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t p = prmt_b32(w, u, (uint32_t)(i | ((4 + i) << 8)));      // byte0 = w.b[i], byte2 = u.b[i]
        const uint32_t v = lop3_and_or(p, 0x0078000fu, 0x41804300u);
        uint32_t d, c, r;
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(bz));
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(c) : "r"(d), "r"(s_lo2));
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(d), "r"(s_hi2), "r"(c));
        out[i] = r;
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// f16: byte i replicated, low nibble under 0x6400 (1024 + n), high nibble in place under
// 0x5400 (64 + n); hz = (1024 + zp, 64 + zp); one correctly rounded multiply by the scale.
__device__ __forceinline__ uint4 dequant_word_f16(uint32_t w, uint32_t hz, uint32_t s2) {
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t p = prmt_b32(w, w, (uint32_t)(i * 0x1111));
        const uint32_t v = lop3_and_or(p, 0x00f0000fu, 0x54006400u);
        uint32_t d, r;
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(hz));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(d), "r"(s2));
        out[i] = r;
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + __expf(-x)); }

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<true>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<false>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct GemmParams {
    const __half* scales;     // [Nw, G]
    const uint8_t* zeros;     // [Nw, ZS] or null
    void* y;                  // [M, Nout]
    uint32_t* status;         // device-visible status word
    int M, Nout, K, G, ZS;
    int up_row_offset;        // SWIGLU: weight row of `up` = weight row of `gate` + this
    int stages;
    int meta_smem;            // 1: the CTA's scales / zero-points are bulk-copied to shared memory
    int meta_zeros_off;       // offset of the zero-points inside the shared-memory block
};

// Dynamic shared memory, all offsets from a 1024-byte aligned base:
//   [A ring: stages x 16 KB][B ring: stages x NB*128 B][packed ring: stages x NB*32 B]
//   [barriers + tmem slot: 256 B][scales NB x G f16, zero-points NB x ZS bytes (if meta_smem)]
// NB = BN (or 2*BN with SwiGLU: gate rows then up rows).
template <int BN, bool SWIGLU, bool BF16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
lux_qgemm_i4_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const GemmParams p) {
    constexpr int NB = SWIGLU ? 2 * BN : BN;                 // B-tile rows = UMMA N
    constexpr int A_BYTES = BM * 128;
    constexpr int B_BYTES = NB * 128;
    constexpr int Q_BYTES = NB * 32;
    constexpr uint32_t TMEM_COLS = NB <= 32 ? 32 : (NB <= 64 ? 64 : (NB <= 128 ? 128 : 256));
    static_assert(NB % 16 == 0 && NB >= 16 && NB <= 256, "UMMA N for M=128");
    static_assert((NB * 2) % (NUM_DQ_WARPS * 32) == 0 || (NUM_DQ_WARPS * 32) % (NB * 2) == 0, "dequant mapping");

    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by OFFSET from the __shared__ symbol, so that every access below
    // stays a 32-bit shared-memory access (a round trip through an integer would turn them
    // into generic 64-bit ones).
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int S = p.stages;
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + (size_t)S * A_BYTES;
    unsigned char* q_ring = b_ring + (size_t)S * B_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_ring + (size_t)S * Q_BYTES);
    // bars[0..S) full_ld, [S..2S) full_b, [2S..3S) empty, [3S] acc_full, [3S+1] meta_full
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    unsigned char* meta = reinterpret_cast<unsigned char*>(bars) + 512;      // 16-byte aligned

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN;            // first output column (weight row) of this tile
    const int m0 = blockIdx.y * BM;
    const int KB = p.K / BK;

    const uint32_t bar0 = smem_u32(bars);
    auto full_ld = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto full_b = [&](int s) { return bar0 + 8u * (uint32_t)(S + s); };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * S + s); };
    const uint32_t acc_full = bar0 + 8u * (uint32_t)(3 * S);
    const uint32_t meta_full = bar0 + 8u * (uint32_t)(3 * S + 1);

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_ld(s), 1);
            mbar_init(full_b(s), NUM_DQ_WARPS);
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(meta_full, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // =============================== TMA producer ===================================
        if (lane == 0) {
            if (p.meta_smem) {
                // The tile's scales [rows, G] and zero-points [rows, ZS] are contiguous row
                // blocks: fetch them once, before the weight stream starts.
                const uint32_t sb = (uint32_t)(BN * p.G * 2), zb = p.zeros ? (uint32_t)(BN * p.ZS) : 0u;
                mbar_expect_tx(meta_full, (SWIGLU ? 2u : 1u) * (sb + zb));
                bulk_g2s(smem_u32(meta), p.scales + (size_t)n0 * p.G, sb, meta_full);
                if (SWIGLU) bulk_g2s(smem_u32(meta + sb), p.scales + (size_t)(n0 + p.up_row_offset) * p.G, sb, meta_full);
                if (p.zeros) {
                    bulk_g2s(smem_u32(meta + p.meta_zeros_off), p.zeros + (size_t)n0 * p.ZS, zb, meta_full);
                    if (SWIGLU)
                        bulk_g2s(smem_u32(meta + p.meta_zeros_off + zb), p.zeros + (size_t)(n0 + p.up_row_offset) * p.ZS,
                                 zb, meta_full);
                }
            }
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < KB; kb++) {
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) break;
                mbar_expect_tx(full_ld(s), A_BYTES + Q_BYTES);
                tma_load_2d(smem_u32(a_ring + (size_t)s * A_BYTES), &map_x, kb * BK, m0, full_ld(s));
                tma_load_2d(smem_u32(q_ring + (size_t)s * Q_BYTES), &map_w, kb * (BK / 2), n0, full_ld(s));
                if (SWIGLU)
                    tma_load_2d(smem_u32(q_ring + (size_t)s * Q_BYTES + BN * 32), &map_w, kb * (BK / 2),
                                n0 + p.up_row_offset, full_ld(s));
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer =====================================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BF16, NB);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < KB && ok; kb++) {
                ok = mbar_wait(full_ld(s), ph, abort_flag) && mbar_wait(full_b(s), ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(a_ring + (size_t)s * A_BYTES));
                const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(b_ring + (size_t)s * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 16; k++) {
                    // +32 bytes per 16 K inside the swizzle row: +2 in the 16-byte address field
                    umma_f16(tmem_base, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                             (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty(s));        // stage reusable once these MMAs have read it
                if (++s == S) { s = 0; ph ^= 1u; }
            }
            if (ok) umma_commit(acc_full);    // accumulators complete
        }
    } else {
        // =============================== dequantizers ===================================
        const int dq = tid - 64;                              // 0..255
        constexpr int DQ_THREADS = NUM_DQ_WARPS * 32;
        constexpr int UNITS = NB * 2;                         // (row, 32-K half) units per block
        constexpr int UPT = (UNITS + DQ_THREADS - 1) / DQ_THREADS;
        bool ok = true;
        // per-unit constants, refreshed when the group changes (every second block)
        uint32_t zc[UPT], sc_a[UPT], sc_b[UPT];
        int s = 0;
        uint32_t ph = 0;
        if (p.meta_smem) ok = warp_wait(meta_full, 0u, abort_flag, lane);
        const __half* meta_s = reinterpret_cast<const __half*>(meta);
        const unsigned char* meta_z = meta + p.meta_zeros_off;
        for (int kb = 0; kb < KB && ok; kb++) {
            if ((kb & 1) == 0) {
                const int g = kb >> 1;
#pragma unroll
                for (int u = 0; u < UPT; u++) {
                    const int unit = dq + u * DQ_THREADS;
                    const int r = min(unit >> 1, NB - 1);
                    __half sh;
                    uint32_t zp = 8u;
                    if (p.meta_smem) {
                        sh = meta_s[(size_t)r * p.G + g];
                        if (p.zeros) zp = ((uint32_t)meta_z[(size_t)r * p.ZS + (g >> 1)] >> ((g & 1) * 4)) & 0xFu;
                    } else {
                        int wrow = n0 + (SWIGLU && r >= BN ? r - BN + p.up_row_offset : r);
                        const int limit = SWIGLU ? p.Nout + p.up_row_offset : p.Nout;
                        wrow = min(wrow, limit - 1);
                        sh = __ldg(p.scales + (size_t)wrow * p.G + g);
                        if (p.zeros) zp = (__ldg(p.zeros + (size_t)wrow * p.ZS + (g >> 1)) >> ((g & 1) * 4)) & 0xFu;
                    }
                    if (BF16) {
                        const uint32_t sbits = __float_as_uint(__half2float(sh));
                        const uint32_t hi = sbits & 0xFFFF0000u;                    // top 8 significand bits
                        const float lo = __half2float(sh) - __uint_as_float(hi);     // remaining 3 bits, exact
                        const uint32_t lo16 = __float_as_uint(lo) >> 16;            // exact in bf16
                        sc_a[u] = (hi >> 16) * 0x00010001u;
                        sc_b[u] = lo16 * 0x00010001u;
                        zc[u] = (0x4300u | zp) | ((0x4180u | (zp << 3)) << 16);     // (128 + zp, 16 + zp)
                    } else {
                        sc_a[u] = (uint32_t)__half_as_ushort(sh) * 0x00010001u;
                        sc_b[u] = 0u;
                        zc[u] = (0x6400u | zp) | ((0x5400u | (zp << 4)) << 16);     // (1024 + zp, 64 + zp)
                    }
                }
            }
            ok = warp_wait(full_ld(s), ph, abort_flag, lane);   // warp-uniform outcome
            if (!ok) break;
            const unsigned char* qs = q_ring + (size_t)s * Q_BYTES;
            unsigned char* bs = b_ring + (size_t)s * B_BYTES;
#pragma unroll
            for (int u = 0; u < UPT; u++) {
                const int unit = dq + u * DQ_THREADS;
                if (unit < UNITS) {
                    const int r = unit >> 1, h = unit & 1;
                    const uint4 q = *reinterpret_cast<const uint4*>(qs + r * 32 + h * 16);
                    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
                    unsigned char* row = bs + r * 128;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint4 v = BF16 ? dequant_word_bf16(words[j], zc[u], sc_a[u], sc_b[u])
                                             : dequant_word_f16(words[j], zc[u], sc_a[u]);
                        const int chunk = (4 * h + j) ^ (r & 7);                     // 128B swizzle
                        *reinterpret_cast<uint4*>(row + chunk * 16) = v;
                    }
                }
            }
            fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(full_b(s));
            if (++s == S) { s = 0; ph ^= 1u; }
        }

        // =============================== epilogue =======================================
        if (ok) ok = warp_wait(acc_full, 0u, abort_flag, lane);
        if (ok) {
            tc_fence_after();
            const int quad = warp & 3;                          // TMEM lanes this warp may read
            const int half = (warp - 2) >> 2;                   // which half of the columns
            const int row = m0 + quad * 32 + lane;
            constexpr int COLS_PER_WARP = BN / 2;
            constexpr int CHUNK = COLS_PER_WARP < 32 ? COLS_PER_WARP : 32;
            static_assert(CHUNK == 32, "BN >= 64 expected");
#pragma unroll 1
            for (int c0 = half * COLS_PER_WARP; c0 < (half + 1) * COLS_PER_WARP; c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, acc);
                if (SWIGLU) {
                    uint32_t up[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(BN + c0), up);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        acc[i] = __float_as_uint(silu_f32(__uint_as_float(acc[i])) * __uint_as_float(up[i]));
                } else {
                    tmem_ld_wait();
                }
                if (row < p.M) {
                    const size_t esz = 2;
                    unsigned char* dst = reinterpret_cast<unsigned char*>(p.y) + ((size_t)row * p.Nout + n0 + c0) * esz;
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        if (n0 + c0 + v * 8 + 8 <= p.Nout) {
                            uint4 o;
                            o.x = pack2<BF16>(__uint_as_float(acc[v * 8 + 0]), __uint_as_float(acc[v * 8 + 1]));
                            o.y = pack2<BF16>(__uint_as_float(acc[v * 8 + 2]), __uint_as_float(acc[v * 8 + 3]));
                            o.z = pack2<BF16>(__uint_as_float(acc[v * 8 + 4]), __uint_as_float(acc[v * 8 + 5]));
                            o.w = pack2<BF16>(__uint_as_float(acc[v * 8 + 6]), __uint_as_float(acc[v * 8 + 7]));
                            *reinterpret_cast<uint4*>(dst + v * 16) = o;
                        }
                    }
                }
            }
            tc_fence_before();
        }
    }

    __syncthreads();
    if (*abort_flag) {
        // A wait gave up: record it, give copies that are still in flight time to land in
        // this CTA's shared memory (bounded), then fall through to the TMEM release.
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C050001u);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

bool encode_2d(CUtensorMap* map, CUtensorMapDataType dt, size_t esz, const void* base, uint64_t inner, uint64_t outer,
               uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    auto fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * esz};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

// Generic tiled tensor-map encoder shared with the other TMA-fed kernels.  dims/box are
// innermost first; strides_bytes has rank-1 entries (dimension 0 is dense).
bool encode_tensor_map_u8(void* map, int rank, const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                          const uint32_t* box, bool swizzle128) {
    auto fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5];
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; i++) st[i] = strides_bytes[i];
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank,
                    const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

namespace {

template <int BN, bool SW, bool BF16>
cudaError_t launch_inst(const CUtensorMap& mx, const CUtensorMap& mw, GemmParams p, dim3 grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemm_i4_tc<BN, SW, BF16>;
    // Raise the dynamic shared-memory limit once per device (not on every launch, so that
    // launches stay legal inside a stream capture).
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured[dev & 63].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(smem, std::memory_order_relaxed);
    }
    kfn<<<grid, NUM_THREADS, smem, st>>>(mx, mw, p);
    return cudaGetLastError();
}

}  // namespace

LuxBackendError launch_qgemm_i4_tc(Context* ctx, const QArgs& a) {
    const bool bf16 = a.x_dtype == LUX_QDTYPE_BF16;
    const int nout = a.swiglu ? a.N / 2 : a.N;
    if (a.K % 128 || nout % 8) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    int bn = g_tune.gemm_tc_bn > 0 ? g_tune.gemm_tc_bn : 128;
    bn = (bn >= 128 && !a.swiglu) ? 128 : (a.swiglu ? (bn >= 128 ? 128 : 64) : 64);
    const int nb = a.swiglu ? 2 * bn : bn;
    const size_t stage_bytes = (size_t)BM * 128 + (size_t)nb * 128 + (size_t)nb * 32;
    // Scales and zero-points of the CTA's rows go to shared memory when every block is a
    // 16-byte aligned, 16-byte multiple copy and the table leaves room for >= 3 stages.
    const int zs = (a.G + 1) / 2;
    const size_t meta_scale_bytes = (size_t)nb * a.G * 2;
    const size_t meta_bytes = meta_scale_bytes + (a.zeros ? (size_t)nb * zs : 0);
    const size_t budget = 226 * 1024;
    bool meta_smem = nout % bn == 0 && ((size_t)bn * a.G * 2) % 16 == 0 && ((size_t)bn * zs) % 16 == 0 &&
                     (!a.swiglu || (((size_t)nout * a.G * 2) % 16 == 0 && ((size_t)nout * zs) % 16 == 0)) &&
                     1024 + 3 * stage_bytes + 512 + meta_bytes <= budget;
    const size_t tail = 512 + (meta_smem ? meta_bytes : 0);
    int stages = g_tune.gemm_tc_stages > 0 ? g_tune.gemm_tc_stages : 6;
    while (stages > 2 && 1024 + (size_t)stages * stage_bytes + tail > budget) stages--;
    stages = std::min(stages, std::max(2, a.K / BK));
    const size_t smem = 1024 + (size_t)stages * stage_bytes + tail;

    CUtensorMap mx, mw;
    if (!encode_2d(&mx, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x,
                   (uint64_t)a.K, (uint64_t)a.M, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return LUX_BACKEND_ERROR_INTERNAL;
    if (!encode_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)a.K / 2, (uint64_t)a.N, BK / 2, (uint32_t)bn,
                   CU_TENSOR_MAP_SWIZZLE_NONE))
        return LUX_BACKEND_ERROR_INTERNAL;

    GemmParams p{};
    p.scales = (const __half*)a.scales;
    p.zeros = a.zeros;
    p.y = a.y;
    p.status = ctx->d_status;
    p.M = a.M;
    p.Nout = nout;
    p.K = a.K;
    p.G = a.G;
    p.ZS = (a.G + 1) / 2;
    p.up_row_offset = a.swiglu ? nout : 0;
    p.stages = stages;
    p.meta_smem = meta_smem ? 1 : 0;
    p.meta_zeros_off = (int)meta_scale_bytes;

    dim3 grid((nout + bn - 1) / bn, (a.M + BM - 1) / BM);
    cudaError_t e;
    if (a.swiglu) {
        if (bn == 128) e = bf16 ? launch_inst<128, true, true>(mx, mw, p, grid, smem, ctx->stream)
                                : launch_inst<128, true, false>(mx, mw, p, grid, smem, ctx->stream);
        else           e = bf16 ? launch_inst<64, true, true>(mx, mw, p, grid, smem, ctx->stream)
                                : launch_inst<64, true, false>(mx, mw, p, grid, smem, ctx->stream);
    } else {
        if (bn == 128) e = bf16 ? launch_inst<128, false, true>(mx, mw, p, grid, smem, ctx->stream)
                                : launch_inst<128, false, false>(mx, mw, p, grid, smem, ctx->stream);
        else           e = bf16 ? launch_inst<64, false, true>(mx, mw, p, grid, smem, ctx->stream)
                                : launch_inst<64, false, false>(mx, mw, p, grid, smem, ctx->stream);
    }
    count_launch(bf16 ? "lux_qgemm_i4_tc_bf16" : "lux_qgemm_i4_tc_f16");
    return map_cuda(e, "lux_qgemm_i4_tc");
}

const void* kernel_addr_qgemm_i4_tc_bf16() { return (const void*)lux_qgemm_i4_tc<128, false, true>; }
const void* kernel_addr_qgemm_i4_tc_f16() { return (const void*)lux_qgemm_i4_tc<128, false, false>; }

}  // namespace luxcuda
