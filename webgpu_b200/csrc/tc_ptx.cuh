// PTX wrappers and dequantization helpers shared by the tcgen05 GEMM kernels
// (qgemm_tc.cu: converted weights as the shared-memory B operand; qgemm_tc_wa.cu: converted
// weights as the tensor-memory A operand).
#pragma once

#include "common.cuh"

#include <cuda.h>

namespace luxcuda {
namespace tcptx {

constexpr int BM = 128;              // UMMA M: rows of the A operand = TMEM lanes of the accumulator
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
// The same wait for roles that run ahead of the tensor core: a failed poll is followed by a
// short sleep, so that threads waiting for a ring slot do not keep the mbarrier unit busy while
// the MMA-issuing thread needs it (its satisfied polls took 300-400 cycles next to nine
// spinning threads, 20 alone).
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 31u) == 31u && *abort_flag) return false;
        __nanosleep(128);
    }
    *abort_flag = 1u;
    return false;
}
__device__ __forceinline__ bool warp_wait_relaxed(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait_relaxed(bar, parity, abort_flag);
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
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

// ---- A operand in tensor memory, cluster helpers (qgemm_tc_wa.cu) -------------------------

// D[tmem] (+)= A[tmem] . B[smem]^T: A is 128 lanes x (K/2) 32-bit columns, two consecutive K
// elements per column with the lower K in the low half.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
// Each lane writes 32 consecutive 32-bit columns of its own TMEM lane (32 * (warp % 4) + lane).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over all threads of the cluster (not a spin: every thread of every CTA
// reaches it on every path, aborted ones included).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace tcptx
}  // namespace luxcuda
