// qint_gemm_tc.cu -- int8 x int8 -> int32 matmul on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), behind lux_cuda_matmul_int8 and
// lux_cuda_matmul_int4_int8 for shapes large enough to fill tiles.
//
// The shader (luxcpp/webgpu kernels/wgsl/gpu/quantized.wgsl:497-555) walks 16 x 16 tiles with one
// scalar multiply-add per thread and k; the mma.sync kernel in qint_matmul.cu reaches 220 TOP/s on
// this GPU, a twentieth of what its tensor cores do through tcgen05.  Integer arithmetic is exact
// (int32 accumulation, wrapping like the shader's i32), so the result is bit-identical either way.
//
// C[M, N] = A[M, K] . B[K, N]:
//   * A is row-major with K contiguous: a K-major operand.  B is row-major [K, N] with N contiguous:
//     an MN-major operand, which kind::i8 accepts (bit 16 of the instruction descriptor), so B is read
//     as it lies -- two TMA boxes of 128 columns x 128 rows of k per stage, each box one column of
//     128-byte swizzle atoms.  When N is not a multiple of 16 bytes a row of B cannot be a tensor
//     map's row, and a first kernel writes B^T [N, K] into the context's scratch (64 x 64 byte tiles
//     through shared memory), which is then read K-major (measured, 4096^3: 83.5 us through B^T,
//     73.0 us without; 256 x 28672 x 4096: 103.8 -> 48.5 us).  For int4 x int8 another kernel
//     sign-extends A's two's complement nibbles (quantized.wgsl:150-158) to bytes;
//   * a CTA owns a 256 x 256 tile of C (128 x 256 when M <= 128): two int32 accumulators of 256
//     columns each in tensor memory, fed by the same B tile;
//   * warp 0 (one thread): TMA producer, one 256 x 128-byte box of A and 32 KB of B per stage
//     (128 k; 128-byte swizzle), three stages (four with one accumulator);
//   * warp 1 (one thread): per stage one wait, four tcgen05.mma.kind::i8 (128 x 256 x 32) per
//     accumulator and one tcgen05.commit that frees the stage;
//   * warps 2-5: epilogue, tcgen05.ld 32 columns at a time, 128-byte stores per thread.
// K tails and ragged M / N are covered by the TMA's zero fill and by masked stores.  Every mbarrier
// wait is bounded (the abort flag, status 0x7C05000B).  No cluster, no multicast.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace luxcuda {

bool encode_tensor_map_u8(void* map, int rank, const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                          const uint32_t* box, bool swizzle128);

namespace {

using namespace tcptx;

constexpr int I8_BM = 128, I8_BN = 256, I8_KB = 128;       // tile of C; k (= bytes) per stage
constexpr int I8_A_BYTES = I8_BM * I8_KB, I8_B_BYTES = I8_BN * I8_KB;
constexpr int I8_THREADS = 6 * 32;
// MA = row tiles of 128 per CTA (1 or 2): two accumulators share every B tile, which cuts the bytes a CTA
// pulls from L2 per multiply-add by a third (the one-tile form asks for 92 bytes per clock and SM at the
// tensor pipe's rate and ran at half of it)
__host__ __device__ constexpr int i8_stages(int ma) { return ma == 2 ? 3 : 4; }
__host__ __device__ constexpr size_t i8_smem(int ma) { return 1024 + (size_t)i8_stages(ma) * (ma * I8_A_BYTES + I8_B_BYTES) + 256; }

// Instruction descriptor for kind::i8: D = s32 (bits 4-5 = 2), A and B signed 8-bit (bits 7-9 and
// 10-12 = 1), both K-major, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t i8_idesc() {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(I8_BN >> 3) << 17) | ((uint32_t)(I8_BM >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}

struct I8Params {
    int* c;
    uint32_t* status;
    int M, N, K;
    int b_mn;      // B is read as it lies, [K, N] with N contiguous (an MN-major operand); 0: map_b describes B^T
};

// Shared-memory descriptor of the B stage as an MN-major operand under the 128-byte swizzle.  In
// 16-byte units the canonical layout is ((8, n), (8, k)) : ((1, LBO), (8, SBO)): 128 contiguous
// bytes of N, eight rows of K 128 bytes apart (one swizzle atom, which is what a TMA box of
// 128 bytes x rows writes), the next eight rows of K SBO = 1024 bytes on, the next 128 columns of N
// LBO = one box (128 rows x 128 bytes) on.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | ((uint32_t)((I8_KB * 128) >> 4) << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

template <int MA>
__global__ void __launch_bounds__(I8_THREADS, 1)
lux_matmul_int8_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const I8Params p) {
    constexpr int I8_STAGES = i8_stages(MA);
    constexpr int A_STAGE = MA * I8_A_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + (size_t)I8_STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + (size_t)I8_STAGES * I8_B_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * I8_STAGES + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * I8_BN, m0 = blockIdx.y * (MA * I8_BM);
    const int KB = (p.K + I8_KB - 1) / I8_KB;
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(I8_STAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (uint32_t)(2 * I8_STAGES);

    if (tid == 0) {
        for (int s = 0; s < I8_STAGES; s++) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), MA * 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < KB; kb++) {
                const int s = kb % I8_STAGES;
                if (kb >= I8_STAGES && !mbar_wait_relaxed(empty(s), (uint32_t)((kb / I8_STAGES) - 1) & 1u, abort_flag)) break;
                mbar_expect_tx(full(s), (uint32_t)(A_STAGE + I8_B_BYTES));        // boxes past an edge are zero-filled and still counted
                tma_load_2d(smem_u32(a_ring + (size_t)s * A_STAGE), &map_a, kb * I8_KB, m0, full(s));
                if (p.b_mn) {
                    // two boxes of 128 columns of N x 128 rows of K, as they lie in B
                    tma_load_2d(smem_u32(b_ring + (size_t)s * I8_B_BYTES), &map_b, n0, kb * I8_KB, full(s));
                    tma_load_2d(smem_u32(b_ring + (size_t)s * I8_B_BYTES + I8_B_BYTES / 2), &map_b, n0 + 128, kb * I8_KB, full(s));
                } else {
                    tma_load_2d(smem_u32(b_ring + (size_t)s * I8_B_BYTES), &map_b, kb * I8_KB, n0, full(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = i8_idesc() | (p.b_mn ? (1u << 16) : 0u);       // bit 16: B is MN-major
            const uint64_t b_step = p.b_mn ? (uint64_t)((32 * 128) >> 4) : 2u;     // 32 k: 32 rows of the box, or 32 bytes of the swizzle row
            bool ok = true;
            for (int kb = 0; kb < KB; kb++) {
                const int s = kb % I8_STAGES;
                ok = mbar_wait(full(s), (uint32_t)(kb / I8_STAGES) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t b_addr = smem_u32(b_ring + (size_t)s * I8_B_BYTES);
                const uint64_t b_desc = p.b_mn ? make_mnmajor_sw128_desc(b_addr) : make_kmajor_sw128_desc(b_addr);
#pragma unroll
                for (int a = 0; a < MA; a++) {
                    // accumulator a: rows a * 128 .. of the A box, TMEM columns a * 256 ..
                    const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(a_ring + (size_t)s * A_STAGE + (size_t)a * I8_A_BYTES));
#pragma unroll
                    for (int k = 0; k < I8_KB / 32; k++)  // 32 k = 32 bytes inside the 128-byte swizzle row: +2 in the address field
                        umma_i8(tmem_base + (uint32_t)(a * 256), a_desc + (uint64_t)(2 * k), b_desc + b_step * (uint64_t)k, idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty(s));
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        // epilogue warps: TMEM lane quarter = warp % 4 (a warp reaches only its own quarter)
        const int quad = warp & 3;
        // (sleeping between polls: these four warps wait for the whole main loop, and tight polls next to
        // the MMA-issuing thread make its own satisfied waits several times dearer)
        bool ok = warp_wait_relaxed(acc_full, 0u, abort_flag, lane);
        if (ok) {
            tc_fence_after();
            const bool vec = (p.N & 3) == 0;
            uint32_t* patch = reinterpret_cast<uint32_t*>(a_ring) + (warp - 2) * (32 * 33);   // the loads are over: the ring is free
#pragma unroll 1
            for (int cc = 0; cc < MA * I8_BN; cc += 32) {
                const int a = cc / I8_BN, c0 = cc - a * I8_BN;
                const int row = m0 + a * I8_BM + quad * 32 + lane;
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * 256);
                if (n0 + c0 >= p.N || m0 + a * I8_BM >= p.M) continue;   // warp-uniform
                uint32_t v[32];
                tmem_ld32(lane_addr + (uint32_t)c0, v);
                tmem_ld_wait();
                if (vec && n0 + c0 + 32 <= p.N) {
                    // through this warp's 32 x 33-word patch of the (idle) ring, so that a store instruction
                    // writes four whole 128-byte pieces of four rows instead of 16 bytes of 32 rows
#pragma unroll
                    for (int j = 0; j < 32; j++) patch[lane * 33 + j] = v[j];
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; it++) {
                        const int r = it * 4 + (lane >> 3), q = lane & 7;
                        const int grow = m0 + a * I8_BM + quad * 32 + r;
                        const uint32_t* src = patch + r * 33 + q * 4;
                        if (grow < p.M)
                            *reinterpret_cast<int4*>(p.c + (size_t)grow * p.N + n0 + c0 + q * 4) = make_int4((int)src[0], (int)src[1], (int)src[2], (int)src[3]);
                    }
                    __syncwarp();
                } else if (row < p.M) {
                    int* dst = p.c + (size_t)row * p.N + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (n0 + c0 + j < p.N) dst[j] = (int)v[j];
                }
            }
            tc_fence_before();
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && p.status) atomicOr(p.status, 0x7C05000Bu);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, MA * 256);
    }
}

// B [K, N] (N contiguous) -> B^T [N, K] (K contiguous), bytes; 64 x 64 tiles.  A full tile goes
// through 4 x 4 byte blocks transposed in registers (prmt) and 16-byte stores; edge tiles byte by byte.
__device__ __forceinline__ uint32_t prmt_i8(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__global__ void __launch_bounds__(256) lux_transpose_i8(const uint8_t* __restrict__ b, uint8_t* __restrict__ bt, int K, int N) {
    __shared__ uint32_t st[64][17];                        // [n][k / 4], one word of padding per row
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64, t = threadIdx.x;
    if (k0 + 64 <= K && n0 + 64 <= N && (N & 3) == 0) {
        const int kr = t >> 4, nc = t & 15;                // rows k0 + 4 kr .. + 3, columns n0 + 4 nc .. + 3
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) w[i] = *reinterpret_cast<const uint32_t*>(b + (size_t)(k0 + 4 * kr + i) * N + n0 + 4 * nc);
        const uint32_t t0 = prmt_i8(w[0], w[1], 0x5140), t1 = prmt_i8(w[2], w[3], 0x5140);
        const uint32_t t2 = prmt_i8(w[0], w[1], 0x7362), t3 = prmt_i8(w[2], w[3], 0x7362);
        st[4 * nc + 0][kr] = prmt_i8(t0, t1, 0x5410);
        st[4 * nc + 1][kr] = prmt_i8(t0, t1, 0x7632);
        st[4 * nc + 2][kr] = prmt_i8(t2, t3, 0x5410);
        st[4 * nc + 3][kr] = prmt_i8(t2, t3, 0x7632);
        __syncthreads();
        const int n = t >> 2, q = t & 3;                   // output row n0 + n, bytes k0 + 16 q .. + 15
        const uint4 v = make_uint4(st[n][4 * q], st[n][4 * q + 1], st[n][4 * q + 2], st[n][4 * q + 3]);
        *reinterpret_cast<uint4*>(bt + (size_t)(n0 + n) * K + k0 + 16 * q) = v;       // K % 16 == 0 and a 256-byte aligned base
        return;
    }
    uint8_t (*tile)[68] = reinterpret_cast<uint8_t (*)[68]>(st);
    for (int i = t; i < 64 * 64; i += 256) {
        const int r = i >> 6, c = i & 63;
        tile[r][c] = (k0 + r < K && n0 + c < N) ? b[(size_t)(k0 + r) * N + n0 + c] : (uint8_t)0;
    }
    __syncthreads();
    for (int i = t; i < 64 * 64; i += 256) {
        const int n = i >> 6, k = i & 63;
        if (n0 + n < N && k0 + k < K) bt[(size_t)(n0 + n) * K + k0 + k] = tile[k][n];
    }
}

// int4 [M, K/2] (two's complement nibbles, element 2j in the low nibble of byte j) -> int8 [M, K]
__global__ void __launch_bounds__(256) lux_unpack_s4_s8(const uint8_t* __restrict__ a4, uint8_t* __restrict__ a8, size_t bytes) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < bytes; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t v = a4[i];
        const uint32_t lo = v & 0xFu, hi = v >> 4;
        const uint32_t slo = lo | ((lo & 8u) ? 0xF0u : 0u), shi = hi | ((hi & 8u) ? 0xF0u : 0u);
        *reinterpret_cast<uint16_t*>(a8 + 2 * i) = (uint16_t)(slo | (shi << 8));
    }
}

}  // namespace

// Returns NOT_SUPPORTED for shapes this kernel does not take (the caller falls back to the
// mma.sync kernels): fewer than a tile's worth of work, K not a multiple of 16, unaligned views.
LuxBackendError launch_matmul_int8_tcgen05(Context* ctx, const void* a, const void* b, int* c, int M, int N, int K, bool a_int4) {
    if (K % 16 || (size_t)M * N < (size_t)I8_BM * I8_BN || K < 256) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    // B as it lies when its rows can be a tensor map's (N a multiple of 16 bytes); else through B^T
    const bool b_mn = N % 16 == 0 && g_tune.int_matmul_kernel != 2;
    const size_t bt_bytes = b_mn ? 0 : (((size_t)N * K + 255) & ~(size_t)255), a8_bytes = a_int4 ? (((size_t)M * K + 255) & ~(size_t)255) : 0;
    if (bt_bytes + a8_bytes) {
        // scratch for B^T (and the unpacked A): grown on demand, kept with the context
        std::lock_guard<std::mutex> lock(ctx->mu);
        if (ctx->d_int_bytes < bt_bytes + a8_bytes) {
            cudaStreamSynchronize(ctx->stream);
            if (ctx->d_int) cudaFree(ctx->d_int);
            ctx->d_int = nullptr;
            ctx->d_int_bytes = 0;
            if (cudaMalloc(&ctx->d_int, bt_bytes + a8_bytes) != cudaSuccess) {
                (void)cudaGetLastError();
                return LUX_BACKEND_ERROR_NOT_SUPPORTED;          // the mma.sync kernel needs no scratch
            }
            ctx->d_int_bytes = bt_bytes + a8_bytes;
        }
    }
    uint8_t* bt = (uint8_t*)ctx->d_int;
    uint8_t* a8 = bt + bt_bytes;
    if (!b_mn) {
        lux_transpose_i8<<<dim3((N + 63) / 64, (K + 63) / 64), 256, 0, ctx->stream>>>((const uint8_t*)b, bt, K, N);
        count_launch();
    }
    if (a_int4) {
        const size_t bytes = (size_t)M * K / 2;
        lux_unpack_s4_s8<<<(unsigned)std::min<size_t>((bytes + 255) / 256, (size_t)ctx->sm_count * 16), 256, 0, ctx->stream>>>((const uint8_t*)a, a8, bytes);
        count_launch();
    }
    CUtensorMap ma_map, mb;
    const uint64_t adims[2] = {(uint64_t)K, (uint64_t)M}, bdims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)K};
    const int ma = M > I8_BM ? 2 : 1;
    const uint32_t abox[2] = {(uint32_t)I8_KB, (uint32_t)(ma * I8_BM)}, bbox[2] = {(uint32_t)I8_KB, (uint32_t)I8_BN};
    if (!encode_tensor_map_u8(&ma_map, 2, a_int4 ? (const void*)a8 : a, adims, strides, abox, true)) return LUX_BACKEND_ERROR_INTERNAL;
    if (b_mn) {
        const uint64_t dims_mn[2] = {(uint64_t)N, (uint64_t)K}, strides_mn[1] = {(uint64_t)N};
        const uint32_t box_mn[2] = {128u, (uint32_t)I8_KB};
        if (!encode_tensor_map_u8(&mb, 2, b, dims_mn, strides_mn, box_mn, true)) return LUX_BACKEND_ERROR_INTERNAL;
    } else if (!encode_tensor_map_u8(&mb, 2, bt, bdims, strides, bbox, true)) {
        return LUX_BACKEND_ERROR_INTERNAL;
    }
    static std::atomic<bool> configured[64];
    int dev = ctx->device & 63;
    if (!configured[dev].load(std::memory_order_relaxed)) {
        if (cudaFuncSetAttribute(lux_matmul_int8_tcgen05<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)i8_smem(1)) != cudaSuccess ||
            cudaFuncSetAttribute(lux_matmul_int8_tcgen05<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)i8_smem(2)) != cudaSuccess)
            return map_cuda(cudaGetLastError(), "lux_matmul_int8_tcgen05");
        configured[dev].store(true, std::memory_order_relaxed);
    }
    I8Params p{c, ctx->d_status, M, N, K, b_mn ? 1 : 0};
    const dim3 grid((N + I8_BN - 1) / I8_BN, (M + ma * I8_BM - 1) / (ma * I8_BM));
    if (ma == 2) lux_matmul_int8_tcgen05<2><<<grid, I8_THREADS, i8_smem(2), ctx->stream>>>(ma_map, mb, p);
    else lux_matmul_int8_tcgen05<1><<<grid, I8_THREADS, i8_smem(1), ctx->stream>>>(ma_map, mb, p);
    count_launch(a_int4 ? "lux_matmul_int4_int8_tcgen05" : "lux_matmul_int8_tcgen05");
    return LUX_BACKEND_OK;
}

const void* kernel_addr_matmul_int8_tcgen05() { return (const void*)lux_matmul_int8_tcgen05<2>; }

}  // namespace luxcuda
