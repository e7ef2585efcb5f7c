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
#include "tc_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <type_traits>

namespace luxcuda {

namespace {

using namespace tcptx;


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
// MA = batch tiles (128 rows each) per CTA: the converted weight tile of a stage feeds MA
// accumulators, so a weight tile is converted once per MA*128 batch rows.
template <int BN, bool SWIGLU, bool BF16, int MA>
__global__ void __launch_bounds__(NUM_THREADS, 1)
lux_qgemm_i4_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const GemmParams p) {
    constexpr int NB = SWIGLU ? 2 * BN : BN;                 // B-tile rows = UMMA N
    constexpr int A_BYTES = MA * BM * 128;                   // MA tiles of 128 rows x 64 K, one TMA box
    constexpr int B_BYTES = NB * 128;
    constexpr int Q_BYTES = NB * 32;
    constexpr int ACC_COLS = MA * NB;                        // accumulator a at columns [a*NB, +NB)
    constexpr uint32_t TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));
    static_assert(ACC_COLS <= 512, "TMEM holds 512 columns");
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
    // bars[0..S) full_ld (per stage), [S..S+S/2) full_b and [2S..2S+S/2) empty (per PAIR of
    // stages = 128 K), [3S] acc_full, [3S+1] meta_full.  S is even.
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    unsigned char* meta = reinterpret_cast<unsigned char*>(bars) + 512;      // 16-byte aligned

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN;            // first output column (weight row) of this tile
    const int m0 = blockIdx.y * (MA * BM);
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
            if ((s & 1) == 0) {
                mbar_init(full_b(s >> 1), 2 * NUM_DQ_WARPS);   // every converting warp, once per stage of the pair
                mbar_init(empty(s >> 1), 1);
            }
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
                if ((s & 1) == 0 && !mbar_wait_relaxed(empty(s >> 1), ph ^ 1u, abort_flag)) break;
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
            // One wait and one commit per PAIR of stages (128 K): a satisfied mbarrier wait costs
            // this thread 200-250 cycles and a commit ~100, which per 64-K stage (with a second
            // wait for the loads) added up to more than the stage's MMAs.  The converters wait
            // for a stage's loads (x tile included) before they arrive, so their barrier alone
            // tells that the x tile has landed too.
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < KB && ok; kb += 2) {
                ok = mbar_wait(full_b(s >> 1), ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(a_ring + (size_t)(s + b) * A_BYTES));
                    const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(b_ring + (size_t)(s + b) * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        // +32 bytes per 16 K inside the swizzle row: +2 in the 16-byte address field;
                        // batch tile a is 16 KB (1024 in the address field) further on
#pragma unroll
                        for (int a = 0; a < MA; a++)
                            umma_f16(tmem_base + (uint32_t)(a * NB), a_desc + (uint64_t)(a * 1024 + 2 * k),
                                     b_desc + (uint64_t)(2 * k), idesc, (kb | b | k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(empty(s >> 1));   // both stages reusable once these MMAs have read them
                s += 2;
                if (s == S) { s = 0; ph ^= 1u; }
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
            if (lane == 0) mbar_arrive(full_b(s >> 1));
            if (++s == S) { s = 0; ph ^= 1u; }
        }

        // =============================== epilogue =======================================
        if (ok) ok = warp_wait(acc_full, 0u, abort_flag, lane);
        if (ok) {
            tc_fence_after();
            const int quad = warp & 3;                          // TMEM lanes this warp may read
            const int half = (warp - 2) >> 2;                   // which half of the columns
#pragma unroll 1
            for (int at = 0; at < MA; at++) {
            const int row = m0 + at * BM + quad * 32 + lane;
            const uint32_t tacc = tmem_base + (uint32_t)(at * NB);
            constexpr int COLS_PER_WARP = BN / 2;
            constexpr int CHUNK = COLS_PER_WARP < 32 ? COLS_PER_WARP : 32;
            static_assert(CHUNK == 32, "BN >= 64 expected");
#pragma unroll 1
            for (int c0 = half * COLS_PER_WARP; c0 < (half + 1) * COLS_PER_WARP; c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(tacc + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, acc);
                if (SWIGLU) {
                    uint32_t up[32];
                    tmem_ld32(tacc + ((uint32_t)(quad * 32) << 16) + (uint32_t)(BN + c0), up);
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
            }   // batch tiles
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
    if (!fn || rank < 1 || rank > 5) return false;
    // A decode loop encodes the same few maps over and over (one per layer and operand): the encoded
    // 128 bytes depend on nothing but these arguments, so the last 64 are kept.
    struct Key { const void* base; uint64_t d[5], st[4]; uint32_t b[5]; int rank; bool sw; };
    struct Slot { Key key; alignas(64) CUtensorMap map; bool used; };
    static Slot cache[64];
    static unsigned next_slot = 0;
    static std::mutex mu;
    Key k;
    std::memset(&k, 0, sizeof k);                      // padding too: the keys are compared bytewise
    k.base = base; k.rank = rank; k.sw = swizzle128;
    for (int i = 0; i < rank; i++) { k.d[i] = dims[i]; k.b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) k.st[i] = strides_bytes[i];
    std::lock_guard<std::mutex> lock(mu);
    for (const Slot& sl : cache)
        if (sl.used && std::memcmp(&sl.key, &k, sizeof k) == 0) {
            std::memcpy(map, &sl.map, sizeof(CUtensorMap));
            return true;
        }
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5];
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; i++) st[i] = strides_bytes[i];
    Slot& sl = cache[next_slot++ % 64];
    CUresult r = fn(&sl.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank,
                    const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    sl.used = r == CUDA_SUCCESS;
    if (!sl.used) return false;
    std::memcpy(&sl.key, &k, sizeof k);
    std::memcpy(map, &sl.map, sizeof(CUtensorMap));
    return true;
}

namespace {

template <int BN, bool SW, bool BF16, int MA>
cudaError_t launch_inst(const CUtensorMap& mx, const CUtensorMap& mw, GemmParams p, dim3 grid, size_t smem, cudaStream_t st) {
    auto kfn = lux_qgemm_i4_tc<BN, SW, BF16, MA>;
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

    // Tile choice (measured on B200; the conversion of the weight tile is what bounds this kernel).
    // SwiGLU above 128 batch rows: 64 outputs (128 weight rows) per CTA and two batch tiles, so a
    // converted tile serves 256 rows (Llama-70B gate_up quarter at M = 256: 74 us against 107 us
    // with 128 outputs and one batch tile).  Otherwise 128 weight rows and one batch tile: two
    // batch tiles leave a 128-wide tile only two pairs of stages (config 3: 56 us against 40 us).
    const bool wide_batch = a.swiglu && a.M > BM;
    int bn = g_tune.gemm_tc_bn > 0 ? g_tune.gemm_tc_bn : (wide_batch ? 64 : 128);
    bn = (bn >= 128 && !a.swiglu) ? 128 : (a.swiglu ? (bn >= 128 ? 128 : 64) : 64);
    const int nb = a.swiglu ? 2 * bn : bn;
    // Two batch tiles per CTA need two accumulators in TMEM (2 * nb <= 512 columns) and, because
    // the ring is handed over in pairs of stages, room for four stages.
    int ma = wide_batch ? 2 : 1;
    if (g_tune.gemm_tc_ma == 1 || g_tune.gemm_tc_ma == 2) ma = g_tune.gemm_tc_ma;
    if (ma == 2 && (2 * nb > 512 ||
                    1024 + 4 * ((size_t)2 * BM * 128 + (size_t)nb * 128 + (size_t)nb * 32) + 512 > (size_t)226 * 1024))
        ma = 1;
    const size_t stage_bytes = (size_t)ma * BM * 128 + (size_t)nb * 128 + (size_t)nb * 32;
    // Scales and zero-points of the CTA's rows go to shared memory when every block is a
    // 16-byte aligned, 16-byte multiple copy and the table leaves room for >= 4 stages.
    const int zs = (a.G + 1) / 2;
    const size_t meta_scale_bytes = (size_t)nb * a.G * 2;
    const size_t meta_bytes = meta_scale_bytes + (a.zeros ? (size_t)nb * zs : 0);
    const size_t budget = 226 * 1024;
    bool meta_smem = nout % bn == 0 && ((size_t)bn * a.G * 2) % 16 == 0 && ((size_t)bn * zs) % 16 == 0 &&
                     (!a.swiglu || (((size_t)nout * a.G * 2) % 16 == 0 && ((size_t)nout * zs) % 16 == 0)) &&
                     1024 + 4 * stage_bytes + 512 + meta_bytes <= budget;
    const size_t tail = 512 + (meta_smem ? meta_bytes : 0);
    int stages = g_tune.gemm_tc_stages > 0 ? g_tune.gemm_tc_stages : 6;
    while (stages > 2 && 1024 + (size_t)stages * stage_bytes + tail > budget) stages--;
    stages = std::min(stages, std::max(2, a.K / BK));
    stages &= ~1;                                     // the ring is handed over in pairs of stages (128 K)
    const size_t smem = 1024 + (size_t)stages * stage_bytes + tail;

    CUtensorMap mx, mw;
    if (!encode_2d(&mx, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x,
                   (uint64_t)a.K, (uint64_t)a.M, BK, (uint32_t)(ma * BM), CU_TENSOR_MAP_SWIZZLE_128B))
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

    dim3 grid((nout + bn - 1) / bn, (a.M + ma * BM - 1) / (ma * BM));
    cudaError_t e;
    auto go = [&](auto bn_tag, auto sw_tag, auto ma_tag) {
        constexpr int BN_ = decltype(bn_tag)::value;
        constexpr bool SW_ = decltype(sw_tag)::value;
        constexpr int MA_ = decltype(ma_tag)::value;
        if constexpr (MA_ * (SW_ ? 2 * BN_ : BN_) <= 512)
            return bf16 ? launch_inst<BN_, SW_, true, MA_>(mx, mw, p, grid, smem, ctx->stream)
                        : launch_inst<BN_, SW_, false, MA_>(mx, mw, p, grid, smem, ctx->stream);
        else
            return cudaErrorInvalidValue;
    };
    using I64 = std::integral_constant<int, 64>;
    using I128 = std::integral_constant<int, 128>;
    using I1 = std::integral_constant<int, 1>;
    using I2 = std::integral_constant<int, 2>;
    if (a.swiglu) {
        if (bn == 128) e = ma == 2 ? go(I128{}, std::true_type{}, I2{}) : go(I128{}, std::true_type{}, I1{});
        else           e = ma == 2 ? go(I64{}, std::true_type{}, I2{}) : go(I64{}, std::true_type{}, I1{});
    } else {
        if (bn == 128) e = ma == 2 ? go(I128{}, std::false_type{}, I2{}) : go(I128{}, std::false_type{}, I1{});
        else           e = ma == 2 ? go(I64{}, std::false_type{}, I2{}) : go(I64{}, std::false_type{}, I1{});
    }
    count_launch(bf16 ? "lux_qgemm_i4_tc_bf16" : "lux_qgemm_i4_tc_f16");
    return map_cuda(e, "lux_qgemm_i4_tc");
}

const void* kernel_addr_qgemm_i4_tc_bf16() { return (const void*)lux_qgemm_i4_tc<128, false, true, 1>; }
const void* kernel_addr_qgemm_i4_tc_f16() { return (const void*)lux_qgemm_i4_tc<128, false, false, 1>; }

}  // namespace luxcuda
