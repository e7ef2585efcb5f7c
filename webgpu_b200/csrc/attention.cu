// attention.cu -- rotary embedding, scaled-dot-product attention, KV-cache append and attention over
// a contiguous or a paged KV cache, all f32 (lux/gpu/attention_ext.h).
//
// What the WGSL does (luxcpp/webgpu kernels/wgsl/gpu/scaled_dot_product_attention.wgsl:81-199, 386-489;
// steel/attention/paged.wgsl:55-405): one 256-thread workgroup per (batch, head, query) walks the
// keys three times, the third time recomputing every score once per output dimension.  Here one
// pass does it, and the pass is shaped by what bounds a decode step on this GPU, the read of the
// KV cache from HBM:
//   * a CTA owns one (sequence, KV head, block of query rows, slice of the keys).  All query heads
//     that share the KV head (and all appended tokens) are rows of the same CTA, so the cache is
//     read from HBM once per KV head, not once per query head;
//   * a producer warp streams 32-key chunks of K and V into a ring in shared memory with bulk
//     copies (cp.async.bulk, one per contiguous run: a whole chunk for a contiguous cache, one per
//     page for a paged one, the page numbers taken from a copy of the block table in shared
//     memory), each chunk signalled through an mbarrier; two CTAs of nine warps share an SM, each
//     with a ring of three chunks (D = 128);
//   * eight consumer warps share a chunk: a key is handled by 8 lanes, each holding 16-byte columns
//     of the row, so a warp takes 4 keys per step; every lane keeps two query rows in registers
//     and runs the running-maximum softmax (the rule of sdpa_flash, :217-362) on its own keys; lanes,
//     warps and, for long contexts, CTAs are merged at the end by the same rule (the partition
//     statistics of paged_attention_v2, paged.wgsl:351-405, are this merge);
//   * only ONE thread per CTA polls an mbarrier (warp 0, for the chunk to land).  Everything else
//     waits on named barriers (bar.sync / bar.arrive), where the hardware parks a warp until the
//     count is reached: the other consumer warps for "chunk ready", the producer for "stage free".
//     With every warp polling its mbarrier the kernel ran at 2.2-5.1 TB/s depending on how many
//     warps happened to be waiting; parked, at 5.0-6.5 TB/s on the same shapes (polls travel the same
//     queue as shared-memory loads and shuffles, and starved the warps that had work);
//   * keys are split over CTAs when there are fewer (sequence, KV head) pairs than SM slots, and
//     each CTA walks its chunks from a different starting point; a small second kernel, resident
//     early through programmatic dependent launch, merges the slices.
// The one polling wait is bounded: if it gives up it sets the CTA's abort flag, every warp leaves
// its loop (the consumers first release the stages the producer may be parked on), the device
// status word reports 0x7C050008 and the output of that CTA is not written.
#include <algorithm>
#include <cmath>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "tc_ptx.cuh"
#include "lux/gpu/attention_ext.h"

namespace luxcuda {

namespace {

using namespace tcptx;

constexpr int ATT_CW = 8;                       // consumer warps
constexpr int ATT_THREADS = (ATT_CW + 1) * 32;  // + the producer warp
constexpr int ATT_CK = 32;                      // keys per staged chunk
constexpr int ATT_MAX_STAGES = 6;
constexpr int ATT_CTAS_PER_SM = 2;
constexpr int ATT_TABLE = 2048;                 // block-table entries a CTA keeps in shared memory
constexpr int ATT_HEADER = 128;                 // barriers + abort flag
constexpr size_t ATT_SMEM_BUDGET = 110u << 10;        // per CTA: two CTAs share an SM
constexpr float ATT_NEG = -3.0e38f;             // "no key seen yet" in the base-2 score domain
constexpr float ATT_LOG2E = 1.4426950408889634f;
constexpr float ATT_LN2 = 0.6931471805599453f;
constexpr uint32_t ATT_STATUS_WAIT = 0x7C050008u;     // a bounded wait of the attention kernel gave up
constexpr uint32_t ATT_STATUS_BLOCK = 0x7C050009u;    // a block-table entry outside the cache (read as block 0)
constexpr uint32_t ATT_STATUS_POSITION = 0x7C05000Au; // a rope position outside the cos/sin cache (pair not written)

struct AttnParams {
    const float* q;
    const float* k;
    const float* v;
    float* out;
    float* lse;                  // may be null
    const int32_t* block_tables; // paged only
    const int32_t* context_lens; // paged only
    float* part;                 // [out row][nsplit][head_dim + 2] when nsplit > 1
    uint32_t* status;
    uint32_t batch, heads, kv_heads, group, seq_q, head_dim;
    uint32_t kv_len;             // keys a row may see (contiguous caches); paged: context_lens decides
    uint32_t kv_stride;          // rows between the bases of two KV heads of a contiguous cache
    uint32_t causal, causal_base;// causal: query i sees min(causal_base + i + 1, kv_len) keys
    uint32_t block_size, max_blocks_per_seq, num_blocks;   // paged (block_size 0: contiguous)
    uint32_t rgp;                // row groups per CTA (1, 2, 4 or 8): rows per CTA = RT * rgp
    uint32_t row_blocks, nsplit, split_keys, stages;
    float qscale;                // scale * log2(e)
};

// 2^x for x <= 0 (results below the normal range flush to 0), one MUFU operation
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Named barriers: a warp that waits on one is parked by the hardware and issues nothing, unlike a
// warp polling an mbarrier, whose polls share the queue that shared-memory loads and shuffles go
// through.  With eight warps polling for every chunk the warps that had work ran 2-3 times slower.
constexpr int ATT_BAR_READY = 1;           // consumer warps: the chunk has landed (warp 0 polled for it)
constexpr int ATT_BAR_FREE0 = 2;           // + stage: every consumer warp is done with the stage (producer waits)

__device__ __forceinline__ uint32_t row_len(const AttnParams& p, uint32_t qi, uint32_t kv_len) {
    return p.causal ? min(p.causal_base + qi + 1u, kv_len) : kv_len;
}

template <int VPL, int RT, bool FULL>
__global__ void __launch_bounds__(ATT_THREADS, ATT_CTAS_PER_SM) lux_attn_stream_f32(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t bar_full = smem_u32(smem);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + 16 * ATT_MAX_STAGES);
    int32_t* table = reinterpret_cast<int32_t*>(smem + ATT_HEADER);
    float* stages = reinterpret_cast<float*>(smem + ATT_HEADER + (p.block_size ? ATT_TABLE * 4 : 0));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t D = p.head_dim, NS = p.stages;
    const size_t stage_floats = (size_t)2 * ATT_CK * D;

    pdl_launch_dependents();                   // the merge kernel may take its place; it waits for this grid

    uint32_t idx = blockIdx.x;
    const uint32_t split = idx % p.nsplit; idx /= p.nsplit;
    const uint32_t rb = idx % p.row_blocks; idx /= p.row_blocks;
    const uint32_t g = idx % p.kv_heads, b = idx / p.kv_heads;

    uint32_t kv_len = p.kv_len;
    if (p.block_size) {
        const int32_t cl = p.context_lens[b];
        if (cl <= 0) return;                   // paged.wgsl:66-67: the rows stay as they are
        kv_len = min((uint32_t)cl, p.max_blocks_per_seq * p.block_size);
    }
    // rows of this CTA: row r of the KV head is (query qi = r / group, head g * group + r % group),
    // so a block of rows holds neighbouring queries and a causal block stops at its last row's keys
    const uint32_t R = p.group * p.seq_q, rpb = RT * p.rgp, row0 = rb * rpb;
    const uint32_t last_row = min(R, row0 + rpb) - 1u;
    const uint32_t lmax = row_len(p, last_row / p.group, kv_len);
    const uint32_t k_begin = split * p.split_keys;
    const uint32_t k_end = min(lmax, k_begin + p.split_keys);
    const uint32_t nchunks = k_end > k_begin ? (k_end - k_begin + ATT_CK - 1) / ATT_CK : 0u;
    const uint32_t tbl0 = p.block_size ? k_begin / p.block_size : 0u;
    // Every CTA walks its chunks from a different starting point (and wraps around), so that the CTAs
    // of a wave, which start together and advance at the same pace, are not all at the same offset
    // of equally spaced slices.
    const uint32_t rot = nchunks ? (blockIdx.x * 2654435761u >> 8) % nchunks : 0u;
    auto chunk_at = [&](uint32_t c) { const uint32_t cc = c + rot; return cc >= nchunks ? cc - nchunks : cc; };

    if (tid == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < NS; s++) {
            mbar_init(bar_full + 8u * s, 1u);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (p.block_size && nchunks) {
        const uint32_t nblk = (k_end - 1u) / p.block_size - tbl0 + 1u;      // <= ATT_TABLE by the launcher's split
        const int32_t* src = p.block_tables + (size_t)b * p.max_blocks_per_seq + tbl0;
        for (uint32_t i = tid; i < nblk; i += ATT_THREADS) {
            int32_t e = src[i];
            if ((uint32_t)e >= p.num_blocks) {
                e = 0;
                if (p.status) atomicOr(p.status, ATT_STATUS_BLOCK);
            }
            table[i] = e;
        }
    }
    __syncthreads();

    // per-lane state of the consumer warps (the producer warp carries it unused)
    const int sub = lane & 7, kg = lane >> 3;
    float4 q[RT][VPL], o[RT][VPL];
    float m[RT], l[RT];
    uint32_t len[RT];
    bool col_ok[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) col_ok[j] = (uint32_t)(j * 8 + sub) * 4u < D;

    if (warp == ATT_CW) {
        // ---- producer: one chunk = keys [t0, t0 + nk) of K and of V ------------------------------
        for (uint32_t c = 0; c < nchunks; c++) {
            const uint32_t s = c % NS;
            if (c >= NS) {
                named_bar_sync<ATT_BAR_FREE0>(s, ATT_THREADS);          // all consumer warps have left the stage
                if (*abort_flag) break;
            }
            const uint32_t t0 = k_begin + chunk_at(c) * ATT_CK, nk = min((uint32_t)ATT_CK, k_end - t0);
            const uint32_t bar = bar_full + 8u * s;
            float* ks = stages + s * stage_floats;
            float* vs = ks + (size_t)ATT_CK * D;
            if (lane == 0) mbar_expect_tx(bar, 2u * nk * D * 4u);
            __syncwarp();
            if (!p.block_size) {
                if (lane == 0) {
                    const size_t off = (((size_t)b * p.kv_heads + g) * p.kv_stride + t0) * D;
                    bulk_g2s(smem_u32(ks), p.k + off, nk * D * 4u, bar);
                    bulk_g2s(smem_u32(vs), p.v + off, nk * D * 4u, bar);
                }
            } else {
                // one copy per page the chunk touches; lane i takes the i-th page
                const uint32_t blk = t0 / p.block_size + (uint32_t)lane;
                const uint32_t ta = max(t0, blk * p.block_size), tb = min(t0 + nk, (blk + 1u) * p.block_size);
                if (ta < tb) {
                    const size_t off = (((size_t)table[blk - tbl0] * p.kv_heads + g) * p.block_size + (ta - blk * p.block_size)) * D;
                    bulk_g2s(smem_u32(ks + (size_t)(ta - t0) * D), p.k + off, (tb - ta) * D * 4u, bar);
                    bulk_g2s(smem_u32(vs + (size_t)(ta - t0) * D), p.v + off, (tb - ta) * D * 4u, bar);
                }
            }
        }
    } else {
        // ---- consumers -------------------------------------------------------------------------
        const uint32_t rg = (uint32_t)warp % p.rgp, kslot = (uint32_t)warp / p.rgp, wpg = ATT_CW / p.rgp;
#pragma unroll
        for (int i = 0; i < RT; i++) {
            const uint32_t r = row0 + rg * RT + i;
            const bool valid = r < R;
            const uint32_t qi = valid ? r / p.group : 0u, head = g * p.group + (valid ? r % p.group : 0u);
            len[i] = valid ? row_len(p, qi, kv_len) : 0xffffffffu;       // a padding row: q = 0, never written, never masks a chunk
            const float* qr = p.q + (((size_t)b * p.heads + head) * p.seq_q + qi) * D;
            m[i] = ATT_NEG;
            l[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (valid && col_ok[j]) t = __ldg(reinterpret_cast<const float4*>(qr) + j * 8 + sub);
                q[i][j] = make_float4(t.x * p.qscale, t.y * p.qscale, t.z * p.qscale, t.w * p.qscale);
                o[i][j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // One step: the warp's four keys (one per group of 8 lanes) against its RT rows.  The
        // running maximum of a lane is only raised when a score passes it by more than 8 (in the
        // base-2 domain), so weights stay below 2^8 and the common step has no rescaling in it:
        // scores, one exp2 per row, the weighted sum.  MASKED steps (the last chunk of a slice, a
        // causal edge) check each key against the chunk and each row's length.
        const uint32_t row_bytes = D * 4u, lane_off = (uint32_t)sub * 16u;
        auto lds4 = [](uint32_t addr) {
            float4 r;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(addr));
            return r;
        };
        auto step = [&](auto masked, uint32_t kaddr, uint32_t vaddr, bool inb, uint32_t t) {
            constexpr bool MASKED = decltype(masked)::value;
            float sc[RT];
#pragma unroll
            for (int i = 0; i < RT; i++) sc[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                float4 kk = make_float4(0.f, 0.f, 0.f, 0.f);
                if ((FULL || col_ok[j]) && (!MASKED || inb)) kk = lds4(kaddr + (uint32_t)j * 128u);
#pragma unroll
                for (int i = 0; i < RT; i++)
                    sc[i] = fmaf(q[i][j].x, kk.x, fmaf(q[i][j].y, kk.y, fmaf(q[i][j].z, kk.z, fmaf(q[i][j].w, kk.w, sc[i]))));
            }
#pragma unroll
            for (int i = 0; i < RT; i++) {
                sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 1);
                sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 2);
                sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 4);
            }
            bool vis[RT], up = false, any = false;
#pragma unroll
            for (int i = 0; i < RT; i++) {
                vis[i] = !MASKED || (inb && t < len[i]);
                up |= vis[i] && sc[i] > m[i] + 8.0f;
                any |= vis[i];
            }
            if (__any_sync(0xffffffffu, up)) {
#pragma unroll
                for (int i = 0; i < RT; i++) {
                    const float mn = vis[i] ? fmaxf(m[i], sc[i]) : m[i];
                    const float alpha = ex2(m[i] - mn);
                    l[i] *= alpha;
#pragma unroll
                    for (int j = 0; j < VPL; j++) {
                        o[i][j].x *= alpha; o[i][j].y *= alpha; o[i][j].z *= alpha; o[i][j].w *= alpha;
                    }
                    m[i] = mn;
                }
            }
            float pw[RT];
#pragma unroll
            for (int i = 0; i < RT; i++) {
                pw[i] = ex2(sc[i] - m[i]);
                if (MASKED && !vis[i]) pw[i] = 0.0f;
                l[i] += pw[i];
            }
            if (!MASKED || any) {
#pragma unroll
                for (int j = 0; j < VPL; j++) {
                    float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (FULL || col_ok[j]) vv = lds4(vaddr + (uint32_t)j * 128u);
#pragma unroll
                    for (int i = 0; i < RT; i++) {
                        o[i][j].x = fmaf(pw[i], vv.x, o[i][j].x);
                        o[i][j].y = fmaf(pw[i], vv.y, o[i][j].y);
                        o[i][j].z = fmaf(pw[i], vv.z, o[i][j].z);
                        o[i][j].w = fmaf(pw[i], vv.w, o[i][j].w);
                    }
                }
            }
        };
        uint32_t min_len = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < RT; i++) min_len = min(min_len, len[i]);
        const uint32_t stage0 = smem_u32(stages), stage_bytes = 2u * ATT_CK * row_bytes, v_off = ATT_CK * row_bytes;
        for (uint32_t c = 0; c < nchunks; c++) {
            const uint32_t s = c % NS;
            // one poller per CTA: warp 0 waits for the copies, the named barrier releases the other seven
            if (warp == 0) warp_wait(bar_full + 8u * s, (c / NS) & 1u, abort_flag, lane);
            named_bar_sync_c<ATT_BAR_READY>(ATT_CW * 32);
            if (*abort_flag) {
                // the producer may be parked on the stages this warp would still have released
                for (uint32_t cc = c; cc < c + NS && cc + NS < nchunks; cc++) named_bar_arrive<ATT_BAR_FREE0>(cc % NS, ATT_THREADS);
                break;
            }
            const uint32_t t0 = k_begin + chunk_at(c) * ATT_CK, nk = min((uint32_t)ATT_CK, k_end - t0);
            const uint32_t kchunk = stage0 + s * stage_bytes + lane_off;
            if (nk == ATT_CK && t0 + ATT_CK <= min_len) {
                for (uint32_t kb = kslot * 4u; kb < ATT_CK; kb += wpg * 4u) {
                    const uint32_t ka = kchunk + (kb + (uint32_t)kg) * row_bytes;
                    step(std::false_type{}, ka, ka + v_off, true, 0u);
                }
            } else {
                for (uint32_t kb = kslot * 4u; kb < nk; kb += wpg * 4u) {
                    const uint32_t key = kb + (uint32_t)kg, ka = kchunk + key * row_bytes;
                    step(std::true_type{}, ka, ka + v_off, key < nk, t0 + key);
                }
            }
            // done with the stage (not needed for the last NS chunks: nobody refills them)
            if (c + NS < nchunks) named_bar_arrive<ATT_BAR_FREE0>(s, ATT_THREADS);
        }
        // the four key slots of the warp, merged by the running-maximum rule
#pragma unroll
        for (int i = 0; i < RT; i++) {
            float mm = fmaxf(m[i], __shfl_xor_sync(0xffffffffu, m[i], 8));
            mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
            const float alpha = ex2(m[i] - mm);
            m[i] = mm;
            l[i] *= alpha;
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                float* e = reinterpret_cast<float*>(&o[i][j]);
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    float val = e[x] * alpha;
                    val += __shfl_xor_sync(0xffffffffu, val, 8);
                    val += __shfl_xor_sync(0xffffffffu, val, 16);
                    e[x] = val;
                }
            }
        }
    }

    __syncthreads();               // every chunk has landed and been read: the ring is free
    if (*abort_flag) {
        // A bounded wait gave up: report it and give copies still in flight time to land in this
        // CTA's shared memory before it is released.  Nothing is written.
        if (tid == 0 && p.status) atomicOr(p.status, ATT_STATUS_WAIT);
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
        return;
    }
    // warps of one row group -> shared memory (over the ring), then one thread per output element
    float* mrg = stages;                                   // [warp][RT][D + 2]
    const uint32_t MS = D + 2u;
    if (warp < ATT_CW && kg == 0) {
#pragma unroll
        for (int i = 0; i < RT; i++) {
            float* dst = mrg + ((size_t)warp * RT + i) * MS;
#pragma unroll
            for (int j = 0; j < VPL; j++)
                if (col_ok[j]) {
                    // D + 2 floats per row: rows are 8-byte aligned, not 16
                    float* d4 = dst + (j * 8 + sub) * 4;
                    d4[0] = o[i][j].x; d4[1] = o[i][j].y; d4[2] = o[i][j].z; d4[3] = o[i][j].w;
                }
            if (sub == 0) {
                dst[D] = m[i];
                dst[D + 1] = l[i];
            }
        }
    }
    __syncthreads();
    const uint32_t wpg = ATT_CW / p.rgp;
    for (uint32_t e = tid; e < rpb * D; e += ATT_THREADS) {
        const uint32_t ir = e / D, d = e - ir * D, r = row0 + ir;
        if (r >= R) continue;
        const uint32_t rgi = ir / RT, ii = ir % RT;
        float M = ATT_NEG;
        for (uint32_t w = 0; w < wpg; w++) M = fmaxf(M, mrg[((size_t)(w * p.rgp + rgi) * RT + ii) * MS + D]);
        float L = 0.0f, acc = 0.0f;
        for (uint32_t w = 0; w < wpg; w++) {
            const float* src = mrg + ((size_t)(w * p.rgp + rgi) * RT + ii) * MS;
            const float wgt = ex2(src[D] - M);
            L = fmaf(src[D + 1], wgt, L);
            acc = fmaf(src[d], wgt, acc);
        }
        const uint32_t qi = r / p.group, head = g * p.group + r % p.group;
        const size_t orow = ((size_t)b * p.heads + head) * p.seq_q + qi;
        if (p.nsplit == 1) {
            p.out[orow * D + d] = L > 0.0f ? acc / L : 0.0f;
            if (d == 0 && p.lse) p.lse[orow] = L > 0.0f ? fmaf(M, ATT_LN2, logf(L)) : -3.402823e+38f;
        } else {
            float* dst = p.part + (orow * p.nsplit + split) * MS;
            dst[d] = acc;
            if (d == 0) {
                dst[D] = M;
                dst[D + 1] = L;
            }
        }
    }
}

// Merge of the key slices of one output row (paged_attention_v2_reduce, paged.wgsl:351-405, with
// the statistics in the base-2 domain).  One CTA per row; resident early, it waits for the slices.
__global__ void __launch_bounds__(128) lux_attn_merge_f32(const float* __restrict__ part, float* __restrict__ out, float* __restrict__ lse,
                                                          const int32_t* __restrict__ context_lens, uint32_t rows_per_seq,
                                                          uint32_t nsplit, uint32_t D) {
    __shared__ float wgt[256];
    __shared__ float stat[2];
    pdl_wait();
    const uint32_t row = blockIdx.x, MS = D + 2u;
    if (context_lens && context_lens[row / rows_per_seq] <= 0) return;
    const float* base = part + (size_t)row * nsplit * MS;
    if (threadIdx.x < 32) {
        float M = ATT_NEG;
        for (uint32_t s = threadIdx.x; s < nsplit; s += 32) M = fmaxf(M, base[(size_t)s * MS + D]);
        for (int off = 16; off; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        float L = 0.0f;
        for (uint32_t s = threadIdx.x; s < nsplit; s += 32) {
            const float w = exp2f(base[(size_t)s * MS + D] - M);
            wgt[s] = w;
            L = fmaf(base[(size_t)s * MS + D + 1], w, L);
        }
        for (int off = 16; off; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        if (threadIdx.x == 0) {
            stat[0] = M;
            stat[1] = L;
        }
    }
    __syncthreads();
    const float L = stat[1], inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t s = 0; s < nsplit; s++) acc = fmaf(base[(size_t)s * MS + d], wgt[s], acc);
        out[(size_t)row * D + d] = acc * inv;
    }
    if (threadIdx.x == 0 && lse) lse[row] = L > 0.0f ? fmaf(stat[0], ATT_LN2, logf(L)) : -3.402823e+38f;
}

// Any head_dim, any alignment: one CTA per output row, 256 keys per step (a thread per key for the
// scores, a thread per output dimension for the weighted sum), the same running-maximum rule.
__device__ __forceinline__ const float* plain_row(const AttnParams& p, const float* base, uint32_t b, uint32_t g, uint32_t t,
                                                  const int32_t* table) {
    if (!p.block_size) return base + (((size_t)b * p.kv_heads + g) * p.kv_stride + t) * p.head_dim;
    int32_t e = table[t / p.block_size];
    if ((uint32_t)e >= p.num_blocks) e = 0;
    return base + (((size_t)e * p.kv_heads + g) * p.block_size + t % p.block_size) * p.head_dim;
}

__global__ void __launch_bounds__(256) lux_attn_plain_f32(const AttnParams p) {
    extern __shared__ float sm[];
    float* o = sm;                       // [head_dim]
    float* pw = sm + p.head_dim;         // [256]
    __shared__ float red[8];
    const uint32_t D = p.head_dim, tid = threadIdx.x;
    uint32_t idx = blockIdx.x;
    const uint32_t qi = idx % p.seq_q; idx /= p.seq_q;
    const uint32_t head = idx % p.heads, b = idx / p.heads, g = head / p.group;
    uint32_t kv_len = p.kv_len;
    const int32_t* table = nullptr;
    if (p.block_size) {
        const int32_t cl = p.context_lens[b];
        if (cl <= 0) return;
        kv_len = min((uint32_t)cl, p.max_blocks_per_seq * p.block_size);
        table = p.block_tables + (size_t)b * p.max_blocks_per_seq;
    }
    const uint32_t len = row_len(p, qi, kv_len);
    const size_t orow = ((size_t)b * p.heads + head) * p.seq_q + qi;
    const float* qr = p.q + orow * D;
    for (uint32_t d = tid; d < D; d += 256) o[d] = 0.0f;
    float m = ATT_NEG, l = 0.0f;
    for (uint32_t t0 = 0; t0 < len; t0 += 256) {
        const uint32_t t = t0 + tid;
        float s = ATT_NEG;
        if (t < len) {
            const float* kr = plain_row(p, p.k, b, g, t, table);
            float dot = 0.0f;
            for (uint32_t d = 0; d < D; d++) dot = fmaf(qr[d], kr[d], dot);
            s = dot * p.qscale;
        }
        float tm = s;
        for (int off = 16; off; off >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, off));
        if ((tid & 31) == 0) red[tid >> 5] = tm;
        __syncthreads();
        tm = red[0];
        for (int w = 1; w < 8; w++) tm = fmaxf(tm, red[w]);
        const float mn = fmaxf(m, tm), alpha = exp2f(m - mn);
        const float e = t < len ? exp2f(s - mn) : 0.0f;
        pw[tid] = e;
        float ts = e;
        for (int off = 16; off; off >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, off);
        __syncthreads();                                   // red[] read by everyone, pw[] written
        if ((tid & 31) == 0) red[tid >> 5] = ts;
        __syncthreads();
        ts = 0.0f;
        for (int w = 0; w < 8; w++) ts += red[w];
        l = fmaf(l, alpha, ts);
        m = mn;
        const uint32_t n = min(256u, len - t0);
        for (uint32_t d = tid; d < D; d += 256) {
            float acc = o[d] * alpha;
            for (uint32_t j = 0; j < n; j++) acc = fmaf(pw[j], plain_row(p, p.v, b, g, t0 + j, table)[d], acc);
            o[d] = acc;
        }
        __syncthreads();
    }
    for (uint32_t d = tid; d < D; d += 256) p.out[orow * D + d] = l > 0.0f ? o[d] / l : 0.0f;
    if (tid == 0 && p.lse) p.lse[orow] = l > 0.0f ? fmaf(m, ATT_LN2, logf(l)) : -3.402823e+38f;
}

// ---- rotary embedding ------------------------------------------------------------------------------

struct RopeParams {
    const float* x;
    float* out;
    const float* x2;               // second tensor of the fused q/k call (null otherwise), rotated in place
    float* out2;
    const float* cos_cache;
    const float* sin_cache;
    const uint32_t* position_ids;
    uint32_t* status;
    uint32_t batch, seq, heads, heads2, half;
    uint32_t position_offset, cache_positions, ntk, backward;
    float theta, head_dim_f;
};

// correctly rounded theta^(-2 i / head_dim) for all but a vanishing share of arguments: the f32
// exponent of the shader (rope.wgsl:56-60), the power in double, one rounding
__device__ __forceinline__ float rope_freq(uint32_t i, float head_dim_f, float theta) {
    const float exponent = __fdiv_rn(__fmul_rn(-2.0f, (float)i), head_dim_f);
    return (float)pow((double)theta, (double)exponent);
}

__global__ void __launch_bounds__(256) lux_rope_f32(const RopeParams p) {
    const size_t per_tok = (size_t)(p.heads + p.heads2) * p.half;
    const size_t total = (size_t)p.batch * p.seq * per_tok;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t tok = e / per_tok;
        uint32_t rem = (uint32_t)(e - tok * per_tok);
        const uint32_t s = (uint32_t)(tok % p.seq);
        uint32_t position = p.position_ids ? p.position_ids[tok] : p.position_offset + s;
        if (p.ntk) position = s;                          // rope_ntk_scaled uses the index alone (rope.wgsl:337-339)
        const float* src = p.x;
        float* dst = p.out;
        uint32_t heads = p.heads;
        if (rem >= p.heads * p.half) {
            rem -= p.heads * p.half;
            src = p.x2;
            dst = p.out2;
            heads = p.heads2;
        }
        const uint32_t i = rem % p.half;
        float c, sn;
        if (p.cos_cache) {
            if (position >= p.cache_positions) {
                if (p.status) atomicOr(p.status, ATT_STATUS_POSITION);
                continue;
            }
            c = __ldg(p.cos_cache + (size_t)position * p.half + i);
            sn = __ldg(p.sin_cache + (size_t)position * p.half + i);
        } else {
            const float angle = __fmul_rn((float)position, rope_freq(i, p.head_dim_f, p.theta));
            c = cosf(angle);
            sn = sinf(angle);
        }
        const size_t i0 = (tok * heads) * (2 * (size_t)p.half) + 2 * (size_t)rem;
        const float2 xv = *reinterpret_cast<const float2*>(src + i0);
        float2 y;
        if (!p.backward) {
            y.x = __fsub_rn(__fmul_rn(xv.x, c), __fmul_rn(xv.y, sn));
            y.y = __fadd_rn(__fmul_rn(xv.x, sn), __fmul_rn(xv.y, c));
        } else {
            y.x = __fadd_rn(__fmul_rn(xv.x, c), __fmul_rn(xv.y, sn));
            y.y = __fadd_rn(__fmul_rn(-xv.x, sn), __fmul_rn(xv.y, c));
        }
        *reinterpret_cast<float2*>(dst + i0) = y;
    }
}

__global__ void __launch_bounds__(256) lux_rope_cache_f32(float* __restrict__ cos_out, float* __restrict__ sin_out, uint32_t max_seq_len,
                                                          uint32_t half, float head_dim_f, float theta) {
    const size_t total = (size_t)max_seq_len * half;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const uint32_t pos = (uint32_t)(e / half), i = (uint32_t)(e % half);
        const float angle = __fmul_rn((float)pos, rope_freq(i, head_dim_f, theta));
        cos_out[e] = cosf(angle);
        sin_out[e] = sinf(angle);
    }
}

// update_kv_cache: one thread per element (pairs of caches, same index arithmetic)
__global__ void __launch_bounds__(256) lux_kv_append_f32(const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ k_cache,
                                                         float* __restrict__ v_cache, uint32_t bh, uint32_t seq_q, uint32_t cache_len,
                                                         uint32_t max_cache_len, uint32_t D) {
    const size_t total = (size_t)bh * seq_q * D;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const uint32_t d = (uint32_t)(e % D);
        const size_t t = e / D;
        const uint32_t s = (uint32_t)(t % seq_q);
        const size_t h = t / seq_q;
        const uint64_t pos = (uint64_t)cache_len + s;
        if (pos >= max_cache_len) continue;                // cache overflow is dropped (:523-525)
        const size_t dst = (h * max_cache_len + pos) * D + d;
        k_cache[dst] = k[e];
        v_cache[dst] = v[e];
    }
}

// ---- host side -------------------------------------------------------------------------------------

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
uint32_t pow2ceil(uint32_t v) {
    uint32_t r = 1;
    while (r < v) r <<= 1;
    return r;
}

using AttnKernel = void (*)(const AttnParams);
template <int VPL, int RT> AttnKernel stream_kernel(bool full) {
    return full ? lux_attn_stream_f32<VPL, RT, true> : lux_attn_stream_f32<VPL, RT, false>;
}
// full: head_dim is exactly VPL * 32, so no lane has a column to skip
AttnKernel pick_stream(int vpl, int rt, bool full) {
    switch (vpl * 10 + rt) {
        case 11: return stream_kernel<1, 1>(full); case 12: return stream_kernel<1, 2>(full);
        case 21: return stream_kernel<2, 1>(full); case 22: return stream_kernel<2, 2>(full);
        case 31: return stream_kernel<3, 1>(full); case 32: return stream_kernel<3, 2>(full);
        case 41: return stream_kernel<4, 1>(full); case 42: return stream_kernel<4, 2>(full);
        case 81: return stream_kernel<8, 1>(full);
    }
    return nullptr;
}

// Fills the launch geometry of p and launches.  max_keys: the longest context any row can have.
LuxBackendError attn_launch(Context* ctx, AttnParams& p, uint32_t max_keys, uint32_t flags, const char* what) {
    cudaSetDevice(ctx->device);
    p.status = ctx->d_status;
    const uint32_t D = p.head_dim;
    const size_t out_rows = (size_t)p.batch * p.heads * p.seq_q;
    if (out_rows == 0) return LUX_BACKEND_OK;
    const bool stream_ok = D % 4 == 0 && D <= 256 && aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && out_rows <= 0x7fffffffu;
    if (!stream_ok) {
        if (out_rows > 0x7fffffffu) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        const size_t smem = ((size_t)D + 256) * 4;
        if (smem > 200u << 10) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        if (smem > 48u << 10) cudaFuncSetAttribute(lux_attn_plain_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        p.nsplit = 1;
        lux_attn_plain_f32<<<(unsigned)out_rows, 256, smem, ctx->stream>>>(p);
        count_launch("lux_attn_plain_f32");
        return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, what);
    }
    int vpl = (int)((D + 31) / 32);
    if (vpl > 4) vpl = 8;
    const uint32_t R = p.group * p.seq_q;
    // two query rows per lane: more would halve the shared-memory reads per row, but the registers
    // of four rows leave one CTA of nine warps per SM, too few to hide the latency of each step
    // (measured: causal prefill of 2048 tokens, Llama-3-8B heads, 15.2 TFLOP/s against 20.4)
    const int rt = R >= 2 && vpl <= 4 ? 2 : 1;
    p.rgp = pow2ceil(std::min<uint32_t>((R + rt - 1) / rt, ATT_CW));
    const uint32_t rpb = rt * p.rgp;
    p.row_blocks = (R + rpb - 1) / rpb;
    const size_t items = (size_t)p.batch * p.kv_heads * p.row_blocks;
    // Slices of the keys.  CTAs run two per SM, so the grid should fill whole waves of 2 x SMs; a slice
    // costs a CTA start-up and a row in the merge, about as much as streaming 64 keys, and is at
    // least 128 keys long.  The block-table copy caps the pages a slice may span.
    auto geometry = [&](uint32_t want) {
        p.split_keys = std::max<uint32_t>(((max_keys + want - 1) / want + ATT_CK - 1) / ATT_CK * ATT_CK, ATT_CK);
        p.nsplit = std::max<uint32_t>((max_keys + p.split_keys - 1) / p.split_keys, 1u);
    };
    uint32_t min_split = 1;
    if (p.block_size) {
        // a slice (a multiple of the chunk) spans at most split_keys / block_size + 2 pages
        const uint64_t cap = (uint64_t)(ATT_TABLE - 2) * p.block_size / ATT_CK * ATT_CK;
        min_split = (uint32_t)std::max<uint64_t>((max_keys + cap - 1) / cap, 1);
    }
    uint32_t best = min_split;
    double best_score = -1.0;
    const uint32_t sm = (uint32_t)ctx->sm_count * ATT_CTAS_PER_SM;
    for (uint32_t n = min_split; n <= 256; n++) {
        geometry(n);
        if (p.nsplit != n) continue;                                   // rounding to chunks merged this count into a smaller one
        if (n > min_split && p.split_keys < 128) break;
        const double ctas = (double)items * n, waves = std::ceil(ctas / sm);
        const double score = ctas / (waves * sm) * p.split_keys / (p.split_keys + 64.0);
        if (score > best_score * 1.02) {                               // a larger count has to earn its merge
            best_score = score;
            best = n;
        }
        if (ctas > 8.0 * sm) break;
    }
    geometry(g_tune.attn_splits > 0 ? std::max<uint32_t>((uint32_t)g_tune.attn_splits, min_split) : best);
    if (p.nsplit > 256) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;     // a context beyond 256 x 2046 pages
    const size_t part_bytes = p.nsplit > 1 ? out_rows * p.nsplit * (D + 2) * 4 : 0;
    if (part_bytes > ctx->d_attn_bytes) {
        // fewer slices than wanted rather than an allocation inside a call
        const uint32_t fit = (uint32_t)(ctx->d_attn_bytes / (out_rows * (D + 2) * 4));
        if (std::max(fit, 1u) < min_split) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
        geometry(std::max(fit, 1u));
    }
    p.part = p.nsplit > 1 ? (float*)ctx->d_attn : nullptr;
    const size_t stage_bytes = (size_t)2 * ATT_CK * D * 4;
    const size_t fixed = ATT_HEADER + (p.block_size ? ATT_TABLE * 4 : 0);
    // heads wider than 128 take the whole SM's shared memory (one CTA per SM)
    const size_t budget = D > 128 ? 2 * ATT_SMEM_BUDGET : ATT_SMEM_BUDGET;
    p.stages = (uint32_t)std::min<size_t>(ATT_MAX_STAGES, (budget - fixed) / stage_bytes);
    const size_t smem = fixed + p.stages * stage_bytes;
    const bool full = D == (uint32_t)vpl * 32u;
    AttnKernel kfn = pick_stream(vpl, rt, full);
    if (!kfn || p.stages < 2) return LUX_BACKEND_ERROR_INTERNAL;
    static std::mutex mu;
    static bool attr_set[16][9][3][2];
    {
        std::lock_guard<std::mutex> lk(mu);
        bool& done = attr_set[ctx->device & 15][vpl][rt][full ? 1 : 0];
        if (!done) {
            if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * ATT_SMEM_BUDGET)) != cudaSuccess)
                return map_cuda(cudaGetLastError(), what);
            done = true;
        }
    }
    const size_t ctas = items * p.nsplit;
    if (ctas > 0x7fffffffu) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    kfn<<<(unsigned)ctas, ATT_THREADS, smem, ctx->stream>>>(p);
    count_launch("lux_attn_stream_f32");
    if (p.nsplit > 1) {
        cudaError_t e = launch_pdl(g_tune.pdl != 2, lux_attn_merge_f32, dim3((unsigned)out_rows), dim3(128), 0, ctx->stream, 1, (const float*)p.part,
                                   p.out, p.lse, p.context_lens, p.heads * p.seq_q, p.nsplit, D);
        if (e != cudaSuccess) return map_cuda(e, what);
        count_launch("lux_attn_merge_f32");
    }
    return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, what);
}

bool holds(const Buffer* b, size_t elems, size_t elem_bytes = 4) { return b && b->ptr && b->size / elem_bytes >= elems; }
// products of u32 arguments as a size, saturating
size_t mul(std::initializer_list<uint64_t> v) {
    unsigned __int128 r = 1;
    for (uint64_t x : v) {
        r *= x;
        if (r > (unsigned __int128)0x3fffffffffffffffull) return (size_t)0x3fffffffffffffffull;
    }
    return (size_t)r;
}

}  // namespace

// entries of the kernel table (kernel_table.cu): the Llama-shaped instance of the streaming kernel
const void* kernel_addr_attn_stream_f32() { return (const void*)lux_attn_stream_f32<4, 2, true>; }
const void* kernel_addr_attn_merge_f32() { return (const void*)lux_attn_merge_f32; }
const void* kernel_addr_attn_plain_f32() { return (const void*)lux_attn_plain_f32; }
const void* kernel_addr_rope_f32() { return (const void*)lux_rope_f32; }
const void* kernel_addr_kv_append_f32() { return (const void*)lux_kv_append_f32; }

}  // namespace luxcuda

using namespace luxcuda;

extern "C" LuxBackendError lux_cuda_rope_precompute_cache_f32(LuxBackendContext* context, LuxBackendBuffer* cos_out, LuxBackendBuffer* sin_out,
                                                              uint32_t max_seq_len, uint32_t head_dim, float theta_base, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bc = as_buf(cos_out), *bs = as_buf(sin_out);
    if (!ctx || !bc || !bs || head_dim == 0 || head_dim % 2 || !(theta_base > 0.0f)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t total = mul({max_seq_len, head_dim / 2});
    if (!holds(bc, total) || !holds(bs, total)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (total == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((total + 255) / 256, (size_t)ctx->sm_count * 8);
    lux_rope_cache_f32<<<(unsigned)blocks, 256, 0, ctx->stream>>>((float*)bc->ptr, (float*)bs->ptr, max_seq_len, head_dim / 2, (float)head_dim,
                                                                 theta_base);
    count_launch("lux_rope_cache_f32");
    return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, "rope_precompute_cache_f32");
}

namespace {
LuxBackendError rope_common(Context* ctx, RopeParams& p, Buffer* bc, Buffer* bs, uint32_t head_dim, uint32_t flags, const char* what) {
    if ((bc != nullptr) != (bs != nullptr)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    p.half = head_dim / 2;
    p.head_dim_f = (float)head_dim;
    p.cos_cache = bc ? (const float*)bc->ptr : nullptr;
    p.sin_cache = bs ? (const float*)bs->ptr : nullptr;
    p.cache_positions = 0;
    if (bc) {
        if (!bc->ptr || !bs->ptr) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        p.cache_positions = (uint32_t)std::min<size_t>(std::min(bc->size, bs->size) / 4 / p.half, 0xffffffffu);
        if (!p.position_ids && (uint64_t)p.position_offset + p.seq > p.cache_positions) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    p.backward = (flags & LUX_ROPE_FLAG_BACKWARD) ? 1u : 0u;
    p.status = ctx->d_status;
    const size_t total = mul({p.batch, p.seq, (uint64_t)p.heads + p.heads2, p.half});
    if (total == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((total + 255) / 256, (size_t)ctx->sm_count * 16);
    lux_rope_f32<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p);
    count_launch("lux_rope_f32");
    return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, what);
}
}  // namespace

extern "C" LuxBackendError lux_cuda_rope_f32(LuxBackendContext* context, LuxBackendBuffer* x, LuxBackendBuffer* out, LuxBackendBuffer* cos_cache,
                                             LuxBackendBuffer* sin_cache, LuxBackendBuffer* position_ids, uint32_t batch_size,
                                             uint32_t seq_len, uint32_t num_heads, uint32_t head_dim, float theta_base,
                                             uint32_t position_offset, float ntk_scale, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bx = as_buf(x), *bo = as_buf(out), *bp = as_buf(position_ids);
    if (!ctx || !bx || !bo || head_dim == 0 || head_dim % 2) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t total = mul({batch_size, seq_len, num_heads, head_dim});
    if (!holds(bx, total) || !holds(bo, total)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bp && !holds(bp, mul({batch_size, seq_len}))) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(bx->ptr) | reinterpret_cast<uintptr_t>(bo->ptr)) & 7u) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const bool cached = cos_cache || sin_cache;
    if (!cached && !(theta_base > 0.0f)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (ntk_scale > 0.0f && (cached || head_dim <= 2)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    RopeParams p{};
    p.x = (const float*)bx->ptr;
    p.out = (float*)bo->ptr;
    p.position_ids = bp ? (const uint32_t*)bp->ptr : nullptr;
    p.batch = batch_size;
    p.seq = seq_len;
    p.heads = num_heads;
    p.heads2 = 0;
    p.position_offset = position_offset;
    p.theta = theta_base;
    if (ntk_scale > 0.0f) {
        // scaled base, rope.wgsl:335, formed once on the host
        p.theta = theta_base * powf(ntk_scale, (float)head_dim / ((float)head_dim - 2.0f));
        p.ntk = 1;
    }
    return rope_common(ctx, p, as_buf(cos_cache), as_buf(sin_cache), head_dim, flags, "rope_f32");
}

extern "C" LuxBackendError lux_cuda_rope_qk_f32(LuxBackendContext* context, LuxBackendBuffer* q, LuxBackendBuffer* k, LuxBackendBuffer* cos_cache,
                                                LuxBackendBuffer* sin_cache, uint32_t batch_size, uint32_t seq_len, uint32_t num_heads,
                                                uint32_t num_kv_heads, uint32_t head_dim, uint32_t position_offset, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bq = as_buf(q), *bk = as_buf(k);
    if (!ctx || !bq || !bk || !cos_cache || !sin_cache || head_dim == 0 || head_dim % 2) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!holds(bq, mul({batch_size, seq_len, num_heads, head_dim})) || !holds(bk, mul({batch_size, seq_len, num_kv_heads, head_dim})))
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(bq->ptr) | reinterpret_cast<uintptr_t>(bk->ptr)) & 7u) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    RopeParams p{};
    p.x = (const float*)bq->ptr;
    p.out = (float*)bq->ptr;
    p.x2 = (const float*)bk->ptr;
    p.out2 = (float*)bk->ptr;
    p.batch = batch_size;
    p.seq = seq_len;
    p.heads = num_heads;
    p.heads2 = num_kv_heads;
    p.position_offset = position_offset;
    p.theta = 1.0f;
    return rope_common(ctx, p, as_buf(cos_cache), as_buf(sin_cache), head_dim, flags, "rope_qk_f32");
}

extern "C" LuxBackendError lux_cuda_sdpa_f32(LuxBackendContext* context, LuxBackendBuffer* q, LuxBackendBuffer* k, LuxBackendBuffer* v,
                                             LuxBackendBuffer* out, LuxBackendBuffer* lse, uint32_t batch_size, uint32_t num_heads,
                                             uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t seq_len_kv, uint32_t head_dim, float scale,
                                             uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bq = as_buf(q), *bk = as_buf(k), *bv = as_buf(v), *bo = as_buf(out), *bl = as_buf(lse);
    if (!ctx || !bq || !bk || !bv || !bo || head_dim == 0 || num_kv_heads == 0 || num_heads % num_kv_heads) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t qn = mul({batch_size, num_heads, seq_len_q, head_dim}), kn = mul({batch_size, num_kv_heads, seq_len_kv, head_dim});
    if (!holds(bq, qn) || !holds(bo, qn)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (kn && (!holds(bk, kn) || !holds(bv, kn))) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bl && !holds(bl, mul({batch_size, num_heads, seq_len_q}))) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    AttnParams p{};
    p.q = (const float*)bq->ptr;
    p.k = (const float*)bk->ptr;
    p.v = (const float*)bv->ptr;
    p.out = (float*)bo->ptr;
    p.lse = bl ? (float*)bl->ptr : nullptr;
    p.batch = batch_size;
    p.heads = num_heads;
    p.kv_heads = num_kv_heads;
    p.group = num_heads / num_kv_heads;
    p.seq_q = seq_len_q;
    p.head_dim = head_dim;
    p.kv_len = seq_len_kv;
    p.kv_stride = seq_len_kv;
    p.causal = (flags & LUX_ATTN_FLAG_CAUSAL) ? 1u : 0u;
    p.causal_base = 0;
    p.qscale = scale * ATT_LOG2E;
    return attn_launch(ctx, p, seq_len_kv, flags, "sdpa_f32");
}

extern "C" LuxBackendError lux_cuda_update_kv_cache_f32(LuxBackendContext* context, LuxBackendBuffer* k, LuxBackendBuffer* v,
                                                        LuxBackendBuffer* k_cache, LuxBackendBuffer* v_cache, uint32_t batch_size,
                                                        uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t cache_len, uint32_t max_cache_len,
                                                        uint32_t head_dim, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bk = as_buf(k), *bv = as_buf(v), *bkc = as_buf(k_cache), *bvc = as_buf(v_cache);
    if (!ctx || !bk || !bv || !bkc || !bvc || head_dim == 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t n = mul({batch_size, num_kv_heads, seq_len_q, head_dim}), cn = mul({batch_size, num_kv_heads, max_cache_len, head_dim});
    if (!holds(bk, n) || !holds(bv, n) || !holds(bkc, cn) || !holds(bvc, cn)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    const size_t blocks = std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
    lux_kv_append_f32<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)bk->ptr, (const float*)bv->ptr, (float*)bkc->ptr, (float*)bvc->ptr,
                                                                batch_size * num_kv_heads, seq_len_q, cache_len, max_cache_len, head_dim);
    count_launch("lux_kv_append_f32");
    return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, "update_kv_cache_f32");
}

extern "C" LuxBackendError lux_cuda_sdpa_kv_cache_f32(LuxBackendContext* context, LuxBackendBuffer* q, LuxBackendBuffer* k_cache,
                                                      LuxBackendBuffer* v_cache, LuxBackendBuffer* out, uint32_t batch_size, uint32_t num_heads,
                                                      uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t cache_len, uint32_t max_cache_len,
                                                      uint32_t head_dim, float scale, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bq = as_buf(q), *bk = as_buf(k_cache), *bv = as_buf(v_cache), *bo = as_buf(out);
    if (!ctx || !bq || !bk || !bv || !bo || head_dim == 0 || num_kv_heads == 0 || num_heads % num_kv_heads || seq_len_q == 0)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((uint64_t)cache_len + seq_len_q > max_cache_len) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t qn = mul({batch_size, num_heads, seq_len_q, head_dim}), cn = mul({batch_size, num_kv_heads, max_cache_len, head_dim});
    if (!holds(bq, qn) || !holds(bo, qn) || !holds(bk, cn) || !holds(bv, cn)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    AttnParams p{};
    p.q = (const float*)bq->ptr;
    p.k = (const float*)bk->ptr;
    p.v = (const float*)bv->ptr;
    p.out = (float*)bo->ptr;
    p.batch = batch_size;
    p.heads = num_heads;
    p.kv_heads = num_kv_heads;
    p.group = num_heads / num_kv_heads;
    p.seq_q = seq_len_q;
    p.head_dim = head_dim;
    p.kv_len = cache_len + seq_len_q;
    p.kv_stride = max_cache_len;
    p.causal = (flags & LUX_ATTN_FLAG_CAUSAL) ? 1u : 0u;
    p.causal_base = cache_len;
    p.qscale = scale * ATT_LOG2E;
    return attn_launch(ctx, p, p.kv_len, flags, "sdpa_kv_cache_f32");
}

extern "C" LuxBackendError lux_cuda_paged_attention_f32(LuxBackendContext* context, LuxBackendBuffer* q, LuxBackendBuffer* k_cache,
                                                        LuxBackendBuffer* v_cache, LuxBackendBuffer* block_tables,
                                                        LuxBackendBuffer* context_lens, LuxBackendBuffer* out, uint32_t num_seqs,
                                                        uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t block_size,
                                                        uint32_t max_blocks_per_seq, float scale, uint32_t flags) {
    Context* ctx = as_ctx(context);
    Buffer *bq = as_buf(q), *bk = as_buf(k_cache), *bv = as_buf(v_cache), *bt = as_buf(block_tables), *bc = as_buf(context_lens),
           *bo = as_buf(out);
    if (!ctx || !bq || !bk || !bv || !bt || !bc || !bo || head_dim == 0 || num_kv_heads == 0 || num_heads % num_kv_heads || block_size == 0 ||
        max_blocks_per_seq == 0)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t qn = mul({num_seqs, num_heads, head_dim});
    if (!holds(bq, qn) || !holds(bo, qn) || !holds(bt, mul({num_seqs, max_blocks_per_seq})) || !holds(bc, num_seqs))
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t block_elems = mul({num_kv_heads, block_size, head_dim});
    const size_t num_blocks = std::min(bk->size, bv->size) / 4 / block_elems;
    const uint64_t max_keys = (uint64_t)max_blocks_per_seq * block_size;
    if (num_blocks == 0 || !bk->ptr || !bv->ptr || max_keys > 0x7fffffffu) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    AttnParams p{};
    p.q = (const float*)bq->ptr;
    p.k = (const float*)bk->ptr;
    p.v = (const float*)bv->ptr;
    p.out = (float*)bo->ptr;
    p.block_tables = (const int32_t*)bt->ptr;
    p.context_lens = (const int32_t*)bc->ptr;
    p.batch = num_seqs;
    p.heads = num_heads;
    p.kv_heads = num_kv_heads;
    p.group = num_heads / num_kv_heads;
    p.seq_q = 1;
    p.head_dim = head_dim;
    p.kv_len = (uint32_t)max_keys;
    p.block_size = block_size;
    p.max_blocks_per_seq = max_blocks_per_seq;
    p.num_blocks = (uint32_t)std::min<size_t>(num_blocks, 0x7fffffffu);
    p.qscale = scale * ATT_LOG2E;
    return attn_launch(ctx, p, (uint32_t)max_keys, flags, "paged_attention_f32");
}
