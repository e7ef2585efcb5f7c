// lux_peer_allreduce_push -- one-node, one-shot all-reduce (sum) of a 16-bit tensor over peer
// memory, for the tensor-parallel FFN's partial outputs (16 KB at batch 1, 4 MB at batch 256):
// at these sizes latency, not link bandwidth, is what a ring or a tree would lose.
//
// Every rank owns a WINDOW in its own HBM that its peers can write (CUDA IPC mapping, or plain
// peer pointers inside one process):
//
//     [2 parities][world source ranks][slot: one 8-byte word {2 elements, epoch} per 2 elements]
//
// One kernel per call, as many CTAs as the tensor has 4 KB pieces (at most one per SM); a thread
// owns 16-byte pieces of the tensor from start to finish:
//   1. push   it packs a piece into 8-byte words {two 16-bit elements, epoch} and stores them (two
//             words per 16-byte store) into slot [parity][my rank] of EVERY rank's window, its own
//             included.  An aligned 8-byte store arrives whole, so a word whose epoch field matches
//             carries valid data: no fence and no separate "done" flag are needed (the scheme of
//             NCCL's LL protocol).  Plain stores only -- no loads from peer memory, no TMA, no
//             multicast;
//   2. reduce it polls the same piece of every source rank in its OWN window (all loads of a round
//             issued before any is tested, L1 bypassed) until every epoch field matches, sums the
//             source ranks in rank order in f32 and writes the piece of the local tensor, so all
//             ranks hold bit-identical results.
// The wait is bounded by a deadline on the SM's cycle counter for the whole call (about 1 s by
// default).  If it passes, the kernel sets the context's status word (the host then reports
// DEVICE_LOST) and marks the communicator FAILED in device memory: pieces whose words never came
// keep their old contents, and every later call on that communicator returns at once with the same
// status instead of waiting again -- after a failure the ranks' epochs may differ, so the
// communicator must be destroyed and created anew on every rank.
// The control words {epoch, CTAs done, failed, CTAs done (fused producer)} live in device memory;
// the last CTA to finish advances the epoch, so the call can be captured in a CUDA graph and
// replayed.  Two parities suffice: a rank can be at most one epoch ahead of a peer, because
// finishing epoch n needs every peer's epoch-n words, which a peer stores only after it has
// finished reading epoch n-1.
// The kernel is launched with the programmatic-launch attribute: its CTAs are resident when the
// kernel that produces the tensor finishes, and wait for it with griddepcontrol.wait.
//
// The reference has no multi-device path (no NCCL / MPI call site in luxcpp/webgpu); this is
// the push all-reduce its tensor-parallel replacement needs.
#include "common.cuh"

#include <algorithm>
#include <cstring>

namespace luxcuda {

namespace {

constexpr int MAX_WORLD = 8;
constexpr int AR_THREADS = 256;

struct PeerComm {
    int device = 0;
    int rank = 0, world = 0;
    size_t max_bytes = 0;
    unsigned char* window = nullptr;          // this rank's window (owned)
    unsigned char* peer[MAX_WORLD] = {};      // every rank's window as seen from here (peer[rank] == window)
    bool opened[MAX_WORLD] = {};              // mapped with cudaIpcOpenMemHandle (to be closed)
    uint32_t* ctl = nullptr;                  // device control words (owned): see PEER_CTL_* in common.cuh
    bool connected = false;
};

struct PushParams {
    unsigned char* peer[MAX_WORLD];
    void* buf;
    uint32_t* ctl;
    uint32_t* status;
    unsigned long long max_bytes;
    unsigned long long count;                 // 16-bit elements
    unsigned long long wait_ns;               // deadline of the whole call
    int rank, world;
    int early;                                // PUSH = false only: do not wait for the producer kernel to end before polling
};

// a slot holds max_bytes of payload as 8-byte words {4 bytes of payload, 4 bytes of epoch}
__host__ __device__ inline size_t slot_bytes(size_t max_bytes) { return 2 * max_bytes; }
// the slots, then 256 bytes that hold an identification tag; the ALLOCATION is rounded up to a
// multiple of 2 MiB so that it owns its driver block: cudaIpcOpenMemHandle maps whole blocks and
// returns the block's base, which is the window only if nothing else shares the block
__host__ __device__ inline size_t window_bytes(int world, size_t max_bytes) {
    return (size_t)2 * world * slot_bytes(max_bytes) + 256;
}
inline size_t window_alloc_bytes(int world, size_t max_bytes) {
    const size_t two_mib = (size_t)2 << 20;
    return (window_bytes(world, max_bytes) + two_mib - 1) / two_mib * two_mib;
}
struct WindowTag { uint32_t magic, rank, world, max_bytes_lo; };
constexpr uint32_t TAG_MAGIC = 0x4C555850u;   // "LUXP"
inline size_t tag_offset(int world, size_t max_bytes) { return (size_t)2 * world * slot_bytes(max_bytes); }
__device__ __forceinline__ unsigned char* slot_ptr(unsigned char* win, int world, size_t max_bytes, int parity, int src) {
    return win + ((size_t)parity * world + src) * slot_bytes(max_bytes);
}

template <bool BF16> __device__ __forceinline__ float2 widen2(uint32_t v);
template <> __device__ __forceinline__ float2 widen2<false>(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
template <> __device__ __forceinline__ float2 widen2<true>(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v)); }
template <bool BF16> __device__ __forceinline__ uint32_t narrow2(float a, float b);
template <> __device__ __forceinline__ uint32_t narrow2<false>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t narrow2<true>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
// 16 bytes = two self-validating 8-byte words; volatile: straight to / from L2
__device__ __forceinline__ void store_words(uint4* dst, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 load_words(const uint4* src) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
    return v;
}

// count is a multiple of 8 (16-byte pieces of the tensor); buf is 16-byte aligned
// PUSH = false: the producer kernel's epilogue has already stored this rank's words (same epoch)
template <bool BF16, bool PUSH>
__global__ void __launch_bounds__(AR_THREADS) lux_peer_allreduce_push(const PushParams p) {
    __shared__ int s_failed;
    const int tid = threadIdx.x;
    if (tid == 0) s_failed = 0;
    pdl_launch_dependents();
    // With PUSH the producer of buf must have finished.  Without, every word this kernel reads carries
    // its epoch and buf is only written: it may start polling while the producer still runs.
    if (PUSH || !p.early) pdl_wait();
    const uint32_t epoch = peer_ctl_load(p.ctl + PEER_CTL_EPOCH) + 1u;   // the same value in every CTA
    if (peer_ctl_load(p.ctl + PEER_CTL_FAILED)) {
        // an earlier call gave up: the ranks' epochs may differ, nothing can be trusted any more
        if (tid == 0 && blockIdx.x == 0 && p.status) atomicOr(p.status, 0x7C050005u);
        return;
    }
    __syncthreads();                                              // s_failed is initialised
    const int parity = (int)(epoch & 1u);
    const size_t pieces = (size_t)p.count / 8;                    // 16-byte pieces of the tensor
    const size_t stride = (size_t)gridDim.x * AR_THREADS;
    const size_t first = (size_t)blockIdx.x * AR_THREADS + tid;
    const uint4* src = reinterpret_cast<const uint4*>(p.buf);
    unsigned char* mine = p.peer[p.rank];
    const unsigned long long t0 = peer_timer_ns();

    // 1. push: piece i becomes four words = two 16-byte stores, into my slot of every window
    for (size_t i = first; PUSH && i < pieces; i += stride) {
        const uint4 v = src[i];
        const uint4 lo = make_uint4(v.x, epoch, v.y, epoch), hi = make_uint4(v.z, epoch, v.w, epoch);
#pragma unroll
        for (int r = 0; r < MAX_WORLD; r++) {
            if (r < p.world) {
                uint4* dst = reinterpret_cast<uint4*>(slot_ptr(p.peer[r], p.world, p.max_bytes, parity, p.rank)) + 2 * i;
                store_words(dst, lo);
                store_words(dst + 1, hi);
            }
        }
    }
    // 2. reduce: every source rank's words of a piece, all requested before any is tested
    bool failed = false;
    for (size_t i = first; i < pieces && !failed; i += stride) {
        uint4 lo[MAX_WORLD], hi[MAX_WORLD];
        for (uint32_t it = 1;; ++it) {
            bool all = true;
#pragma unroll
            for (int r = 0; r < MAX_WORLD; r++) {
                if (r < p.world) {
                    const uint4* w = reinterpret_cast<const uint4*>(slot_ptr(mine, p.world, p.max_bytes, parity, r)) + 2 * i;
                    lo[r] = load_words(w);
                    hi[r] = load_words(w + 1);
                }
            }
#pragma unroll
            for (int r = 0; r < MAX_WORLD; r++)
                if (r < p.world) all = all && lo[r].y == epoch && lo[r].w == epoch && hi[r].y == epoch && hi[r].w == epoch;
            if (all) break;
            if ((it & 15u) == 0u && (*(volatile int*)&s_failed || peer_timer_ns() - t0 > p.wait_ns)) { failed = true; break; }
            if (!PUSH && p.early) __nanosleep(200);          // beside a producer that still computes
        }
        if (failed) break;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < MAX_WORLD; r++) {
            if (r < p.world) {
                const uint32_t d[4] = {lo[r].x, lo[r].z, hi[r].x, hi[r].z};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = widen2<BF16>(d[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 o;
        o.x = narrow2<BF16>(acc[0], acc[1]);
        o.y = narrow2<BF16>(acc[2], acc[3]);
        o.z = narrow2<BF16>(acc[4], acc[5]);
        o.w = narrow2<BF16>(acc[6], acc[7]);
        reinterpret_cast<uint4*>(p.buf)[i] = o;
    }
    if (failed) atomicExch(&s_failed, 1);
    __syncthreads();
    if (tid == 0) peer_ctl_finish(p.ctl, PEER_CTL_DONE, gridDim.x, epoch, s_failed != 0, p.status);
}

PeerComm* as_comm(LuxPeerComm* c) { return reinterpret_cast<PeerComm*>(c); }

}  // namespace

const void* kernel_addr_peer_allreduce_push() { return (const void*)lux_peer_allreduce_push<false, true>; }

unsigned long long peer_wait_ns() {
    // peer_wait_limit is given in microseconds; the default bounds a whole call to one second
    return g_tune.peer_wait_limit > 0 ? (unsigned long long)g_tune.peer_wait_limit * 1000ull : 1000000000ull;
}

bool peer_comm_push_target(LuxPeerComm* comm, size_t count, int device, PushTarget* out) {
    PeerComm* c = reinterpret_cast<PeerComm*>(comm);
    if (!c || !out || c->world < 2 || !c->connected || c->device != device) return false;
    if (count == 0 || count % 8 || count * 2 > c->max_bytes) return false;
    for (int r = 0; r < MAX_WORLD; r++) out->peer[r] = r < c->world ? c->peer[r] : nullptr;
    out->ctl = c->ctl;
    out->wait_ns = peer_wait_ns();
    out->max_bytes = c->max_bytes;
    out->rank = c->rank;
    out->world = c->world;
    out->reduce_here = 1;
    return true;
}

LuxBackendError peer_allreduce_launch(Context* ctx, LuxPeerComm* comm, void* buf, size_t buf_bytes, size_t count,
                                      int dtype, bool push) {
    PeerComm* c = reinterpret_cast<PeerComm*>(comm);
    if (!ctx || !c || !buf || count == 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (dtype != LUX_QDTYPE_F16 && dtype != LUX_QDTYPE_BF16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (!c->connected && c->world > 1) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (count % 8 || (reinterpret_cast<uintptr_t>(buf) & 15)) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (count * 2 > c->max_bytes || count * 2 > buf_bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (ctx->device != c->device) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    PushParams p{};
    for (int r = 0; r < c->world; r++) p.peer[r] = c->peer[r];
    p.buf = buf;
    p.ctl = c->ctl;
    p.status = ctx->d_status;
    p.max_bytes = c->max_bytes;
    p.count = count;
    p.rank = c->rank;
    p.world = c->world;
    p.wait_ns = peer_wait_ns();
    p.early = !push && g_tune.tp_reduce_early == 1 ? 1 : 0;
    // one CTA per 4 KB of the tensor, at most one per SM: 16 KB (batch 1) takes 4 CTAs, 4 MB all SMs
    const size_t pieces = count / 8;
    const unsigned grid = (unsigned)std::min<size_t>((size_t)ctx->sm_count, (pieces + AR_THREADS - 1) / AR_THREADS);
    const bool pdl = g_tune.pdl != 2;          // reads no weight operand: the pending-writer mark does not concern it
    const bool bf16 = dtype == LUX_QDTYPE_BF16;
    auto kfn = push ? (bf16 ? lux_peer_allreduce_push<true, true> : lux_peer_allreduce_push<false, true>)
                    : (bf16 ? lux_peer_allreduce_push<true, false> : lux_peer_allreduce_push<false, false>);
    const cudaError_t le = launch_pdl(pdl, kfn, dim3(grid), dim3(AR_THREADS), 0, ctx->stream, 1, p);
    if (le != cudaSuccess) return map_cuda(le, "lux_peer_allreduce_push");
    count_launch("lux_peer_allreduce_push");
    return map_cuda(cudaGetLastError(), "lux_peer_allreduce_push");
}

}  // namespace luxcuda

using namespace luxcuda;

extern "C" {

LuxBackendError lux_cuda_peer_comm_create(LuxBackendContext* context, int rank, int world, size_t max_bytes,
                                          LuxPeerComm** out, void* handle_out) {
    Context* ctx = reinterpret_cast<Context*>(context);
    if (!ctx || !out || world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || max_bytes == 0)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    max_bytes = (max_bytes + 255) & ~(size_t)255;
    cudaSetDevice(ctx->device);
    PeerComm* c = new (std::nothrow) PeerComm();
    if (!c) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    c->device = ctx->device;
    c->rank = rank;
    c->world = world;
    c->max_bytes = max_bytes;
    const size_t bytes = window_alloc_bytes(world, max_bytes);
    if (cudaMalloc(&c->window, bytes) != cudaSuccess || cudaMalloc(&c->ctl, PEER_CTL_WORDS * sizeof(uint32_t)) != cudaSuccess) {
        if (c->window) cudaFree(c->window);
        delete c;
        (void)cudaGetLastError();
        return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    }
    cudaMemset(c->window, 0, bytes);
    cudaMemset(c->ctl, 0, PEER_CTL_WORDS * sizeof(uint32_t));
    const WindowTag tag{TAG_MAGIC, (uint32_t)rank, (uint32_t)world, (uint32_t)max_bytes};
    cudaMemcpy(c->window + tag_offset(world, max_bytes), &tag, sizeof tag, cudaMemcpyHostToDevice);
    cudaDeviceSynchronize();
    c->peer[rank] = c->window;
    if (handle_out) {
        static_assert(sizeof(cudaIpcMemHandle_t) == LUX_PEER_HANDLE_BYTES, "handle size");
        cudaIpcMemHandle_t h;
        std::memset(&h, 0, sizeof h);
        if (world > 1 && cudaIpcGetMemHandle(&h, c->window) != cudaSuccess) {
            // no IPC on this system: the caller can still connect with raw peer pointers
            (void)cudaGetLastError();
            std::memset(&h, 0, sizeof h);
        }
        std::memcpy(handle_out, &h, sizeof h);
    }
    *out = reinterpret_cast<LuxPeerComm*>(c);
    return LUX_BACKEND_OK;
}

LuxBackendError lux_cuda_peer_comm_connect(LuxPeerComm* comm, const void* handles) {
    PeerComm* c = as_comm(comm);
    if (!c || !handles) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(c->device);
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const unsigned char*)handles + (size_t)r * LUX_PEER_HANDLE_BYTES, sizeof h);
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            std::fprintf(stderr, "[lux-cuda] cudaIpcOpenMemHandle(rank %d): %s\n", r, cudaGetErrorString(e));
            return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        }
        c->peer[r] = (unsigned char*)ptr;
        c->opened[r] = true;
        // the mapping must really be rank r's window (same geometry, its tag where ours is)
        WindowTag tag{};
        e = cudaMemcpy(&tag, c->peer[r] + tag_offset(c->world, c->max_bytes), sizeof tag, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess || tag.magic != TAG_MAGIC || tag.rank != (uint32_t)r || tag.world != (uint32_t)c->world ||
            tag.max_bytes_lo != (uint32_t)c->max_bytes) {
            (void)cudaGetLastError();
            std::fprintf(stderr, "[lux-cuda] peer window of rank %d does not identify itself (mapping refused)\n", r);
            return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        }
    }
    c->connected = true;
    return LUX_BACKEND_OK;
}

LuxBackendError lux_cuda_peer_comm_connect_ptrs(LuxPeerComm* comm, void* const* windows) {
    PeerComm* c = as_comm(comm);
    if (!c || !windows) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) continue;
        if (!windows[r]) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        c->peer[r] = (unsigned char*)windows[r];
    }
    c->connected = true;
    return LUX_BACKEND_OK;
}

void* lux_cuda_peer_comm_window(LuxPeerComm* comm) { return comm ? as_comm(comm)->window : nullptr; }
size_t lux_cuda_peer_comm_window_bytes(LuxPeerComm* comm) {
    return comm ? window_bytes(as_comm(comm)->world, as_comm(comm)->max_bytes) : 0;
}

LuxBackendError lux_cuda_peer_allreduce(LuxBackendContext* context, LuxPeerComm* comm, LuxBackendBuffer* buffer,
                                        size_t count, LuxQDType dtype, uint32_t flags) {
    Context* ctx = reinterpret_cast<Context*>(context);
    Buffer* b = reinterpret_cast<Buffer*>(buffer);
    if (!ctx || !comm || !b || !b->ptr) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    std::lock_guard<std::mutex> lock(ctx->mu);
    LuxBackendError e = peer_allreduce_launch(ctx, comm, b->ptr, b->size, count, (int)dtype, true);
    if (e != LUX_BACKEND_OK) return e;
    return finish_op(ctx, (flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, "lux_cuda_peer_allreduce");
}

void lux_cuda_peer_comm_destroy(LuxPeerComm* comm) {
    PeerComm* c = as_comm(comm);
    if (!c) return;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; r++)
        if (c->opened[r] && c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
    if (c->window) cudaFree(c->window);
    if (c->ctl) cudaFree(c->ctl);
    (void)cudaGetLastError();
    delete c;
}

}  // extern "C"
