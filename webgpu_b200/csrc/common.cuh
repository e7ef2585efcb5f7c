// Shared declarations of libluxgpu_backend_cuda.so: the context and buffer structs
// behind the opaque LuxBackend* handles, error mapping and launch bookkeeping.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <utility>

#include "lux/gpu/backend_plugin.h"
#include "lux/gpu/qmatmul_ext.h"

namespace luxcuda {

// Counterpart of WGPUBackendBuffer{buffer,size} (luxcpp/webgpu src/webgpu_plugin.cpp:516-519).
struct Buffer {
    void*  ptr;
    size_t size;
    int    device;
    bool   owned;    // false for lux_cuda_buffer_wrap handles
};

// Counterpart of WGPUBackendContext (src/webgpu_plugin.cpp:584-622): one device, one
// queue.  The reference keeps a 256-byte uniform buffer per context for kernel
// parameters; CUDA passes parameters by value, so the per-context device state here is
// the status word for bounded device-side waits and the staging used by host-pointer ops.
struct Context {
    int            device = 0;
    cudaStream_t   own_stream = nullptr;
    cudaStream_t   stream = nullptr;        // own_stream unless lux_cuda_context_set_stream
    cudaDeviceProp prop{};
    std::string    name;
    uint32_t*      d_status = nullptr;      // device status word (0 = ok)
    uint32_t*      h_status = nullptr;      // pinned mirror
    void*          h_stage = nullptr;       // pinned staging for host-pointer ops
    void*          d_stage_y = nullptr;     // the same buffer as the device sees it (null: not mapped)
    size_t         h_stage_bytes = 0;
    void*          d_stage = nullptr;       // device staging for host-pointer ops
    size_t         d_stage_bytes = 0;
    uint32_t       last_status = 0;
    uint32_t*      d_absmax = nullptr;      // device word for lux_cuda_dynamic_quantize's tensor-wide max (allocated with the context)
    void*          d_splitk = nullptr;      // split-K exchange of the weights-in-TMEM GEMM: 128 KB per CTA pair,
    size_t         d_splitk_bytes = 0;      // allocated with the context (no entry point allocates for it)
    void*          d_int = nullptr;         // lux_cuda_matmul_int8 on the tcgen05 path: B transposed (and A unpacked), grown on demand
    size_t         d_int_bytes = 0;
    void*          d_attn = nullptr;        // partial results of attention calls that split the keys over CTAs:
    size_t         d_attn_bytes = 0;        // 16 MB, allocated with the context (a call takes fewer slices rather than allocate)
    std::mutex     mu;                      // guards the staging buffers
    int            sm_count = 148;
    // A kernel of this library that WRITES a buffer a later matmul may bind as weights, scales or
    // zero-points (unpack, dequantize, quantize) has been enqueued without a wait.  The next matmul
    // is then launched without the programmatic-launch attribute, because its prologue reads those
    // operands before griddepcontrol.wait (see launch_pdl below).
    bool           writer_pending = false;
};

inline Context* as_ctx(LuxBackendContext* c) { return reinterpret_cast<Context*>(c); }
inline Buffer*  as_buf(LuxBackendBuffer* b) { return reinterpret_cast<Buffer*>(b); }

extern std::atomic<uint64_t> g_launches;
extern std::atomic<const char*> g_last_kernel;
inline void count_launch(unsigned n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
// counts one launch and remembers which kernel it was (a string literal)
inline void count_launch(const char* kernel) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    g_last_kernel.store(kernel, std::memory_order_relaxed);
}

// Maps a CUDA error to the plugin's error vocabulary, logging in the reference's
// stderr style ("[lux-webgpu] ...", src/webgpu_plugin.cpp:695).
inline LuxBackendError map_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return LUX_BACKEND_OK;
    std::fprintf(stderr, "[lux-cuda] %s: %s\n", what, cudaGetErrorString(e));
    if (e == cudaErrorMemoryAllocation) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    if (e == cudaErrorInvalidValue || e == cudaErrorInvalidDevice) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    return LUX_BACKEND_ERROR_INTERNAL;
}

#define LUX_CUDA_TRY(expr)                                                   \
    do {                                                                     \
        cudaError_t _e = (expr);                                             \
        if (_e != cudaSuccess) return ::luxcuda::map_cuda(_e, #expr);        \
    } while (0)

// Checks the launch, and unless `no_sync` waits for the stream like the reference's
// dispatchCompute does (src/webgpu_plugin.cpp:1028-1050).
LuxBackendError finish_op(Context* ctx, bool no_sync, const char* what);

// Tunables a benchmark may override (0 = use the built-in heuristic).
struct Tunables {
    int gemv_i4_warps = 0;       // warps per CTA of the int4 skinny kernel
    int gemv_i4_row_tiles = 0;   // 16-row tiles per CTA
    int gemv_i8_warps = 0;
    int tp_reduce_early = 0;     // reduce-only all-reduce kernel: 1 = poll without waiting for the producer kernel to end
    int tp_fused_push = 0;       // lux_cuda_qmlp_tp at batch <= 2: 0 the down kernel pushes and a reduce-only kernel follows;
                                 // 1 the down kernel pushes, waits and sums itself; 2 separate all-reduce kernel
    int peer_wait_limit = 0;     // push all-reduce: microseconds before a call's wait for its peers gives up (default 10^6)
    int gemv_i8_kernel = 0;      // 0 auto, 1 lux_qgemv_i8_g32_f32, 2 lux_qgemv_i8_g32_units_fx
    int gemv_i4_kernel = 0;      // 0 auto, 1 lux_qskinny_i4_g128, 2 lux_qgemv_i4_g128_stream, 3 lux_qgemv_i4_g128_units
    int gemv_stream_cg = 0;      // stream kernel: groups per stage / 8 (1, 2 or 4)
    int gemv_stream_stages = 0;  // stream kernel: ring depth cap
    int gemv_stream_warps = 0;   // stream kernel: consumer warps (8 or 16)
    int gemv_units_ks = 0;       // units kernel: groups per unit (a multiple of the chunk that divides K/128)
    int gemv_units_stages = 0;   // units kernel: cap on the FIFO depth per warp (chunks)
    int gemv_units_cg = 0;       // units kernel: groups per chunk (2 or 4)
    int gemv_units_pre = 0;      // units kernel: chunks requested per warp before its loop starts (default 1)
    int gemv_units_fx = 0;       // units kernel, batch <= 2: 0/1 block-fixed-point int8 variant, 2 f16 variant
    int gemv_units_warps = 0;    // fixed-point units kernels: 8 half-SM CTAs (where the plan fits), 0/16 whole-SM CTAs
    int host_pageable = 0;       // host-pointer entry point: 0/1 hand x_host to the copy as it is (<= 64 KB), 2 stage it in pinned memory
    int gemv_units_planes = 0;   // fixed-point units kernels: byte planes of the activations, 3 or 4 (0 = 4 where it costs no FIFO depth)
    int gemm_tc_bn = 0;          // N tile of the tcgen05 GEMM
    int gemm_tc_stages = 0;
    int gemm_tc_splitk = 0;      // weights-in-TMEM GEMM: K splits over a CTA cluster, 1, 2 or 4 (0 = choose)
    int gemm_tc_groups = 0;      // weights-in-TMEM GEMM: converter groups of four warps, 2..4
    int pdl = 0;                 // programmatic dependent launch of the persistent kernels: 0/1 on, 2 off
    int gemm_min_m = 0;          // smallest batch the weights-in-TMEM GEMM takes from the streaming kernels (0 = built-in)
    int gemm_tc_kernel = 0;      // 0 auto, 1 lux_qgemm_i4_tc, 2 lux_qgemm_i4_tc_wa wherever it applies
    int int_matmul_kernel = 0;   // lux_cuda_matmul_int8 / _int4_int8: 0 tcgen05 for large shapes, 1 mma.sync kernels only, 2 tcgen05 always through B^T
    int attn_splits = 0;         // attention: slices of the keys per (sequence, KV head, row block); 0 = choose
    int gemm_wa_narrow = 0;      // weights-in-TMEM GEMM, batch <= 64: 0 narrow tile (two CTAs per SM) when the launch has more CTAs
                                 // than SMs, 1 always, 2 never
    int gemm_wa_prefetch = 0;    // weights-in-TMEM GEMM: L2 prefetch distance of the weight rows in 128-K units (0 = 2, -1 = off)
    int gemm_tc_ma = 0;          // GEMM: batch tiles (128 rows) per CTA, 1 or 2 (0 = choose)
};
extern Tunables g_tune;

// ---- programmatic dependent launch --------------------------------------------------------
// The persistent GEMV kernels and the weights-in-TMEM GEMM are launched with the programmatic
// stream serialization attribute: the grid may be set up while the previous kernel of the stream
// is still running, so that its CTAs start the moment SMs free up instead of one launch latency
// after the previous grid has drained.  Each of these kernels
//   * calls pdl_launch_dependents() first (the next such kernel may be set up behind it), and
//   * touches only static model state (weights, scales, zero-points) until pdl_wait(), which
//     returns when every earlier kernel of the stream has completed and its writes are visible;
//     activations are read, and anything is written, only after it.
// In a kernel launched without the attribute both calls do nothing.
#ifdef __CUDACC__

// Named barriers with the barrier number as an immediate (a number held in a register makes the
// compiler reserve all sixteen of the CTA's barriers).  `base` + `i`, i in 0..7.
#ifdef __CUDACC__
template <int ID> __device__ __forceinline__ void named_bar_sync_c(uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(threads) : "memory");
}
template <int ID> __device__ __forceinline__ void named_bar_arrive_c(uint32_t threads) {
    asm volatile("bar.arrive %0, %1;" ::"n"(ID), "r"(threads) : "memory");
}
template <int BASE> __device__ __forceinline__ void named_bar_sync(uint32_t i, uint32_t threads) {
    switch (i) {
        case 0: named_bar_sync_c<BASE + 0>(threads); break;
        case 1: named_bar_sync_c<BASE + 1>(threads); break;
        case 2: named_bar_sync_c<BASE + 2>(threads); break;
        case 3: named_bar_sync_c<BASE + 3>(threads); break;
        case 4: named_bar_sync_c<BASE + 4>(threads); break;
        default: named_bar_sync_c<BASE + 5>(threads); break;
    }
}
template <int BASE> __device__ __forceinline__ void named_bar_arrive(uint32_t i, uint32_t threads) {
    switch (i) {
        case 0: named_bar_arrive_c<BASE + 0>(threads); break;
        case 1: named_bar_arrive_c<BASE + 1>(threads); break;
        case 2: named_bar_arrive_c<BASE + 2>(threads); break;
        case 3: named_bar_arrive_c<BASE + 3>(threads); break;
        case 4: named_bar_arrive_c<BASE + 4>(threads); break;
        default: named_bar_arrive_c<BASE + 5>(threads); break;
    }
}
#endif

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

//
// Contract for the operands read before pdl_wait(): weights, scales and zero-points must be complete
// when the call is enqueued -- or the call carries LUX_QMATMUL_FLAG_WEIGHTS_VOLATILE, or the tunable
// pdl = 2 is set.  Where the library can see the hazard itself (one of its own writer kernels is
// pending on the context) it drops the attribute for the next launch on its own: pdl_allowed().
struct Context;
inline bool pdl_allowed(Context* ctx, bool weights_volatile);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(bool allow, void (*kfn)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              unsigned cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_z;
        n++;
    }
    if (allow) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kfn, std::forward<Args>(args)...);
}
#endif

// ---- kernel launchers (defined in the .cu file named after each kernel family) ------
LuxBackendError launch_matmul_int8_tcgen05(Context* ctx, const void* a, const void* b, int* c, int M, int N, int K, bool a_int4);

// Where a kernel's epilogue pushes its 16-bit outputs for the push all-reduce (allreduce_push.cu):
// every rank's window, this rank's number, the communicator's epoch counter.  world <= 1: no push.
struct PushTarget {
    unsigned char* peer[8];
    uint32_t* ctl;                  // the communicator's control words in device memory (PEER_CTL_*)
    unsigned long long max_bytes;
    unsigned long long wait_ns;     // deadline of a wait for the peers' words
    int rank, world;
    int reduce_here;                // 1: the producer kernel also waits for the peers and writes the sum;
                                    // 0: it only pushes, and a reduce-only all-reduce kernel follows
};
// control words of a push communicator
enum { PEER_CTL_EPOCH = 0,          // number of completed reductions
       PEER_CTL_DONE = 1,           // CTAs of the all-reduce kernel that have finished the current one
       PEER_CTL_FAILED = 2,         // a wait gave up: sticky, every later call returns at once
       PEER_CTL_DONE_FUSED = 3,     // the same count for a producer kernel that reduces in its epilogue
       PEER_CTL_WORDS = 4 };
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t peer_ctl_load(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// The waits are bounded on the SM's own cycle counter: a register read, unlike the global
// nanosecond timer, whose reads from tens of thousands of threads at once queue up for microseconds.
// The bound is given in nanoseconds and counted at 2 cycles per nanosecond (the SM clock runs at
// 1.3-2 GHz, so "one second" is 1 to 1.5 s: it is a safety limit, not a measurement).
__device__ __forceinline__ unsigned long long peer_timer_ns() { return (unsigned long long)clock64() >> 1; }
// One thread per CTA, after the CTA's part of a reduction: records a failure, and the last CTA of
// the grid to arrive advances the epoch (only while the communicator is intact) and re-arms the count.
__device__ __forceinline__ void peer_ctl_finish(uint32_t* ctl, int done_word, unsigned ctas, uint32_t epoch, bool failed,
                                                uint32_t* status) {
    if (failed) {
        atomicExch(ctl + PEER_CTL_FAILED, 1u);
        if (status) atomicOr(status, 0x7C050005u);
    }
    __threadfence();
    if (atomicAdd(ctl + done_word, 1u) == ctas - 1u) {
        atomicExch(ctl + done_word, 0u);
        if (peer_ctl_load(ctl + PEER_CTL_FAILED) == 0u) atomicExch(ctl + PEER_CTL_EPOCH, epoch);
        __threadfence();
    }
}
#endif

struct QArgs {
    int M, N, K, G;              // G = K / group
    const void* x;
    const uint8_t* w;
    const void* scales;
    const uint8_t* zeros;        // may be null
    void* y;
    int x_dtype, scale_dtype, y_dtype;
    bool swiglu;
    const PushTarget* push = nullptr;   // set: push the outputs into the peers' windows instead of writing y
    bool weights_volatile = false;      // LUX_QMATMUL_FLAG_WEIGHTS_VOLATILE: w / scales / zeros may still be being written
};

// Whether the next matmul launch on `ctx` may carry the programmatic-launch attribute.  A launch
// without it waits for everything before it on the stream, so it also clears the pending-writer mark.
inline bool pdl_allowed(Context* ctx, bool weights_volatile) {
    if (weights_volatile || ctx->writer_pending) {
        ctx->writer_pending = false;
        return false;
    }
    return g_tune.pdl != 2;
}

// allreduce_push.cu: the push target of a connected communicator (false if it cannot take `count`
// 16-bit elements), and the all-reduce launch with or without its own push phase
bool peer_comm_push_target(LuxPeerComm* comm, size_t count, int device, PushTarget* out);
LuxBackendError peer_allreduce_launch(Context* ctx, LuxPeerComm* comm, void* buf, size_t buf_bytes, size_t count,
                                      int dtype, bool push);

LuxBackendError launch_qgemv_i8(Context* ctx, const QArgs& a);
LuxBackendError launch_qgemv_i8_units(Context* ctx, const QArgs& a);    // NOT_SUPPORTED if the shape does not fit
LuxBackendError launch_qskinny_i4(Context* ctx, const QArgs& a);
LuxBackendError launch_qgemv_i4_stream(Context* ctx, const QArgs& a);   // NOT_SUPPORTED if the shape does not fit
LuxBackendError launch_qgemv_i4_units(Context* ctx, const QArgs& a);    // NOT_SUPPORTED if the shape does not fit
LuxBackendError launch_qgemm_i4_tc(Context* ctx, const QArgs& a);
LuxBackendError launch_qgemm_i4_tc_wa(Context* ctx, const QArgs& a);    // NOT_SUPPORTED if the shape does not fit
LuxBackendError launch_qdequant(Context* ctx, const QArgs& a, int bits);

// tensor_ops.cu: the f32 slots the reference's shader library backs but its plugin leaves unwired
LuxBackendError op_div_f32(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n);
LuxBackendError op_transpose_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, int rows, int cols);
LuxBackendError op_softmax_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim);
LuxBackendError op_log_softmax_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim);
LuxBackendError op_exp_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_log_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_sqrt_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_neg_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_abs_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_tanh_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_sigmoid_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_relu_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_gelu_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_copy_f32(LuxBackendContext*, LuxBackendBuffer* src, LuxBackendBuffer* dst, size_t n);
LuxBackendError op_silu_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
LuxBackendError op_layer_norm_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* gamma, LuxBackendBuffer* beta,
                                  LuxBackendBuffer* out, size_t batch, size_t dim, float eps);
LuxBackendError op_rms_norm_f32(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* weight, LuxBackendBuffer* out,
                                size_t batch, size_t dim, float eps);
LuxBackendError launch_qunpack(Context* ctx, const QArgs& a, int bits);

// Encodes a tiled uint8 tensor map (CUtensorMap, 128 bytes, 64-byte aligned) through the
// driver entry point; dims/box innermost first, strides_bytes for dimensions 1..rank-1.
bool encode_tensor_map_u8(void* map, int rank, const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                          const uint32_t* box, bool swizzle128);

}  // namespace luxcuda
