// libluxgpu_backend_cuda.so -- plugin entry, context, buffers and the f32 tensor slots.
//
// Exports lux_gpu_backend_init with the same descriptor + 65-slot vtable shape that
// luxcpp/webgpu's src/webgpu_plugin.cpp:4022-4154 fills, so luxcpp/gpu's loader can
// dlopen this file in place of libluxgpu_backend_webgpu.so.  WebGPU instance/adapter/
// device/queue become a CUDA device + stream; WGPUBuffer becomes cudaMalloc memory;
// runtime WGSL compilation disappears (kernels are precompiled for sm_100a).
#include "common.cuh"

#include <algorithm>
#include <cstring>
#include <new>

namespace luxcuda {

std::atomic<uint64_t> g_launches{0};
std::atomic<const char*> g_last_kernel{""};
Tunables g_tune;

LuxBackendError finish_op(Context* ctx, bool no_sync, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return map_cuda(e, what);
    if (no_sync) return LUX_BACKEND_OK;
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        std::fprintf(stderr, "[lux-cuda] %s: %s\n", what, cudaGetErrorString(e));
        // The reference reports a wait that never completes as DEVICE_LOST
        // (src/webgpu_plugin.cpp:1046-1048); a failed stream wait is the CUDA analogue.
        return LUX_BACKEND_ERROR_DEVICE_LOST;
    }
    ctx->writer_pending = false;             // everything enqueued so far has completed
    if (ctx->h_status && *(volatile uint32_t*)ctx->h_status != 0) {
        ctx->last_status = *(volatile uint32_t*)ctx->h_status;
        *(volatile uint32_t*)ctx->h_status = 0;
        return LUX_BACKEND_ERROR_DEVICE_LOST;
    }
    ctx->last_status = 0;                    // what lux_cuda_last_device_status reports belongs to the latest wait
    return LUX_BACKEND_OK;
}

// ---------------------------------------------------------------------------------
// f32 kernels behind the four wired tensor slots (reference: inline WGSL at
// src/webgpu_plugin.cpp:92-205).  Thin by design; not the hot path.
// ---------------------------------------------------------------------------------

enum BinOp { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2 };

template <int OP>
__global__ void lux_binary_f32(const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float x = a[i], y = b[i];
        out[i] = OP == OP_ADD ? x + y : (OP == OP_SUB ? x - y : x * y);
    }
}

// out[M,N] = a[M,K] . b[K,N], row-major, 32x32 tiles, f32 accumulate in ascending k.
__global__ void lux_matmul_f32(const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ out, int M, int K, int N) {
    __shared__ float ta[32][33];
    __shared__ float tb[32][33];
    int row = blockIdx.y * 32 + threadIdx.y;
    int col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        int ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        ta[threadIdx.y][threadIdx.x] = (row < M && ka < K) ? a[(size_t)row * K + ka] : 0.0f;
        tb[threadIdx.y][threadIdx.x] = (kb < K && col < N) ? b[(size_t)kb * N + col] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; k++) acc += ta[threadIdx.y][k] * tb[k][threadIdx.x];
        __syncthreads();
    }
    if (row < M && col < N) out[(size_t)row * N + col] = acc;
}

}  // namespace luxcuda

using namespace luxcuda;

// ---------------------------------------------------------------------------------
// Lifecycle (src/webgpu_plugin.cpp:1218-1353)
// ---------------------------------------------------------------------------------

static LuxBackendContext* cuda_create_context(int device_index) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device_index < 0 || device_index >= count) {
        cudaGetLastError();
        return nullptr;
    }
    if (cudaSetDevice(device_index) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    auto* ctx = new (std::nothrow) Context();
    if (!ctx) return nullptr;
    ctx->device = device_index;
    bool ok = cudaGetDeviceProperties(&ctx->prop, device_index) == cudaSuccess;
    // This library carries sm_100a code only; refuse other devices instead of failing
    // at the first launch.
    ok = ok && ctx->prop.major == 10;
    ok = ok && cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) == cudaSuccess;
    // The status word lives in pinned host memory that the device can write: a kernel
    // whose bounded wait gives up stores a code there, and the host reads it after the
    // stream wait without another copy.
    ok = ok && cudaHostAlloc(&ctx->h_status, sizeof(uint32_t), cudaHostAllocMapped) == cudaSuccess;
    ok = ok && cudaHostGetDevicePointer((void**)&ctx->d_status, ctx->h_status, 0) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->d_absmax, sizeof(uint32_t)) == cudaSuccess;
    // Split-K partial sums of the tensor-core GEMM: one 128 KB slot per CTA pair, at most one pair
    // per two SMs.  Allocated here so that no matmul entry point ever allocates device memory.
    if (ok) {
        // two K splits: 128 KB per pair, a pair per two SMs; four: 384 KB per quartet, one per four SMs
        ctx->d_splitk_bytes = std::max((size_t)(ctx->prop.multiProcessorCount / 2) * (128u << 10),
                                       (size_t)(ctx->prop.multiProcessorCount / 4) * (384u << 10));
        ok = cudaMalloc(&ctx->d_splitk, ctx->d_splitk_bytes) == cudaSuccess;
    }
    if (ok) {
        ctx->d_attn_bytes = 16u << 20;
        ok = cudaMalloc(&ctx->d_attn, ctx->d_attn_bytes) == cudaSuccess;
    }
    if (!ok) {
        cudaGetLastError();
        if (ctx->d_attn) cudaFree(ctx->d_attn);
        if (ctx->d_splitk) cudaFree(ctx->d_splitk);
        if (ctx->d_absmax) cudaFree(ctx->d_absmax);
        if (ctx->h_status) cudaFreeHost(ctx->h_status);
        if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return nullptr;
    }
    *ctx->h_status = 0;
    ctx->stream = ctx->own_stream;
    ctx->name = ctx->prop.name;
    ctx->sm_count = ctx->prop.multiProcessorCount;
    return reinterpret_cast<LuxBackendContext*>(ctx);
}

static void cuda_destroy_context(LuxBackendContext* context) {
    auto* ctx = as_ctx(context);
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    if (ctx->d_stage) cudaFree(ctx->d_stage);
    if (ctx->d_int) cudaFree(ctx->d_int);
    if (ctx->d_attn) cudaFree(ctx->d_attn);
    if (ctx->d_splitk) cudaFree(ctx->d_splitk);
    if (ctx->d_absmax) cudaFree(ctx->d_absmax);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    cudaGetLastError();
    delete ctx;
}

// ---------------------------------------------------------------------------------
// Device info & sync (src/webgpu_plugin.cpp:1359-1430)
// ---------------------------------------------------------------------------------

static LuxBackendError cuda_get_device_count(int* count) {
    if (!count) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
    *count = n;
    return LUX_BACKEND_OK;
}

static LuxBackendError cuda_get_device_info(LuxBackendContext* context, LuxBackendDeviceInfo* info) {
    if (!info) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    auto* ctx = as_ctx(context);
    if (!ctx) return LUX_BACKEND_ERROR_INTERNAL;      // same split as the reference (:1370-1373)
    size_t free_b = 0, total_b = 0;
    cudaSetDevice(ctx->device);
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) {
        cudaGetLastError();
        total_b = ctx->prop.totalGlobalMem;
        free_b = total_b;
    }
    info->name = ctx->name.c_str();
    info->vendor = "NVIDIA";
    info->memory_total = total_b;
    info->memory_available = free_b;
    info->compute_units = ctx->prop.multiProcessorCount;
    info->max_workgroup_size = ctx->prop.maxThreadsPerBlock;
    info->is_discrete = true;
    info->is_unified_memory = false;
    return LUX_BACKEND_OK;
}

static LuxBackendError cuda_sync(LuxBackendContext* context) {
    auto* ctx = as_ctx(context);
    if (!ctx) return LUX_BACKEND_ERROR_INTERNAL;
    cudaSetDevice(ctx->device);
    return finish_op(ctx, false, "sync");
}

// ---------------------------------------------------------------------------------
// Buffers (src/webgpu_plugin.cpp:1432-1566)
// ---------------------------------------------------------------------------------

static LuxBackendBuffer* cuda_buffer_alloc(LuxBackendContext* context, size_t bytes) {
    auto* ctx = as_ctx(context);
    if (!ctx) return nullptr;
    cudaSetDevice(ctx->device);
    auto* buf = new (std::nothrow) Buffer{nullptr, bytes, ctx->device, true};
    if (!buf) return nullptr;
    // A zero-size WGPUBuffer is legal; keep a valid handle with a 1-byte allocation.
    if (cudaMalloc(&buf->ptr, bytes ? bytes : 1) != cudaSuccess) {
        cudaGetLastError();
        delete buf;
        return nullptr;
    }
    return reinterpret_cast<LuxBackendBuffer*>(buf);
}

static LuxBackendBuffer* cuda_buffer_alloc_with_data(LuxBackendContext* context, const void* data, size_t bytes) {
    auto* ctx = as_ctx(context);
    if (!ctx) return nullptr;
    LuxBackendBuffer* h = cuda_buffer_alloc(context, bytes);
    if (!h) return nullptr;
    if (data && bytes) {
        auto* buf = as_buf(h);
        cudaError_t e = cudaMemcpyAsync(buf->ptr, data, bytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            cudaGetLastError();
            cudaFree(buf->ptr);
            delete buf;
            return nullptr;
        }
    }
    return h;
}

static void cuda_buffer_free(LuxBackendContext*, LuxBackendBuffer* buffer) {
    auto* buf = as_buf(buffer);
    if (!buf) return;
    if (buf->owned && buf->ptr) {
        cudaSetDevice(buf->device);
        cudaFree(buf->ptr);
        cudaGetLastError();
    }
    delete buf;
}

static LuxBackendError cuda_buffer_copy_to_host(LuxBackendContext* context, LuxBackendBuffer* buffer, void* dst, size_t bytes) {
    auto* ctx = as_ctx(context);
    auto* buf = as_buf(buffer);
    if (!ctx || !buf || !dst) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    size_t n = std::min(bytes, buf->size);                 // clamp as the reference does (:1495)
    if (n == 0) return finish_op(ctx, false, "buffer_copy_to_host");
    LUX_CUDA_TRY(cudaMemcpyAsync(dst, buf->ptr, n, cudaMemcpyDeviceToHost, ctx->stream));
    return finish_op(ctx, false, "buffer_copy_to_host");
}

static LuxBackendError cuda_buffer_copy_from_host(LuxBackendContext* context, LuxBackendBuffer* buffer, const void* src, size_t bytes) {
    auto* ctx = as_ctx(context);
    auto* buf = as_buf(buffer);
    if (!ctx || !buf || !src) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    size_t n = std::min(bytes, buf->size);                 // clamp (:1553)
    if (n == 0) return LUX_BACKEND_OK;
    LUX_CUDA_TRY(cudaMemcpyAsync(buf->ptr, src, n, cudaMemcpyHostToDevice, ctx->stream));
    // wgpuQueueWriteBuffer snapshots the source before returning; waiting here gives
    // the caller the same freedom to reuse `src` immediately.
    return finish_op(ctx, false, "buffer_copy_from_host");
}

static void* cuda_buffer_get_host_ptr(LuxBackendContext*, LuxBackendBuffer*) {
    return nullptr;    // discrete memory: no host mapping, as in the reference (:1564-1566)
}

// ---------------------------------------------------------------------------------
// f32 tensor slots (src/webgpu_plugin.cpp:1647-1771)
// ---------------------------------------------------------------------------------

template <int OP>
static LuxBackendError binary_op(LuxBackendContext* context, LuxBackendBuffer* a, LuxBackendBuffer* b,
                                 LuxBackendBuffer* out, size_t n) {
    auto* ctx = as_ctx(context);
    auto *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
    if (!ctx || !ba || !bb || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (ba->size < n * 4 || bb->size < n * 4 || bo->size < n * 4) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    cudaSetDevice(ctx->device);
    size_t blocks = std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
    lux_binary_f32<OP><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
        (const float*)ba->ptr, (const float*)bb->ptr, (float*)bo->ptr, n);
    count_launch();
    return finish_op(ctx, false, "binary_f32");
}

static LuxBackendError cuda_op_add_f32(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary_op<OP_ADD>(c, a, b, o, n); }
static LuxBackendError cuda_op_sub_f32(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary_op<OP_SUB>(c, a, b, o, n); }
static LuxBackendError cuda_op_mul_f32(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary_op<OP_MUL>(c, a, b, o, n); }

static LuxBackendError cuda_op_matmul_f32(LuxBackendContext* context, LuxBackendBuffer* a, LuxBackendBuffer* b,
                                          LuxBackendBuffer* out, int M, int K, int N) {
    auto* ctx = as_ctx(context);
    auto *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
    if (!ctx || !ba || !bb || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (M <= 0 || K <= 0 || N <= 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (ba->size < (size_t)M * K * 4 || bb->size < (size_t)K * N * 4 || bo->size < (size_t)M * N * 4)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    dim3 grid((N + 31) / 32, (M + 31) / 32), block(32, 32);
    lux_matmul_f32<<<grid, block, 0, ctx->stream>>>((const float*)ba->ptr, (const float*)bb->ptr, (float*)bo->ptr, M, K, N);
    count_launch();
    return finish_op(ctx, false, "matmul_f32");
}

// ---------------------------------------------------------------------------------
// Slots outside this backend's scope.  The reference's own convention for "not here,
// fall back to the CPU" is LUX_BACKEND_ERROR_NOT_SUPPORTED
// (src/webgpu_plugin.cpp:2087-2092, 3596-3602).
// ---------------------------------------------------------------------------------
#define NS return LUX_BACKEND_ERROR_NOT_SUPPORTED
static LuxBackendError ns_ntt(LuxBackendContext*, uint64_t*, size_t, uint64_t) { NS; }
static LuxBackendError ns_poly_mul(LuxBackendContext*, const uint64_t*, const uint64_t*, uint64_t*, size_t, uint64_t) { NS; }
static LuxBackendError ns_bootstrap(LuxBackendContext*, const uint64_t*, uint64_t*, const uint64_t*, const uint64_t*, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint64_t) { NS; }
static LuxBackendError ns_keyswitch(LuxBackendContext*, const uint64_t*, uint64_t*, const uint64_t*, uint32_t, uint32_t, uint32_t, uint32_t, uint64_t) { NS; }
static LuxBackendError ns_blind_rotate(LuxBackendContext*, uint64_t*, const uint64_t*, const uint64_t*, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint64_t) { NS; }
static LuxBackendError ns_poseidon2(LuxBackendContext*, const uint64_t*, uint64_t*, size_t, size_t) { NS; }
static LuxBackendError ns_hash(LuxBackendContext*, const uint8_t*, uint8_t*, const size_t*, size_t) { NS; }
static LuxBackendError ns_curve(LuxBackendContext*, const void*, const void*, void*, size_t, bool) { NS; }
static LuxBackendError ns_pairing(LuxBackendContext*, const void*, const void*, void*, size_t) { NS; }
static LuxBackendError ns_msm(LuxBackendContext*, const void*, const void*, void*, size_t, int) { NS; }
static LuxBackendError ns_kzg_commit(LuxBackendContext*, const void*, const void*, void*, size_t, int) { NS; }
static LuxBackendError ns_kzg_open(LuxBackendContext*, const void*, const void*, const void*, void*, size_t, int) { NS; }
static LuxBackendError ns_kzg_verify(LuxBackendContext*, const void*, const void*, const void*, const void*, const void*, bool*, int) { NS; }
static LuxBackendError ns_ecrecover(LuxBackendContext*, const void*, void*, size_t) { NS; }
// post-quantum, threshold and Schnorr batches: callable stubs in the reference too (:3973-4016)
static LuxBackendError ns_verify3(LuxBackendContext*, const uint8_t* const*, const uint8_t* const*, const uint8_t* const*, bool*, size_t) { NS; }
static LuxBackendError ns_batch2_out(LuxBackendContext*, const uint8_t* const*, const uint8_t* const*, uint8_t**, size_t) { NS; }
static LuxBackendError ns_ringtail_combine(LuxBackendContext*, const uint8_t* const*, const int32_t*, uint8_t**, size_t, size_t) { NS; }
static LuxBackendError ns_frost_verify(LuxBackendContext*, const uint8_t* const*, const uint8_t* const*, const uint8_t* const*, const uint8_t* const*, bool*, size_t) { NS; }
static LuxBackendError ns_cggmp21_sign(LuxBackendContext*, const uint8_t* const*, const uint8_t*, uint8_t**, size_t) { NS; }
#undef NS

// ---------------------------------------------------------------------------------
// Vtable, in the reference's slot order (src/webgpu_plugin.cpp:4022-4123)
// ---------------------------------------------------------------------------------
// The f32 slots the WebGPU plugin leaves nullptr: wired here with this reconstruction's signatures
// (see backend_plugin.h), or left nullptr like the reference with -DLUX_CUDA_F32_SLOTS_NULL.
#ifdef LUX_CUDA_F32_SLOTS_NULL
#define LUX_F32_SLOT(fn) nullptr
#else
#define LUX_F32_SLOT(fn) luxcuda::fn
#endif
static const lux_gpu_backend_vtbl cuda_vtbl = {
    .create_context  = cuda_create_context,
    .destroy_context = cuda_destroy_context,

    .get_device_count = cuda_get_device_count,
    .get_device_info  = cuda_get_device_info,
    .sync             = cuda_sync,

    .buffer_alloc           = cuda_buffer_alloc,
    .buffer_alloc_with_data = cuda_buffer_alloc_with_data,
    .buffer_free            = cuda_buffer_free,
    .buffer_copy_to_host    = cuda_buffer_copy_to_host,
    .buffer_copy_from_host  = cuda_buffer_copy_from_host,
    .buffer_get_host_ptr    = cuda_buffer_get_host_ptr,

    .op_add_f32 = cuda_op_add_f32,
    .op_sub_f32 = cuda_op_sub_f32,
    .op_mul_f32 = cuda_op_mul_f32,
    .op_div_f32 = LUX_F32_SLOT(op_div_f32),

    .op_matmul_f32    = cuda_op_matmul_f32,
    .op_transpose_f32 = LUX_F32_SLOT(op_transpose_f32),

    .op_reduce_sum_f32      = nullptr,
    .op_reduce_max_f32      = nullptr,
    .op_reduce_min_f32      = nullptr,
    .op_reduce_mean_f32     = nullptr,
    .op_reduce_sum_axis_f32 = nullptr,
    .op_reduce_max_axis_f32 = nullptr,

    .op_softmax_f32     = LUX_F32_SLOT(op_softmax_f32),
    .op_log_softmax_f32 = LUX_F32_SLOT(op_log_softmax_f32),

    .op_exp_f32     = LUX_F32_SLOT(op_exp_f32),
    .op_log_f32     = LUX_F32_SLOT(op_log_f32),
    .op_sqrt_f32    = LUX_F32_SLOT(op_sqrt_f32),
    .op_neg_f32     = LUX_F32_SLOT(op_neg_f32),
    .op_abs_f32     = LUX_F32_SLOT(op_abs_f32),
    .op_tanh_f32    = LUX_F32_SLOT(op_tanh_f32),
    .op_sigmoid_f32 = LUX_F32_SLOT(op_sigmoid_f32),
    .op_relu_f32    = LUX_F32_SLOT(op_relu_f32),
    .op_gelu_f32    = LUX_F32_SLOT(op_gelu_f32),

    .op_copy_f32 = LUX_F32_SLOT(op_copy_f32),

    .op_layer_norm_f32 = LUX_F32_SLOT(op_layer_norm_f32),
    .op_rms_norm_f32   = LUX_F32_SLOT(op_rms_norm_f32),

    .op_ntt_forward = ns_ntt,
    .op_ntt_inverse = ns_ntt,

    .op_poly_mul       = ns_poly_mul,
    .op_tfhe_bootstrap = ns_bootstrap,
    .op_tfhe_keyswitch = ns_keyswitch,
    .op_blind_rotate   = ns_blind_rotate,

    .op_poseidon2_hash = ns_poseidon2,
    .op_blake3_hash    = ns_hash,
    .op_keccak256_hash = ns_hash,

    .op_bls12_381_add     = ns_curve,
    .op_bls12_381_mul     = ns_curve,
    .op_bls12_381_pairing = ns_pairing,

    .op_bn254_add = ns_curve,
    .op_bn254_mul = ns_curve,

    .op_msm = ns_msm,

    .op_kzg_commit = ns_kzg_commit,
    .op_kzg_open   = ns_kzg_open,
    .op_kzg_verify = ns_kzg_verify,

    .op_ecrecover_batch = ns_ecrecover,

    .op_mldsa_verify_batch          = ns_verify3,
    .op_mlkem_decapsulate_batch     = ns_batch2_out,
    .op_slhdsa_verify_batch         = ns_verify3,
    .op_ringtail_partial_sign_batch = ns_batch2_out,
    .op_ringtail_combine_batch      = ns_ringtail_combine,
    .op_frost_partial_verify_batch  = ns_frost_verify,
    .op_cggmp21_partial_sign_batch  = ns_cggmp21_sign,
    .op_ed25519_verify_batch        = ns_verify3,
    .op_sr25519_verify_batch        = ns_verify3,
};

static_assert(sizeof(lux_gpu_backend_vtbl) == LUX_GPU_BACKEND_VTBL_SLOTS * sizeof(void*),
              "vtable must have exactly the reference's 65 pointer-sized slots");

// ---------------------------------------------------------------------------------
// Entry point (src/webgpu_plugin.cpp:4129-4154)
// ---------------------------------------------------------------------------------
static bool cuda_backend_init_impl(lux_gpu_backend_desc* out) {
    if (!out) return false;
    out->abi_version     = LUX_GPU_BACKEND_ABI_VERSION;
    out->vtbl_size       = sizeof(lux_gpu_backend_vtbl);
    out->backend_name    = "cuda";
    out->backend_version = "0.1.0-b200";
    // Only what this backend really runs on the GPU is advertised; everything else
    // answers NOT_SUPPORTED so the host falls back.
    out->capabilities    = LUX_CAP_TENSOR_OPS | LUX_CAP_MATMUL | LUX_CAP_CUSTOM_KERNELS;
    out->vtbl            = &cuda_vtbl;
    return true;
}

LUX_GPU_DECLARE_BACKEND(cuda_backend_init_impl)

// ---------------------------------------------------------------------------------
// Interop entry points of lux/gpu/qmatmul_ext.h
// ---------------------------------------------------------------------------------
extern "C" {

LuxBackendError lux_cuda_context_set_stream(LuxBackendContext* context, void* stream) {
    auto* ctx = as_ctx(context);
    if (!ctx) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    ctx->stream = stream ? reinterpret_cast<cudaStream_t>(stream) : ctx->own_stream;
    return LUX_BACKEND_OK;
}

void* lux_cuda_context_get_stream(LuxBackendContext* context) {
    auto* ctx = as_ctx(context);
    return ctx ? reinterpret_cast<void*>(ctx->stream) : nullptr;
}

LuxBackendBuffer* lux_cuda_buffer_wrap(LuxBackendContext* context, void* device_ptr, size_t bytes) {
    auto* ctx = as_ctx(context);
    if (!ctx || !device_ptr) return nullptr;
    auto* buf = new (std::nothrow) Buffer{device_ptr, bytes, ctx->device, false};
    return reinterpret_cast<LuxBackendBuffer*>(buf);
}

void* lux_cuda_buffer_device_ptr(LuxBackendBuffer* buf) { return buf ? as_buf(buf)->ptr : nullptr; }
size_t lux_cuda_buffer_size(LuxBackendBuffer* buf) { return buf ? as_buf(buf)->size : 0; }

uint64_t lux_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* lux_cuda_last_kernel_name(void) { return g_last_kernel.load(std::memory_order_relaxed); }

uint32_t lux_cuda_last_device_status(LuxBackendContext* context) {
    auto* ctx = as_ctx(context);
    return ctx ? ctx->last_status : 0;
}

}  // extern "C"
