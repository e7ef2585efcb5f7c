// C-ABI launch layer of the quantized-matmul extension (lux/gpu/qmatmul_ext.h):
// validates like the reference's op bridges do (arguments first, then sizes;
// luxcpp/webgpu src/webgpu_plugin.cpp:1721-1731), picks a precompiled kernel, launches
// it on the context's stream and, unless asked not to, waits for it.
#include "common.cuh"

#include <algorithm>
#include <cstring>

using namespace luxcuda;

namespace {

size_t dtype_size(uint32_t d) { return d == LUX_QDTYPE_F32 ? 4 : 2; }

struct Checked {
    QArgs a;
    int bits;
    int route;
    bool no_sync;
};

// Shape / dtype rules shared by every entry point.  `need_x` is false for dequant/unpack.
LuxBackendError check_desc(const LuxQMatmulDesc* d, bool has_zeros, bool need_x, Checked* out) {
    if (!d || d->struct_size < sizeof(LuxQMatmulDesc)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->N == 0 || d->K == 0 || (need_x && d->M == 0)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->bits != 4 && d->bits != 8) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->group_size == 0 || d->K % d->group_size) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->x_dtype > LUX_QDTYPE_BF16 || d->scale_dtype > LUX_QDTYPE_BF16 || d->y_dtype > LUX_QDTYPE_BF16)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const bool swiglu = (d->flags & LUX_QMATMUL_FLAG_SWIGLU) != 0;
    if (swiglu && (d->N % 2)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;

    int route = LUX_QROUTE_NONE;
    if (d->bits == 8) {
        if (d->group_size == 32 && d->scale_dtype == LUX_QDTYPE_F32 && !has_zeros && !swiglu &&
            (!need_x || (d->x_dtype == LUX_QDTYPE_F32 && d->y_dtype == LUX_QDTYPE_F32)) && d->K % 64 == 0)
            route = LUX_QROUTE_GEMV_I8;
    } else {
        if (d->group_size == 128 && d->scale_dtype == LUX_QDTYPE_F16) {
            if (!need_x) {
                route = LUX_QROUTE_SKINNY_I4;
            } else if (d->x_dtype == d->y_dtype && d->x_dtype != LUX_QDTYPE_F32) {
                if (d->M <= 32 && d->x_dtype == LUX_QDTYPE_F16) route = LUX_QROUTE_SKINNY_I4;
                else route = LUX_QROUTE_GEMM_I4_TC;
            }
        }
    }
    if (route == LUX_QROUTE_NONE) return LUX_BACKEND_ERROR_NOT_SUPPORTED;

    out->bits = (int)d->bits;
    out->route = route;
    out->no_sync = (d->flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0;
    QArgs& a = out->a;
    a.M = (int)d->M; a.N = (int)d->N; a.K = (int)d->K; a.G = (int)(d->K / d->group_size);
    a.x_dtype = (int)d->x_dtype; a.scale_dtype = (int)d->scale_dtype; a.y_dtype = (int)d->y_dtype;
    a.swiglu = swiglu;
    a.weights_volatile = (d->flags & LUX_QMATMUL_FLAG_WEIGHTS_VOLATILE) != 0;
    return LUX_BACKEND_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

LuxBackendError bind_weights(Checked& c, Buffer* w, Buffer* scales, Buffer* zeros) {
    QArgs& a = c.a;
    const size_t w_bytes = (size_t)a.N * a.K * c.bits / 8;
    const size_t s_bytes = (size_t)a.N * a.G * dtype_size(a.scale_dtype);
    const size_t z_bytes = (size_t)a.N * ((a.G + 1) / 2);
    if (w->size < w_bytes || scales->size < s_bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (zeros && zeros->size < z_bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    // several kernels fetch rows of all three tables with 16-byte bulk copies
    if (!aligned16(w->ptr) || !aligned16(scales->ptr) || (zeros && !aligned16(zeros->ptr))) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    a.w = (const uint8_t*)w->ptr;
    a.scales = scales->ptr;
    a.zeros = zeros ? (const uint8_t*)zeros->ptr : nullptr;
    return LUX_BACKEND_OK;
}

LuxBackendError dispatch(Context* ctx, const Checked& c) {
    switch (c.route) {
        case LUX_QROUTE_GEMV_I8: {
            // batch 1 and 2: the warp-autonomous fixed-point kernel wherever its plan fits
            if (g_tune.gemv_i8_kernel == 2 || (g_tune.gemv_i8_kernel == 0 && c.a.M <= 2)) {
                LuxBackendError e = launch_qgemv_i8_units(ctx, c.a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED || g_tune.gemv_i8_kernel == 2) return e;
            }
            return launch_qgemv_i8(ctx, c.a);
        }
        case LUX_QROUTE_SKINNY_I4: {
            // Both kernels compute the same thing.  Measured on B200: the TMA ring kernel wins
            // for batches of 4..16 and for big layers (long rows or many megabytes of weights);
            // the register-staged kernel wins for batch 1..3 on small layers and covers every
            // shape the ring kernel does not take.
            const QArgs& a = c.a;
            // Batch 1 and 2: the warp-autonomous kernel in its fixed-point variant is the fastest
            // wherever its shared-memory plan fits.
            if (g_tune.gemv_i4_kernel == 3 || (g_tune.gemv_i4_kernel == 0 && a.M <= 4)) {
                LuxBackendError e = launch_qgemv_i4_units(ctx, a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED || g_tune.gemv_i4_kernel == 3) return e;
            }
            // From five batch rows on, the tensor-core kernel with the weights in tensor memory streams
            // the weights faster than the mma.sync kernels below, whose unpacking grows with the batch
            // (config 4 gate_up / down at batch 5: 27.4 / 19.8 us against 31.4 / 25.7 us, at batch 11:
            // 27.5 / 19.9 us against 46.3 / 69.6 us; its time does not depend on the batch up to 64).  Three
            // and four rows stay with the fixed-point kernel above (gate_up 19.1 us) or the ring kernel.
            const int min_m = g_tune.gemm_min_m > 0 ? g_tune.gemm_min_m : 5;
            if (a.M >= min_m && g_tune.gemv_i4_kernel == 0 && g_tune.gemm_tc_kernel != 1 && !a.push) {
                LuxBackendError e = launch_qgemm_i4_tc_wa(ctx, a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED) return e;
            }
            const size_t wbytes = (size_t)a.N * a.K / 2;
            const bool prefer_ring = a.M >= 4 || a.K >= 8192 || wbytes >= ((size_t)40 << 20);
            if (g_tune.gemv_i4_kernel == 2 || (g_tune.gemv_i4_kernel == 0 && prefer_ring)) {
                LuxBackendError e = launch_qgemv_i4_stream(ctx, a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED || g_tune.gemv_i4_kernel == 2) return e;
            }
            return launch_qskinny_i4(ctx, a);
        }
        case LUX_QROUTE_GEMM_I4_TC: {
            // bf16 decode (up to four rows): the fixed-point GEMV takes bf16 activations as it takes
            // f16 ones, streams the weights at the same rate and keeps the weights exact, where the
            // tensor-core kernels below round them to bf16
            if (c.a.x_dtype == LUX_QDTYPE_BF16 && c.a.M <= 4 && g_tune.gemv_i4_kernel == 0 && g_tune.gemm_tc_kernel == 0 && !c.a.push) {
                LuxBackendError e = launch_qgemv_i4_units(ctx, c.a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED) return e;
            }
            // The kernel that keeps the converted weights in tensor memory (one conversion per 256
            // batch rows, 128 x 256 MMAs; for smaller batches 128 x M) wherever the shape fits it:
            // measured faster than the B-operand kernel at every batch from 64 up (config 4 layers at
            // M = 64: 12-38 us against 34-109 us; config 3: 18 us against 40 us).
            if (g_tune.gemm_tc_kernel == 2 || g_tune.gemm_tc_kernel == 0) {
                LuxBackendError e = launch_qgemm_i4_tc_wa(ctx, c.a);
                if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED) return e;
            }
            return launch_qgemm_i4_tc(ctx, c.a);
        }
        default:                    return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
}

size_t y_cols(const QArgs& a) { return a.swiglu ? (size_t)a.N / 2 : (size_t)a.N; }

// Grows the context's staging pair (pinned host + device) used by host-pointer ops.
LuxBackendError ensure_stage(Context* ctx, size_t bytes) {
    if (ctx->h_stage_bytes >= bytes && ctx->d_stage_bytes >= bytes) return LUX_BACKEND_OK;
    size_t want = std::max<size_t>(bytes, 1 << 20);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->h_stage) { cudaFreeHost(ctx->h_stage); ctx->h_stage = nullptr; ctx->h_stage_bytes = 0; }
    if (ctx->d_stage) { cudaFree(ctx->d_stage); ctx->d_stage = nullptr; ctx->d_stage_bytes = 0; }
    LUX_CUDA_TRY(cudaHostAlloc(&ctx->h_stage, want, cudaHostAllocMapped));   // device-visible: small results are written into it directly
    ctx->h_stage_bytes = want;
    ctx->d_stage_y = nullptr;
    if (cudaHostGetDevicePointer(&ctx->d_stage_y, ctx->h_stage, 0) != cudaSuccess) { (void)cudaGetLastError(); ctx->d_stage_y = nullptr; }
    LUX_CUDA_TRY(cudaMalloc(&ctx->d_stage, want));
    ctx->d_stage_bytes = want;
    return LUX_BACKEND_OK;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" {

LuxBackendError lux_cuda_qmatmul_route(const LuxQMatmulDesc* desc, int has_zeros, int* route_out) {
    if (!route_out) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Checked c{};
    LuxBackendError e = check_desc(desc, has_zeros != 0, true, &c);
    *route_out = e == LUX_BACKEND_OK ? c.route : LUX_QROUTE_NONE;
    return e;
}

LuxBackendError lux_cuda_qmatmul(LuxBackendContext* context, const LuxQMatmulDesc* desc,
                                 LuxBackendBuffer* x, LuxBackendBuffer* w, LuxBackendBuffer* scales,
                                 LuxBackendBuffer* zeros, LuxBackendBuffer* y) {
    Context* ctx = as_ctx(context);
    Buffer *bx = as_buf(x), *bw = as_buf(w), *bs = as_buf(scales), *bz = as_buf(zeros), *by = as_buf(y);
    if (!ctx || !bx || !bw || !bs || !by) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Checked c{};
    LuxBackendError e = check_desc(desc, bz != nullptr, true, &c);
    if (e != LUX_BACKEND_OK) return e;
    e = bind_weights(c, bw, bs, bz);
    if (e != LUX_BACKEND_OK) return e;
    QArgs& a = c.a;
    if (bx->size < (size_t)a.M * a.K * dtype_size(a.x_dtype)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (by->size < (size_t)a.M * y_cols(a) * dtype_size(a.y_dtype)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!aligned16(bx->ptr) || !aligned16(by->ptr)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    a.x = bx->ptr;
    a.y = by->ptr;
    cudaSetDevice(ctx->device);
    e = dispatch(ctx, c);
    if (e != LUX_BACKEND_OK) return e;
    return finish_op(ctx, c.no_sync, "lux_cuda_qmatmul");
}

LuxBackendError lux_cuda_qmatmul_host(LuxBackendContext* context, const LuxQMatmulDesc* desc,
                                      const void* x_host, LuxBackendBuffer* w, LuxBackendBuffer* scales,
                                      LuxBackendBuffer* zeros, void* y_host) {
    Context* ctx = as_ctx(context);
    Buffer *bw = as_buf(w), *bs = as_buf(scales), *bz = as_buf(zeros);
    if (!ctx || !x_host || !bw || !bs || !y_host) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Checked c{};
    LuxBackendError e = check_desc(desc, bz != nullptr, true, &c);
    if (e != LUX_BACKEND_OK) return e;
    e = bind_weights(c, bw, bs, bz);
    if (e != LUX_BACKEND_OK) return e;
    QArgs& a = c.a;
    const size_t xb = (size_t)a.M * a.K * dtype_size(a.x_dtype);
    const size_t yb = (size_t)a.M * y_cols(a) * dtype_size(a.y_dtype);
    const size_t y_off = round_up(xb, 256);
    cudaSetDevice(ctx->device);
    std::lock_guard<std::mutex> lock(ctx->mu);
    e = ensure_stage(ctx, y_off + yb);
    if (e != LUX_BACKEND_OK) return e;
    // Decode-sized calls are all fixed cost, so every step that can go, goes:
    //   * x: up to 64 KB the runtime sends a host-to-device copy from ordinary memory inside the
    //     command stream itself and returns, so x_host is handed over as it is (no staging copy,
    //     no DMA read back over the bus); larger activations go through the pinned buffer;
    //   * y: a small result is written by the kernel straight into the pinned buffer (posted writes
    //     over the bus), which takes the device-to-host copy off the critical path;
    //   * completion: one cudaStreamSynchronize.  (Measured and dropped: a completion flag in pinned
    //     memory written by the kernel's last CTA and polled by the host was 3.5 us SLOWER per call
    //     than the stream wait; carrying x in the kernel's parameter block instead of copying it
    //     was 4 us slower, 8 KB of parameters costing more than the copy they replace; letting the
    //     kernel read x from the mapped pinned buffer, with no copy command at all, took 52 us against
    //     29: every CTA then fetches its own copy of x over the bus; a one-CTA copy kernel in place of
    //     the copy command, so that the matmul starts early behind it, 28.2 us against 27.6.)
    const bool direct = yb <= ((size_t)256 << 10) && ctx->d_stage_y;
    a.y = direct ? (void*)((char*)ctx->d_stage_y + y_off) : (void*)((char*)ctx->d_stage + y_off);
    {
        if (xb <= ((size_t)64 << 10) && g_tune.host_pageable != 2) {
            LUX_CUDA_TRY(cudaMemcpyAsync(ctx->d_stage, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
        } else {
            std::memcpy(ctx->h_stage, x_host, xb);
            LUX_CUDA_TRY(cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, xb, cudaMemcpyHostToDevice, ctx->stream));
        }
        a.x = ctx->d_stage;
        e = dispatch(ctx, c);
        if (e != LUX_BACKEND_OK) return e;
    }
    if (!direct)
        LUX_CUDA_TRY(cudaMemcpyAsync((char*)ctx->h_stage + y_off, a.y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    e = finish_op(ctx, false, "lux_cuda_qmatmul_host");
    if (e != LUX_BACKEND_OK) return e;
    std::memcpy(y_host, (char*)ctx->h_stage + y_off, yb);
    return LUX_BACKEND_OK;
}

LuxBackendError lux_cuda_qdequant(LuxBackendContext* context, const LuxQMatmulDesc* desc,
                                  LuxBackendBuffer* w, LuxBackendBuffer* scales, LuxBackendBuffer* zeros,
                                  LuxBackendBuffer* out) {
    Context* ctx = as_ctx(context);
    Buffer *bw = as_buf(w), *bs = as_buf(scales), *bz = as_buf(zeros), *bo = as_buf(out);
    if (!ctx || !bw || !bs || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Checked c{};
    LuxBackendError e = check_desc(desc, bz != nullptr, false, &c);
    if (e != LUX_BACKEND_OK) return e;
    if (c.a.swiglu || c.a.K % 32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    e = bind_weights(c, bw, bs, bz);
    if (e != LUX_BACKEND_OK) return e;
    if (bo->size < (size_t)c.a.N * c.a.K * dtype_size(c.a.y_dtype) || !aligned16(bo->ptr))
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    c.a.y = bo->ptr;
    cudaSetDevice(ctx->device);
    e = launch_qdequant(ctx, c.a, c.bits);
    if (e != LUX_BACKEND_OK) return e;
    ctx->writer_pending = true;          // cleared by the wait in finish_op unless NO_SYNC
    return finish_op(ctx, c.no_sync, "lux_cuda_qdequant");
}

LuxBackendError lux_cuda_qunpack(LuxBackendContext* context, const LuxQMatmulDesc* desc,
                                 LuxBackendBuffer* w, LuxBackendBuffer* zeros, LuxBackendBuffer* out_i8) {
    Context* ctx = as_ctx(context);
    Buffer *bw = as_buf(w), *bz = as_buf(zeros), *bo = as_buf(out_i8);
    if (!ctx || !bw || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Checked c{};
    LuxBackendError e = check_desc(desc, bz != nullptr, false, &c);
    if (e != LUX_BACKEND_OK) return e;
    QArgs& a = c.a;
    if (a.swiglu || a.K % 32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bw->size < (size_t)a.N * a.K * c.bits / 8 || !aligned16(bw->ptr)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bz && bz->size < (size_t)a.N * ((a.G + 1) / 2)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (bo->size < (size_t)a.N * a.K) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    a.w = (const uint8_t*)bw->ptr;
    a.zeros = bz ? (const uint8_t*)bz->ptr : nullptr;
    a.scales = nullptr;
    a.y = bo->ptr;
    cudaSetDevice(ctx->device);
    e = launch_qunpack(ctx, a, c.bits);
    if (e != LUX_BACKEND_OK) return e;
    ctx->writer_pending = true;          // cleared by the wait in finish_op unless NO_SYNC
    return finish_op(ctx, c.no_sync, "lux_cuda_qunpack");
}

// The tensor-parallel FFN of one rank: gate_up + SwiGLU, down, and the all-reduce of the partial
// outputs through the push communicator.  When the down projection runs in the warp-autonomous
// fixed-point kernel (batch <= 2), its final reduction stores the outputs straight into every
// rank's window (fused compute + push) and the all-reduce kernel that follows only waits and sums:
// its CTAs are resident before `down` ends (programmatic launch), and while they wait for the
// peers' words the NEXT matmul's CTAs already take the SMs `down` has left and request their
// weights.  (tp_fused_push = 1 makes the down kernel wait and sum itself, two launches per FFN:
// measured 1 us slower per step on two GPUs, because the waiting CTAs keep the SMs from the next
// kernel's prefetch.)  Otherwise down writes y and the all-reduce kernel pushes it.
LuxBackendError lux_cuda_qmlp_tp(LuxBackendContext* context, const LuxQMlpDesc* d, LuxBackendBuffer* x,
                                 LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
                                 LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down,
                                 LuxBackendBuffer* h_scratch, LuxBackendBuffer* y, LuxPeerComm* comm) {
    Context* ctx = as_ctx(context);
    if (!ctx || !d || d->struct_size < sizeof(LuxQMlpDesc) || !comm) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!x || !w_gate_up || !s_gate_up || !w_down || !s_down || !h_scratch || !y) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->act_dtype != LUX_QDTYPE_F16 && d->act_dtype != LUX_QDTYPE_BF16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    LuxQMatmulDesc gu{};
    gu.struct_size = sizeof(gu);
    gu.M = d->M; gu.N = 2 * d->I; gu.K = d->K;
    gu.bits = 4; gu.group_size = d->group_size;
    gu.x_dtype = d->act_dtype; gu.scale_dtype = LUX_QDTYPE_F16; gu.y_dtype = d->act_dtype;
    gu.flags = LUX_QMATMUL_FLAG_SWIGLU | LUX_QMATMUL_FLAG_NO_SYNC;
    LuxBackendError e = lux_cuda_qmatmul(context, &gu, x, w_gate_up, s_gate_up, z_gate_up, h_scratch);
    if (e != LUX_BACKEND_OK) return e;
    LuxQMatmulDesc dn = gu;
    dn.N = d->H; dn.K = d->I;
    dn.flags = LUX_QMATMUL_FLAG_NO_SYNC;
    const size_t count = (size_t)d->M * d->H;
    Buffer* by = as_buf(y);
    bool fused = false;
    PushTarget target{};
    if (d->M <= 2 && d->act_dtype == LUX_QDTYPE_F16 && g_tune.tp_fused_push != 2 &&
        peer_comm_push_target(comm, count, ctx->device, &target)) {
        Buffer *bh = as_buf(h_scratch), *bw = as_buf(w_down), *bs = as_buf(s_down), *bz = as_buf(z_down);
        Checked c{};
        e = check_desc(&dn, bz != nullptr, true, &c);
        if (e == LUX_BACKEND_OK) e = bind_weights(c, bw, bs, bz);
        if (e == LUX_BACKEND_OK && c.route == LUX_QROUTE_SKINNY_I4 && bh->ptr && by->ptr && aligned16(bh->ptr) &&
            aligned16(by->ptr) && bh->size >= (size_t)d->M * d->I * 2 && by->size >= count * 2) {
            c.a.x = bh->ptr;
            c.a.y = by->ptr;
            target.reduce_here = g_tune.tp_fused_push == 1 ? 1 : 0;
            c.a.push = &target;
            cudaSetDevice(ctx->device);
            e = launch_qgemv_i4_units(ctx, c.a);
            if (e == LUX_BACKEND_OK) fused = true;
            else if (e != LUX_BACKEND_ERROR_NOT_SUPPORTED) return e;
        }
    }
    if (!fused) {
        e = lux_cuda_qmatmul(context, &dn, h_scratch, w_down, s_down, z_down, y);
        if (e != LUX_BACKEND_OK) return e;
    }
    if (!fused || !target.reduce_here) {
        cudaSetDevice(ctx->device);
        e = peer_allreduce_launch(ctx, comm, by->ptr, by->size, count, (int)d->act_dtype, !fused);
        if (e != LUX_BACKEND_OK) return e;
    }
    return finish_op(ctx, (d->flags & LUX_QMATMUL_FLAG_NO_SYNC) != 0, "lux_cuda_qmlp_tp");
}

LuxBackendError lux_cuda_qmlp(LuxBackendContext* context, const LuxQMlpDesc* d, LuxBackendBuffer* x,
                              LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
                              LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down,
                              LuxBackendBuffer* h_scratch, LuxBackendBuffer* y) {
    if (!context || !d || d->struct_size < sizeof(LuxQMlpDesc)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!x || !w_gate_up || !s_gate_up || !w_down || !s_down || !h_scratch || !y) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (d->act_dtype != LUX_QDTYPE_F16 && d->act_dtype != LUX_QDTYPE_BF16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    // Two launches on one stream: gate_up with the SwiGLU epilogue, then down.
    LuxQMatmulDesc gu{};
    gu.struct_size = sizeof(gu);
    gu.M = d->M; gu.N = 2 * d->I; gu.K = d->K;
    gu.bits = 4; gu.group_size = d->group_size;
    gu.x_dtype = d->act_dtype; gu.scale_dtype = LUX_QDTYPE_F16; gu.y_dtype = d->act_dtype;
    gu.flags = LUX_QMATMUL_FLAG_SWIGLU | LUX_QMATMUL_FLAG_NO_SYNC;
    LuxBackendError e = lux_cuda_qmatmul(context, &gu, x, w_gate_up, s_gate_up, z_gate_up, h_scratch);
    if (e != LUX_BACKEND_OK) return e;
    LuxQMatmulDesc dn = gu;
    dn.N = d->H; dn.K = d->I;
    dn.flags = d->flags & LUX_QMATMUL_FLAG_NO_SYNC;
    return lux_cuda_qmatmul(context, &dn, h_scratch, w_down, s_down, z_down, y);
}

// Benchmark / tuning hook: override a launch heuristic (0 restores the default).
// Not part of the drop-in surface; unknown keys are rejected.
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_tune_set(const char* key, int value) {
    if (!key) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    struct { const char* k; int* v; } table[] = {
        {"gemv_i4_warps", &g_tune.gemv_i4_warps},   {"gemv_i4_row_tiles", &g_tune.gemv_i4_row_tiles},
        {"gemv_i8_warps", &g_tune.gemv_i8_warps},   {"gemv_i8_kernel", &g_tune.gemv_i8_kernel}, {"peer_wait_limit", &g_tune.peer_wait_limit}, {"tp_fused_push", &g_tune.tp_fused_push}, {"tp_reduce_early", &g_tune.tp_reduce_early},   {"gemm_tc_bn", &g_tune.gemm_tc_bn},
        {"gemv_i4_kernel", &g_tune.gemv_i4_kernel}, {"gemv_stream_cg", &g_tune.gemv_stream_cg},
        {"gemv_stream_stages", &g_tune.gemv_stream_stages}, {"gemv_stream_warps", &g_tune.gemv_stream_warps},
        {"gemv_units_ks", &g_tune.gemv_units_ks}, {"gemv_units_stages", &g_tune.gemv_units_stages}, {"gemv_units_cg", &g_tune.gemv_units_cg}, {"gemv_units_pre", &g_tune.gemv_units_pre}, {"gemv_units_fx", &g_tune.gemv_units_fx}, {"gemv_units_warps", &g_tune.gemv_units_warps}, {"gemv_units_planes", &g_tune.gemv_units_planes}, {"host_pageable", &g_tune.host_pageable},
        {"gemm_tc_stages", &g_tune.gemm_tc_stages}, {"gemm_tc_splitk", &g_tune.gemm_tc_splitk}, {"gemm_tc_ma", &g_tune.gemm_tc_ma}, {"gemm_wa_narrow", &g_tune.gemm_wa_narrow}, {"gemm_wa_prefetch", &g_tune.gemm_wa_prefetch}, {"attn_splits", &g_tune.attn_splits}, {"int_matmul_kernel", &g_tune.int_matmul_kernel}, {"gemm_tc_groups", &g_tune.gemm_tc_groups}, {"gemm_tc_kernel", &g_tune.gemm_tc_kernel}, {"gemm_min_m", &g_tune.gemm_min_m}, {"pdl", &g_tune.pdl},
    };
    for (auto& t : table)
        if (std::strcmp(t.k, key) == 0) { *t.v = value; return LUX_BACKEND_OK; }
    return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
}

}  // extern "C"
