/*
 * lux/gpu/qmatmul_ext.h -- weight-only group-quantized matmul, exported by
 * libluxgpu_backend_cuda.so BESIDE the backend vtable.
 *
 * The luxcpp/gpu backend vtable has no quantized-matmul slot
 * (luxcpp/webgpu src/webgpu_plugin.cpp:4022-4123), and the WebGPU plugin ships its
 * kernel-level entry points as extra extern "C" symbols next to the vtable
 * (src/webgpu_kernel_loader.cpp:205-291).  This header follows that convention:
 * a host resolves these symbols with dlsym from the same handle it got
 * lux_gpu_backend_init from.  Operands are LuxBackendBuffer handles created through
 * the vtable; every function validates its arguments first and returns a
 * LuxBackendError; nothing throws across the boundary
 * (conventions of src/webgpu_plugin.cpp:1658-1660, 1721-1771).
 *
 * Arithmetic contract (what the kernels compute; the WGSL each rule replaces):
 *   int4 element i of a little-endian u32 is (word >> 4i) & 0xF, i.e. byte j holds
 *   element 2j in its LOW nibble ............. kernels/wgsl/gpu/quantized_nax.wgsl:125-132
 *   int8 element i is byte i, sign-extended .. kernels/wgsl/gpu/quantized_nax.wgsl:143-151
 *   dequantized weight = f32(q - zero_point) * scale, integer subtract first, one
 *   multiply ................................. kernels/wgsl/gpu/quantized_nax.wgsl:312-330, 364-381
 *   group index = (row*K + col) / group_size . kernels/wgsl/gpu/quantized_nax.wgsl:587-589
 *   y = sum_k w*x accumulated in f32 ......... kernels/wgsl/gpu/quantized_nax.wgsl:577-621
 *   SwiGLU = silu(gate) * up with `up` rows stored after the `gate` rows
 *   .......................................... kernels/wgsl/steel/gemm/steel_gemm_fused.wgsl:91-94, 452-558
 *
 * Memory layout (row-major, K a multiple of group_size, G = K / group_size):
 *   x       [M, K]            f32 | f16 | bf16
 *   W int4  [N, K/2]  uint8   two values per byte, low nibble first
 *   W int8  [N, K]    int8
 *   scales  [N, G]            f32 | f16
 *   zeros   [N, ceil(G/2)] uint8, 4-bit zero-points two per byte, low nibble first;
 *           NULL means symmetric: zero-point 8 for int4 (quantized_nax.wgsl:105-112),
 *           0 for int8
 *   y       [M, N]            f32 | f16 | bf16     (y = x . dequant(W)^T)
 */
#ifndef LUX_GPU_QMATMUL_EXT_H
#define LUX_GPU_QMATMUL_EXT_H

#include "lux/gpu/backend_plugin.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum LuxQDType {
    LUX_QDTYPE_F32  = 0,
    LUX_QDTYPE_F16  = 1,
    LUX_QDTYPE_BF16 = 2
} LuxQDType;

enum {
    /* Enqueue on the context's stream and return without waiting.  The default is
     * the vtable's behaviour: return after the GPU has finished
     * (src/webgpu_plugin.cpp:1028-1050 blocks in dispatchCompute). */
    LUX_QMATMUL_FLAG_NO_SYNC = 1u << 0,
    /* W holds [gate ; up] stacked on the output axis (N = 2*I).  The kernel writes
     * y[M, I] = silu(x.gate^T) * (x.up^T), both products kept in f32
     * (steel_gemm_silu_mul, steel/gemm/steel_gemm_fused.wgsl:452-558). */
    LUX_QMATMUL_FLAG_SWIGLU  = 1u << 1,
    /* The weight, scale or zero-point buffer of this call may still be being written by
     * earlier work on the same stream (a dequantize / unpack / quantize call made with
     * NO_SYNC, a caller's own kernel, an asynchronous copy).  Without this flag the matmul
     * kernels may be launched so that their prologue -- which requests weights, scales and
     * zero-points, never activations -- overlaps the tail of the previous kernel on the
     * stream (programmatic dependent launch); with it the launch is ordered after all
     * earlier work like any other.  The library sets it by itself after its own writer
     * calls; a caller whose own stream work produces these operands must set it. */
    LUX_QMATMUL_FLAG_WEIGHTS_VOLATILE = 1u << 2,
    /* lux_cuda_qquantize, asymmetric int4 only: store clamp(round(v / scale) + zp, 0, 15).  NOT the
     * reference's arithmetic: its shader stores clamp(round(v / scale), 0, 15) (see there). */
    LUX_QQUANT_FLAG_SHIFTED = 1u << 3
};

typedef struct LuxQMatmulDesc {
    uint32_t struct_size;   /* sizeof(LuxQMatmulDesc); lets the struct grow */
    uint32_t M, N, K;       /* N counts weight rows (2*I with FLAG_SWIGLU) */
    uint32_t bits;          /* 4 or 8 */
    uint32_t group_size;    /* 128 for int4, 32 for int8 */
    uint32_t x_dtype;       /* LuxQDType */
    uint32_t scale_dtype;   /* LuxQDType */
    uint32_t y_dtype;       /* LuxQDType */
    uint32_t flags;
} LuxQMatmulDesc;

/* Which kernel a call was (or would be) routed to. */
typedef enum LuxQMatmulRoute {
    LUX_QROUTE_NONE        = 0,
    LUX_QROUTE_GEMV_I8     = 1,   /* int8 g32, f32 in/out, streaming GEMV              */
    LUX_QROUTE_SKINNY_I4   = 2,   /* int4 g128, M <= 32, streaming GEMV / skinny GEMM  */
    LUX_QROUTE_GEMM_I4_TC  = 3    /* int4 g128, M >= 33 (bf16: any M), tcgen05 / TMEM GEMM; bf16 at
                                     M <= 4 is served by the fixed-point GEMV where its plan fits */
} LuxQMatmulRoute;

/* y = x . dequant(W)^T.  Replaces the role of matmul_nax_grouped
 * (kernels/wgsl/gpu/quantized_nax.wgsl:550-626) dispatched the way op_matmul_f32 is
 * (src/webgpu_plugin.cpp:1721-1771).  Supported combinations:
 *   bits=8 group=32  x=f32        scales=f32 y=f32   zeros=NULL           any M (GEMV per row)
 *   bits=4 group=128 x=f16|bf16   scales=f16 y=x     zeros NULL or given  any M
 * Anything else returns LUX_BACKEND_ERROR_NOT_SUPPORTED (the reference's signal for
 * "fall back", src/webgpu_plugin.cpp:2087-2092). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmatmul(
    LuxBackendContext* ctx, const LuxQMatmulDesc* desc,
    LuxBackendBuffer* x, LuxBackendBuffer* w, LuxBackendBuffer* scales,
    LuxBackendBuffer* zeros, LuxBackendBuffer* y);

/* Same computation with HOST activations, following the reference's host-pointer op
 * convention (src/webgpu_plugin.cpp:1117-1198: caller owns host memory, the plugin
 * owns the transient device memory): copies x_host in, runs, copies y back, waits.
 * Weights, scales and zeros stay device buffers (they are model state). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmatmul_host(
    LuxBackendContext* ctx, const LuxQMatmulDesc* desc,
    const void* x_host, LuxBackendBuffer* w, LuxBackendBuffer* scales,
    LuxBackendBuffer* zeros, void* y_host);

/* Reports the route lux_cuda_qmatmul would take; never launches. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmatmul_route(
    const LuxQMatmulDesc* desc, int has_zeros, int* route_out);

/* out[N, K] = f32(q - zp) * scale, written as f32, or rounded once more to
 * f16/bf16 (round-to-nearest-even) when desc->y_dtype says so; desc->M and x_dtype
 * are ignored.  Replaces dequantize_nax_int4_asym / dequantize_nax_int8_group
 * (kernels/wgsl/gpu/quantized_nax.wgsl:312-330, 364-386). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qdequant(
    LuxBackendContext* ctx, const LuxQMatmulDesc* desc,
    LuxBackendBuffer* w, LuxBackendBuffer* scales, LuxBackendBuffer* zeros,
    LuxBackendBuffer* out);

/* out[n] = integer (q - zp) as int8, one per weight: the unpack step alone
 * (unpack_nax_int4_asym_x8 / unpack_nax_int8_x4, quantized_nax.wgsl:125-151). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qunpack(
    LuxBackendContext* ctx, const LuxQMatmulDesc* desc,
    LuxBackendBuffer* w, LuxBackendBuffer* zeros, LuxBackendBuffer* out_i8);

/* The quantize side: x[N, K] (f32, or f16 / bf16 widened exactly; desc->x_dtype) becomes packed
 * weights, a scale table and a zero-point table in the layout above, ready for lux_cuda_qmatmul.
 * Replaces compute_group_scales + quantize_nax_int4_sym / quantize_nax_int4_asym /
 * quantize_nax_int8_group (kernels/wgsl/gpu/quantized_nax.wgsl:157-232, 236-259, 288-310, 336-362)
 * in one pass, bit for bit: IEEE division, round-half-to-even, saturating conversion, min / max
 * seeded with +-1e30, "scale == 0 -> 1", zero-point = clamp(round(-min / scale), 0, 15).
 *   bits=4 group=128: zeros_out given -> asymmetric, NULL -> symmetric (stored nibble = q + 8);
 *                     desc->scale_dtype f32 (the reference's GroupScale.scale) or f16 (the scale is
 *                     rounded to f16 first and the values are quantized with the rounded number)
 *   bits=8 group=32 : symmetric, f32 scales, zeros_out NULL
 * The reference's asymmetric int4 shader never shifts by the zero-point before clamping (:303 with
 * :118): it stores clamp(round(v / scale), 0, 15), so negative inputs become 0 and a round trip
 * through lux_cuda_qdequant is offset by -zp * scale.  That behaviour is reproduced;
 * LUX_QQUANT_FLAG_SHIFTED asks for clamp(round(v / scale) + zp, 0, 15) instead.
 * desc->M and y_dtype are ignored.  The next matmul on this context is ordered behind this call
 * even with LUX_QMATMUL_FLAG_NO_SYNC (see LUX_QMATMUL_FLAG_WEIGHTS_VOLATILE). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qquantize(
    LuxBackendContext* ctx, const LuxQMatmulDesc* desc, LuxBackendBuffer* x,
    LuxBackendBuffer* w_out, LuxBackendBuffer* scales_out, LuxBackendBuffer* zeros_out);

/* ---- the activation-quantized integer path (W8A8 / W4A8) ----------------------------------
 * Exact integer arithmetic: results are bit-identical to the shaders.
 *
 * lux_cuda_dynamic_quantize: per-tensor symmetric quantization of n f32 activations
 * (dynamic_quantize, kernels/wgsl/gpu/quantized_nax.wgsl:644-718): scale = max|x| / 127 (bits 8) or
 * / 7 (bits 4), 1 if that is 0; q = clamp(round(x / scale)).  `out` receives n int8 bytes, or
 * ceil(n / 2) bytes of int4 in the weight-only format's +8 offset (pack_nax_int4_sym_x8);
 * `scale_out` one f32.
 * lux_cuda_matmul_int8: C[M, N] (i32) = A[M, K] (int8) . B[K, N] (int8), both row-major
 * (matmul_int8, kernels/wgsl/gpu/quantized.wgsl:497-555).
 * lux_cuda_matmul_int4_int8: the same with A as packed int4, element 2j in the low nibble of byte
 * j, nibbles in TWO'S COMPLEMENT (unpack_int4x8, quantized.wgsl:150-158 -- not the +8 offset of the
 * weight-only format) (matmul_int4_int8, :590-647).
 * lux_cuda_requantize_int32_to_int8: out[i] (i32) = clamp(i32(round(f32(in[i]) * input_scale /
 * output_scale) + zero_point), -128, 127) (requantize_int32_to_int8, :573-588).
 * Any shape; K % 16 == 0, N % 16 == 0 and 16-byte aligned buffers take the tensor-core kernel
 * (mma.sync int8), everything else a plain one. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_dynamic_quantize(LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* out,
                                                                LuxBackendBuffer* scale_out, size_t n, uint32_t bits);
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_matmul_int8(LuxBackendContext* ctx, LuxBackendBuffer* a, LuxBackendBuffer* b,
                                                           LuxBackendBuffer* c, int M, int N, int K);
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_matmul_int4_int8(LuxBackendContext* ctx, LuxBackendBuffer* w4, LuxBackendBuffer* b,
                                                                LuxBackendBuffer* c, int M, int N, int K);
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_requantize_int32_to_int8(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out,
                                                                        size_t n, float input_scale, float output_scale,
                                                                        int32_t output_zero_point);

/* out = in / (1 + exp(-in)), element-wise f32 (silu, kernels/wgsl/gpu/unary.wgsl:375-381).  The
 * backend vtable has slots for sigmoid, relu and gelu but none for SiLU, the activation of the
 * Llama FFN, so it ships as a symbol beside the vtable like the quantized ops. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_op_silu_f32(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);

/* Llama-style FFN on one GPU or one tensor-parallel shard:
 *   h[M, I] = silu(x.gate^T) * (x.up^T)    W_gate_up [2*I, K]  (gate rows, then up rows)
 *   y[M, H] = h . dequant(W_down)^T        W_down    [H, I]
 * int4 g128, f16 or bf16 activations.  `h` is caller-provided scratch of M*I elements.
 * On a shard, I is the local intermediate size and y is the PARTIAL sum the caller
 * all-reduces. */
typedef struct LuxQMlpDesc {
    uint32_t struct_size;
    uint32_t M, K, I, H;    /* K: model dim in, I: local intermediate, H: model dim out */
    uint32_t group_size;    /* 128 */
    uint32_t act_dtype;     /* LUX_QDTYPE_F16 | LUX_QDTYPE_BF16 */
    uint32_t flags;         /* LUX_QMATMUL_FLAG_NO_SYNC */
} LuxQMlpDesc;

LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmlp(
    LuxBackendContext* ctx, const LuxQMlpDesc* desc, LuxBackendBuffer* x,
    LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
    LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down,
    LuxBackendBuffer* h_scratch, LuxBackendBuffer* y);

/* The FFN above for callers that must not allocate device memory.  NO COUNTERPART IN THE
 * REFERENCE: luxcpp/webgpu has no allocation-free variant of any op.
 *
 * Who needs it: a host that gave all device memory to its own arena at start-up (a later
 * cudaMalloc would fail or fragment it), and latency-critical decode loops, where
 * cudaMalloc / cudaFree synchronise the whole device.  Instead of a caller-provided `h`,
 * the SwiGLU output goes to a fixed array inside this library's device image
 * (LUX_QMLP_NOALLOC_MAX_BYTES, held by every GPU that loads the library until exit).
 * Rules: M * I * 2 bytes must fit that array, else INVALID_ARGUMENT; every call on a device
 * shares the one array, so calls that overlap on the GPU race; the first call on a device
 * resolves the array's address and should be made outside any stream capture.  It calls no
 * cudaMalloc, cudaFree or other allocating routine. */
#define LUX_QMLP_NOALLOC_MAX_BYTES (1u << 20)
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmlp_noalloc(
    LuxBackendContext* ctx, const LuxQMlpDesc* desc, LuxBackendBuffer* x,
    LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
    LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down,
    LuxBackendBuffer* y);

/* -- interop needed by a host that already owns CUDA state (one process per GPU) ---- */

/* Run this context's work on an existing stream (a cudaStream_t passed as void*;
 * NULL restores the context's own non-blocking stream; to name the default stream pass
 * cudaStreamLegacy or cudaStreamPerThread, not 0).  The reference has one implicit queue per
 * context (src/webgpu_plugin.cpp:584-622); this is its CUDA counterpart. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_context_set_stream(LuxBackendContext* ctx, void* stream);
LUX_GPU_PLUGIN_EXPORT void* lux_cuda_context_get_stream(LuxBackendContext* ctx);

/* Wrap device memory the caller owns as a non-owning LuxBackendBuffer; buffer_free
 * releases only the handle.  Same handle layout as buffer_alloc
 * (WGPUBackendBuffer{buffer,size}, src/webgpu_plugin.cpp:516-519). */
LUX_GPU_PLUGIN_EXPORT LuxBackendBuffer* lux_cuda_buffer_wrap(LuxBackendContext* ctx, void* device_ptr, size_t bytes);
LUX_GPU_PLUGIN_EXPORT void*  lux_cuda_buffer_device_ptr(LuxBackendBuffer* buf);
LUX_GPU_PLUGIN_EXPORT size_t lux_cuda_buffer_size(LuxBackendBuffer* buf);

/* ---- one-node push all-reduce over peer memory (tensor-parallel FFN) --------------------
 * No reference counterpart: luxcpp/webgpu has no multi-device path.  One process per GPU.
 * Every rank creates a communicator (a window in its own memory that peers write into),
 * exchanges the 64-byte handles by any means (the Python host uses torch.distributed),
 * connects, and then calls lux_cuda_peer_allreduce on every rank for every reduction, in the
 * same order.  The kernel pushes self-validating 8-byte words {payload, epoch} with plain
 * stores, waits a bounded time for the peers' words and sums in rank order (bit-identical results on all ranks); a peer that never
 * arrives leaves the tensor unchanged and is reported as LUX_BACKEND_ERROR_DEVICE_LOST by the
 * next synchronising call (status 0x7C050005).  Works under CUDA-graph capture and replay. */
typedef struct LuxPeerComm LuxPeerComm;
#define LUX_PEER_HANDLE_BYTES 64
/* max_bytes: largest tensor (in bytes) that will be reduced.  handle_out: 64 bytes to send to the
 * other ranks (may be NULL when connecting with pointers). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_peer_comm_create(LuxBackendContext* ctx, int rank, int world,
                                                                size_t max_bytes, LuxPeerComm** out, void* handle_out);
/* handles: world * 64 bytes, rank order (the own entry is ignored); opens the peers' windows
 * through CUDA IPC.  NOT_SUPPORTED if the system refuses the mapping. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_peer_comm_connect(LuxPeerComm* comm, const void* handles);
/* For hosts that drive several GPUs from one process with peer access enabled: windows[r] is
 * lux_cuda_peer_comm_window() of rank r's communicator (the own entry is ignored). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_peer_comm_connect_ptrs(LuxPeerComm* comm, void* const* windows);
LUX_GPU_PLUGIN_EXPORT void*  lux_cuda_peer_comm_window(LuxPeerComm* comm);
LUX_GPU_PLUGIN_EXPORT size_t lux_cuda_peer_comm_window_bytes(LuxPeerComm* comm);
/* In-place sum of `count` f16 / bf16 elements (count % 8 == 0, 16-byte aligned buffer,
 * count * 2 <= max_bytes) across the ranks, on the context's stream.  flags:
 * LUX_QMATMUL_FLAG_NO_SYNC to return without waiting. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_peer_allreduce(LuxBackendContext* ctx, LuxPeerComm* comm,
                                                              LuxBackendBuffer* buf, size_t count, LuxQDType dtype,
                                                              uint32_t flags);
/* The tensor-parallel FFN of one rank in one call: lux_cuda_qmlp on this rank's shards followed by
 * the all-reduce of y through `comm` (same argument meaning as lux_cuda_qmlp; y holds the reduced
 * result on every rank).  At batch <= 2 with f16 activations the down projection's kernel stores
 * its outputs straight into every rank's window (fused compute + collective) and a second small
 * kernel waits for the peers and sums; otherwise it is lux_cuda_qmlp + lux_cuda_peer_allreduce.
 * Call on every rank, in the same order as any other reduction on `comm`. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_qmlp_tp(
    LuxBackendContext* ctx, const LuxQMlpDesc* desc, LuxBackendBuffer* x,
    LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
    LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down,
    LuxBackendBuffer* h_scratch, LuxBackendBuffer* y, LuxPeerComm* comm);
/* Every rank must have finished its last reduction (e.g. a host barrier) before any rank destroys. */
LUX_GPU_PLUGIN_EXPORT void lux_cuda_peer_comm_destroy(LuxPeerComm* comm);

/* Number of kernel launches this library has issued since load (all contexts). */
LUX_GPU_PLUGIN_EXPORT uint64_t lux_cuda_launch_count(void);

/* Name of the quantized-matmul kernel launched most recently by this library (all contexts;
 * "" before the first one).  The library picks a kernel per shape; benchmarks and profiles
 * use this to say which one they measured.  The string is static. */
LUX_GPU_PLUGIN_EXPORT const char* lux_cuda_last_kernel_name(void);

/* Benchmark / tuning hook: overrides one launch heuristic (value 0 restores the
 * default).  Keys: gemv_i8_kernel (1 row-per-warp-group, 2 warp-autonomous units), gemv_i4_kernel
 * (1 register-staged, 2 bulk-copy ring, 3 warp-autonomous units), gemv_i4_warps, gemv_i4_row_tiles, gemv_stream_warps, gemv_stream_cg, gemv_stream_stages,
 * gemv_units_ks, gemv_units_stages, gemv_units_cg, gemv_units_pre, gemv_units_fx, gemv_i8_warps, gemm_tc_bn,
 * gemm_tc_stages, gemm_tc_ma, gemm_tc_kernel (1 lux_qgemm_i4_tc, 2 lux_qgemm_i4_tc_wa wherever it applies), gemm_tc_splitk (1, 2, 4),
 * gemm_tc_groups, gemm_min_m (smallest batch handed to lux_qgemm_i4_tc_wa, default 5), pdl (2: no programmatic dependent launch), peer_wait_limit, tp_fused_push, tp_reduce_early,
 * gemv_units_warps, gemv_units_planes, gemm_wa_narrow, gemm_wa_prefetch (-1 off), host_pageable, attn_splits, int_matmul_kernel (1 mma.sync kernels only, 2 tcgen05 through a transposed copy of B).  Unknown keys return INVALID_ARGUMENT.  Process-wide;
 * not part of the drop-in surface. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_tune_set(const char* key, int value);

/* What the context's most recent synchronising call found in the device status word: 0 if every
 * device-side check since the synchronising call before it passed, else the code of the check that
 * failed (a bounded wait that gave up, a block-table entry or rope position out of range); the call
 * itself returned LUX_BACKEND_ERROR_DEVICE_LOST. */
LUX_GPU_PLUGIN_EXPORT uint32_t lux_cuda_last_device_status(LuxBackendContext* ctx);

#ifdef __cplusplus
}
#endif

#endif /* LUX_GPU_QMATMUL_EXT_H */
