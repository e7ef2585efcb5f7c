// Kernel table: the CUDA counterpart of the lux_wgpu_kernel_* C API
// (luxcpp/webgpu src/webgpu_kernel_loader.cpp:205-291).  The WebGPU loader turns WGSL
// text into a pipeline at run time; every kernel here is already compiled for sm_100a
// and embedded in this shared library, so a "kernel" is a name, a function address and
// the block size it is launched with.
#include "common.cuh"

#include <cstring>
#include <new>

#include "lux/gpu/cuda_kernel_loader.h"

namespace luxcuda {
const void* kernel_addr_qskinny_i4();
const void* kernel_addr_qskinny_i4_swiglu();
const void* kernel_addr_qgemv_i8();
const void* kernel_addr_qgemv_i8_units_fx();
const void* kernel_addr_qgemv_i4_stream();
const void* kernel_addr_qgemv_i4_units();
const void* kernel_addr_qgemv_i4_units_fx();
const void* kernel_addr_peer_allreduce_push();
const void* kernel_addr_qdequant_i4();
const void* kernel_addr_qdequant_i8();
const void* kernel_addr_matmul_int8();
const void* kernel_addr_matmul_int4_int8();
const void* kernel_addr_qquantize_i4();
const void* kernel_addr_qquantize_i8();
const void* kernel_addr_qgemm_i4_tc_bf16();
const void* kernel_addr_qgemm_i4_tc_f16();
const void* kernel_addr_qgemm_i4_tc_wa_bf16();
const void* kernel_addr_qgemm_i4_tc_wa_f16();
const void* kernel_addr_qgemm_i4_tc_wa_bf16_swiglu();
const void* kernel_addr_qgemm_i4_tc_wa_f16_swiglu();
const void* kernel_addr_qgemv_i4_units_fx_swiglu();
const void* kernel_addr_qgemv_i4_units_fx_batch2();
const void* kernel_addr_qgemv_i4_units_fx_batch4();
const void* kernel_addr_matmul_int8_tcgen05();
const void* kernel_addr_attn_stream_f32();
const void* kernel_addr_attn_merge_f32();
const void* kernel_addr_attn_plain_f32();
const void* kernel_addr_rope_f32();
const void* kernel_addr_kv_append_f32();
}  // namespace luxcuda

namespace {

struct Entry {
    const char* name;
    const void* (*addr)();
    uint32_t bx, by, bz;      // launch block size (the reference's workgroup size)
};

const Entry kTable[] = {
    {"lux_qgemv_i8_g32_f32",       luxcuda::kernel_addr_qgemv_i8,           256, 1, 1},
    {"lux_qgemv_i8_g32_units_fx",  luxcuda::kernel_addr_qgemv_i8_units_fx,  512, 1, 1},
    {"lux_qgemv_i4_g128_stream",   luxcuda::kernel_addr_qgemv_i4_stream,    544, 1, 1},
    {"lux_qgemv_i4_g128_units",    luxcuda::kernel_addr_qgemv_i4_units,     512, 1, 1},
    {"lux_qgemv_i4_g128_units_fx", luxcuda::kernel_addr_qgemv_i4_units_fx,  512, 1, 1},
    {"lux_qskinny_i4_g128",        luxcuda::kernel_addr_qskinny_i4,         128, 1, 1},
    {"lux_qskinny_i4_g128_swiglu", luxcuda::kernel_addr_qskinny_i4_swiglu,  128, 1, 1},
    {"lux_peer_allreduce_push",    luxcuda::kernel_addr_peer_allreduce_push, 1024, 1, 1},
    {"lux_qdequant_i4_g128",       luxcuda::kernel_addr_qdequant_i4,        256, 1, 1},
    {"lux_qdequant_i8_g32",        luxcuda::kernel_addr_qdequant_i8,        256, 1, 1},
    {"lux_matmul_int8",            luxcuda::kernel_addr_matmul_int8,        256, 1, 1},
    {"lux_matmul_int4_int8",       luxcuda::kernel_addr_matmul_int4_int8,   256, 1, 1},
    {"lux_qquantize_i4_g128",      luxcuda::kernel_addr_qquantize_i4,       256, 1, 1},
    {"lux_qquantize_i8_g32",       luxcuda::kernel_addr_qquantize_i8,       256, 1, 1},
    {"lux_qgemm_i4_tc_bf16",       luxcuda::kernel_addr_qgemm_i4_tc_bf16,   320, 1, 1},
    {"lux_qgemm_i4_tc_f16",        luxcuda::kernel_addr_qgemm_i4_tc_f16,    320, 1, 1},
    {"lux_qgemm_i4_tc_wa_bf16",    luxcuda::kernel_addr_qgemm_i4_tc_wa_bf16, 320, 1, 1},
    {"lux_qgemm_i4_tc_wa_f16",     luxcuda::kernel_addr_qgemm_i4_tc_wa_f16,  320, 1, 1},
    {"lux_qgemm_i4_tc_wa_bf16_swiglu", luxcuda::kernel_addr_qgemm_i4_tc_wa_bf16_swiglu, 320, 1, 1},
    {"lux_qgemm_i4_tc_wa_f16_swiglu",  luxcuda::kernel_addr_qgemm_i4_tc_wa_f16_swiglu,  320, 1, 1},
    {"lux_qgemv_i4_g128_units_fx_swiglu", luxcuda::kernel_addr_qgemv_i4_units_fx_swiglu, 512, 1, 1},
    {"lux_qgemv_i4_g128_units_fx_batch2", luxcuda::kernel_addr_qgemv_i4_units_fx_batch2, 512, 1, 1},
    {"lux_qgemv_i4_g128_units_fx_batch4", luxcuda::kernel_addr_qgemv_i4_units_fx_batch4, 512, 1, 1},
    {"lux_matmul_int8_tcgen05",    luxcuda::kernel_addr_matmul_int8_tcgen05, 192, 1, 1},
    {"lux_attn_stream_f32",        luxcuda::kernel_addr_attn_stream_f32,    288, 1, 1},
    {"lux_attn_merge_f32",         luxcuda::kernel_addr_attn_merge_f32,     128, 1, 1},
    {"lux_attn_plain_f32",         luxcuda::kernel_addr_attn_plain_f32,     256, 1, 1},
    {"lux_rope_f32",               luxcuda::kernel_addr_rope_f32,           256, 1, 1},
    {"lux_kv_append_f32",          luxcuda::kernel_addr_kv_append_f32,      256, 1, 1},
};
constexpr size_t kCount = sizeof(kTable) / sizeof(kTable[0]);

// Mirrors WgpuKernel{..., entry_point, workgroup_size_*} (webgpu_kernel_loader.cpp:28-42).
struct CudaKernel {
    const Entry* entry;
    const void* fn;
};

}  // namespace

extern "C" {

LuxKernel* lux_cuda_kernel_get(const char* entry_point) {
    if (!entry_point) return nullptr;
    for (size_t i = 0; i < kCount; i++) {
        if (std::strcmp(kTable[i].name, entry_point) == 0) {
            auto* k = new (std::nothrow) CudaKernel{&kTable[i], kTable[i].addr()};
            return reinterpret_cast<LuxKernel*>(k);
        }
    }
    return nullptr;
}

void lux_cuda_kernel_destroy(LuxKernel* kernel) { delete reinterpret_cast<CudaKernel*>(kernel); }

const char* lux_cuda_kernel_entry_point(LuxKernel* kernel) {
    auto* k = reinterpret_cast<CudaKernel*>(kernel);
    return k ? k->entry->name : nullptr;
}

const void* lux_cuda_kernel_function(LuxKernel* kernel) {
    auto* k = reinterpret_cast<CudaKernel*>(kernel);
    return k ? k->fn : nullptr;
}

LuxBackendError lux_cuda_kernel_attributes(LuxKernel* kernel, LuxCudaKernelAttributes* out) {
    auto* k = reinterpret_cast<CudaKernel*>(kernel);
    if (!k || !out) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    cudaFuncAttributes fa{};
    if (cudaFuncGetAttributes(&fa, k->fn) != cudaSuccess) {
        cudaGetLastError();
        return LUX_BACKEND_ERROR_INTERNAL;
    }
    out->registers_per_thread = fa.numRegs;
    out->static_smem_bytes = (int)fa.sharedSizeBytes;
    out->max_dynamic_smem_bytes = fa.maxDynamicSharedSizeBytes;
    out->max_threads_per_block = fa.maxThreadsPerBlock;
    out->const_bytes = (int)fa.constSizeBytes;
    out->local_bytes = (int)fa.localSizeBytes;
    out->binary_arch = fa.binaryVersion;
    return LUX_BACKEND_OK;
}

void lux_cuda_kernel_workgroup_size(LuxKernel* kernel, uint32_t* x, uint32_t* y, uint32_t* z) {
    auto* k = reinterpret_cast<CudaKernel*>(kernel);
    if (x) *x = k ? k->entry->bx : 1;
    if (y) *y = k ? k->entry->by : 1;
    if (z) *z = k ? k->entry->bz : 1;
}

size_t lux_cuda_kernel_count(void) { return kCount; }

const char* lux_cuda_kernel_name(size_t index) { return index < kCount ? kTable[index].name : nullptr; }

}  // extern "C"
