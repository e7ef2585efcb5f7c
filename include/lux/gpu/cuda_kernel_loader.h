/*
 * lux/gpu/cuda_kernel_loader.h -- kernel table of libluxgpu_backend_cuda.so.
 *
 * Counterpart of the seven lux_wgpu_kernel_* functions
 * (luxcpp/webgpu src/webgpu_kernel_loader.cpp:205-291).  The WebGPU loader compiles
 * WGSL text at run time into a WgpuKernel{module, pipeline, layout, entry_point,
 * workgroup size}; this backend ships every kernel precompiled for sm_100a inside the
 * shared library, so "compile" becomes a lookup by entry-point name and the handle
 * carries the launchable function plus its static resource usage.
 */
#ifndef LUX_GPU_CUDA_KERNEL_LOADER_H
#define LUX_GPU_CUDA_KERNEL_LOADER_H

#include <stddef.h>
#include <stdint.h>

#include "lux/gpu/backend_plugin.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct LuxKernel LuxKernel;   /* opaque, as in lux/gpu/kernel_loader.h */

typedef struct LuxCudaKernelAttributes {
    int registers_per_thread;
    int static_smem_bytes;
    int max_dynamic_smem_bytes;
    int max_threads_per_block;
    int const_bytes;
    int local_bytes;          /* per-thread spill + stack */
    int binary_arch;          /* e.g. 100 */
} LuxCudaKernelAttributes;

/* Replaces lux_wgpu_kernel_compile / lux_wgpu_kernel_load_file (:209-248): there is no
 * source to compile, so the kernel is found by entry-point name.  NULL if unknown.
 * The handle must be released with lux_cuda_kernel_destroy. */
LUX_GPU_PLUGIN_EXPORT LuxKernel* lux_cuda_kernel_get(const char* entry_point);

/* lux_wgpu_kernel_destroy (:250). */
LUX_GPU_PLUGIN_EXPORT void lux_cuda_kernel_destroy(LuxKernel* kernel);

/* lux_wgpu_kernel_entry_point (:254-257). */
LUX_GPU_PLUGIN_EXPORT const char* lux_cuda_kernel_entry_point(LuxKernel* kernel);

/* lux_wgpu_kernel_pipeline (:260-270): the launchable object.  Here: the address
 * cudaLaunchKernel / cudaFuncGetAttributes accept. */
LUX_GPU_PLUGIN_EXPORT const void* lux_cuda_kernel_function(LuxKernel* kernel);

/* lux_wgpu_kernel_bind_group_layout (:273-283) describes how resources bind; a CUDA
 * kernel's counterpart is its static resource usage.  Needs a current CUDA device;
 * returns LUX_BACKEND_ERROR_INTERNAL if the attributes cannot be queried. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_kernel_attributes(LuxKernel* kernel, LuxCudaKernelAttributes* out);

/* lux_wgpu_kernel_workgroup_size (:286-298): threads per block this kernel is
 * launched with; (1,1,1) for a NULL handle, like the reference. */
LUX_GPU_PLUGIN_EXPORT void lux_cuda_kernel_workgroup_size(LuxKernel* kernel, uint32_t* x, uint32_t* y, uint32_t* z);

/* Enumeration (the reference iterates a registry, :363-370). */
LUX_GPU_PLUGIN_EXPORT size_t      lux_cuda_kernel_count(void);
LUX_GPU_PLUGIN_EXPORT const char* lux_cuda_kernel_name(size_t index);

#ifdef __cplusplus
}
#endif

#endif /* LUX_GPU_CUDA_KERNEL_LOADER_H */
