// lux_cuda_qmlp_noalloc -- the quantized FFN for callers that must not allocate.
//
// lux_cuda_qmlp needs an M x I scratch buffer for the SwiGLU output between its two
// matmuls, and its callers normally get that buffer from buffer_alloc (cudaMalloc).  Some
// hosts cannot do that at the point where they call the FFN: a serving loop that has
// handed every byte of device memory to its own arena at start-up (a later cudaMalloc
// fails or fragments the arena), and latency-critical decode steps, where cudaMalloc /
// cudaFree synchronise the whole device and would stall every stream.  For them the
// scratch lives in this library's own image: a fixed-size __device__ array that exists
// from the moment the library is loaded on a GPU until the process exits.
//
// Consequences the caller must know:
//   * the array is ONE per device and is shared by every call: two calls that overlap on
//     the GPU (different streams or contexts of the same device) race on it;
//   * its contents persist from call to call; this entry point overwrites the M x I region
//     it uses before reading it, so nothing needs clearing;
//   * M * I * 2 bytes must fit in LUX_QMLP_NOALLOC_MAX_BYTES, otherwise the call is
//     rejected with LUX_BACKEND_ERROR_INVALID_ARGUMENT;
//   * the first call on a device looks up the array's device address
//     (cudaGetSymbolAddress); make that first call outside any stream capture.
#include "common.cuh"

#include <mutex>

using namespace luxcuda;

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address is fetched below, once per device.
static __device__ __align__(256) unsigned char g_qmlp_scratch[LUX_QMLP_NOALLOC_MAX_BYTES];

namespace {

std::mutex g_scratch_mu;
void* g_scratch_ptr[64] = {};      // device address of g_qmlp_scratch, per device ordinal

// Returns the device address of the scratch array on `device` (which must be current).
LuxBackendError scratch_address(int device, void** out) {
    if (device < 0 || device >= 64) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_ptr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_qmlp_scratch);
        if (e != cudaSuccess || !ptr) {
            std::fprintf(stderr, "[lux-cuda] lux_cuda_qmlp_noalloc: cudaGetSymbolAddress failed: %s\n",
                         cudaGetErrorString(e));
            cudaGetLastError();
            return LUX_BACKEND_ERROR_INTERNAL;
        }
        g_scratch_ptr[device] = ptr;
    }
    *out = g_scratch_ptr[device];
    return LUX_BACKEND_OK;
}

}  // namespace

extern "C" LuxBackendError lux_cuda_qmlp_noalloc(
    LuxBackendContext* context, const LuxQMlpDesc* d, LuxBackendBuffer* x,
    LuxBackendBuffer* w_gate_up, LuxBackendBuffer* s_gate_up, LuxBackendBuffer* z_gate_up,
    LuxBackendBuffer* w_down, LuxBackendBuffer* s_down, LuxBackendBuffer* z_down, LuxBackendBuffer* y) {
    Context* ctx = as_ctx(context);
    if (!ctx || !d || d->struct_size < sizeof(LuxQMlpDesc)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t need = (size_t)d->M * d->I * 2;
    if (d->M == 0 || d->I == 0 || need > (size_t)LUX_QMLP_NOALLOC_MAX_BYTES) {
        std::fprintf(stderr,
                     "[lux-cuda] lux_cuda_qmlp_noalloc: M*I*2 = %zu bytes does not fit the built-in scratch of %zu bytes; "
                     "use lux_cuda_qmlp with a caller-provided buffer\n",
                     need, (size_t)LUX_QMLP_NOALLOC_MAX_BYTES);
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (cudaSetDevice(ctx->device) != cudaSuccess) {
        cudaGetLastError();
        return LUX_BACKEND_ERROR_INTERNAL;
    }
    void* scratch = nullptr;
    LuxBackendError e = scratch_address(ctx->device, &scratch);
    if (e != LUX_BACKEND_OK) return e;
    // A buffer handle on the stack that points at the built-in array: nothing is allocated,
    // and the two-launch FFN runs exactly as it does with a caller-provided scratch.
    Buffer h{scratch, need, ctx->device, false};
    return lux_cuda_qmlp(context, d, x, w_gate_up, s_gate_up, z_gate_up, w_down, s_down, z_down,
                         reinterpret_cast<LuxBackendBuffer*>(&h), y);
}
