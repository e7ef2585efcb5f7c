/*
 * lux/gpu/backend_plugin.h -- backend plugin boundary of luxcpp/gpu, RECONSTRUCTED.
 *
 * The original header belongs to the sibling project luxcpp/gpu and is not shipped with
 * luxcpp/webgpu.  Every declaration below was rebuilt from the way the WebGPU plugin
 * uses it (citations are paths inside luxcpp/webgpu):
 *
 *   - vtable slot order and signatures ..... src/webgpu_plugin.cpp:4022-4123 and the
 *                                            defining functions cited per slot
 *   - descriptor fields ..................... src/webgpu_plugin.cpp:4129-4152
 *   - device-info fields .................... src/webgpu_plugin.cpp:1369-1389
 *   - error enumerators ..................... used throughout src/webgpu_plugin.cpp
 *   - capability bits ....................... docs/architecture.md:111-124
 *   - entry-point name ...................... README.md:281-282, docs/architecture.md:89-107
 *
 * UNPINNED VALUES.  Three things cannot be observed from the plugin source and are
 * therefore guesses, isolated here so that a maintainer with the real header can fix
 * them in one place (or simply compile this backend against the real header, which the
 * build supports with -DLUX_GPU_USE_SYSTEM_BACKEND_PLUGIN_H):
 *     1. LUX_GPU_BACKEND_ABI_VERSION (plugin comments call the current ABI "v3"),
 *     2. the numeric values of LuxBackendError (docs/api.md:662-670 used as the hint),
 *     3. the declaration order of lux_gpu_backend_desc and LuxBackendDeviceInfo fields
 *        (assignment order in the plugin, and docs/api.md:32-43, used as the hint).
 * The vtable slot ORDER is pinned: C++20 designated initialisers must follow declaration
 * order, and the plugin spells out all 65 slots.
 */
#ifndef LUX_GPU_BACKEND_PLUGIN_H
#define LUX_GPU_BACKEND_PLUGIN_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* -- unpinned: see the header comment ------------------------------------------------ */
#ifndef LUX_GPU_BACKEND_ABI_VERSION
#define LUX_GPU_BACKEND_ABI_VERSION 3u
#endif

typedef enum LuxBackendError {
    LUX_BACKEND_OK                     = 0,
    LUX_BACKEND_ERROR_INVALID_ARGUMENT = 1,
    LUX_BACKEND_ERROR_OUT_OF_MEMORY    = 2,
    LUX_BACKEND_ERROR_INTERNAL         = 3,
    LUX_BACKEND_ERROR_DEVICE_LOST      = 4,
    LUX_BACKEND_ERROR_KERNEL_FAILED    = 5,
    LUX_BACKEND_ERROR_NOT_SUPPORTED    = 6
} LuxBackendError;

/* -- capability bits (docs/architecture.md:111-124) ---------------------------------- */
#define LUX_CAP_TENSOR_OPS     (1u << 0)
#define LUX_CAP_MATMUL         (1u << 1)
#define LUX_CAP_NTT            (1u << 2)
#define LUX_CAP_MSM            (1u << 3)
#define LUX_CAP_CUSTOM_KERNELS (1u << 4)
#define LUX_CAP_UNIFIED_MEMORY (1u << 5)
#define LUX_CAP_FHE            (1u << 6)
#define LUX_CAP_TFHE           (1u << 7)
#define LUX_CAP_BLS12_381      (1u << 12)
#define LUX_CAP_BN254          (1u << 13)
#define LUX_CAP_KZG            (1u << 14)
#define LUX_CAP_POSEIDON2      (1u << 15)
/* Used by the plugin (src/webgpu_plugin.cpp:4145-4146) but undocumented: bit positions
 * are guesses.  This backend never advertises them. */
#define LUX_CAP_POLY_MUL       (1u << 8)
#define LUX_CAP_BLIND_ROTATE   (1u << 9)

/* -- opaque handles (the plugin reinterpret_casts its own structs,
 *    src/webgpu_plugin.cpp:1310, 1452) ------------------------------------------------ */
typedef struct LuxBackendContext LuxBackendContext;
typedef struct LuxBackendBuffer  LuxBackendBuffer;
typedef struct LuxBackendKernel  LuxBackendKernel;   /* dead since ABI v3 (:1569) */

/* Fields written at src/webgpu_plugin.cpp:1375-1382; order unpinned. */
typedef struct LuxBackendDeviceInfo {
    const char* name;               /* points into context-owned storage */
    const char* vendor;
    uint64_t    memory_total;
    uint64_t    memory_available;
    bool        is_discrete;
    bool        is_unified_memory;
    int         compute_units;
    int         max_workgroup_size;
} LuxBackendDeviceInfo;

/* -- the 65-slot vtable, in the plugin's order ---------------------------------------- */
typedef struct lux_gpu_backend_vtbl {
    /* lifecycle (src/webgpu_plugin.cpp:1218, 1317) */
    LuxBackendContext* (*create_context)(int device_index);
    void               (*destroy_context)(LuxBackendContext*);

    /* device info & sync (:1359, 1369, 1391) */
    LuxBackendError (*get_device_count)(int* count);
    LuxBackendError (*get_device_info)(LuxBackendContext*, LuxBackendDeviceInfo*);
    LuxBackendError (*sync)(LuxBackendContext*);

    /* buffers (:1433-1566) */
    LuxBackendBuffer* (*buffer_alloc)(LuxBackendContext*, size_t bytes);
    LuxBackendBuffer* (*buffer_alloc_with_data)(LuxBackendContext*, const void* data, size_t bytes);
    void              (*buffer_free)(LuxBackendContext*, LuxBackendBuffer*);
    LuxBackendError   (*buffer_copy_to_host)(LuxBackendContext*, LuxBackendBuffer*, void* dst, size_t bytes);
    LuxBackendError   (*buffer_copy_from_host)(LuxBackendContext*, LuxBackendBuffer*, const void* src, size_t bytes);
    void*             (*buffer_get_host_ptr)(LuxBackendContext*, LuxBackendBuffer*);

    /* f32 tensor ops.  add / sub / mul / matmul are wired in the plugin (:1694-1771) and their
     * signatures are observed.  The other slots of this block are nullptr there (:4044-4072), so
     * their parameter lists CANNOT be observed: the ones below are this reconstruction's choice,
     * made to match the wired ops (buffers first, sizes last) and the parameter blocks of the
     * shaders that would back them (unary.wgsl, copy.wgsl, softmax.wgsl, logsumexp.wgsl,
     * layer_norm.wgsl, rms_norm.wgsl).  UNPINNED like the values at the top of this header: a
     * maintainer with the real header either confirms them or builds this backend with
     * -DLUX_CUDA_F32_SLOTS_NULL, which leaves these slots nullptr exactly as the WebGPU plugin does
     * (the same functions stay reachable as lux_cuda_op_* symbols, qmatmul_ext.h).  The six
     * reduction slots stay untyped and nullptr. */
    LuxBackendError (*op_add_f32)(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_sub_f32)(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_mul_f32)(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_div_f32)(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, size_t n);

    LuxBackendError (*op_matmul_f32)(LuxBackendContext*, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out, int M, int K, int N);
    /* out[cols, rows] = in[rows, cols]^T */
    LuxBackendError (*op_transpose_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, int rows, int cols);

    void* op_reduce_sum_f32;
    void* op_reduce_max_f32;
    void* op_reduce_min_f32;
    void* op_reduce_mean_f32;
    void* op_reduce_sum_axis_f32;
    void* op_reduce_max_axis_f32;

    /* over the last axis of [batch, dim] */
    LuxBackendError (*op_softmax_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim);
    LuxBackendError (*op_log_softmax_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim);

    LuxBackendError (*op_exp_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_log_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_sqrt_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_neg_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_abs_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_tanh_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_sigmoid_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_relu_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);
    LuxBackendError (*op_gelu_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n);

    LuxBackendError (*op_copy_f32)(LuxBackendContext*, LuxBackendBuffer* src, LuxBackendBuffer* dst, size_t n);

    /* over the last axis of [batch, dim]; gamma, beta, weight are [dim] */
    LuxBackendError (*op_layer_norm_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* gamma, LuxBackendBuffer* beta,
                                         LuxBackendBuffer* out, size_t batch, size_t dim, float eps);
    LuxBackendError (*op_rms_norm_f32)(LuxBackendContext*, LuxBackendBuffer* in, LuxBackendBuffer* weight, LuxBackendBuffer* out,
                                       size_t batch, size_t dim, float eps);

    /* NTT (:1773, 1918) */
    LuxBackendError (*op_ntt_forward)(LuxBackendContext*, uint64_t* data, size_t n, uint64_t modulus);
    LuxBackendError (*op_ntt_inverse)(LuxBackendContext*, uint64_t* data, size_t n, uint64_t modulus);

    /* FHE (:2130, 3380, 3410, 3430) */
    LuxBackendError (*op_poly_mul)(LuxBackendContext*, const uint64_t* a, const uint64_t* b, uint64_t* result, size_t n, uint64_t modulus);
    LuxBackendError (*op_tfhe_bootstrap)(LuxBackendContext*, const uint64_t* lwe_in, uint64_t* lwe_out, const uint64_t* bsk, const uint64_t* test_poly,
                                         uint32_t n_lwe, uint32_t N, uint32_t k, uint32_t l, uint32_t base_log, uint64_t q);
    LuxBackendError (*op_tfhe_keyswitch)(LuxBackendContext*, const uint64_t* lwe_in, uint64_t* lwe_out, const uint64_t* ksk,
                                         uint32_t n_in, uint32_t n_out, uint32_t l, uint32_t base_log, uint64_t q);
    LuxBackendError (*op_blind_rotate)(LuxBackendContext*, uint64_t* acc, const uint64_t* bsk, const uint64_t* lwe_a,
                                       uint32_t n_lwe, uint32_t N, uint32_t k, uint32_t l, uint32_t base_log, uint64_t q);

    /* hashes (:3605, 3658, 3715) */
    LuxBackendError (*op_poseidon2_hash)(LuxBackendContext*, const uint64_t* in, uint64_t* out, size_t rate, size_t num_hashes);
    LuxBackendError (*op_blake3_hash)(LuxBackendContext*, const uint8_t* in, uint8_t* out, const size_t* lens, size_t n);
    LuxBackendError (*op_keccak256_hash)(LuxBackendContext*, const uint8_t* in, uint8_t* out, const size_t* lens, size_t n);

    /* curves (:3775-3915) */
    LuxBackendError (*op_bls12_381_add)(LuxBackendContext*, const void* a, const void* b, void* out, size_t n, bool is_g2);
    LuxBackendError (*op_bls12_381_mul)(LuxBackendContext*, const void* pts, const void* scalars, void* out, size_t n, bool is_g2);
    LuxBackendError (*op_bls12_381_pairing)(LuxBackendContext*, const void* g1, const void* g2, void* out, size_t n);
    LuxBackendError (*op_bn254_add)(LuxBackendContext*, const void* a, const void* b, void* out, size_t n, bool is_g2);
    LuxBackendError (*op_bn254_mul)(LuxBackendContext*, const void* pts, const void* scalars, void* out, size_t n, bool is_g2);

    /* MSM (:2074) */
    LuxBackendError (*op_msm)(LuxBackendContext*, const void* scalars, const void* points, void* result, size_t n, int curve_type);

    /* KZG (:3948-3958) */
    LuxBackendError (*op_kzg_commit)(LuxBackendContext*, const void*, const void*, void*, size_t, int);
    LuxBackendError (*op_kzg_open)(LuxBackendContext*, const void*, const void*, const void*, void*, size_t, int);
    LuxBackendError (*op_kzg_verify)(LuxBackendContext*, const void*, const void*, const void*, const void*, const void*, bool*, int);

    /* ecrecover (:3960) */
    LuxBackendError (*op_ecrecover_batch)(LuxBackendContext*, const void*, void*, size_t);

    /* post-quantum / threshold / Schnorr batches (:3973-4016): every one is a callable
     * NOT_SUPPORTED stub in the plugin ("CPU backend handles these"), with these parameters. */
    LuxBackendError (*op_mldsa_verify_batch)(LuxBackendContext*, const uint8_t* const* pks, const uint8_t* const* msgs,
                                             const uint8_t* const* sigs, bool* results, size_t n);
    LuxBackendError (*op_mlkem_decapsulate_batch)(LuxBackendContext*, const uint8_t* const* sks, const uint8_t* const* cts,
                                                  uint8_t** shared, size_t n);
    LuxBackendError (*op_slhdsa_verify_batch)(LuxBackendContext*, const uint8_t* const* pks, const uint8_t* const* msgs,
                                              const uint8_t* const* sigs, bool* results, size_t n);
    LuxBackendError (*op_ringtail_partial_sign_batch)(LuxBackendContext*, const uint8_t* const* shares,
                                                      const uint8_t* const* msgs, uint8_t** partials, size_t n);
    LuxBackendError (*op_ringtail_combine_batch)(LuxBackendContext*, const uint8_t* const* partials, const int32_t* indices,
                                                 uint8_t** sigs, size_t n, size_t threshold);
    LuxBackendError (*op_frost_partial_verify_batch)(LuxBackendContext*, const uint8_t* const*, const uint8_t* const*,
                                                     const uint8_t* const*, const uint8_t* const*, bool* results, size_t n);
    LuxBackendError (*op_cggmp21_partial_sign_batch)(LuxBackendContext*, const uint8_t* const* shares, const uint8_t* msg_hash,
                                                     uint8_t** partials, size_t n);
    LuxBackendError (*op_ed25519_verify_batch)(LuxBackendContext*, const uint8_t* const* pks, const uint8_t* const* msgs,
                                               const uint8_t* const* sigs, bool* results, size_t n);
    LuxBackendError (*op_sr25519_verify_batch)(LuxBackendContext*, const uint8_t* const* pks, const uint8_t* const* msgs,
                                               const uint8_t* const* sigs, bool* results, size_t n);
} lux_gpu_backend_vtbl;

#define LUX_GPU_BACKEND_VTBL_SLOTS 65

/* Filled by lux_gpu_backend_init (src/webgpu_plugin.cpp:4132-4147); order unpinned. */
typedef struct lux_gpu_backend_desc {
    uint32_t                    abi_version;
    uint32_t                    vtbl_size;
    const char*                 backend_name;
    const char*                 backend_version;
    uint64_t                    capabilities;
    const lux_gpu_backend_vtbl* vtbl;
} lux_gpu_backend_desc;

typedef bool (*lux_gpu_backend_init_fn)(lux_gpu_backend_desc* out);

#if defined(_WIN32)
#define LUX_GPU_PLUGIN_EXPORT __declspec(dllexport)
#else
#define LUX_GPU_PLUGIN_EXPORT __attribute__((visibility("default")))
#endif

/* Same shape as the macro the plugin ends with (src/webgpu_plugin.cpp:4154): exports
 * the one symbol the loader resolves with dlsym. */
#define LUX_GPU_DECLARE_BACKEND(impl_fn)                                              \
    extern "C" LUX_GPU_PLUGIN_EXPORT bool lux_gpu_backend_init(lux_gpu_backend_desc* out) { \
        return impl_fn(out);                                                          \
    }

#ifdef __cplusplus
}
#endif

#endif /* LUX_GPU_BACKEND_PLUGIN_H */
