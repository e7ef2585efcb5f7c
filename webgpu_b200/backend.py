"""Host-side loader for ``libluxgpu_backend_cuda.so``.

Plays the part luxcpp/gpu's plugin loader plays for the reference: ``dlopen`` the
backend, resolve ``lux_gpu_backend_init``, check the descriptor, and call through the
vtable (luxcpp/webgpu docs/architecture.md:87-107, README.md:11-14).  The quantized
matmul entry points are resolved from the same handle, the way a host resolves the
reference's ``lux_wgpu_kernel_*`` symbols (src/webgpu_kernel_loader.cpp:205-291).

Everything here is ctypes over the C ABI declared in ``include/lux/gpu/*.h``; there is
no CPU fallback: if the shared library is missing or a call is not supported, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libluxgpu_backend_cuda.so")

# -- mirrors of include/lux/gpu/backend_plugin.h -----------------------------------------

ABI_VERSION = 3
VTBL_SLOTS = 65

OK, INVALID_ARGUMENT, OUT_OF_MEMORY, INTERNAL, DEVICE_LOST, KERNEL_FAILED, NOT_SUPPORTED = range(7)
ERROR_NAMES = {
    OK: "LUX_BACKEND_OK", INVALID_ARGUMENT: "LUX_BACKEND_ERROR_INVALID_ARGUMENT",
    OUT_OF_MEMORY: "LUX_BACKEND_ERROR_OUT_OF_MEMORY", INTERNAL: "LUX_BACKEND_ERROR_INTERNAL",
    DEVICE_LOST: "LUX_BACKEND_ERROR_DEVICE_LOST", KERNEL_FAILED: "LUX_BACKEND_ERROR_KERNEL_FAILED",
    NOT_SUPPORTED: "LUX_BACKEND_ERROR_NOT_SUPPORTED",
}

CAP_TENSOR_OPS, CAP_MATMUL, CAP_CUSTOM_KERNELS = 1 << 0, 1 << 1, 1 << 4

F32, F16, BF16 = 0, 1, 2
NOALLOC_MAX_BYTES = 1 << 20          # LUX_QMLP_NOALLOC_MAX_BYTES
FLAG_NO_SYNC, FLAG_SWIGLU, FLAG_WEIGHTS_VOLATILE, FLAG_QUANT_SHIFTED = 1, 2, 4, 8
FLAG_ATTN_CAUSAL, FLAG_ROPE_BACKWARD = 16, 32               # lux/gpu/attention_ext.h
ROUTE_NONE, ROUTE_GEMV_I8, ROUTE_SKINNY_I4, ROUTE_GEMM_I4_TC = range(4)

VTBL_FIELDS = [
    "create_context", "destroy_context", "get_device_count", "get_device_info", "sync",
    "buffer_alloc", "buffer_alloc_with_data", "buffer_free", "buffer_copy_to_host",
    "buffer_copy_from_host", "buffer_get_host_ptr",
    "op_add_f32", "op_sub_f32", "op_mul_f32", "op_div_f32", "op_matmul_f32", "op_transpose_f32",
    "op_reduce_sum_f32", "op_reduce_max_f32", "op_reduce_min_f32", "op_reduce_mean_f32",
    "op_reduce_sum_axis_f32", "op_reduce_max_axis_f32", "op_softmax_f32", "op_log_softmax_f32",
    "op_exp_f32", "op_log_f32", "op_sqrt_f32", "op_neg_f32", "op_abs_f32", "op_tanh_f32",
    "op_sigmoid_f32", "op_relu_f32", "op_gelu_f32", "op_copy_f32", "op_layer_norm_f32",
    "op_rms_norm_f32", "op_ntt_forward", "op_ntt_inverse", "op_poly_mul", "op_tfhe_bootstrap",
    "op_tfhe_keyswitch", "op_blind_rotate", "op_poseidon2_hash", "op_blake3_hash",
    "op_keccak256_hash", "op_bls12_381_add", "op_bls12_381_mul", "op_bls12_381_pairing",
    "op_bn254_add", "op_bn254_mul", "op_msm", "op_kzg_commit", "op_kzg_open", "op_kzg_verify",
    "op_ecrecover_batch", "op_mldsa_verify_batch", "op_mlkem_decapsulate_batch",
    "op_slhdsa_verify_batch", "op_ringtail_partial_sign_batch", "op_ringtail_combine_batch",
    "op_frost_partial_verify_batch", "op_cggmp21_partial_sign_batch", "op_ed25519_verify_batch",
    "op_sr25519_verify_batch",
]
assert len(VTBL_FIELDS) == VTBL_SLOTS


class Vtbl(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in VTBL_FIELDS]


class BackendDesc(C.Structure):
    _fields_ = [
        ("abi_version", C.c_uint32), ("vtbl_size", C.c_uint32),
        ("backend_name", C.c_char_p), ("backend_version", C.c_char_p),
        ("capabilities", C.c_uint64), ("vtbl", C.POINTER(Vtbl)),
    ]


class DeviceInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char_p), ("vendor", C.c_char_p),
        ("memory_total", C.c_uint64), ("memory_available", C.c_uint64),
        ("is_discrete", C.c_bool), ("is_unified_memory", C.c_bool),
        ("compute_units", C.c_int), ("max_workgroup_size", C.c_int),
    ]


class QMatmulDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "struct_size", "M", "N", "K", "bits", "group_size", "x_dtype", "scale_dtype", "y_dtype", "flags")]


class QMlpDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "struct_size", "M", "K", "I", "H", "group_size", "act_dtype", "flags")]


class KernelAttributes(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "registers_per_thread", "static_smem_bytes", "max_dynamic_smem_bytes",
        "max_threads_per_block", "const_bytes", "local_bytes", "binary_arch")]


# Every symbol include/lux/gpu/*.h declares.
EXPORTED_SYMBOLS = [
    "lux_gpu_backend_init",
    "lux_cuda_qmatmul", "lux_cuda_qmatmul_host", "lux_cuda_qmatmul_route", "lux_cuda_qdequant",
    "lux_cuda_qunpack", "lux_cuda_qquantize", "lux_cuda_op_silu_f32", "lux_cuda_dynamic_quantize",
    "lux_cuda_matmul_int8", "lux_cuda_matmul_int4_int8", "lux_cuda_requantize_int32_to_int8", "lux_cuda_qmlp", "lux_cuda_qmlp_noalloc", "lux_cuda_context_set_stream", "lux_cuda_context_get_stream",
    "lux_cuda_buffer_wrap", "lux_cuda_buffer_device_ptr", "lux_cuda_buffer_size",
    "lux_cuda_launch_count", "lux_cuda_last_kernel_name", "lux_cuda_tune_set", "lux_cuda_last_device_status",
    "lux_cuda_kernel_get", "lux_cuda_kernel_destroy", "lux_cuda_kernel_entry_point",
    "lux_cuda_kernel_function", "lux_cuda_kernel_attributes", "lux_cuda_kernel_workgroup_size",
    "lux_cuda_kernel_count", "lux_cuda_kernel_name",
    "lux_cuda_peer_comm_create", "lux_cuda_peer_comm_connect", "lux_cuda_peer_comm_connect_ptrs",
    "lux_cuda_peer_comm_window", "lux_cuda_peer_comm_window_bytes", "lux_cuda_peer_allreduce",
    "lux_cuda_peer_comm_destroy", "lux_cuda_qmlp_tp",
    "lux_cuda_rope_precompute_cache_f32", "lux_cuda_rope_f32", "lux_cuda_rope_qk_f32", "lux_cuda_sdpa_f32",
    "lux_cuda_update_kv_cache_f32", "lux_cuda_sdpa_kv_cache_f32", "lux_cuda_paged_attention_f32",
]
PEER_HANDLE_BYTES = 64


class BackendError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {ERROR_NAMES.get(code, code)}")
        self.code = code


def _check(code: int, what: str) -> None:
    if code != OK:
        raise BackendError(code, what)


_vp, _sz, _int = C.c_void_p, C.c_size_t, C.c_int
_SIGS = {   # vtable slot -> (restype, argtypes); unwired slots are not callable
    "create_context": (_vp, [_int]),
    "destroy_context": (None, [_vp]),
    "get_device_count": (_int, [C.POINTER(_int)]),
    "get_device_info": (_int, [_vp, C.POINTER(DeviceInfo)]),
    "sync": (_int, [_vp]),
    "buffer_alloc": (_vp, [_vp, _sz]),
    "buffer_alloc_with_data": (_vp, [_vp, _vp, _sz]),
    "buffer_free": (None, [_vp, _vp]),
    "buffer_copy_to_host": (_int, [_vp, _vp, _vp, _sz]),
    "buffer_copy_from_host": (_int, [_vp, _vp, _vp, _sz]),
    "buffer_get_host_ptr": (_vp, [_vp, _vp]),
    "op_add_f32": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_sub_f32": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_mul_f32": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_matmul_f32": (_int, [_vp, _vp, _vp, _vp, _int, _int, _int]),
    "op_div_f32": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_transpose_f32": (_int, [_vp, _vp, _vp, _int, _int]),
    "op_softmax_f32": (_int, [_vp, _vp, _vp, _sz, _sz]),
    "op_log_softmax_f32": (_int, [_vp, _vp, _vp, _sz, _sz]),
    "op_exp_f32": (_int, [_vp, _vp, _vp, _sz]), "op_log_f32": (_int, [_vp, _vp, _vp, _sz]),
    "op_sqrt_f32": (_int, [_vp, _vp, _vp, _sz]), "op_neg_f32": (_int, [_vp, _vp, _vp, _sz]),
    "op_abs_f32": (_int, [_vp, _vp, _vp, _sz]), "op_tanh_f32": (_int, [_vp, _vp, _vp, _sz]),
    "op_sigmoid_f32": (_int, [_vp, _vp, _vp, _sz]), "op_relu_f32": (_int, [_vp, _vp, _vp, _sz]),
    "op_gelu_f32": (_int, [_vp, _vp, _vp, _sz]), "op_copy_f32": (_int, [_vp, _vp, _vp, _sz]),
    "op_layer_norm_f32": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float]),
    "op_rms_norm_f32": (_int, [_vp, _vp, _vp, _vp, _sz, _sz, C.c_float]),
    "op_ntt_forward": (_int, [_vp, _vp, _sz, C.c_uint64]),
    "op_msm": (_int, [_vp, _vp, _vp, _vp, _sz, _int]),
    "op_mldsa_verify_batch": (_int, [_vp, _vp, _vp, _vp, _vp, _sz]),
    "op_mlkem_decapsulate_batch": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_slhdsa_verify_batch": (_int, [_vp, _vp, _vp, _vp, _vp, _sz]),
    "op_ringtail_partial_sign_batch": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_ringtail_combine_batch": (_int, [_vp, _vp, _vp, _vp, _sz, _sz]),
    "op_frost_partial_verify_batch": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _sz]),
    "op_cggmp21_partial_sign_batch": (_int, [_vp, _vp, _vp, _vp, _sz]),
    "op_ed25519_verify_batch": (_int, [_vp, _vp, _vp, _vp, _vp, _sz]),
    "op_sr25519_verify_batch": (_int, [_vp, _vp, _vp, _vp, _vp, _sz]),
}


class Backend:
    """A loaded backend plugin: descriptor, vtable and extension entry points."""

    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} not found: build it with `make -C webgpu_b200/csrc` "
                "(or __graft_entry__.build()); there is no CPU fallback")
        self.path = path
        self.lib = C.CDLL(path, mode=C.RTLD_LOCAL)
        init = self.lib.lux_gpu_backend_init
        init.restype = C.c_bool
        init.argtypes = [C.POINTER(BackendDesc)]
        self.desc = BackendDesc()
        if not init(C.byref(self.desc)):
            raise RuntimeError("lux_gpu_backend_init returned false")
        if self.desc.abi_version != ABI_VERSION:
            raise RuntimeError(f"ABI version {self.desc.abi_version} != {ABI_VERSION}")
        if self.desc.vtbl_size != C.sizeof(Vtbl):
            raise RuntimeError(f"vtable size {self.desc.vtbl_size} != {C.sizeof(Vtbl)}")
        self.name = self.desc.backend_name.decode()
        self.version = self.desc.backend_version.decode()
        self.capabilities = int(self.desc.capabilities)
        self.vt = {}
        raw = self.desc.vtbl.contents
        for field in VTBL_FIELDS:
            addr = getattr(raw, field)
            if addr and field in _SIGS:
                res, args = _SIGS[field]
                self.vt[field] = C.CFUNCTYPE(res, *args)(addr)
            else:
                self.vt[field] = None
        self.raw_vtbl = raw
        L = self.lib
        bufs5 = [_vp] * 5
        L.lux_cuda_qmatmul.argtypes = [_vp, C.POINTER(QMatmulDesc)] + bufs5
        L.lux_cuda_qmatmul_host.argtypes = [_vp, C.POINTER(QMatmulDesc)] + bufs5
        L.lux_cuda_qmatmul_route.argtypes = [C.POINTER(QMatmulDesc), _int, C.POINTER(_int)]
        L.lux_cuda_qdequant.argtypes = [_vp, C.POINTER(QMatmulDesc), _vp, _vp, _vp, _vp]
        L.lux_cuda_qunpack.argtypes = [_vp, C.POINTER(QMatmulDesc), _vp, _vp, _vp]
        L.lux_cuda_qquantize.argtypes = [_vp, C.POINTER(QMatmulDesc), _vp, _vp, _vp, _vp]
        L.lux_cuda_op_silu_f32.argtypes = [_vp, _vp, _vp, _sz]
        L.lux_cuda_dynamic_quantize.argtypes = [_vp, _vp, _vp, _vp, _sz, C.c_uint32]
        L.lux_cuda_matmul_int8.argtypes = [_vp, _vp, _vp, _vp, _int, _int, _int]
        L.lux_cuda_matmul_int4_int8.argtypes = [_vp, _vp, _vp, _vp, _int, _int, _int]
        L.lux_cuda_requantize_int32_to_int8.argtypes = [_vp, _vp, _vp, _sz, C.c_float, C.c_float, C.c_int32]
        u32, f32 = C.c_uint32, C.c_float
        L.lux_cuda_rope_precompute_cache_f32.argtypes = [_vp, _vp, _vp, u32, u32, f32, u32]
        L.lux_cuda_rope_f32.argtypes = [_vp] * 6 + [u32] * 4 + [f32, u32, f32, u32]
        L.lux_cuda_rope_qk_f32.argtypes = [_vp] * 5 + [u32] * 7
        L.lux_cuda_sdpa_f32.argtypes = [_vp] * 6 + [u32] * 6 + [f32, u32]
        L.lux_cuda_update_kv_cache_f32.argtypes = [_vp] * 5 + [u32] * 7
        L.lux_cuda_sdpa_kv_cache_f32.argtypes = [_vp] * 5 + [u32] * 7 + [f32, u32]
        L.lux_cuda_paged_attention_f32.argtypes = [_vp] * 7 + [u32] * 6 + [f32, u32]
        L.lux_cuda_qmlp.argtypes = [_vp, C.POINTER(QMlpDesc)] + [_vp] * 9
        L.lux_cuda_qmlp_noalloc.argtypes = [_vp, C.POINTER(QMlpDesc)] + [_vp] * 8
        L.lux_cuda_peer_comm_create.restype = C.c_int
        L.lux_cuda_peer_comm_create.argtypes = [_vp, C.c_int, C.c_int, C.c_size_t, C.POINTER(_vp), _vp]
        L.lux_cuda_peer_comm_connect.restype = C.c_int
        L.lux_cuda_peer_comm_connect.argtypes = [_vp, _vp]
        L.lux_cuda_peer_comm_connect_ptrs.restype = C.c_int
        L.lux_cuda_peer_comm_connect_ptrs.argtypes = [_vp, C.POINTER(_vp)]
        L.lux_cuda_peer_comm_window.restype = _vp
        L.lux_cuda_peer_comm_window.argtypes = [_vp]
        L.lux_cuda_peer_comm_window_bytes.restype = C.c_size_t
        L.lux_cuda_peer_comm_window_bytes.argtypes = [_vp]
        L.lux_cuda_peer_allreduce.restype = C.c_int
        L.lux_cuda_peer_allreduce.argtypes = [_vp, _vp, _vp, C.c_size_t, C.c_uint32, C.c_uint32]
        L.lux_cuda_qmlp_tp.restype = C.c_int
        L.lux_cuda_qmlp_tp.argtypes = [_vp, C.POINTER(QMlpDesc)] + [_vp] * 10
        L.lux_cuda_peer_comm_destroy.restype = None
        L.lux_cuda_peer_comm_destroy.argtypes = [_vp]
        L.lux_cuda_context_set_stream.argtypes = [_vp, _vp]
        L.lux_cuda_context_get_stream.argtypes = [_vp]
        L.lux_cuda_context_get_stream.restype = _vp
        L.lux_cuda_buffer_wrap.argtypes = [_vp, _vp, _sz]
        L.lux_cuda_buffer_wrap.restype = _vp
        L.lux_cuda_buffer_device_ptr.argtypes = [_vp]
        L.lux_cuda_buffer_device_ptr.restype = _vp
        L.lux_cuda_buffer_size.argtypes = [_vp]
        L.lux_cuda_buffer_size.restype = _sz
        L.lux_cuda_launch_count.restype = C.c_uint64
        L.lux_cuda_last_kernel_name.restype = C.c_char_p
        L.lux_cuda_tune_set.argtypes = [C.c_char_p, _int]
        L.lux_cuda_last_device_status.argtypes = [_vp]
        L.lux_cuda_last_device_status.restype = C.c_uint32
        L.lux_cuda_kernel_get.argtypes = [C.c_char_p]
        L.lux_cuda_kernel_get.restype = _vp
        L.lux_cuda_kernel_destroy.argtypes = [_vp]
        L.lux_cuda_kernel_destroy.restype = None
        L.lux_cuda_kernel_entry_point.argtypes = [_vp]
        L.lux_cuda_kernel_entry_point.restype = C.c_char_p
        L.lux_cuda_kernel_function.argtypes = [_vp]
        L.lux_cuda_kernel_function.restype = _vp
        L.lux_cuda_kernel_attributes.argtypes = [_vp, C.POINTER(KernelAttributes)]
        L.lux_cuda_kernel_workgroup_size.argtypes = [_vp] + [C.POINTER(C.c_uint32)] * 3
        L.lux_cuda_kernel_workgroup_size.restype = None
        L.lux_cuda_kernel_count.restype = _sz
        L.lux_cuda_kernel_name.argtypes = [_sz]
        L.lux_cuda_kernel_name.restype = C.c_char_p

    # -- device-free queries ---------------------------------------------------------
    def device_count(self) -> int:
        n = _int(0)
        _check(self.vt["get_device_count"](C.byref(n)), "get_device_count")
        return n.value

    def route(self, desc: QMatmulDesc, has_zeros: bool) -> tuple[int, int]:
        r = _int(0)
        code = self.lib.lux_cuda_qmatmul_route(C.byref(desc), int(has_zeros), C.byref(r))
        return code, r.value

    def kernel_names(self) -> list[str]:
        return [self.lib.lux_cuda_kernel_name(i).decode() for i in range(self.lib.lux_cuda_kernel_count())]

    def launch_count(self) -> int:
        return int(self.lib.lux_cuda_launch_count())

    def last_kernel_name(self) -> str:
        """Which quantized-matmul kernel the library launched most recently."""
        return self.lib.lux_cuda_last_kernel_name().decode()

    def tune(self, key: str, value: int) -> None:
        _check(self.lib.lux_cuda_tune_set(key.encode(), int(value)), f"tune_set({key})")

    def create_context(self, device_index: int = 0) -> "Context":
        h = self.vt["create_context"](device_index)
        if not h:
            raise RuntimeError(f"create_context({device_index}) failed: no sm_100 device at that index?")
        return Context(self, h)


_backend = None


def load(path: str = LIB_PATH) -> Backend:
    """Load (once per process) and return the backend."""
    global _backend
    if _backend is None or _backend.path != path:
        _backend = Backend(path)
    return _backend


def make_desc(M, N, K, bits, group, x_dtype, scale_dtype, y_dtype, flags=0) -> QMatmulDesc:
    return QMatmulDesc(C.sizeof(QMatmulDesc), M, N, K, bits, group, x_dtype, scale_dtype, y_dtype, flags)


def np_dtype_code(a: np.ndarray, bf16: bool = False) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(a.dtype)


_NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16}


class Buffer:
    """A LuxBackendBuffer handle.  Freed explicitly or when garbage-collected."""

    def __init__(self, ctx: "Context", handle: int, nbytes: int):
        self.ctx, self.handle, self.nbytes = ctx, handle, nbytes

    @property
    def device_ptr(self) -> int:
        return int(self.ctx.backend.lib.lux_cuda_buffer_device_ptr(self.handle) or 0)

    def to_host(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        _check(self.ctx.backend.vt["buffer_copy_to_host"](self.ctx.handle, self.handle, out.ctypes.data, out.nbytes),
               "buffer_copy_to_host")
        return out

    def from_host(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        _check(self.ctx.backend.vt["buffer_copy_from_host"](self.ctx.handle, self.handle, a.ctypes.data, a.nbytes),
               "buffer_copy_from_host")

    def free(self) -> None:
        if self.handle:
            self.ctx.backend.vt["buffer_free"](self.ctx.handle, self.handle)
            self.handle = None

    def __del__(self):
        try:
            if self.handle and self.ctx.handle:
                self.free()
        except Exception:
            pass


@dataclass
class DeviceQLayer:
    """Device-resident quantized layer (weights are model state: uploaded once)."""
    bits: int
    group: int
    N: int
    K: int
    w: Buffer
    scales: Buffer
    zeros: Buffer | None
    scale_dtype: int

    @property
    def weight_bytes(self) -> int:
        return self.w.nbytes + self.scales.nbytes + (self.zeros.nbytes if self.zeros else 0)


class Context:
    def __init__(self, backend: Backend, handle: int):
        self.backend, self.handle = backend, handle
        self._host_calls = {}

    # vtable wrappers
    def destroy(self) -> None:
        if self.handle:
            self.backend.vt["destroy_context"](self.handle)
            self.handle = None

    def device_info(self) -> dict:
        info = DeviceInfo()
        _check(self.backend.vt["get_device_info"](self.handle, C.byref(info)), "get_device_info")
        return {f: (getattr(info, f).decode() if isinstance(getattr(info, f), bytes) else getattr(info, f))
                for f, _ in DeviceInfo._fields_}

    def sync(self) -> None:
        _check(self.backend.vt["sync"](self.handle), "sync")

    def alloc(self, nbytes: int) -> Buffer:
        h = self.backend.vt["buffer_alloc"](self.handle, nbytes)
        if not h:
            raise BackendError(OUT_OF_MEMORY, f"buffer_alloc({nbytes})")
        return Buffer(self, h, nbytes)

    def upload(self, a: np.ndarray) -> Buffer:
        a = np.ascontiguousarray(a)
        h = self.backend.vt["buffer_alloc_with_data"](self.handle, a.ctypes.data, a.nbytes)
        if not h:
            raise BackendError(OUT_OF_MEMORY, f"buffer_alloc_with_data({a.nbytes})")
        return Buffer(self, h, a.nbytes)

    def wrap(self, device_ptr: int, nbytes: int) -> Buffer:
        h = self.backend.lib.lux_cuda_buffer_wrap(self.handle, device_ptr, nbytes)
        if not h:
            raise BackendError(INVALID_ARGUMENT, "lux_cuda_buffer_wrap")
        return Buffer(self, h, nbytes)

    CUDA_STREAM_LEGACY = 1      # cudaStreamLegacy: the handle that names the default stream explicitly

    def set_stream(self, stream_ptr: int | None) -> None:
        """None restores the context's own (non-blocking) stream.  0 is what frameworks report for
        the default stream; it is passed on as cudaStreamLegacy, because a NULL handle means
        "own stream" at the C boundary and work there would not be ordered with the caller's."""
        if stream_ptr is not None and stream_ptr == 0:
            stream_ptr = self.CUDA_STREAM_LEGACY
        _check(self.backend.lib.lux_cuda_context_set_stream(self.handle, stream_ptr), "set_stream")

    def binary_f32(self, op: str, a: Buffer, b: Buffer, out: Buffer, n: int) -> None:
        _check(self.backend.vt[f"op_{op}_f32"](self.handle, a.handle, b.handle, out.handle, n), f"op_{op}_f32")

    def unary_f32(self, op: str, x: Buffer, out: Buffer, n: int) -> None:
        """exp, log, sqrt, neg, abs, tanh, sigmoid, relu, gelu, copy through the vtable; silu through its symbol."""
        if op == "silu":
            _check(self.backend.lib.lux_cuda_op_silu_f32(self.handle, x.handle, out.handle, n), "lux_cuda_op_silu_f32")
        else:
            _check(self.backend.vt[f"op_{op}_f32"](self.handle, x.handle, out.handle, n), f"op_{op}_f32")

    def transpose_f32(self, x: Buffer, out: Buffer, rows: int, cols: int) -> None:
        _check(self.backend.vt["op_transpose_f32"](self.handle, x.handle, out.handle, rows, cols), "op_transpose_f32")

    def softmax_f32(self, x: Buffer, out: Buffer, batch: int, dim: int, log: bool = False) -> None:
        name = "op_log_softmax_f32" if log else "op_softmax_f32"
        _check(self.backend.vt[name](self.handle, x.handle, out.handle, batch, dim), name)

    def layer_norm_f32(self, x: Buffer, gamma: Buffer, beta: Buffer, out: Buffer, batch: int, dim: int, eps: float) -> None:
        _check(self.backend.vt["op_layer_norm_f32"](self.handle, x.handle, gamma.handle, beta.handle, out.handle, batch, dim, eps),
               "op_layer_norm_f32")

    def rms_norm_f32(self, x: Buffer, weight: Buffer, out: Buffer, batch: int, dim: int, eps: float) -> None:
        _check(self.backend.vt["op_rms_norm_f32"](self.handle, x.handle, weight.handle, out.handle, batch, dim, eps),
               "op_rms_norm_f32")

    def matmul_f32(self, a: Buffer, b: Buffer, out: Buffer, M: int, K: int, N: int) -> None:
        _check(self.backend.vt["op_matmul_f32"](self.handle, a.handle, b.handle, out.handle, M, K, N), "op_matmul_f32")

    # quantized extension
    def upload_layer(self, layer) -> DeviceQLayer:
        """layer: anything with bits, group, N, K, w, scales, zeros (numpy)."""
        z = self.upload(layer.zeros) if layer.zeros is not None else None
        return DeviceQLayer(layer.bits, layer.group, layer.N, layer.K, self.upload(layer.w),
                            self.upload(layer.scales), z, np_dtype_code(layer.scales))

    def _desc(self, L: DeviceQLayer, M: int, x_dtype: int, y_dtype: int, flags: int) -> QMatmulDesc:
        return make_desc(M, L.N, L.K, L.bits, L.group, x_dtype, L.scale_dtype, y_dtype, flags)

    def qmatmul(self, x: Buffer, L: DeviceQLayer, y: Buffer, M: int, x_dtype: int, y_dtype: int | None = None,
                flags: int = 0) -> None:
        d = self._desc(L, M, x_dtype, x_dtype if y_dtype is None else y_dtype, flags)
        _check(self.backend.lib.lux_cuda_qmatmul(self.handle, C.byref(d), x.handle, L.w.handle, L.scales.handle,
                                                 L.zeros.handle if L.zeros else None, y.handle), "lux_cuda_qmatmul")

    def qmatmul_host(self, x: np.ndarray, L: DeviceQLayer, y_dtype: int | None = None, flags: int = 0,
                     out: np.ndarray | None = None) -> np.ndarray:
        if not x.flags.c_contiguous:
            x = np.ascontiguousarray(x)
        M = x.shape[0]
        xd = np_dtype_code(x)
        yd = xd if y_dtype is None else y_dtype
        if out is None:
            out = np.empty((M, L.N // 2 if flags & FLAG_SWIGLU else L.N), _NP_OF[yd])
        # the descriptor and the weight handles of a (layer, batch, types) combination never change:
        # a decode loop pays for building them once
        key = (id(L), M, xd, yd, flags)
        hit = self._host_calls.get(key)
        if hit is None:
            d = self._desc(L, M, xd, yd, flags)
            hit = (C.byref(d), d, L.w.handle, L.scales.handle, L.zeros.handle if L.zeros else None, L)
            if len(self._host_calls) > 256:
                self._host_calls.clear()
            self._host_calls[key] = hit
        code = self.backend.lib.lux_cuda_qmatmul_host(self.handle, hit[0], x.ctypes.data, hit[2], hit[3], hit[4],
                                                      out.ctypes.data)
        if code != OK:
            raise BackendError(code, "lux_cuda_qmatmul_host")
        return out

    def qmatmul_host_bound(self, x: np.ndarray, L: DeviceQLayer, out: np.ndarray, y_dtype: int | None = None, flags: int = 0):
        """A decode loop's form of qmatmul_host: the arguments of lux_cuda_qmatmul_host for FIXED host
        arrays x and out are marshalled once, and the returned function makes the call (it reads x and
        fills out each time it is called; it returns out).  The arrays must stay alive and in place."""
        assert x.flags.c_contiguous and out.flags.c_contiguous and out.flags.writeable
        xd = np_dtype_code(x)
        d = self._desc(L, x.shape[0], xd, xd if y_dtype is None else y_dtype, flags)
        fn = self.backend.lib.lux_cuda_qmatmul_host
        args = (C.c_void_p(self.handle), C.byref(d), C.c_void_p(x.ctypes.data), C.c_void_p(L.w.handle), C.c_void_p(L.scales.handle),
                C.c_void_p(L.zeros.handle) if L.zeros else None, C.c_void_p(out.ctypes.data))
        keep = (d, x, out, L)

        def call(_fn=fn, _args=args, _keep=keep):
            code = _fn(*_args)
            if code != OK:
                raise BackendError(code, "lux_cuda_qmatmul_host")
            return _keep[2]
        return call

    def qdequant(self, L: DeviceQLayer, out_dtype: int = F32) -> np.ndarray:
        out = self.alloc(L.N * L.K * (4 if out_dtype == F32 else 2))
        d = self._desc(L, 0, F32, out_dtype, 0)
        _check(self.backend.lib.lux_cuda_qdequant(self.handle, C.byref(d), L.w.handle, L.scales.handle,
                                                  L.zeros.handle if L.zeros else None, out.handle), "lux_cuda_qdequant")
        res = out.to_host(_NP_OF[out_dtype], (L.N, L.K))
        out.free()
        return res

    def qunpack(self, L: DeviceQLayer) -> np.ndarray:
        out = self.alloc(L.N * L.K)
        d = self._desc(L, 0, F32, F32, 0)
        _check(self.backend.lib.lux_cuda_qunpack(self.handle, C.byref(d), L.w.handle,
                                                 L.zeros.handle if L.zeros else None, out.handle), "lux_cuda_qunpack")
        res = out.to_host(np.int8, (L.N, L.K))
        out.free()
        return res

    def qquantize(self, x: np.ndarray, bits: int, symmetric: bool = False, scale_dtype: int | None = None,
                  flags: int = 0) -> DeviceQLayer:
        """Quantizes a host matrix [N, K] (f32 / f16 / bf16 bit patterns) ON THE DEVICE into a layer the
        matmul entry points take (lux_cuda_qquantize)."""
        x = np.ascontiguousarray(x)
        N, K = x.shape
        group = 128 if bits == 4 else 32
        if scale_dtype is None:
            scale_dtype = F16 if bits == 4 else F32
        G = K // group
        xb = self.upload(x)
        w = self.alloc(N * K * bits // 8)
        sc = self.alloc(N * G * (4 if scale_dtype == F32 else 2))
        z = self.alloc(N * ((G + 1) // 2)) if (bits == 4 and not symmetric) else None
        d = make_desc(0, N, K, bits, group, np_dtype_code(x), scale_dtype, F32, flags)
        _check(self.backend.lib.lux_cuda_qquantize(self.handle, C.byref(d), xb.handle, w.handle, sc.handle,
                                                   z.handle if z else None), "lux_cuda_qquantize")
        return DeviceQLayer(bits, group, N, K, w, sc, z, scale_dtype)

    # activation-quantized integer path
    def dynamic_quantize(self, x: Buffer, out: Buffer, scale: Buffer, n: int, bits: int = 8) -> None:
        _check(self.backend.lib.lux_cuda_dynamic_quantize(self.handle, x.handle, out.handle, scale.handle, n, bits),
               "lux_cuda_dynamic_quantize")

    def matmul_int8(self, a: Buffer, b: Buffer, c: Buffer, M: int, N: int, K: int, a_bits: int = 8) -> None:
        fn = self.backend.lib.lux_cuda_matmul_int8 if a_bits == 8 else self.backend.lib.lux_cuda_matmul_int4_int8
        _check(fn(self.handle, a.handle, b.handle, c.handle, M, N, K), "lux_cuda_matmul_int8")

    def requantize(self, x: Buffer, out: Buffer, n: int, input_scale: float, output_scale: float, zero_point: int) -> None:
        _check(self.backend.lib.lux_cuda_requantize_int32_to_int8(self.handle, x.handle, out.handle, n, input_scale,
                                                                  output_scale, zero_point), "lux_cuda_requantize_int32_to_int8")

    # attention side (lux/gpu/attention_ext.h); every tensor is an f32 Buffer in the shader's layout
    def rope_precompute_cache(self, cos: Buffer, sin: Buffer, max_seq_len: int, head_dim: int, theta_base: float, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_rope_precompute_cache_f32(self.handle, cos.handle, sin.handle, max_seq_len, head_dim,
                                                                   theta_base, flags), "lux_cuda_rope_precompute_cache_f32")

    def rope(self, x: Buffer, out: Buffer, batch: int, seq: int, heads: int, head_dim: int, cos: Buffer | None = None,
             sin: Buffer | None = None, position_ids: Buffer | None = None, theta_base: float = 10000.0,
             position_offset: int = 0, ntk_scale: float = 0.0, flags: int = 0) -> None:
        h = lambda b: b.handle if b is not None else None
        _check(self.backend.lib.lux_cuda_rope_f32(self.handle, x.handle, out.handle, h(cos), h(sin), h(position_ids), batch, seq,
                                                  heads, head_dim, theta_base, position_offset, ntk_scale, flags), "lux_cuda_rope_f32")

    def rope_qk(self, q: Buffer, k: Buffer, cos: Buffer, sin: Buffer, batch: int, seq: int, heads: int, kv_heads: int,
                head_dim: int, position_offset: int = 0, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_rope_qk_f32(self.handle, q.handle, k.handle, cos.handle, sin.handle, batch, seq, heads,
                                                     kv_heads, head_dim, position_offset, flags), "lux_cuda_rope_qk_f32")

    def sdpa(self, q: Buffer, k: Buffer, v: Buffer, out: Buffer, batch: int, heads: int, kv_heads: int, seq_q: int, seq_kv: int,
             head_dim: int, scale: float, lse: Buffer | None = None, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_sdpa_f32(self.handle, q.handle, k.handle, v.handle, out.handle,
                                                  lse.handle if lse is not None else None, batch, heads, kv_heads, seq_q, seq_kv,
                                                  head_dim, scale, flags), "lux_cuda_sdpa_f32")

    def update_kv_cache(self, k: Buffer, v: Buffer, k_cache: Buffer, v_cache: Buffer, batch: int, kv_heads: int, seq_q: int,
                        cache_len: int, max_cache_len: int, head_dim: int, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_update_kv_cache_f32(self.handle, k.handle, v.handle, k_cache.handle, v_cache.handle, batch,
                                                             kv_heads, seq_q, cache_len, max_cache_len, head_dim, flags),
               "lux_cuda_update_kv_cache_f32")

    def sdpa_kv_cache(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, out: Buffer, batch: int, heads: int, kv_heads: int,
                      seq_q: int, cache_len: int, max_cache_len: int, head_dim: int, scale: float, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_sdpa_kv_cache_f32(self.handle, q.handle, k_cache.handle, v_cache.handle, out.handle, batch,
                                                           heads, kv_heads, seq_q, cache_len, max_cache_len, head_dim, scale, flags),
               "lux_cuda_sdpa_kv_cache_f32")

    def paged_attention(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, block_tables: Buffer, context_lens: Buffer, out: Buffer,
                        num_seqs: int, heads: int, kv_heads: int, head_dim: int, block_size: int, max_blocks_per_seq: int,
                        scale: float, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_paged_attention_f32(self.handle, q.handle, k_cache.handle, v_cache.handle,
                                                             block_tables.handle, context_lens.handle, out.handle, num_seqs, heads,
                                                             kv_heads, head_dim, block_size, max_blocks_per_seq, scale, flags),
               "lux_cuda_paged_attention_f32")

    def qmlp(self, x: Buffer, gate_up: DeviceQLayer, down: DeviceQLayer, h: Buffer, y: Buffer, M: int,
             act_dtype: int, flags: int = 0) -> None:
        d = QMlpDesc(C.sizeof(QMlpDesc), M, gate_up.K, gate_up.N // 2, down.N, gate_up.group, act_dtype, flags)
        z = lambda L: L.zeros.handle if L.zeros else None
        _check(self.backend.lib.lux_cuda_qmlp(self.handle, C.byref(d), x.handle, gate_up.w.handle,
                                              gate_up.scales.handle, z(gate_up), down.w.handle, down.scales.handle,
                                              z(down), h.handle, y.handle), "lux_cuda_qmlp")

    def qmlp_noalloc(self, x: Buffer, gate_up: DeviceQLayer, down: DeviceQLayer, y: Buffer, M: int,
                     act_dtype: int, flags: int = 0) -> None:
        """The FFN with the library's built-in scratch instead of a caller-provided one
        (for callers that must not allocate); M * I * 2 bytes must fit NOALLOC_MAX_BYTES."""
        d = QMlpDesc(C.sizeof(QMlpDesc), M, gate_up.K, gate_up.N // 2, down.N, gate_up.group, act_dtype, flags)
        z = lambda L: L.zeros.handle if L.zeros else None
        _check(self.backend.lib.lux_cuda_qmlp_noalloc(self.handle, C.byref(d), x.handle, gate_up.w.handle,
                                                      gate_up.scales.handle, z(gate_up), down.w.handle,
                                                      down.scales.handle, z(down), y.handle), "lux_cuda_qmlp_noalloc")

    def last_device_status(self) -> int:
        return int(self.backend.lib.lux_cuda_last_device_status(self.handle))

    # -- one-node push all-reduce over peer memory ------------------------------------------
    def peer_comm_create(self, rank: int, world: int, max_bytes: int):
        """Returns (communicator handle, 64-byte IPC handle to send to the other ranks)."""
        comm = _vp()
        handle = C.create_string_buffer(PEER_HANDLE_BYTES)
        _check(self.backend.lib.lux_cuda_peer_comm_create(self.handle, rank, world, max_bytes, C.byref(comm), handle),
               "lux_cuda_peer_comm_create")
        return comm, handle.raw

    def peer_comm_connect(self, comm, handles: bytes) -> None:
        """`handles`: every rank's 64-byte handle concatenated in rank order."""
        _check(self.backend.lib.lux_cuda_peer_comm_connect(comm, handles), "lux_cuda_peer_comm_connect")

    def peer_comm_connect_ptrs(self, comm, windows) -> None:
        arr = (_vp * len(windows))(*[_vp(w) for w in windows])
        _check(self.backend.lib.lux_cuda_peer_comm_connect_ptrs(comm, arr), "lux_cuda_peer_comm_connect_ptrs")

    def peer_comm_window(self, comm) -> int:
        return int(self.backend.lib.lux_cuda_peer_comm_window(comm) or 0)

    def peer_allreduce(self, comm, buf: "Buffer", count: int, dtype: int, flags: int = 0) -> None:
        _check(self.backend.lib.lux_cuda_peer_allreduce(self.handle, comm, buf.handle, count, dtype, flags),
               "lux_cuda_peer_allreduce")

    def qmlp_tp(self, x: "Buffer", gate_up: "DeviceQLayer", down: "DeviceQLayer", h: "Buffer", y: "Buffer", M: int,
                act_dtype: int, comm, flags: int = 0) -> None:
        """One rank's tensor-parallel FFN: lux_cuda_qmlp on its shards + the all-reduce of y through
        the push communicator (fused into the down kernel's epilogue at batch <= 2)."""
        d = QMlpDesc(C.sizeof(QMlpDesc), M, gate_up.K, gate_up.N // 2, down.N, gate_up.group, act_dtype, flags)
        z = lambda L: L.zeros.handle if L.zeros else None
        _check(self.backend.lib.lux_cuda_qmlp_tp(self.handle, C.byref(d), x.handle, gate_up.w.handle,
                                                 gate_up.scales.handle, z(gate_up), down.w.handle, down.scales.handle,
                                                 z(down), h.handle, y.handle, comm), "lux_cuda_qmlp_tp")

    def peer_comm_destroy(self, comm) -> None:
        self.backend.lib.lux_cuda_peer_comm_destroy(comm)

    def __del__(self):
        # Contexts are destroyed explicitly; buffers hold a reference to their context,
        # so tearing down here could run before a buffer's own finaliser.
        pass
