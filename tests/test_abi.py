"""The drop-in boundary, checked without a GPU: the shared library loads, exports every
symbol the headers declare, and its descriptor / vtable have the reference's shape
(luxcpp/webgpu src/webgpu_plugin.cpp:4022-4154)."""
import ctypes as C
import glob
import os
import re

import pytest

from webgpu_b200 import backend as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Of the 22 slots the reference's own vtable leaves nullptr (src/webgpu_plugin.cpp:4044-4072) this
# backend wires the sixteen either side of a linear layer; the six reductions stay nullptr.
REFERENCE_NULL_SLOTS = {
    "op_reduce_sum_f32", "op_reduce_max_f32", "op_reduce_min_f32",
    "op_reduce_mean_f32", "op_reduce_sum_axis_f32", "op_reduce_max_axis_f32",
}
WIRED_F32_SLOTS = {
    "op_div_f32", "op_transpose_f32", "op_softmax_f32", "op_log_softmax_f32", "op_exp_f32", "op_log_f32",
    "op_sqrt_f32", "op_neg_f32", "op_abs_f32", "op_tanh_f32", "op_sigmoid_f32", "op_relu_f32", "op_gelu_f32",
    "op_copy_f32", "op_layer_norm_f32", "op_rms_norm_f32",
}


def _declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "lux", "gpu", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"LUX_GPU_PLUGIN_EXPORT[^;(]*?\b(lux_\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_library_exports_every_declared_symbol(backend):
    declared = _declared_symbols()
    assert "lux_cuda_qmatmul" in declared and "lux_cuda_kernel_get" in declared
    declared.add("lux_gpu_backend_init")
    assert declared == set(B.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(backend.lib, name) is not None, name


def test_descriptor(backend):
    d = backend.desc
    assert d.abi_version == B.ABI_VERSION
    assert d.vtbl_size == 65 * C.sizeof(C.c_void_p)
    assert backend.name == "cuda"
    assert backend.capabilities & B.CAP_TENSOR_OPS and backend.capabilities & B.CAP_MATMUL
    # nothing out of scope is advertised (NTT 1<<2, MSM 1<<3, FHE 1<<6, TFHE 1<<7 ...)
    assert backend.capabilities & ~(B.CAP_TENSOR_OPS | B.CAP_MATMUL | B.CAP_CUSTOM_KERNELS) == 0


def test_vtable_slots(backend):
    raw = backend.raw_vtbl
    assert len(B.VTBL_FIELDS) == 65
    for field in B.VTBL_FIELDS:
        addr = getattr(raw, field)
        if field in REFERENCE_NULL_SLOTS:
            assert not addr, field
    for field in ("create_context", "destroy_context", "get_device_count", "get_device_info", "sync",
                  "buffer_alloc", "buffer_alloc_with_data", "buffer_free", "buffer_copy_to_host",
                  "buffer_copy_from_host", "buffer_get_host_ptr", "op_add_f32", "op_sub_f32", "op_mul_f32",
                  "op_matmul_f32", "op_ntt_forward", "op_msm", "op_kzg_verify", "op_ecrecover_batch"):
        assert getattr(raw, field), field
    for field in WIRED_F32_SLOTS:
        assert getattr(raw, field), field
        assert backend.vt[field] is not None, field
    assert backend.vt["op_exp_f32"](None, None, None, 4) == B.INVALID_ARGUMENT
    assert backend.vt["op_rms_norm_f32"](None, None, None, None, 1, 8, 1e-6) == B.INVALID_ARGUMENT
    # the post-quantum / threshold / Schnorr batches are callable stubs in the reference
    # (src/webgpu_plugin.cpp:3973-4016, 4110-4122), so a loader may call them without a null check
    for field in B.VTBL_FIELDS[56:]:
        assert getattr(raw, field), field


def test_out_of_scope_slots_answer_not_supported(backend):
    # the reference's "fall back to CPU" signal (src/webgpu_plugin.cpp:2087-2092)
    assert backend.vt["op_ntt_forward"](None, None, 0, 0) == B.NOT_SUPPORTED
    assert backend.vt["op_msm"](None, None, None, None, 0, 0) == B.NOT_SUPPORTED
    for field in ("op_mldsa_verify_batch", "op_slhdsa_verify_batch", "op_ed25519_verify_batch", "op_sr25519_verify_batch"):
        assert backend.vt[field](None, None, None, None, None, 0) == B.NOT_SUPPORTED, field
    for field in ("op_mlkem_decapsulate_batch", "op_ringtail_partial_sign_batch", "op_cggmp21_partial_sign_batch"):
        assert backend.vt[field](None, None, None, None, 0) == B.NOT_SUPPORTED, field
    assert backend.vt["op_ringtail_combine_batch"](None, None, None, None, 0, 0) == B.NOT_SUPPORTED
    assert backend.vt["op_frost_partial_verify_batch"](None, None, None, None, None, None, 0) == B.NOT_SUPPORTED


def test_argument_validation_without_device(backend):
    assert backend.vt["get_device_count"](None) == B.INVALID_ARGUMENT
    assert backend.vt["get_device_info"](None, None) == B.INVALID_ARGUMENT
    info = B.DeviceInfo()
    assert backend.vt["get_device_info"](None, C.byref(info)) == B.INTERNAL      # null context, as the reference
    assert backend.vt["sync"](None) == B.INTERNAL
    assert backend.vt["buffer_alloc"](None, 16) is None
    assert backend.vt["buffer_copy_to_host"](None, None, None, 0) == B.INVALID_ARGUMENT
    assert backend.vt["op_add_f32"](None, None, None, None, 4) == B.INVALID_ARGUMENT
    assert backend.vt["op_matmul_f32"](None, None, None, None, 1, 1, 1) == B.INVALID_ARGUMENT
    assert backend.vt["buffer_get_host_ptr"](None, None) is None
    d = B.make_desc(1, 16, 128, 4, 128, B.F16, B.F16, B.F16)
    assert backend.lib.lux_cuda_qmatmul(None, C.byref(d), None, None, None, None, None) == B.INVALID_ARGUMENT


@pytest.mark.parametrize("kw,has_zeros,code,route", [
    (dict(M=1, N=4096, K=4096, bits=8, group=32, x=B.F32, s=B.F32, y=B.F32), False, B.OK, B.ROUTE_GEMV_I8),
    (dict(M=1, N=14336, K=4096, bits=4, group=128, x=B.F16, s=B.F16, y=B.F16), True, B.OK, B.ROUTE_SKINNY_I4),
    (dict(M=32, N=64, K=256, bits=4, group=128, x=B.F16, s=B.F16, y=B.F16), False, B.OK, B.ROUTE_SKINNY_I4),
    (dict(M=33, N=64, K=256, bits=4, group=128, x=B.F16, s=B.F16, y=B.F16), True, B.OK, B.ROUTE_GEMM_I4_TC),
    (dict(M=512, N=4096, K=4096, bits=4, group=128, x=B.BF16, s=B.F16, y=B.BF16), True, B.OK, B.ROUTE_GEMM_I4_TC),
    (dict(M=1, N=64, K=256, bits=4, group=64, x=B.F16, s=B.F16, y=B.F16), True, B.NOT_SUPPORTED, B.ROUTE_NONE),
    (dict(M=1, N=64, K=256, bits=8, group=32, x=B.F16, s=B.F32, y=B.F16), False, B.NOT_SUPPORTED, B.ROUTE_NONE),
    (dict(M=1, N=64, K=256, bits=8, group=32, x=B.F32, s=B.F32, y=B.F32), True, B.NOT_SUPPORTED, B.ROUTE_NONE),
    (dict(M=1, N=64, K=100, bits=4, group=128, x=B.F16, s=B.F16, y=B.F16), True, B.INVALID_ARGUMENT, B.ROUTE_NONE),
    (dict(M=1, N=64, K=256, bits=5, group=128, x=B.F16, s=B.F16, y=B.F16), True, B.INVALID_ARGUMENT, B.ROUTE_NONE),
    (dict(M=0, N=64, K=256, bits=4, group=128, x=B.F16, s=B.F16, y=B.F16), True, B.INVALID_ARGUMENT, B.ROUTE_NONE),
])
def test_routing(backend, kw, has_zeros, code, route):
    d = B.make_desc(kw["M"], kw["N"], kw["K"], kw["bits"], kw["group"], kw["x"], kw["s"], kw["y"])
    assert backend.route(d, has_zeros) == (code, route)


def test_kernel_table_without_device(backend):
    names = backend.kernel_names()
    assert "lux_qskinny_i4_g128" in names and "lux_qgemm_i4_tc_bf16" in names
    # every name lux_cuda_last_kernel_name can report for a default route is in the table
    for n in ("lux_qgemm_i4_tc_wa_f16", "lux_qgemm_i4_tc_wa_bf16", "lux_qgemv_i4_g128_units_fx", "lux_qgemv_i8_g32_units_fx"):
        assert n in names, n
    L = backend.lib
    assert L.lux_cuda_kernel_get(b"no_such_kernel") is None
    assert L.lux_cuda_kernel_get(None) is None
    k = L.lux_cuda_kernel_get(b"lux_qgemv_i8_g32_f32")
    assert k
    assert L.lux_cuda_kernel_entry_point(k) == b"lux_qgemv_i8_g32_f32"
    assert L.lux_cuda_kernel_function(k)
    x, y, z = C.c_uint32(0), C.c_uint32(0), C.c_uint32(0)
    L.lux_cuda_kernel_workgroup_size(k, C.byref(x), C.byref(y), C.byref(z))
    assert (x.value, y.value, z.value) == (256, 1, 1)
    L.lux_cuda_kernel_workgroup_size(None, C.byref(x), C.byref(y), C.byref(z))
    assert (x.value, y.value, z.value) == (1, 1, 1)          # the reference's answer for a null kernel
    L.lux_cuda_kernel_destroy(k)
    assert L.lux_cuda_kernel_entry_point(None) is None


def test_tune_hook(backend):
    backend.tune("gemv_i4_warps", 4)
    backend.tune("gemv_i4_warps", 0)
    with pytest.raises(B.BackendError):
        backend.tune("no_such_key", 1)


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        B.Backend(str(tmp_path / "libluxgpu_backend_cuda.so"))
