"""ctypes front end of the CPU oracle (oracle/qmatmul_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and by the
CPU-baseline legs of ``bench.py``; the shipped library never touches it.

PARITY UNPINNED: luxcpp/webgpu has no golden vectors for its quantized kernels, so the
oracle is pinned only by known-answer cases derived by hand from the WGSL text
(tests/golden/).

Arrays are numpy; f16 tensors are ``np.float16``; bf16 tensors are ``np.uint16`` bit
patterns (numpy has no bf16 type).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

F32, F16, BF16 = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqmatmul_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with oracle/Makefile if the shared object is missing."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        u32, i32, vp, f32 = C.c_uint32, C.c_int32, C.c_void_p, C.c_float
        L.orc_unpack_int4_asym_x8.argtypes = [u32, i32, C.POINTER(i32)]
        L.orc_unpack_int4_sym_x8.argtypes = [u32, C.POINTER(i32)]
        L.orc_unpack_int8_x4.argtypes = [u32, C.POINTER(i32)]
        L.orc_pack_int4_asym_x8.argtypes = [C.POINTER(i32), i32]
        L.orc_pack_int4_asym_x8.restype = u32
        L.orc_f16_bits_to_f32.argtypes = [u32]
        L.orc_f16_bits_to_f32.restype = f32
        L.orc_f32_to_f16_bits_wgsl.argtypes = [f32]
        L.orc_f32_to_f16_bits_wgsl.restype = u32
        L.orc_f32_to_f16_rne.argtypes = [f32]
        L.orc_f32_to_f16_rne.restype = u32
        L.orc_f32_to_bf16_rne.argtypes = [f32]
        L.orc_f32_to_bf16_rne.restype = u32
        L.orc_bf16_bits_to_f32.argtypes = [u32]
        L.orc_bf16_bits_to_f32.restype = f32
        L.orc_silu.argtypes = [f32]
        L.orc_silu.restype = f32
        L.orc_qunpack.argtypes = [i32, i32, i32, i32, vp, vp, vp]
        L.orc_qdequant.argtypes = [i32, i32, i32, i32, vp, vp, i32, vp, vp, i32]
        L.orc_qmatmul.argtypes = [i32, i32, i32, i32, i32, vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, i32]
        L.orc_swiglu.argtypes = [i32, i32, vp, i32, vp, i32]
        L.orc_num_procs.restype = i32
        L.orc_unary_f32.argtypes = [i32, vp, vp, C.c_size_t]
        L.orc_transpose_f32.argtypes = [vp, vp, i32, i32]
        L.orc_softmax_f32.argtypes = [vp, vp, C.c_size_t, C.c_size_t, i32]
        L.orc_layer_norm_f32.argtypes = [vp, vp, vp, vp, C.c_size_t, C.c_size_t, f32]
        L.orc_rms_norm_f32.argtypes = [vp, vp, vp, C.c_size_t, C.c_size_t, f32]
        L.orc_matmul_int.argtypes = [i32, i32, i32, i32, vp, vp, vp]
        L.orc_requantize_int32_to_int8.argtypes = [vp, vp, C.c_size_t, f32, f32, i32]
        L.orc_dynamic_quantize.argtypes = [vp, C.c_size_t, i32, vp, vp]
        L.orc_compute_group_scales.argtypes = [vp, C.c_size_t, i32, i32, vp]
        L.orc_quantize.argtypes = [vp, C.c_size_t, i32, i32, vp, vp]
        L.orc_rope_freq.argtypes = [u32, u32, f32]
        L.orc_rope_freq.restype = f32
        L.orc_rope_precompute_cache.argtypes = [u32, u32, f32, vp, vp]
        L.orc_rope.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, f32, u32, f32, i32]
        L.orc_sdpa.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, i32]
        L.orc_sdpa_kv_cache.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, f32, i32]
        L.orc_update_kv_cache.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32]
        L.orc_paged_attention.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, u32]
        _lib = L
    return _lib


# -- scalar helpers -------------------------------------------------------------------

def unpack_int4_asym_x8(word: int, zero_point: int) -> list[int]:
    out = (C.c_int32 * 8)()
    lib().orc_unpack_int4_asym_x8(word & 0xFFFFFFFF, zero_point, out)
    return list(out)


def unpack_int4_sym_x8(word: int) -> list[int]:
    out = (C.c_int32 * 8)()
    lib().orc_unpack_int4_sym_x8(word & 0xFFFFFFFF, out)
    return list(out)


def unpack_int8_x4(word: int) -> list[int]:
    out = (C.c_int32 * 4)()
    lib().orc_unpack_int8_x4(word & 0xFFFFFFFF, out)
    return list(out)


def pack_int4_asym_x8(vals, zero_point: int) -> int:
    arr = (C.c_int32 * 8)(*[int(v) for v in vals])
    return int(lib().orc_pack_int4_asym_x8(arr, zero_point))


def f16_bits_to_f32(bits: int) -> float:
    return float(lib().orc_f16_bits_to_f32(bits))


def f32_to_f16_bits_wgsl(v: float) -> int:
    return int(lib().orc_f32_to_f16_bits_wgsl(v))


def f32_to_f16_rne(v: float) -> int:
    return int(lib().orc_f32_to_f16_rne(v))


def f32_to_bf16_rne(v: float) -> int:
    return int(lib().orc_f32_to_bf16_rne(v))


def silu(v: float) -> float:
    return float(lib().orc_silu(v))


# -- array helpers --------------------------------------------------------------------

def dtype_code(a: np.ndarray, bf16: bool = False) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(f"unsupported dtype {a.dtype}")


def _np_out(shape, code):
    return np.empty(shape, {F32: np.float32, F16: np.float16, BF16: np.uint16}[code])


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def to_f32(a: np.ndarray) -> np.ndarray:
    return bf16_to_f32(a) if a.dtype == np.uint16 else a.astype(np.float32)


def qunpack(w: np.ndarray, zeros, bits: int, group: int) -> np.ndarray:
    N = w.shape[0]
    K = w.shape[1] * (2 if bits == 4 else 1)
    w = np.ascontiguousarray(w).view(np.uint8)
    out = np.empty((N, K), np.int8)
    rc = lib().orc_qunpack(N, K, bits, group, _ptr(w), _ptr(zeros), _ptr(out))
    assert rc == 0, rc
    return out


def qdequant(w, scales, zeros, bits: int, group: int, out_code: int = F32) -> np.ndarray:
    N = w.shape[0]
    K = w.shape[1] * (2 if bits == 4 else 1)
    w = np.ascontiguousarray(w).view(np.uint8)
    scales = np.ascontiguousarray(scales)
    out = _np_out((N, K), out_code)
    rc = lib().orc_qdequant(N, K, bits, group, _ptr(w), _ptr(scales), dtype_code(scales),
                            _ptr(zeros), _ptr(out), out_code)
    assert rc == 0, rc
    return out


def qmatmul(x, w, scales, zeros, bits: int, group: int, y_code: int | None = None,
            w_round: int = F32, acc_mode: int = 0, threads: int = 0) -> np.ndarray:
    """y[M,N] = x[M,K] . dequant(W[N,K])^T; see orc_qmatmul for the modes."""
    x = np.ascontiguousarray(x)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] * (2 if bits == 4 else 1) == K
    w = np.ascontiguousarray(w).view(np.uint8)
    scales = np.ascontiguousarray(scales)
    if zeros is not None:
        zeros = np.ascontiguousarray(zeros, np.uint8)
    xc = dtype_code(x)
    if y_code is None:
        y_code = xc
    y = _np_out((M, N), y_code)
    rc = lib().orc_qmatmul(M, N, K, bits, group, _ptr(x), xc, _ptr(w), _ptr(scales),
                           dtype_code(scales), _ptr(zeros), _ptr(y), y_code, w_round,
                           acc_mode, threads)
    assert rc == 0, rc
    return y


def swiglu(gu: np.ndarray, h_code: int | None = None) -> np.ndarray:
    gu = np.ascontiguousarray(gu)
    M, two_i = gu.shape
    code = dtype_code(gu)
    if h_code is None:
        h_code = code
    h = _np_out((M, two_i // 2), h_code)
    lib().orc_swiglu(M, two_i // 2, _ptr(gu), code, _ptr(h), h_code)
    return h


def mlp(x, gate_up, down, group: int = 128, fused: bool = False, w_round: int = F32,
        acc_mode: int = 0, threads: int = 0) -> np.ndarray:
    """Llama FFN: y = (silu(x.Wg^T) * (x.Wu^T)) . Wd^T on int4 weights.

    gate_up / down are (w, scales, zeros) triples; gate_up stacks gate rows then up rows.
    fused=False rounds gate_up's output to the activation dtype before SwiGLU (two
    separate "f32 accumulate, 16-bit output" layers); fused=True keeps gate and up in
    f32 until after SwiGLU (one rounding fewer), which is what a fused epilogue does.
    """
    code = dtype_code(x)
    gu = qmatmul(x, *gate_up, bits=4, group=group, y_code=(F32 if fused else code),
                 w_round=w_round, acc_mode=acc_mode, threads=threads)
    h = swiglu(gu, h_code=code)
    return qmatmul(h, *down, bits=4, group=group, y_code=code, w_round=w_round,
                   acc_mode=acc_mode, threads=threads)


def tp_mlp(x, shards, group: int = 128, fused: bool = True, w_round: int = F32) -> np.ndarray:
    """Tensor-parallel FFN: each shard is (gate_up_triple, down_triple); partial outputs
    are narrowed to the activation dtype per shard (what each GPU hands to the
    all-reduce) and summed in f32 in rank order, then narrowed once."""
    code = dtype_code(x)
    total = None
    for gate_up, down in shards:
        part = to_f32(mlp(x, gate_up, down, group=group, fused=fused, w_round=w_round))
        total = part if total is None else total + part
    if code == F16:
        return total.astype(np.float16)
    if code == BF16:
        return f32_to_bf16(total)
    return total


# -- f32 tensor ops (oracle/tensor_ops_oracle.c) ---------------------------------------

UNARY_OPS = {"exp": 0, "log": 1, "sqrt": 2, "neg": 3, "abs": 4, "tanh": 5, "sigmoid": 6, "relu": 7, "gelu": 8,
             "silu": 9, "copy": 10}


def unary_f32(op: str, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    assert lib().orc_unary_f32(UNARY_OPS[op], _ptr(x), _ptr(out), x.size) == 0
    return out


def transpose_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty((x.shape[1], x.shape[0]), np.float32)
    lib().orc_transpose_f32(_ptr(x), _ptr(out), x.shape[0], x.shape[1])
    return out


def softmax_f32(x: np.ndarray, log: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().orc_softmax_f32(_ptr(x), _ptr(out), x.shape[0], x.shape[1], int(log))
    return out


def layer_norm_f32(x, gamma, beta, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().orc_layer_norm_f32(_ptr(x), _ptr(np.ascontiguousarray(gamma, np.float32)), _ptr(np.ascontiguousarray(beta, np.float32)),
                             _ptr(out), x.shape[0], x.shape[1], eps)
    return out


def rms_norm_f32(x, weight, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm_f32(_ptr(x), _ptr(np.ascontiguousarray(weight, np.float32)), _ptr(out), x.shape[0], x.shape[1], eps)
    return out


# -- attention side (attention_oracle.c) ----------------------------------------------------


def _f32c(a):
    return np.ascontiguousarray(a, np.float32)


def rope_cache(max_seq_len: int, head_dim: int, theta_base: float):
    """rope_precompute_cache: (cos, sin), each [max_seq_len, head_dim / 2]."""
    cos = np.empty((max_seq_len, head_dim // 2), np.float32)
    sin = np.empty_like(cos)
    assert lib().orc_rope_precompute_cache(max_seq_len, head_dim, theta_base, _ptr(cos), _ptr(sin)) == 0
    return cos, sin


def rope(x, cos=None, sin=None, position_ids=None, theta_base: float = 10000.0, position_offset: int = 0,
         ntk_scale: float = 0.0, backward: bool = False) -> np.ndarray:
    """The rotation of gpu/rope.wgsl on x [batch, seq, heads, head_dim] (adjacent pairs)."""
    x = _f32c(x)
    B, S, H, D = x.shape
    out = np.empty_like(x)
    cos = None if cos is None else _f32c(cos)
    sin = None if sin is None else _f32c(sin)
    pid = None if position_ids is None else np.ascontiguousarray(position_ids, np.uint32)
    rc = lib().orc_rope(_ptr(x), _ptr(out), None if cos is None else _ptr(cos), None if sin is None else _ptr(sin),
                        None if pid is None else _ptr(pid), B, S, H, D, theta_base, position_offset, ntk_scale, int(backward))
    assert rc == 0, rc
    return out


def sdpa(q, k, v, scale: float, causal: bool = False, want_lse: bool = False):
    """sdpa_basic / sdpa_mqa: q [B, H, Sq, D], k and v [B, Hkv, Skv, D]."""
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, H, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    out = np.empty_like(q)
    lse = np.empty((B, H, Sq), np.float32) if want_lse else None
    rc = lib().orc_sdpa(_ptr(q), _ptr(k), _ptr(v), _ptr(out), None if lse is None else _ptr(lse), B, H, Hkv, Sq, Skv, D, scale,
                        int(causal))
    assert rc == 0, rc
    return (out, lse) if want_lse else out


def sdpa_kv_cache(q, k_cache, v_cache, cache_len: int, scale: float, causal_append: bool = False) -> np.ndarray:
    """sdpa_kv_cache: q [B, H, Sq, D], caches [B, Hkv, max_len, D] with the new tokens already appended."""
    q, k_cache, v_cache = _f32c(q), _f32c(k_cache), _f32c(v_cache)
    B, H, Sq, D = q.shape
    Hkv, max_len = k_cache.shape[1], k_cache.shape[2]
    out = np.empty_like(q)
    rc = lib().orc_sdpa_kv_cache(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), B, H, Hkv, Sq, cache_len, max_len, D, scale,
                                 int(causal_append))
    assert rc == 0, rc
    return out


def update_kv_cache(k, v, k_cache, v_cache, cache_len: int) -> None:
    """update_kv_cache, in place on the two caches (float32, C-contiguous)."""
    k, v = _f32c(k), _f32c(v)
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous and v_cache.flags.c_contiguous
    B, Hkv, Sq, D = k.shape
    assert lib().orc_update_kv_cache(_ptr(k), _ptr(v), _ptr(k_cache), _ptr(v_cache), B, Hkv, Sq, cache_len, k_cache.shape[2], D) == 0


def paged_attention(q, k_cache, v_cache, block_tables, context_lens, scale: float, partition_size: int = 0, out=None) -> np.ndarray:
    """paged_attention_v1 (partition_size 0) or v2 partial + reduce: q [S, H, D], caches [blocks, Hkv, block_size, D]."""
    q, k_cache, v_cache = _f32c(q), _f32c(k_cache), _f32c(v_cache)
    bt = np.ascontiguousarray(block_tables, np.int32)
    cl = np.ascontiguousarray(context_lens, np.int32)
    S, H, D = q.shape
    out = np.zeros_like(q) if out is None else out
    rc = lib().orc_paged_attention(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(bt), _ptr(cl), _ptr(out), S, H, k_cache.shape[1], D,
                                   k_cache.shape[2], bt.shape[1], scale, partition_size)
    assert rc == 0, rc
    return out


# -- quantize side ---------------------------------------------------------------------

NAX_INT4_SYM, NAX_INT4_ASYM, NAX_INT8_SYM = 0, 1, 2          # quantized_nax.wgsl:31-33
EXT_INT4_ASYM_SHIFTED = 101                                   # not a reference format (see orc_quantize)
GROUP_SCALE = np.dtype([("scale", np.float32), ("zero_point", np.int32), ("group_min", np.float32),
                        ("group_max", np.float32)])          # GroupScale, quantized_nax.wgsl:49-54


def group_scales(x: np.ndarray, group: int, fmt: int) -> np.ndarray:
    """compute_group_scales over the flat array: one GroupScale record per `group` elements."""
    flat = np.ascontiguousarray(x, np.float32).ravel()
    out = np.zeros((flat.size + group - 1) // group, GROUP_SCALE)
    rc = lib().orc_compute_group_scales(_ptr(flat), flat.size, group, fmt, _ptr(out))
    assert rc == 0, rc
    return out


def quantize_packed(x: np.ndarray, group: int, fmt: int, gs: np.ndarray) -> np.ndarray:
    """quantize_nax_int4_sym / _asym / quantize_nax_int8_group: the packed u32 words."""
    flat = np.ascontiguousarray(x, np.float32).ravel()
    per = 4 if fmt == NAX_INT8_SYM else 8
    out = np.zeros(flat.size // per, np.uint32)
    rc = lib().orc_quantize(_ptr(flat), flat.size, group, fmt, _ptr(np.ascontiguousarray(gs)), _ptr(out))
    assert rc == 0, rc
    return out


def quantize(x: np.ndarray, bits: int, group: int, symmetric: bool, scale_code: int = F32, shifted: bool = False):
    """The reference's two quantize passes on a row-major [N, K] f32 matrix (K % group == 0), mapped
    onto the compact layout the matmul kernels read: (w, scales, zeros) with w uint8 [N, K/2] (int4,
    low nibble first) or int8 [N, K], scales [N, K/group], zeros packed two per byte or None.

    `shifted` selects the non-reference asymmetric variant clamp(round(v / scale) + zp, 0, 15).
    scale_code F32 is the reference's arithmetic exactly.  F16 (the benchmark configurations' int4
    scale tables) is an extension: the scale is rounded to f16 first and the values are quantized
    with the rounded scale, so that quantize and dequantize use the same number."""
    x = np.ascontiguousarray(x, np.float32)
    N, K = x.shape
    assert K % group == 0
    fmt = NAX_INT8_SYM if bits == 8 else (NAX_INT4_SYM if symmetric else NAX_INT4_ASYM)
    gs = group_scales(x, group, fmt)
    if scale_code == F16:
        with np.errstate(over="ignore"):
            s16 = gs["scale"].astype(np.float16)
        gs = gs.copy()
        gs["scale"] = s16.astype(np.float32)
        scales = s16.reshape(N, K // group)
    else:
        scales = gs["scale"].reshape(N, K // group).copy()
    with np.errstate(divide="ignore", invalid="ignore"):
        words = quantize_packed(x, group, EXT_INT4_ASYM_SHIFTED if (shifted and fmt == NAX_INT4_ASYM) else fmt, gs)
    if bits == 4:
        w = words.view(np.uint8).reshape(N, K // 2)
    else:
        w = words.view(np.int8).reshape(N, K)
    zeros = None
    if fmt == NAX_INT4_ASYM:
        zp = gs["zero_point"].reshape(N, K // group).astype(np.uint8)
        G = K // group
        if G % 2:
            zp = np.concatenate([zp, np.zeros((N, 1), np.uint8)], axis=1)
        zeros = (zp[:, 0::2] | (zp[:, 1::2] << 4)).astype(np.uint8)
    return w, scales, zeros


# -- activation-quantized integer path --------------------------------------------------

def matmul_int(a: np.ndarray, b: np.ndarray, M: int, N: int, K: int, a_bits: int = 8) -> np.ndarray:
    """C[M, N] i32 = A[M, K] . B[K, N]: A int8 (a_bits 8) or packed two's-complement int4 bytes (a_bits 4)."""
    a = np.ascontiguousarray(a).view(np.uint8)
    b = np.ascontiguousarray(b, np.int8)
    c = np.empty((M, N), np.int32)
    assert lib().orc_matmul_int(M, N, K, a_bits, _ptr(a), _ptr(b), _ptr(c)) == 0
    return c


def requantize_int32_to_int8(x: np.ndarray, input_scale: float, output_scale: float, zero_point: int) -> np.ndarray:
    x = np.ascontiguousarray(x, np.int32)
    out = np.empty_like(x)
    lib().orc_requantize_int32_to_int8(_ptr(x), _ptr(out), x.size, input_scale, output_scale, zero_point)
    return out


def dynamic_quantize(x: np.ndarray, bits: int = 8):
    """(packed bytes, scale): per-tensor symmetric quantization of activations."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size if bits == 8 else (x.size + 1) // 2, np.uint8)
    scale = np.zeros(1, np.float32)
    assert lib().orc_dynamic_quantize(_ptr(x), x.size, bits, _ptr(out), _ptr(scale)) == 0
    return out, float(scale[0])


def rel_l2(a: np.ndarray, ref: np.ndarray) -> float:
    a = to_f32(a).astype(np.float64)
    ref = to_f32(ref).astype(np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / (den if den > 0 else 1.0))


def num_procs() -> int:
    return int(lib().orc_num_procs())
