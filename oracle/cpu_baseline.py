"""ctypes front end of the timed CPU baseline (oracle/cpu_baseline.c).

TEST / BENCHMARK INFRASTRUCTURE ONLY: imported by ``bench.py``'s ``cpu_baseline`` and
``--impl reference`` legs and by the test that holds it to the oracle.  It is the oracle's
arithmetic (the reference's shader math) written the way a CPU backend would write it:
scale and zero-point hoisted per group, vectorisable inner loop, OpenMP over rows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqmatmul_cpu_baseline.so")
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            subprocess.check_call(["make", "-C", _HERE, "-s"])
        L = C.CDLL(_LIB_PATH)
        i32, vp = C.c_int32, C.c_void_p
        L.cpub_qmatmul_i4.argtypes = [i32, i32, i32, vp, vp, vp, vp, vp, i32]
        L.cpub_mlp_i4.argtypes = [i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32]
        L.cpub_num_procs.restype = i32
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_procs() -> int:
    return int(lib().cpub_num_procs())


def qmatmul_i4(x: np.ndarray, w, scales, zeros, threads: int = 0) -> np.ndarray:
    """y[M, N] f16 = x[M, K] f16 . dequant(W)^T, int4 g128."""
    x = np.ascontiguousarray(x, np.float16)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), np.float16)
    rc = lib().cpub_qmatmul_i4(M, N, K, _p(x), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(scales)),
                               _p(None if zeros is None else np.ascontiguousarray(zeros)), _p(y), threads)
    assert rc == 0, rc
    return y


def mlp_i4(x: np.ndarray, gate_up, down, threads: int = 0) -> np.ndarray:
    """Llama FFN on int4 g128 (w, scales, zeros) triples; gate rows then up rows in gate_up."""
    x = np.ascontiguousarray(x, np.float16)
    M, K = x.shape
    I, H = gate_up[0].shape[0] // 2, down[0].shape[0]
    y = np.empty((M, H), np.float16)
    a = [np.ascontiguousarray(t) if t is not None else None for t in (*gate_up, *down)]
    rc = lib().cpub_mlp_i4(M, K, I, H, _p(x), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(a[5]), _p(y), threads)
    assert rc == 0, rc
    return y
