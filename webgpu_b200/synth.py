"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset is involved: every tensor is fully specified by its
distribution and a seed).

One numpy PCG64 stream per tensor, derived from (seed, tensor tag), so tensors do not
shift when another tensor's shape changes.  bf16 tensors are ``np.uint16`` bit patterns.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass

import numpy as np


def _rng(seed: int, tag: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(tag.encode())]))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def activations(M: int, K: int, dtype: str, seed: int = 0, tag: str = "x") -> np.ndarray:
    """x ~ N(0,1) as f32 / f16 / bf16(bit patterns)."""
    x = _rng(seed, tag).standard_normal((M, K), dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    raise ValueError(dtype)


@dataclass
class QLayer:
    """A quantized linear layer y = x . dequant(W)^T in the library's memory layout."""
    bits: int
    group: int
    N: int
    K: int
    w: np.ndarray                 # int4: uint8 [N, K/2] low nibble first; int8: int8 [N, K]
    scales: np.ndarray            # [N, K/group] f16 (int4) or f32 (int8)
    zeros: np.ndarray | None      # uint8 [N, ceil(G/2)] nibbles low first; None = symmetric

    @property
    def triple(self):
        return (self.w, self.scales, self.zeros)

    @property
    def weight_bytes(self) -> int:
        z = 0 if self.zeros is None else self.zeros.nbytes
        return self.w.nbytes + self.scales.nbytes + z


def int8_layer(N: int, K: int, seed: int = 0, tag: str = "w8", group: int = 32) -> QLayer:
    """W int8 uniform in [-127,127]; one f32 scale |N(0,0.02)|/127 per `group` K."""
    w = _rng(seed, tag + ".w").integers(-127, 128, size=(N, K), dtype=np.int8)
    s = np.abs(_rng(seed, tag + ".s").standard_normal((N, K // group), dtype=np.float32)) * np.float32(0.02)
    s = (s / np.float32(127.0)).astype(np.float32)
    return QLayer(8, group, N, K, w, s, None)


def pack_nibbles(vals: np.ndarray) -> np.ndarray:
    """[..., n] values 0..15 -> [..., ceil(n/2)] bytes, element 2j in the low nibble."""
    vals = np.asarray(vals, np.uint8)
    if vals.shape[-1] % 2:
        pad = np.zeros(vals.shape[:-1] + (1,), np.uint8)
        vals = np.concatenate([vals, pad], axis=-1)
    return (vals[..., 0::2] | (vals[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray, n: int) -> np.ndarray:
    packed = np.asarray(packed, np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out[..., :n]


def int4_layer(N: int, K: int, seed: int = 0, tag: str = "w4", group: int = 128,
               symmetric: bool = False) -> QLayer:
    """Nibbles uniform 0..15 packed low first; f16 scale |N(0,0.02)|/7 and a 4-bit
    zero-point uniform 0..15 per `group` K.  A scale that rounds to 0 in f16 is kept."""
    G = K // group
    w = _rng(seed, tag + ".w").integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    s = np.abs(_rng(seed, tag + ".s").standard_normal((N, G), dtype=np.float32)) * np.float32(0.02)
    s = (s / np.float32(7.0)).astype(np.float16)
    zeros = None
    if not symmetric:
        zp = _rng(seed, tag + ".z").integers(0, 16, size=(N, G), dtype=np.uint8)
        zeros = pack_nibbles(zp)
    return QLayer(4, group, N, K, w, s, zeros)


# -- the benchmark configurations -----------------------------------------------------

def config1(seed: int = 0):
    """int8 symmetric g32 GEMV 4096x4096, f32 in/out."""
    return activations(1, 4096, "f32", seed, "cfg1.x"), int8_layer(4096, 4096, seed, "cfg1")


def config2(seed: int = 0, M: int = 1):
    """int4 asymmetric g128 GEMV, Llama-3-8B MLP up shape 4096 -> 14336, f16."""
    return activations(M, 4096, "f16", seed, "cfg2.x"), int4_layer(14336, 4096, seed, "cfg2")


def config3(seed: int = 0, M: int = 512):
    """int4 g128 prefill GEMM, X bf16 [512,4096], W [4096,4096]."""
    return activations(M, 4096, "bf16", seed, "cfg3.x"), int4_layer(4096, 4096, seed, "cfg3")


SWEEP_LAYERS = {                     # Llama-3-8B decode linears: name -> (K in, N out)
    "qkv": (4096, 6144),
    "o": (4096, 4096),
    "gate_up": (4096, 28672),
    "down": (14336, 4096),
}
SWEEP_M = (1, 4, 16, 64)


def config4(name: str, M: int, seed: int = 0):
    K, N = SWEEP_LAYERS[name]
    return activations(M, K, "f16", seed, f"cfg4.{name}.x"), int4_layer(N, K, seed, f"cfg4.{name}")


MLP70B = dict(K=8192, I=28672, H=8192)        # Llama-3-70B FFN
MLP70B_M = (1, 32, 256)


def mlp_layers(K: int, I: int, H: int, seed: int = 0, tag: str = "cfg5"):
    """gate_up [2I, K] (gate rows then up rows) and down [H, I], int4 g128 asymmetric."""
    return int4_layer(2 * I, K, seed, tag + ".gate_up"), int4_layer(H, I, seed, tag + ".down")
