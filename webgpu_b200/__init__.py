"""B200-native quantized-matmul backend behind luxcpp/gpu's plugin boundary.

The product is ``webgpu_b200/lib/libluxgpu_backend_cuda.so`` (sources in ``csrc/``,
C ABI in ``include/lux/gpu/``).  This package is the Python host side: a ctypes loader
that plays the role of luxcpp/gpu's plugin loader (``backend``), seeded synthetic
inputs (``synth``) and the tensor-parallel MLP driver over ``torch.distributed``
(``tp``).  Nothing here computes on the CPU in place of the library.
"""
from .backend import load, Backend, Context, Buffer, BackendError  # noqa: F401

__all__ = ["load", "Backend", "Context", "Buffer", "BackendError"]
__version__ = "0.1.0"
