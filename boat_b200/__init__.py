"""boat_b200 - Boat's multi-head-attention training step on B200 (sm_100a).

The product is the shared library ``libboat_b200.so`` built from ``csrc/``: Boat's C API for
the attention path (``boat_tensor_*``, ``boat_attention_*``, ``boat_var_attention`` ...)
in C, on top of hand-written CUDA kernels behind the ``boat_cuda_*`` ABI
(``include/boat_cuda.h``).  This Python package is only a ctypes loader plus helpers for
tests and the benchmark; it contains no arithmetic and no fallback: without the built
library, or without a GPU, calls fail.
"""
from .capi import load, lib_path, LibraryMissing
from .build import build

__all__ = ["load", "lib_path", "build", "LibraryMissing"]
