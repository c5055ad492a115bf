"""vexel_b200: B200-native CUDA backend for the Vexel inference engine.

The product is the C-ABI shared library built from csrc/ (include/vexel_cuda.h).  This package holds
the build step, a thin ctypes binding used by the tests and the benchmark, and helpers that produce
synthetic GGUF-format weights.  There is no CPU fallback: loading fails if the library is missing.
"""
from .capi import Lib, Backend, Model, ModelConfig, VxError  # noqa: F401
