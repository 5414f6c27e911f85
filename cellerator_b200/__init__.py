"""B200 (sm_100a) backend for Cellerator's quantized sparse-matrix path.

The product is the native library `lib/libcellerator_b200.so` (C ABI in
include/cellerator_b200.h) plus the C++ operation-core backend over it; this Python package
is the build script and a ctypes driver used by the tests and the benchmark.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
