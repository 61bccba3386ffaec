"""catlass_b200: B200 (sm_100a) quantized-matmul kernels behind a C ABI.

The product is the shared library built from catlass_b200/csrc (C ABI in include/catlass_b200.h) and the
C++ surface in include/catlass_b200/.  This Python package only builds the library and binds it with
ctypes for the tests and the benchmark; there is no Python or CPU compute path.
"""
from . import capi  # noqa: F401
