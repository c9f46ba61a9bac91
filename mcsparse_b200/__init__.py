"""B200-native CSR SpMV / SpMM behind the mcSparse C API.

The product is ``mcsparse_b200/lib/libmcsparse.so`` (C ABI, declared in ``include/mcsparse.h``).
This package is the Python-side binding used by the tests and the benchmark: it loads the
library with ctypes and mirrors the C entry points one to one. There is no CPU fallback:
importing :mod:`mcsparse_b200.capi` raises if the library has not been built.
"""

from . import capi  # noqa: F401
from .capi import (  # noqa: F401
    McsparseError,
    check,
    lib,
    load_library,
)
from .host import (  # noqa: F401
    CscMatrix,
    CsrMatrix,
    DnMat,
    DnVec,
    Handle,
    HostSpmvPipeline,
    spmm,
    spmm_buffer_size,
    spmm_preprocess,
    spmv,
    spmv_buffer_size,
    spmv_preprocess,
)

__all__ = [
    "capi", "lib", "load_library", "check", "McsparseError", "Handle", "CsrMatrix", "CscMatrix", "DnVec", "DnMat",
    "HostSpmvPipeline",
    "spmv", "spmv_buffer_size", "spmv_preprocess", "spmm", "spmm_buffer_size", "spmm_preprocess",
]
