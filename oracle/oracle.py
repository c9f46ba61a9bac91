"""ctypes/numpy front end of oracle/csr_oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the CPU
baseline / reference arm of bench.py. PARITY UNPINNED BY THE REFERENCE (it has no tests or
fixtures for this path); see the header of csr_oracle.c for what pins these loops instead.
"""

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")


def build(force=False):
    src = os.path.join(_HERE, "csr_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s", "_build/liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.oracle_merge_path_partition.restype = C.c_int64
        _lib.baseline_num_threads.restype = C.c_int
        _lib.oracle_csr_validate.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _np(a, dtype=None):
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    a = np.ascontiguousarray(a)
    return a if dtype is None else a.astype(dtype, copy=False)


def _vt(val):
    if val.dtype == np.float32:
        return "f32"
    if val.dtype == np.float64:
        return "f64"
    if val.dtype == np.complex64:
        return "c32"
    if val.dtype == np.complex128:
        return "c64"
    raise TypeError(val.dtype)


def _pair(z):
    z = complex(z)
    return np.array([z.real, z.imag], np.float64)


def spmv(row_ptr, col, val, x, alpha, beta, y0=None, base=0, conj=False):
    """High-precision y = alpha A x + beta y0 and the tolerance scale d. Returns (y, d): float64, or
    complex128 and float64 for complex values (`conj` multiplies with conj(A))."""
    row_ptr, col, val, x = _np(row_ptr, np.int32), _np(col, np.int32), _np(val), _np(x)
    m = row_ptr.size - 1
    y_in = _np(y0).astype(val.dtype, copy=False) if y0 is not None else np.zeros(max(m, 1), val.dtype)
    if np.iscomplexobj(val):
        x = x.astype(val.dtype, copy=False)
        y = np.empty(m, np.complex128)
        d = np.empty(m, np.float64)
        a, b = _pair(alpha), _pair(beta if y0 is not None else 0.0)
        getattr(lib(), "oracle_csr_spmv_" + _vt(val))(C.c_int64(m), C.c_int(base), _p(row_ptr), _p(col), _p(val), _p(x),
                                                      _p(a), _p(b), C.c_int(int(conj)), _p(y_in), _p(y), _p(d))
        return y, d
    y = np.empty(m, np.float64)
    d = np.empty(m, np.float64)
    fn = getattr(lib(), "oracle_csr_spmv_" + _vt(val))
    fn(C.c_int64(m), C.c_int(base), _p(row_ptr), _p(col), _p(val), _p(x), C.c_double(alpha), C.c_double(beta),
       _p(y_in), _p(y), _p(d))
    return y, d


def spmm(row_ptr, col, val, B, ldb, order_b, n, alpha, beta, C0=None, ldc=None, order_c=2, base=0):
    """High-precision C = alpha A B + beta C0 as a dense (m, n) float64 array, and d of the same shape.
    B and C0 are flat arrays laid out by (ld, order); order 1 = column-major, 2 = row-major."""
    row_ptr, col, val, B = _np(row_ptr, np.int32), _np(col, np.int32), _np(val), _np(B).ravel()
    m = row_ptr.size - 1
    ldc = n if ldc is None else ldc
    c_in = _np(C0).ravel().astype(val.dtype, copy=False) if C0 is not None else np.zeros(1, val.dtype)
    if np.iscomplexobj(val):
        B = B.astype(val.dtype, copy=False)
        out, d = np.empty((m, n), np.complex128), np.empty((m, n), np.float64)
        a, b = _pair(alpha), _pair(beta if C0 is not None else 0.0)
        getattr(lib(), "oracle_csr_spmm_" + _vt(val))(C.c_int64(m), C.c_int64(n), C.c_int(base), _p(row_ptr), _p(col),
                                                      _p(val), _p(B), C.c_int64(ldb), C.c_int(order_b), _p(a), _p(b),
                                                      _p(c_in), C.c_int64(ldc), C.c_int(order_c), _p(out), _p(d))
        return out, d
    out = np.empty((m, n), np.float64)
    d = np.empty((m, n), np.float64)
    fn = getattr(lib(), "oracle_csr_spmm_" + _vt(val))
    fn(C.c_int64(m), C.c_int64(n), C.c_int(base), _p(row_ptr), _p(col), _p(val), _p(B), C.c_int64(ldb),
       C.c_int(order_b), C.c_double(alpha), C.c_double(beta if C0 is not None else 0.0), _p(c_in), C.c_int64(ldc),
       C.c_int(order_c), _p(out), _p(d))
    return out, d


def merge_path_partition(row_ptr, nnz, items_per_tile, base=0):
    """(num_tiles + 1, 2) int32 array of {row, nonzero} tile starts."""
    row_ptr = _np(row_ptr, np.int32)
    m = row_ptr.size - 1
    num_tiles = (m + nnz + items_per_tile - 1) // items_per_tile
    out = np.empty((num_tiles + 1, 2), np.int32)
    got = lib().oracle_merge_path_partition(C.c_int64(m), C.c_int64(nnz), C.c_int(base), _p(row_ptr),
                                            C.c_int(items_per_tile), _p(out))
    assert got == num_tiles
    return out


def shard_row_bounds(row_ptr, nnz, num_shards, base=0):
    row_ptr = _np(row_ptr, np.int32)
    out = np.empty(num_shards + 1, np.int64)
    lib().oracle_shard_row_bounds(C.c_int64(row_ptr.size - 1), C.c_int64(nnz), C.c_int(base), _p(row_ptr),
                                  C.c_int(num_shards), _p(out))
    return out


def shard_local_row_offsets(row_ptr, first_row, num_rows, base=0):
    row_ptr = _np(row_ptr, np.int32)
    out = np.empty(num_rows + 1, np.int32)
    lib().oracle_shard_local_row_offsets(_p(row_ptr), C.c_int64(first_row), C.c_int64(num_rows), C.c_int(base),
                                         _p(out))
    return out


def coo_row_offsets(coo_rows, num_rows, base=0):
    coo_rows = _np(coo_rows, np.int32)
    out = np.empty(num_rows + 1, np.int32)
    lib().oracle_coo_row_offsets(C.c_int64(num_rows), C.c_int64(coo_rows.size), C.c_int(base), _p(coo_rows), _p(out))
    return out


def csr_transpose(row_ptr, col, num_cols, base=0):
    """(t_ptr, t_idx, perm) of the transposed matrix: 0-based CSR arrays and, for every transposed nonzero,
    its position in the source arrays (stable: ascending source rows inside a row of the transpose)."""
    row_ptr, col = _np(row_ptr, np.int32), _np(col, np.int32)
    m, nnz = row_ptr.size - 1, col.size
    t_ptr, t_idx, perm = np.empty(num_cols + 1, np.int32), np.empty(nnz, np.int32), np.empty(nnz, np.int32)
    lib().oracle_csr_transpose(C.c_int64(m), C.c_int64(num_cols), C.c_int64(nnz), C.c_int(base), _p(row_ptr), _p(col),
                               _p(t_ptr), _p(t_idx), _p(perm))
    return t_ptr, t_idx, perm


def csr_validate(rows, cols, row_ptr, col, base=0):
    row_ptr, col = _np(row_ptr, np.int32), _np(col, np.int32)
    return lib().oracle_csr_validate(C.c_int64(rows), C.c_int64(cols), C.c_int64(col.size), C.c_int(base),
                                     _p(row_ptr), _p(col))


def num_threads():
    return lib().baseline_num_threads()


def use_host_cores():
    """Sizes the OpenMP team of the baseline kernels to the cores this process may run on, whatever
    OMP_NUM_THREADS says (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers)."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().baseline_set_threads(cores)
    return num_threads()


def baseline_spmv(row_ptr, col, val, x, alpha, beta, y, base=0):
    """Native-precision OpenMP y = alpha A x + beta y, in place on the numpy array y."""
    ct = C.c_float if val.dtype == np.float32 else C.c_double
    fn = getattr(lib(), "baseline_csr_spmv_" + _vt(val))
    fn(C.c_int64(row_ptr.size - 1), C.c_int(base), _p(row_ptr), _p(col), _p(val), _p(x), ct(alpha), ct(beta), _p(y))


def baseline_spmm(row_ptr, col, val, B, n, alpha, beta, Cmat, base=0):
    """Native-precision OpenMP C = alpha A B + beta C for row-major B (ld n) and C (ld n), in place."""
    ct = C.c_float if val.dtype == np.float32 else C.c_double
    fn = getattr(lib(), "baseline_csr_spmm_" + _vt(val))
    fn(C.c_int64(row_ptr.size - 1), C.c_int64(n), C.c_int(base), _p(row_ptr), _p(col), _p(val), _p(B), C.c_int64(n),
       ct(alpha), ct(beta), _p(Cmat), C.c_int64(n))
