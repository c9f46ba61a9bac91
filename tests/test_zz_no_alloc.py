"""mcsparseB200SpMVNoAlloc: the SpMV entry point for callers that may not allocate device memory.

Such callers (a plugin or solver callback whose host owns all device memory and forbids
cudaMalloc inside the call, or code that cannot afford the implicit synchronisation of an
allocation) cannot provide the work buffer mcsparseSpMV needs, so this variant keeps the work
partition in a fixed array inside the library. The test calls it through the C ABI twice in a
row, on different matrices that share that array, and compares each result with mcsparseSpMV's
on the same inputs; it also checks that the device's free memory (cudaMemGetInfo, which sees any
allocation made inside the library) does not change and that a matrix too large for the fixed array
is refused with the documented status. The file sorts last so that a
run stopping at the first failure has already run every other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

import mcsparse_b200 as mc
from mcsparse_b200 import capi, workloads
from mcsparse_b200.capi import lib
from oracle import oracle
from tests.util import TOL, assert_close

pytestmark = pytest.mark.gpu


def _scalars(dtype, alpha, beta):
    ct = C.c_double if dtype == torch.float64 else C.c_float
    a, b = ct(alpha), ct(beta)
    return a, b, C.cast(C.pointer(a), C.c_void_p), C.cast(C.pointer(b), C.c_void_p)


def _no_alloc_spmv(handle, A, X, Y, dtype, alpha, beta):
    a, b, pa, pb = _scalars(dtype, alpha, beta)
    dt = capi.MACA_R_64F if dtype == torch.float64 else capi.MACA_R_32F
    return lib.mcsparseB200SpMVNoAlloc(handle.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, pa, A.d, X.d, pb, Y.d, dt,
                                       capi.MCSPARSE_SPMV_ALG_DEFAULT)


def test_no_alloc_spmv_matches_spmv_on_two_calls_in_a_row(handle, device):
    cases = []
    for name, factor, alpha, beta in (("C5", 64, 1.0, 0.5), ("C3", 128, -2.0, 0.0)):
        cfg = workloads.scaled(name, factor)
        w = workloads.generate(cfg, device)
        A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
        y_ref, y_new = w.y0.clone(), w.y0.clone()
        X, Yref, Ynew = mc.DnVec(w.x), mc.DnVec(y_ref), mc.DnVec(y_new)
        buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Yref), dtype=torch.uint8, device=device)
        mc.spmv(handle, A, X, Yref, buf, alpha=alpha, beta=beta)
        cases.append((cfg, w, A, X, Ynew, y_ref, y_new, alpha, beta))
    torch.cuda.synchronize()

    # one call first: the first call on a device looks up the address of the built-in work area
    cfg, w, A, X, Ynew, y_ref, y_new, alpha, beta = cases[0]
    capi.check(_no_alloc_spmv(handle, A, X, Ynew, cfg.dtype, alpha, beta), "mcsparseB200SpMVNoAlloc")
    torch.cuda.synchronize()
    y_new.copy_(w.y0)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(device)[0]  # cudaMemGetInfo: sees allocations torch's counters cannot
    before = torch.cuda.memory_stats(device)["allocation.all.allocated"]
    for cfg, w, A, X, Ynew, y_ref, y_new, alpha, beta in cases:  # two calls in a row, one shared work area
        capi.check(_no_alloc_spmv(handle, A, X, Ynew, cfg.dtype, alpha, beta), "mcsparseB200SpMVNoAlloc")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(device)[0] == free_before
    assert torch.cuda.memory_stats(device)["allocation.all.allocated"] == before
    status = C.c_int(-1)  # the status word of the built-in work area: NULL stands for it
    capi.check(lib.mcsparseB200SpMVGetStatus(handle.h, cases[-1][2].d, None, C.byref(status)))
    assert status.value == 0

    for cfg, w, A, X, Ynew, y_ref, y_new, alpha, beta in cases:
        ref, d = oracle.spmv(w.row_ptr, w.col, w.val, w.x, alpha, beta, w.y0)
        assert_close(y_new.cpu().numpy(), ref, d, TOL[cfg.dtype], f"no-alloc SpMV {cfg.name}")
        assert_close(y_new.cpu().numpy(), y_ref.cpu().numpy().astype(np.float64), d, TOL[cfg.dtype],
                     f"no-alloc vs mcsparseSpMV {cfg.name}")

    # and once more on the first matrix after the array was used for the second one
    cfg, w, A, X, Ynew, y_ref, y_new, alpha, beta = cases[0]
    y_new.copy_(w.y0)
    capi.check(_no_alloc_spmv(handle, A, X, Ynew, cfg.dtype, alpha, beta))
    torch.cuda.synchronize()
    assert torch.equal(y_new, y_ref)


def test_no_alloc_spmv_refuses_oversized_matrix(handle, device):
    # 2.2e9 merge items of fp32 would need more than the fixed 16 MiB; no array is touched
    # before the size check, so small placeholders stand in for the matrix.
    rows = 1 << 30
    nnz = (1 << 30) - 8
    dummy_i = torch.zeros(4, dtype=torch.int32, device=device)
    dummy_f = torch.zeros(4, dtype=torch.float64, device=device)
    d = C.c_void_p()
    capi.check(lib.mcsparseCreateCsr(C.byref(d), rows, rows, nnz, C.c_void_p(dummy_i.data_ptr()),
                                     C.c_void_p(dummy_i.data_ptr()), C.c_void_p(dummy_f.data_ptr()),
                                     capi.MCSPARSE_INDEX_32I, capi.MCSPARSE_INDEX_32I, 0, capi.MACA_R_64F))
    x, y = C.c_void_p(), C.c_void_p()
    capi.check(lib.mcsparseCreateDnVec(C.byref(x), rows, C.c_void_p(dummy_f.data_ptr()), capi.MACA_R_64F))
    capi.check(lib.mcsparseCreateDnVec(C.byref(y), rows, C.c_void_p(dummy_f.data_ptr()), capi.MACA_R_64F))
    a, b, pa, pb = _scalars(torch.float64, 1.0, 0.0)
    st = lib.mcsparseB200SpMVNoAlloc(handle.h, 0, pa, d, x, pb, y, capi.MACA_R_64F, 0)
    assert st == capi.MCSPARSE_STATUS_INSUFFICIENT_RESOURCES
    lib.mcsparseDestroySpMat(d)
    lib.mcsparseDestroyDnVec(x)
    lib.mcsparseDestroyDnVec(y)
