"""GPU parity tests of the complex value types (MACA_C_32F / MACA_C_64F) of mcsparseSpMV and mcsparseSpMM."""

import ctypes as C

import numpy as np
import pytest
import torch

import mcsparse_b200 as mc
from mcsparse_b200 import capi
from mcsparse_b200.capi import lib
from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, TOL, assert_close, csr_from_lengths

pytestmark = pytest.mark.gpu
N, T, H = (capi.MCSPARSE_OPERATION_NON_TRANSPOSE, capi.MCSPARSE_OPERATION_TRANSPOSE,
           capi.MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE)
ROW, COL = capi.MCSPARSE_ORDER_ROW, capi.MCSPARSE_ORDER_COL
MACA = {np.complex64: capi.MACA_C_32F, np.complex128: capi.MACA_C_64F}


def cplx(rng, shape, dtype):
    return (rng.uniform(-1, 1, shape) + 1j * rng.uniform(-1, 1, shape)).astype(dtype)


def up(a, device):
    t = torch.empty(a.size + 1, dtype=torch.from_numpy(a[:0]).dtype, device=device)
    t[:a.size] = torch.from_numpy(a).to(device)
    return t[:a.size]


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("beta", [0.0, -0.75 + 0.5j])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_complex_spmv(handle, device, name, dtype, base, beta):
    lengths = ADVERSARIAL_LENGTHS[name]
    m, n = len(lengths), max(max(lengths), 1) + 17
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=29, base=base)
    rng = np.random.default_rng(12)
    x, y0 = cplx(rng, n, dtype), cplx(rng, m, dtype)
    A = mc.CsrMatrix(m, n, up(rp, device), up(col, device), up(val, device), base=base)
    d_y = up(y0.copy(), device)
    X, Y = mc.DnVec(up(x, device)), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
    alpha = 1.25 - 0.5j
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(rp, col, val, x, alpha, beta, y0, base=base)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], name)
    # the work partition for this value type's tile size is bit-exact against the CPU partition
    items, nt, p = C.c_int(), C.c_int64(), C.c_void_p()
    capi.check(lib.mcsparseB200SpMVPartitionView(A.d, C.c_void_p(buf.data_ptr()), C.byref(items), C.byref(nt), C.byref(p)))
    assert items.value in capi.SPMV_TILE_ITEMS[MACA[dtype]]
    part = oracle.merge_path_partition(rp, col.size, items.value, base)
    off = p.value - buf.data_ptr()
    got = buf[off:off + part.size * 4].view(torch.int32).cpu().numpy().reshape(-1, 2)
    np.testing.assert_array_equal(got, part)


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
@pytest.mark.parametrize("op", [T, H])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle", "mixed_medium_long"])
def test_complex_spmv_transposed(handle, device, name, dtype, op):
    lengths = ADVERSARIAL_LENGTHS[name]
    m, n = len(lengths), max(max(lengths), 1) + 9
    base = 1
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=31, base=base)
    rng = np.random.default_rng(13)
    x, y0 = cplx(rng, m, dtype), cplx(rng, n, dtype)
    A = mc.CsrMatrix(m, n, up(rp, device), up(col, device), up(val, device), base=base)
    d_y = up(y0.copy(), device)
    X, Y = mc.DnVec(up(x, device)), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=op), dtype=torch.uint8, device=device)
    alpha, beta = -0.5 + 2.0j, 0.25 - 1.0j
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta, op=op)
    torch.cuda.synchronize()
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
    ref, d = oracle.spmv(t_ptr, t_idx, val[perm], x, alpha, beta, y0, conj=(op == H))
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], f"{name} op {op}")


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
@pytest.mark.parametrize("n,order", [(1, ROW), (2, ROW), (3, ROW), (8, ROW), (64, ROW), (5, COL)])
def test_complex_spmm(handle, device, dtype, n, order):
    lengths = ADVERSARIAL_LENGTHS["lengths_1_to_33"] + ADVERSARIAL_LENGTHS["empty_start_mid_end"] + [300]
    k, m, base = 400, None, n % 2
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=n, base=base)
    m = len(lengths)
    rng = np.random.default_rng(n)
    ldb = (n if order == ROW else k) + (2 if n == 3 else 0)
    ldc = n if order == ROW else m
    majorB, majorC = (k, m) if order == ROW else (n, n)
    B = cplx(rng, majorB * ldb, dtype)
    C0 = cplx(rng, majorC * ldc, dtype)
    t = [up(a, device) for a in (rp, col, val, B, C0.copy())]
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2], base=base)
    Bm, Cm = mc.DnMat(t[3], k, n, ldb, order), mc.DnMat(t[4], m, n, ldc, order)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    alpha, beta = 0.75 + 0.25j, -0.5 + 1.5j
    mc.spmm(handle, A, Bm, Cm, buf, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, B, ldb, order, n, alpha, beta, C0, ldc, order, base=base)
    raw = t[4].cpu().numpy()
    got = raw.reshape(m, ldc)[:, :n] if order == ROW else raw.reshape(n, ldc)[:, :m].T
    assert_close(got, ref, d, TOL[np.dtype(dtype)], f"complex SpMM n={n}")


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "many_short", "one_row_all_nnz", "all_empty"])
def test_legacy_complex_csrmv_csrmvex_csrmm(handle, device, dtype, name):
    """mcsparse{C,Z}csrmv, mcsparseCsrmvEx with complex types, mcsparse{C,Z}csrmm2 / csrmm (column-major B and C)."""
    lengths = ADVERSARIAL_LENGTHS[name]
    m, ncols, base = len(lengths), max(max(lengths), 1) + 5, 1
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=6, base=base)
    rng = np.random.default_rng(9)
    x, y0 = cplx(rng, ncols, dtype), cplx(rng, m, dtype)
    alpha, beta = 0.5 - 0.25j, 1.5 + 2.0j
    ref, d = oracle.spmv(rp, col, val, x, alpha, beta, y0, base=base)
    t = {k: up(v, device) for k, v in dict(rp=rp, col=col, val=val, x=x).items()}
    P = lambda k: mc.host._ptr(t[k])  # non-null also for empty arrays
    descr = C.c_void_p()
    capi.check(lib.mcsparseCreateMatDescr(C.byref(descr)))
    capi.check(lib.mcsparseSetMatIndexBase(descr, base))
    ct = C.c_float if dtype == np.complex64 else C.c_double
    a, b = (ct * 2)(alpha.real, alpha.imag), (ct * 2)(beta.real, beta.imag)
    pa, pb = C.cast(C.byref(a), C.c_void_p), C.cast(C.byref(b), C.c_void_p)
    single = dtype == np.complex64
    nnz = col.size

    y = up(y0.copy(), device)
    fn = lib.mcsparseCcsrmv if single else lib.mcsparseZcsrmv
    capi.check(fn(handle.h, N, m, ncols, nnz, pa, descr, P("val"), P("rp"), P("col"), P("x"), pb, C.c_void_p(y.data_ptr())))
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], "csrmv")

    y = up(y0.copy(), device)
    dt = MACA[dtype]
    sz = C.c_size_t()
    ex_args = (handle.h, capi.MCSPARSE_ALG_MERGE_PATH, N, m, ncols, nnz, pa, dt, descr, P("val"), dt, P("rp"), P("col"),
               P("x"), dt, pb, dt, C.c_void_p(y.data_ptr()), dt, dt)
    capi.check(lib.mcsparseCsrmvEx_bufferSize(*ex_args, C.byref(sz)))
    buf = torch.empty(sz.value, dtype=torch.uint8, device=device)
    capi.check(lib.mcsparseCsrmvEx(*ex_args, C.c_void_p(buf.data_ptr())))
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], "CsrmvEx")

    n, ldb, ldc = 3, ncols + 1, m + 2
    B, C0 = cplx(rng, n * ldb, dtype), cplx(rng, n * ldc, dtype)
    refC, dC = oracle.spmm(rp, col, val, B, ldb, COL, n, alpha, beta, C0, ldc, COL, base=base)
    for fn2, extra in ((lib.mcsparseCcsrmm2 if single else lib.mcsparseZcsrmm2, (N,)),
                       (lib.mcsparseCcsrmm if single else lib.mcsparseZcsrmm, ())):
        dB, dC0 = up(B, device), up(C0.copy(), device)
        capi.check(fn2(handle.h, N, *extra, m, n, ncols, nnz, pa, descr, P("val"), P("rp"), P("col"),
                       C.c_void_p(dB.data_ptr()), ldb, pb, C.c_void_p(dC0.data_ptr()), ldc))
        torch.cuda.synchronize()
        got = dC0.cpu().numpy().reshape(n, ldc)[:, :m].T
        assert_close(got, refC, dC, TOL[np.dtype(dtype)], "csrmm")
    lib.mcsparseDestroyMatDescr(descr)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("beta", [0.0, 0.5 - 1.25j])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle", "many_short"])
def test_real_matrix_complex_vectors(handle, device, name, dtype, base, beta):
    """Real values in A, complex x, y, alpha and beta (compute type complex)."""
    cdtype = np.complex64 if dtype == np.float32 else np.complex128
    lengths = ADVERSARIAL_LENGTHS[name]
    m, n = len(lengths), max(max(lengths), 1) + 3
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=47, base=base)
    rng = np.random.default_rng(17)
    x, y0 = cplx(rng, n, cdtype), cplx(rng, m, cdtype)
    t = [up(a, device) for a in (rp, col, val)]
    A = mc.CsrMatrix(m, n, *t, base=base)
    d_y = up(y0.copy(), device)
    X, Y = mc.DnVec(up(x, device)), mc.DnVec(d_y)
    alpha = -0.75 + 0.5j
    ct = C.c_float if dtype == np.float32 else C.c_double
    a, b = (ct * 2)(alpha.real, alpha.imag), (ct * 2)(complex(beta).real, complex(beta).imag)
    pa, pb = C.cast(C.byref(a), C.c_void_p), C.cast(C.byref(b), C.c_void_p)
    size = C.c_size_t()
    args = (handle.h, N, pa, A.d, X.d, pb, Y.d, MACA[cdtype], 0)
    capi.check(lib.mcsparseSpMV_bufferSize(*args, C.byref(size)))
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    capi.check(lib.mcsparseSpMV(*args, C.c_void_p(buf.data_ptr())))
    torch.cuda.synchronize()
    ref, d = oracle.spmv(rp, col, val.astype(cdtype), x, alpha, beta, y0, base=base)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(cdtype)], name)
    assert lib.mcsparseSpMV_bufferSize(handle.h, T, pa, A.d, Y.d, pb, X.d, MACA[cdtype], 0,
                                       C.byref(size)) == capi.MCSPARSE_STATUS_NOT_SUPPORTED


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_complex_with_64bit_indices(handle, device, dtype):
    """SpMV and SpMM with complex values and 64-bit indices agree bit for bit with the 32-bit run (SpMV at the
    small tile size, the only one 64-bit indices use)."""
    lengths = ADVERSARIAL_LENGTHS["long_then_short"] + ADVERSARIAL_LENGTHS["lengths_1_to_33"]
    m, k, base, n = len(lengths), 9100, 1, 6
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=59, base=base)
    rng = np.random.default_rng(19)
    x, B = cplx(rng, k, dtype), cplx(rng, k * n, dtype)
    alpha = 0.5 + 0.25j
    ys, cs = [], []
    for idx in (np.int32, np.int64):
        A = mc.CsrMatrix(m, k, up(rp.astype(idx), device), up(col.astype(idx), device), up(val, device), base=base)
        d_y = torch.zeros(m, dtype=torch.from_numpy(val[:0]).dtype, device=device)
        X, Y = mc.DnVec(up(x, device)), mc.DnVec(d_y)
        buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
        mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=0.0)
        d_c = torch.zeros(m * n, dtype=d_y.dtype, device=device)
        Bm, Cm = mc.DnMat(up(B, device), k, n, n, ROW), mc.DnMat(d_c, m, n, n, ROW)
        mc.spmm(handle, A, Bm, Cm, torch.empty(256, dtype=torch.uint8, device=device), alpha=alpha, beta=0.0)
        torch.cuda.synchronize()
        ys.append(d_y.cpu().numpy())
        cs.append(d_c.cpu().numpy())
    ref, d = oracle.spmv(rp, col, val, x, alpha, 0.0, base=base)
    assert_close(ys[1], ref, d, TOL[np.dtype(dtype)], "complex SpMV, 64-bit indices")
    refC, dC = oracle.spmm(rp, col, val, B, n, ROW, n, alpha, 0.0, base=base)
    assert_close(cs[1].reshape(m, n), refC, dC, TOL[np.dtype(dtype)], "complex SpMM, 64-bit indices")
    np.testing.assert_array_equal(cs[0], cs[1])


def test_complex_refusals(handle, device):
    """Complex values on the entry points that stay real-only."""
    rp, col, val = csr_from_lengths([2, 3, 0, 1], 5, np.complex64)
    t = [up(a, device) for a in (rp, col, val)]
    A = mc.CsrMatrix(4, 5, *t)
    A64 = mc.CsrMatrix(4, 5, t[0].long(), t[1].long(), t[2])
    x, y = torch.ones(5, dtype=torch.complex64, device=device), torch.zeros(4, dtype=torch.complex64, device=device)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    one = (C.c_float * 2)(1.0, 0.0)
    pa = C.cast(C.byref(one), C.c_void_p)
    size = C.c_size_t()
    c32 = capi.MACA_C_32F
    assert lib.mcsparseSpMV_bufferSize(handle.h, N, pa, A.d, X.d, pa, Y.d, c32, 0, C.byref(size)) == 0
    assert lib.mcsparseSpMV_bufferSize(handle.h, N, pa, A64.d, X.d, pa, Y.d, c32, 0, C.byref(size)) == 0
    assert lib.mcsparseB200SpMVNoAlloc(handle.h, N, pa, A.d, X.d, pa, Y.d, c32, 0) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    # real values with op(A) = A^H stay an invalid combination, as in the reference
    rpr, colr, valr = csr_from_lengths([2, 3, 0, 1], 5, np.float32)
    Ar = mc.CsrMatrix(4, 5, *[up(a, device) for a in (rpr, colr, valr)])
    Xr, Yr = mc.DnVec(torch.ones(4, device=device)), mc.DnVec(torch.zeros(5, device=device))
    onef = C.c_float(1.0)
    assert lib.mcsparseSpMV_bufferSize(handle.h, H, C.byref(onef), Ar.d, Xr.d, C.byref(onef), Yr.d, capi.MACA_R_32F, 0,
                                       C.byref(size)) == capi.MCSPARSE_STATUS_INVALID_VALUE


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
@pytest.mark.parametrize("preprocess", [False, True])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle", "many_short"])
def test_complex_csc_conjugate_transpose(handle, device, name, dtype, preprocess):
    """y = alpha * A^H x + beta * y for a CSC matrix: the CSC arrays are the CSR arrays of A^T, the values are
    conjugated on the fly (the reference conjugates them in place first, mcsp_spmv_gpu.cpp:741-770)."""
    lengths = ADVERSARIAL_LENGTHS[name]  # lengths of A's columns
    n, m = len(lengths), max(max(lengths), 1) + 9  # A is m x n
    base = 1
    cp, ri, val = csr_from_lengths(lengths, m, dtype, seed=17, base=base)
    rng = np.random.default_rng(19)
    x, y0 = cplx(rng, m, dtype), cplx(rng, n, dtype)
    d_val = up(val, device)
    A = mc.CscMatrix(m, n, up(cp, device), up(ri, device), d_val, base=base)
    d_y = up(y0.copy(), device)
    X, Y = mc.DnVec(up(x, device)), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=H), dtype=torch.uint8, device=device)
    alpha, beta = 0.75 - 1.5j, -0.5 + 0.25j
    if preprocess:
        mc.spmv_preprocess(handle, A, X, Y, buf, op=H)
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta, op=H)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(cp, ri, val, x, alpha, beta, y0, base=base, conj=True)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], name)
    assert np.array_equal(d_val.cpu().numpy(), val)  # the values stay as they were
    # beta = 0 does not read y
    d_y.fill_(float("nan"))
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=0.0, op=H)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(cp, ri, val, x, alpha, 0.0, None, base=base, conj=True)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], name + " beta 0")
