"""GPU parity tests of the transposed products of mcsparseSpMV: op(A) = A^T on CSR and CSC inputs,
both through the device conversion that is checked bit for bit against the CPU one."""

import ctypes as C

import numpy as np
import pytest
import torch

import mcsparse_b200 as mc
from mcsparse_b200 import capi, workloads
from mcsparse_b200.capi import lib
from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, TOL, assert_close, csr_from_lengths

pytestmark = pytest.mark.gpu
N, T = capi.MCSPARSE_OPERATION_NON_TRANSPOSE, capi.MCSPARSE_OPERATION_TRANSPOSE


def device_view(A, op, buf, nnz, dtype):
    """(row offsets, column indices, values) of the converted matrix inside the buffer, as numpy arrays."""
    rows, p_ptr, p_idx, p_val = C.c_int64(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    capi.check(lib.mcsparseB200SpMVTransposedView(A.d, op, C.c_void_p(buf.data_ptr()), C.byref(rows), C.byref(p_ptr),
                                                  C.byref(p_idx), C.byref(p_val)))

    def grab(p, count, tdtype):
        off = p.value - buf.data_ptr()
        size = count * torch.empty(0, dtype=tdtype).element_size()
        return buf[off:off + size].view(tdtype).cpu().numpy()

    return (rows.value, grab(p_ptr, rows.value + 1, torch.int32), grab(p_idx, nnz, torch.int32),
            grab(p_val, nnz, torch.from_numpy(np.zeros(0, dtype)).dtype))


def up(a, device):
    """Device copy with a non-null address even when the array is empty (the C API rejects null arrays)."""
    t = torch.empty(a.size + 1, dtype=torch.from_numpy(a[:0]).dtype, device=device)
    t[:a.size] = torch.from_numpy(a).to(device)
    return t[:a.size]


def run(handle, device, A, op, x, y0, alpha, beta, preprocess=False):
    d_x, d_y = torch.from_numpy(x).to(device), torch.from_numpy(y0.copy()).to(device)
    X, Y = mc.DnVec(d_x), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=op), dtype=torch.uint8, device=device)
    if preprocess:
        mc.spmv_preprocess(handle, A, X, Y, buf, op=op)
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta, op=op)
    torch.cuda.synchronize()
    return d_y, buf, (X, Y)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("beta", [0.0, -0.75])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_spmv_transpose_csr(handle, device, name, dtype, base, beta):
    lengths = ADVERSARIAL_LENGTHS[name]
    m, n = len(lengths), max(max(lengths), 1) + 17
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=17, base=base)
    rng = np.random.default_rng(4)
    x, y0 = rng.uniform(-1, 1, m).astype(dtype), rng.uniform(-1, 1, n).astype(dtype)
    t = [up(a, device) for a in (rp, col, val)]
    A = mc.CsrMatrix(m, n, *t, base=base)
    d_y, buf, _ = run(handle, device, A, T, x, y0, 1.25, beta)
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
    ref, d = oracle.spmv(t_ptr, t_idx, val[perm], x, 1.25, beta, y0)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], name)
    rows, g_ptr, g_idx, g_val = device_view(A, T, buf, col.size, dtype)
    assert rows == n
    np.testing.assert_array_equal(g_ptr, t_ptr)
    np.testing.assert_array_equal(g_idx, t_idx)
    np.testing.assert_array_equal(g_val, val[perm])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle", "mostly_empty"])
def test_spmv_csc_input(handle, device, name, dtype, base):
    """A given in CSC form: A @ x goes through the conversion, A^T @ x runs the CSR kernels directly."""
    lengths = ADVERSARIAL_LENGTHS[name]
    m, n = len(lengths), max(max(lengths), 1) + 5
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=23, base=base)
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
    csc = [up(a, device) for a in ((t_ptr + base).astype(np.int32), (t_idx + base).astype(np.int32), val[perm])]
    A = mc.CscMatrix(m, n, *csc, base=base)
    rng = np.random.default_rng(6)
    xn, ym = rng.uniform(-1, 1, n).astype(dtype), rng.uniform(-1, 1, m).astype(dtype)
    d_y, _, _ = run(handle, device, A, N, xn, ym, 0.5, 2.0, preprocess=True)
    ref, d = oracle.spmv(rp, col, val, xn, 0.5, 2.0, ym, base=base)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], f"{name} CSC, A @ x")
    d_y, _, _ = run(handle, device, A, T, ym, xn, 0.5, 2.0)
    ref, d = oracle.spmv(t_ptr, t_idx, val[perm], ym, 0.5, 2.0, xn)
    assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], f"{name} CSC, A^T @ x")


@pytest.mark.parametrize("name,factor", [("C2", 64), ("C3", 64), ("C5", 64)])
def test_spmv_transpose_scaled_configs(handle, device, name, factor):
    """Three radix passes (more than 65536 columns), recorded conversion reused, values updated in place."""
    cfg = workloads.scaled(name, factor)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    x = workloads.dense_values(cfg, device, w.rows, 77)
    y = torch.zeros(w.cols, dtype=cfg.dtype, device=device)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=T), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf, op=T)
    rp, col = w.row_ptr.cpu().numpy(), w.col.cpu().numpy()
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, w.cols)
    results = []
    for scale in (1.0, -2.0, -2.0):
        w.val.mul_(scale)  # in place: the recorded structure stays valid, the values must be re-read
        mc.spmv(handle, A, X, Y, buf, alpha=1.0, beta=0.0, op=T)
        torch.cuda.synchronize()
        val = w.val.cpu().numpy()
        ref, d = oracle.spmv(t_ptr, t_idx, val[perm], x.cpu().numpy(), 1.0, 0.0)
        assert_close(y.cpu().numpy(), ref, d, TOL[cfg.dtype], f"{name} transposed, values x{scale}")
        results.append(y.clone())
    _, g_ptr, g_idx, _ = device_view(A, T, buf, col.size, val.dtype)
    np.testing.assert_array_equal(g_ptr, t_ptr)
    np.testing.assert_array_equal(g_idx, t_idx)
    # same inputs (values x4 of the first call), same conversion, same order of summation
    mc.spmv(handle, A, X, Y, buf, alpha=1.0, beta=0.0, op=T)
    torch.cuda.synchronize()
    assert torch.equal(y, results[-1])


def test_spmv_transpose_refusals(handle, device):
    rp, col, val = csr_from_lengths([2, 3, 0, 1], 5, np.float32)
    t64 = [torch.from_numpy(a).to(device) for a in (rp.astype(np.int64), col.astype(np.int64), val)]
    A64 = mc.CsrMatrix(4, 5, *t64)
    X, Y = mc.DnVec(torch.ones(4, device=device)), mc.DnVec(torch.zeros(5, device=device))
    one = C.c_float(1.0)
    pa = C.cast(C.pointer(one), C.c_void_p)
    size = C.c_size_t()
    # the peer-push and built-in-buffer entry points take op(A) = A only; 64-bit indices are converted like 32-bit ones
    assert lib.mcsparseSpMV_bufferSize(handle.h, T, pa, A64.d, X.d, pa, Y.d, capi.MACA_R_32F, 0, C.byref(size)) == 0
    t32 = [torch.from_numpy(a).to(device) for a in (rp, col, val)]
    A = mc.CsrMatrix(4, 5, *t32)
    assert lib.mcsparseB200SpMVNoAlloc(handle.h, T, pa, A.d, X.d, pa, Y.d, capi.MACA_R_32F,
                                       0) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert lib.mcsparseSpMV_bufferSize(handle.h, T, pa, A.d, X.d, pa, Y.d, capi.MACA_R_32F, 0, C.byref(size)) == 0
    plain = C.c_size_t()
    Xn, Yn = mc.DnVec(torch.ones(5, device=device)), mc.DnVec(torch.zeros(4, device=device))
    assert lib.mcsparseSpMV_bufferSize(handle.h, N, pa, A.d, Xn.d, pa, Yn.d, capi.MACA_R_32F, 0, C.byref(plain)) == 0
    assert size.value > plain.value  # the conversion area is part of the reported size


def test_one_buffer_alternating_between_a_and_a_transposed(handle, device):
    """The same external buffer used for A x and A^T x in turn, with preprocess calls in between: whatever
    was recorded in the buffer for one product must not be trusted by the other."""
    dtype = np.float64
    lengths = ADVERSARIAL_LENGTHS["many_short"] + ADVERSARIAL_LENGTHS["lengths_255_257"] + ADVERSARIAL_LENGTHS["tile_straddle"]
    m = len(lengths)
    n = m  # square, so that one pair of vectors serves both products
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=37)
    A = mc.CsrMatrix(m, n, up(rp, device), up(col, device), up(val, device))
    rng = np.random.default_rng(14)
    x = rng.uniform(-1, 1, n).astype(dtype)
    d_x, d_y = up(x, device), torch.zeros(m, dtype=torch.float64, device=device)
    X, Y = mc.DnVec(d_x), mc.DnVec(d_y)
    size = max(mc.spmv_buffer_size(handle, A, X, Y, op=T), mc.spmv_buffer_size(handle, A, X, Y, op=N))
    buf = torch.empty(size, dtype=torch.uint8, device=device)
    ref_n, d_n = oracle.spmv(rp, col, val, x, 1.0, 0.0)
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n)
    ref_t, d_t = oracle.spmv(t_ptr, t_idx, val[perm], x, 1.0, 0.0)
    for op, pre in [(N, True), (T, True), (N, False), (T, False), (T, True), (N, True), (N, False), (T, False)]:
        if pre:
            mc.spmv_preprocess(handle, A, X, Y, buf, op=op)
        mc.spmv(handle, A, X, Y, buf, op=op)
        torch.cuda.synchronize()
        ref, d = (ref_n, d_n) if op == N else (ref_t, d_t)
        assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], f"op {op} preprocess {pre}")


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex128])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("op", [N, T])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle", "many_short"])
def test_spmv_coo_any_order_and_transposed(handle, device, name, dtype, base, op):
    """COO entries shuffled: the library sorts them (stable, by row; by column for A^T) into the external
    buffer and runs the CSR kernels. The sorted structure is compared bit for bit with a stable CPU sort."""
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    m, n = lengths.size, max(int(lengths.max()), 1) + 13
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=43, base=base)
    rows = (np.repeat(np.arange(m), lengths) + base).astype(np.int32)
    rng = np.random.default_rng(21)
    shuffle = rng.permutation(col.size)
    rows_s, col_s, val_s = rows[shuffle], col[shuffle], val[shuffle]
    d = C.c_void_p()
    t = [up(a, device) for a in (rows_s, col_s, val_s)]
    maca = {np.float32: capi.MACA_R_32F, np.float64: capi.MACA_R_64F, np.complex128: capi.MACA_C_64F}[dtype]
    capi.check(lib.mcsparseCreateCoo(C.byref(d), m, n, col.size, mc.host._ptr(t[0]), mc.host._ptr(t[1]),
                                     mc.host._ptr(t[2]), capi.MCSPARSE_INDEX_32I, base, maca))

    class Holder:
        pass

    A = Holder()
    A.d, A.dtype = d, t[2].dtype
    xlen, ylen = (n, m) if op == N else (m, n)

    def rand(count):
        v = rng.uniform(-1, 1, count)
        return (v + 1j * rng.uniform(-1, 1, count)).astype(dtype) if np.iscomplexobj(val) else v.astype(dtype)

    x, y0 = rand(xlen), rand(ylen)
    alpha, beta = (1.25, -0.5) if not np.iscomplexobj(val) else (1.25 - 0.5j, -0.5 + 0.75j)
    d_y, buf, _ = run(handle, device, A, op, x, y0, alpha, beta, preprocess=True)
    if op == N:
        ref, dd = oracle.spmv(rp, col, val, x, alpha, beta, y0, base=base)
    else:
        t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
        ref, dd = oracle.spmv(t_ptr, t_idx, val[perm], x, alpha, beta, y0)
    assert_close(d_y.cpu().numpy(), ref, dd, TOL[np.dtype(dtype)], f"{name} shuffled COO op {op}")
    if col.size > 1 and (op == T or np.any(np.diff(rows_s) < 0)):  # converted: stable sort by row (or by column)
        key, other = (rows_s, col_s) if op == N else (col_s, rows_s)
        order = np.argsort(key, kind="stable")
        rows_out, g_ptr, g_idx, g_val = device_view(A, op, buf, col.size, dtype)
        assert rows_out == ylen
        np.testing.assert_array_equal(g_ptr, np.concatenate([[0], np.cumsum(np.bincount(key - base, minlength=ylen))]))
        np.testing.assert_array_equal(g_idx, other[order] - base)
        np.testing.assert_array_equal(g_val, val_s[order])
    lib.mcsparseDestroySpMat(d)


@pytest.mark.parametrize("dtype", [np.float64, np.complex64])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "tile_straddle"])
def test_converted_products_with_64bit_indices(handle, device, name, dtype):
    """A^T x on CSR, A x and A^T x on CSC, A x and A^T x on (sorted) COO, all with 64-bit indices: the conversion
    leaves the same 32-bit arrays as for 32-bit inputs, so the results agree bit for bit."""
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    m, n, base = lengths.size, max(int(lengths.max()), 1) + 9, 1
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=53, base=base)
    rows = (np.repeat(np.arange(m), lengths) + base).astype(np.int32)
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
    maca = {np.float64: capi.MACA_R_64F, np.complex64: capi.MACA_C_32F}[dtype]
    rng = np.random.default_rng(23)

    def rand(count):
        v = rng.uniform(-1, 1, count)
        return (v + 1j * rng.uniform(-1, 1, count)).astype(dtype) if np.iscomplexobj(val) else v.astype(dtype)

    xn, xm = rand(n), rand(m)
    alpha, beta = (0.5, 0.0)

    class Holder:
        pass

    def make(kind, idx_dtype):
        it = capi.MCSPARSE_INDEX_64I if idx_dtype == np.int64 else capi.MCSPARSE_INDEX_32I
        d = C.c_void_p()
        if kind == "csr":
            t = [up(rp.astype(idx_dtype), device), up(col.astype(idx_dtype), device), up(val, device)]
            capi.check(lib.mcsparseCreateCsr(C.byref(d), m, n, col.size, mc.host._ptr(t[0]), mc.host._ptr(t[1]),
                                             mc.host._ptr(t[2]), it, it, base, maca))
        elif kind == "csc":
            t = [up((t_ptr + base).astype(idx_dtype), device), up((t_idx + base).astype(idx_dtype), device),
                 up(val[perm], device)]
            capi.check(lib.mcsparseCreateCsc(C.byref(d), m, n, col.size, mc.host._ptr(t[0]), mc.host._ptr(t[1]),
                                             mc.host._ptr(t[2]), it, it, base, maca))
        else:
            t = [up(rows.astype(idx_dtype), device), up(col.astype(idx_dtype), device), up(val, device)]
            capi.check(lib.mcsparseCreateCoo(C.byref(d), m, n, col.size, mc.host._ptr(t[0]), mc.host._ptr(t[1]),
                                             mc.host._ptr(t[2]), it, base, maca))
        A = Holder()
        A.d, A.dtype, A.keep = d, t[2].dtype, t
        return A

    ref_n, d_n = oracle.spmv(rp, col, val, xn, alpha, beta, base=base)
    ref_t, d_t = oracle.spmv(t_ptr, t_idx, val[perm], xm, alpha, beta)
    for kind, ops in (("csr", (T,)), ("csc", (N, T)), ("coo", (N, T))):
        for op in ops:
            out = []
            for idx_dtype in (np.int32, np.int64):
                A = make(kind, idx_dtype)
                x, ylen = (xn, m) if op == N else (xm, n)
                d_y, _, _ = run(handle, device, A, op, x, np.zeros(ylen, dtype), alpha, beta)
                out.append(d_y.cpu().numpy())
                lib.mcsparseDestroySpMat(A.d)
            ref, d = (ref_n, d_n) if op == N else (ref_t, d_t)
            assert_close(out[1], ref, d, TOL[np.dtype(dtype)], f"{kind} op {op} 64-bit")
            if not (kind == "coo" and op == N):  # sorted 32-bit COO takes the direct path, 64-bit COO is re-sorted
                np.testing.assert_array_equal(out[0], out[1])


@pytest.mark.parametrize("dtype", [np.float32, np.complex128])
@pytest.mark.parametrize("op", [N, T])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty"])
def test_spmv_coo_array_of_pairs(handle, device, name, dtype, op):
    """COO given as one array of (row, column) pairs, entries shuffled."""
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    m, n, base = lengths.size, max(int(lengths.max()), 1) + 13, 1
    rp, col, val = csr_from_lengths(lengths, n, dtype, seed=61, base=base)
    rows = (np.repeat(np.arange(m), lengths) + base).astype(np.int32)
    rng = np.random.default_rng(29)
    shuffle = rng.permutation(col.size)
    pairs = np.stack([rows[shuffle], col[shuffle]], axis=1).astype(np.int32).ravel()
    t = [up(pairs, device), up(val[shuffle], device)]
    maca = {np.float32: capi.MACA_R_32F, np.complex128: capi.MACA_C_64F}[dtype]
    d = C.c_void_p()
    capi.check(lib.mcsparseCreateCooAoS(C.byref(d), m, n, col.size, mc.host._ptr(t[0]), mc.host._ptr(t[1]),
                                        capi.MCSPARSE_INDEX_32I, base, maca))
    got = [C.c_int64(), C.c_int64(), C.c_int64(), C.c_void_p(), C.c_void_p(), C.c_int(), C.c_int(), C.c_int()]
    capi.check(lib.mcsparseCooAoSGet(d, *[C.byref(g) for g in got]))
    assert (got[0].value, got[1].value, got[2].value, got[7].value) == (m, n, col.size, maca)

    class Holder:
        pass

    A = Holder()
    A.d, A.dtype = d, t[1].dtype
    xlen, ylen = (n, m) if op == N else (m, n)

    def rand(count):
        v = rng.uniform(-1, 1, count)
        return (v + 1j * rng.uniform(-1, 1, count)).astype(dtype) if np.iscomplexobj(val) else v.astype(dtype)

    x, y0 = rand(xlen), rand(ylen)
    alpha, beta = (1.25, -0.5) if not np.iscomplexobj(val) else (1.25 - 0.5j, -0.5 + 0.75j)
    for pre in (False, True):
        d_y, _, _ = run(handle, device, A, op, x, y0, alpha, beta, preprocess=pre)
        if op == N:
            ref, dd = oracle.spmv(rp, col, val, x, alpha, beta, y0, base=base)
        else:
            t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
            ref, dd = oracle.spmv(t_ptr, t_idx, val[perm], x, alpha, beta, y0)
        assert_close(d_y.cpu().numpy(), ref, dd, TOL[np.dtype(dtype)], f"{name} pairs op {op} preprocess {pre}")
    lib.mcsparseDestroySpMat(d)


def test_transposed_product_keeps_converted_values_on_promise(handle, device):
    """mcsparseB200SpMatKeepConvertedValues: once the caller promises to announce value changes, a transposed
    product reuses the values gathered last time; an in-place edit is then only seen after mcsparseSpMatSetValues."""
    cfg = workloads.scaled("C5", 64)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    x = workloads.dense_values(cfg, device, w.rows, 77)
    y = torch.zeros(w.cols, dtype=cfg.dtype, device=device)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=T), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf, op=T)
    capi.check(lib.mcsparseB200SpMatKeepConvertedValues(A.d, 1))
    mc.spmv(handle, A, X, Y, buf, op=T)  # gathers (nothing gathered yet)
    torch.cuda.synchronize()
    first = y.clone()
    mc.spmv(handle, A, X, Y, buf, op=T)  # reuses
    torch.cuda.synchronize()
    assert torch.equal(y, first)
    w.val.mul_(3.0)  # in place, not announced: the product still runs on the gathered copy
    mc.spmv(handle, A, X, Y, buf, op=T)
    torch.cuda.synchronize()
    assert torch.equal(y, first)
    capi.check(lib.mcsparseSpMatSetValues(A.d, C.c_void_p(w.val.data_ptr())))  # announced: gathered again
    mc.spmv(handle, A, X, Y, buf, op=T)
    torch.cuda.synchronize()
    rp, col = w.row_ptr.cpu().numpy(), w.col.cpu().numpy()
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, w.cols)
    ref, d = oracle.spmv(t_ptr, t_idx, w.val.cpu().numpy()[perm], x.cpu().numpy(), 1.0, 0.0)
    assert_close(y.cpu().numpy(), ref, d, TOL[cfg.dtype], "after the announced change")
    capi.check(lib.mcsparseB200SpMatKeepConvertedValues(A.d, 0))  # promise withdrawn: every product gathers again
    w.val.mul_(0.5)
    mc.spmv(handle, A, X, Y, buf, op=T)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(t_ptr, t_idx, w.val.cpu().numpy()[perm], x.cpu().numpy(), 1.0, 0.0)
    assert_close(y.cpu().numpy(), ref, d, TOL[cfg.dtype], "without the promise")
