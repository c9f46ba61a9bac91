"""GPU parity tests of mcsparseSpMM and the legacy csrmm entry points, through the C ABI."""

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
ROW, COL = capi.MCSPARSE_ORDER_ROW, capi.MCSPARSE_ORDER_COL


def dense(rng, rows, cols, ld, order, dtype):
    """Backing array of a rows x cols matrix with leading dimension ld, padding filled with a sentinel."""
    major = rows if order == ROW else cols
    a = np.full(major * ld, 777.0, dtype)
    v = a.reshape(major, ld)
    minor = cols if order == ROW else rows
    v[:, :minor] = rng.uniform(-1, 1, (major, minor)).astype(dtype)
    return a


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n", [1, 3, 4, 5, 32, 64, 100, 128, 256])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_spmm_row_major(handle, device, dtype, n, beta):
    lengths = ADVERSARIAL_LENGTHS["lengths_1_to_33"] + ADVERSARIAL_LENGTHS["empty_start_mid_end"] + [300]
    k = 400
    base = n % 2
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=n, base=base)
    m = len(lengths)
    rng = np.random.default_rng(n)
    ldb, ldc = n + (4 if n % 3 == 0 else 0), n + (8 if n % 5 == 0 else 0)
    B, C0 = dense(rng, k, n, ldb, ROW, dtype), dense(rng, m, n, ldc, ROW, dtype)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B, C0.copy())]
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2], base=base)
    Bm, Cm = mc.DnMat(t[3], k, n, ldb, ROW), mc.DnMat(t[4], m, n, ldc, ROW)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    mc.spmm(handle, A, Bm, Cm, buf, alpha=-1.5, beta=beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, B, ldb, ROW, n, -1.5, beta, C0, ldc, ROW, base=base)
    got = t[4].cpu().numpy().reshape(m, ldc)
    assert_close(got[:, :n], ref, d, TOL[np.dtype(dtype)], f"n={n}")
    assert (got[:, n:] == 777.0).all(), "padding columns of C must stay untouched"


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("order_b,order_c", [(COL, COL), (ROW, COL), (COL, ROW)])
def test_spmm_other_layouts(handle, device, dtype, order_b, order_c):
    lengths = ADVERSARIAL_LENGTHS["lengths_63_65"] + [0, 1, 2]
    k, n = 90, 12
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=2)
    m = len(lengths)
    rng = np.random.default_rng(1)
    ldb = (n if order_b == ROW else k) + 3
    ldc = (n if order_c == ROW else m) + 2
    B, C0 = dense(rng, k, n, ldb, order_b, dtype), dense(rng, m, n, ldc, order_c, dtype)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B, C0.copy())]
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2])
    Bm, Cm = mc.DnMat(t[3], k, n, ldb, order_b), mc.DnMat(t[4], m, n, ldc, order_c)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    mc.spmm(handle, A, Bm, Cm, buf, alpha=2.0, beta=-1.0)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, B, ldb, order_b, n, 2.0, -1.0, C0, ldc, order_c)
    raw = t[4].cpu().numpy()
    got = raw.reshape(m, ldc)[:, :n] if order_c == ROW else raw.reshape(n, ldc)[:, :m].T
    assert_close(got, ref, d, TOL[np.dtype(dtype)], "layouts")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n,order", [(64, ROW), (12, ROW), (5, COL)])
def test_spmm_64bit_indices(handle, device, dtype, n, order):
    """MCSPARSE_INDEX_64I row offsets and column indices give the 32-bit result bit for bit."""
    lengths = ADVERSARIAL_LENGTHS["lengths_1_to_33"] + ADVERSARIAL_LENGTHS["empty_start_mid_end"] + [300]
    k, m, base = 400, None, 1
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=9, base=base)
    m = len(lengths)
    rng = np.random.default_rng(9)
    ldb = n if order == ROW else k
    ldc = n if order == ROW else m
    B, C0 = dense(rng, k, n, ldb, order, dtype), dense(rng, m, n, ldc, order, dtype)
    out = []
    for idx in (np.int32, np.int64):
        t = [torch.from_numpy(a).to(device) for a in (rp.astype(idx), col.astype(idx), val, B, C0.copy())]
        A = mc.CsrMatrix(m, k, t[0], t[1], t[2], base=base)
        Bm, Cm = mc.DnMat(t[3], k, n, ldb, order), mc.DnMat(t[4], m, n, ldc, order)
        buf = torch.empty(256, dtype=torch.uint8, device=device)
        mc.spmm(handle, A, Bm, Cm, buf, alpha=0.75, beta=-0.5)
        torch.cuda.synchronize()
        out.append(t[4].cpu().numpy())
    np.testing.assert_array_equal(out[0], out[1])
    ref, d = oracle.spmm(rp, col, val, B, ldb, order, n, 0.75, -0.5, C0, ldc, order, base=base)
    got = out[1].reshape(m, ldc) if order == ROW else out[1].reshape(n, ldc).T
    assert_close(got, ref, d, TOL[np.dtype(dtype)], f"64-bit indices, n={n}")


def test_spmm_op_b_transpose(handle, device):
    """op(B) = B^T with B stored n x k column-major is the same memory as k x n row-major."""
    dtype = np.float32
    lengths = [5, 0, 17, 33]
    k, n = 40, 8
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=5)
    rng = np.random.default_rng(5)
    Bkn = rng.uniform(-1, 1, (k, n)).astype(dtype)  # k x n row-major == (n x k) column-major with ld n
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, Bkn.ravel())]
    Cout = torch.zeros(len(lengths) * n, dtype=torch.float32, device=device)
    A = mc.CsrMatrix(len(lengths), k, t[0], t[1], t[2])
    Bm, Cm = mc.DnMat(t[3], n, k, n, COL), mc.DnMat(Cout, len(lengths), n, n, ROW)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    mc.spmm(handle, A, Bm, Cm, buf, op_b=capi.MCSPARSE_OPERATION_TRANSPOSE)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, Bkn, n, ROW, n, 1.0, 0.0)
    assert_close(Cout.cpu().numpy().reshape(-1, n), ref, d, 1e-5, "opB=T")


@pytest.mark.parametrize("n", [64, 128])
def test_spmm_scaled_config(handle, device, n):
    cfg = workloads.scaled("C4", 64)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    Cout = torch.full((w.rows, n), float("nan"), dtype=cfg.dtype, device=device)  # beta = 0 must not read it
    Bm, Cm = mc.DnMat(w.B[n], w.cols, n, n), mc.DnMat(Cout, w.rows, n, n)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    mc.spmm(handle, A, Bm, Cm, buf)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(w.row_ptr, w.col, w.val, w.B[n], n, ROW, n, 1.0, 0.0)
    assert_close(Cout.cpu().numpy(), ref, d, 1e-5, f"C4 n={n}")


def test_spmm_status_codes(handle, device):
    rp, col, val = csr_from_lengths([2, 3], 4, np.float32)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val)]
    A = mc.CsrMatrix(2, 4, *t)
    Bt, Ct = torch.ones(4 * 8, device=device), torch.zeros(2 * 8, device=device)
    B, Cm = mc.DnMat(Bt, 4, 8, 8), mc.DnMat(Ct, 2, 8, 8)
    Bbad = mc.DnMat(Bt, 5, 6, 6)
    Cld = mc.DnMat(Ct, 2, 8, 4)
    one = C.c_float(1.0)
    pa = C.cast(C.pointer(one), C.c_void_p)
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    pb = C.c_void_p(buf.data_ptr())
    f32 = capi.MACA_R_32F
    call = lib.mcsparseSpMM
    assert call(handle.h, 0, 0, pa, A.d, B.d, pa, Cm.d, f32, 0, pb) == 0
    assert call(handle.h, 0, 0, pa, A.d, B.d, pa, Cm.d, f32, 0, None) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, 0, 0, pa, None, B.d, pa, Cm.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, 1, 0, pa, A.d, B.d, pa, Cm.d, f32, 0, pb) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert call(handle.h, 0, 0, pa, A.d, B.d, pa, Cm.d, capi.MACA_R_64F, 0, pb) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert call(handle.h, 0, 0, pa, A.d, Bbad.d, pa, Cm.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, 0, 0, pa, A.d, B.d, pa, Cld.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    sz = C.c_size_t()
    assert lib.mcsparseSpMM_bufferSize(handle.h, 0, 0, pa, A.d, B.d, pa, Cm.d, f32, 0, C.byref(sz)) == 0
    assert sz.value == 128
    assert lib.mcsparseSpMM_preprocess(handle.h, 0, 0, pa, A.d, B.d, pa, Cm.d, f32, 0, pb) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("trans_b", [0, 1])
def test_legacy_csrmm2(handle, device, dtype, trans_b):
    lengths = ADVERSARIAL_LENGTHS["lengths_1_to_33"]
    k, n, base = 50, 7, 1
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=3, base=base)
    m = len(lengths)
    rng = np.random.default_rng(8)
    if trans_b:  # B is n x k column-major, ldb >= n
        ldb = n + 1
        B = dense(rng, n, k, ldb, COL, dtype)
        B_for_oracle, ld_o, order_o = B, ldb, ROW  # same memory read as k x n row-major
    else:  # B is k x n column-major, ldb >= k
        ldb = k + 2
        B = dense(rng, k, n, ldb, COL, dtype)
        B_for_oracle, ld_o, order_o = B, ldb, COL
    ldc = m + 3
    C0 = dense(rng, m, n, ldc, COL, dtype)
    ref, d = oracle.spmm(rp, col, val, B_for_oracle, ld_o, order_o, n, 1.5, 0.5, C0, ldc, COL, base=base)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B, C0.copy())]
    descr = C.c_void_p()
    capi.check(lib.mcsparseCreateMatDescr(C.byref(descr)))
    capi.check(lib.mcsparseSetMatIndexBase(descr, base))
    ct = C.c_float if dtype == np.float32 else C.c_double
    a, b = ct(1.5), ct(0.5)
    P = lambda x: C.c_void_p(x.data_ptr())
    fn = lib.mcsparseScsrmm2 if dtype == np.float32 else lib.mcsparseDcsrmm2
    capi.check(fn(handle.h, 0, trans_b, m, n, k, col.size, C.cast(C.pointer(a), C.c_void_p), descr, P(t[2]), P(t[0]),
                  P(t[1]), P(t[3]), ldb, C.cast(C.pointer(b), C.c_void_p), P(t[4]), ldc))
    torch.cuda.synchronize()
    got = t[4].cpu().numpy().reshape(n, ldc)[:, :m].T
    assert_close(got, ref, d, TOL[np.dtype(dtype)], "csrmm2")
    if not trans_b:
        t[4].copy_(torch.from_numpy(C0))
        fn1 = lib.mcsparseScsrmm if dtype == np.float32 else lib.mcsparseDcsrmm
        capi.check(fn1(handle.h, 0, m, n, k, col.size, C.cast(C.pointer(a), C.c_void_p), descr, P(t[2]), P(t[0]),
                       P(t[1]), P(t[3]), ldb, C.cast(C.pointer(b), C.c_void_p), P(t[4]), ldc))
        torch.cuda.synchronize()
        assert_close(t[4].cpu().numpy().reshape(n, ldc)[:, :m].T, ref, d, TOL[np.dtype(dtype)], "csrmm")
    lib.mcsparseDestroyMatDescr(descr)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("beta", [0.0, 0.5])
@pytest.mark.parametrize("shuffle_rows", [False, True])
@pytest.mark.parametrize("lanes", ["model", "4", "8", "16", "32"])
def test_spmm_column_panels(handle, device, dtype, beta, shuffle_rows, lanes, monkeypatch):
    """With a small L2 budget the preprocess call splits the product into column slabs and panels; the
    result must not change, whatever the slab width (modelled, or forced to 4 ... 32 lanes per row).
    Rows whose columns are not sorted are handled whole by the first panel."""
    monkeypatch.setenv("MCSPARSE_B200_SPMM_PANEL_MB", "1")
    if lanes != "model":
        monkeypatch.setenv("MCSPARSE_B200_SPMM_PANEL_LANES", lanes)
    rng = np.random.default_rng(3)
    m, k, n = 3000, 10000, (128 if lanes == "32" else 64)  # 32 lanes of fp32 are a slab of 128 columns
    lengths = rng.integers(12, 40, size=m).tolist()
    lengths[5], lengths[17], lengths[40] = 0, 1, 700  # an empty row, a single nonzero, pieces longer than the lane group
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=14)
    if shuffle_rows:
        for r in range(0, m, 7):
            seg = slice(rp[r], rp[r + 1])
            perm = rng.permutation(rp[r + 1] - rp[r])
            col[seg], val[seg] = col[seg][perm], val[seg][perm]
    B = rng.uniform(-1, 1, (k, n)).astype(dtype)
    C0 = rng.uniform(-1, 1, (m, n)).astype(dtype)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B.ravel(), C0.ravel().copy())]
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2])
    Bm, Cm = mc.DnMat(t[3], k, n, n), mc.DnMat(t[4], m, n, n)
    size = mc.spmm_buffer_size(handle, A, Bm, Cm)
    # the buffer holds (panels + 1) offsets and panels piece positions per row, and A regrouped panel by panel
    assert size > 2 * m * 4 + col.size * (4 + np.dtype(dtype).itemsize)
    if lanes != "model":  # a panel holds budget / max(128, 16 * lanes) rows of B
        panels = -(-k // ((1 << 20) // max(128, 16 * int(lanes))))
        assert size > (2 * panels + 1) * m * 4 + col.size * (4 + np.dtype(dtype).itemsize)
    buf = torch.empty(size, dtype=torch.uint8, device=device)
    mc.spmm_preprocess(handle, A, Bm, Cm, buf)
    mc.spmm(handle, A, Bm, Cm, buf, alpha=1.25, beta=beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, B, n, ROW, n, 1.25, beta, C0, n, ROW)
    assert_close(t[4].cpu().numpy().reshape(m, n), ref, d, TOL[np.dtype(dtype)], "column panels")
    # the same call without a preprocess (another buffer) takes the single-pass kernel: same result within tolerance
    t[4].copy_(torch.from_numpy(C0.ravel()))
    other = torch.empty(size, dtype=torch.uint8, device=device)
    mc.spmm(handle, A, Bm, Cm, other, alpha=1.25, beta=beta)
    torch.cuda.synchronize()
    assert_close(t[4].cpu().numpy().reshape(m, n), ref, d, TOL[np.dtype(dtype)], "single pass")


def test_spmm_panels_keep_regrouped_values_on_promise(handle, device, monkeypatch):
    """With mcsparseB200SpMatKeepConvertedValues the panelled product reuses the values it regrouped last time:
    an in-place edit is seen only after it was announced (mcsparseSpMatSetValues); without the promise at once."""
    monkeypatch.setenv("MCSPARSE_B200_SPMM_PANEL_MB", "1")
    rng = np.random.default_rng(8)
    m, k, n = 2000, 9000, 64
    rp, col, val = csr_from_lengths(rng.integers(10, 30, size=m).tolist(), k, np.float32, seed=4)
    B = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B.ravel())]
    Cd = torch.zeros(m * n, dtype=torch.float32, device=device)
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2])
    Bm, Cm = mc.DnMat(t[3], k, n, n), mc.DnMat(Cd, m, n, n)
    buf = torch.empty(mc.spmm_buffer_size(handle, A, Bm, Cm), dtype=torch.uint8, device=device)
    mc.spmm_preprocess(handle, A, Bm, Cm, buf)
    ref, d = oracle.spmm(rp, col, val, B, n, ROW, n, 1.0, 0.0)
    ref2, d2 = oracle.spmm(rp, col, 2 * val, B, n, ROW, n, 1.0, 0.0)

    def product():
        mc.spmm(handle, A, Bm, Cm, buf)
        torch.cuda.synchronize()
        return Cd.cpu().numpy().reshape(m, n)

    capi.check(lib.mcsparseB200SpMatKeepConvertedValues(A.d, 1))
    assert_close(product(), ref, d, 1e-5, "first product regroups")
    assert_close(product(), ref, d, 1e-5, "second product reuses")
    t[2].mul_(2)  # edited in place, not announced: the product may still use the old values
    assert_close(product(), ref, d, 1e-5, "unannounced edit")
    capi.check(lib.mcsparseSpMatSetValues(A.d, C.c_void_p(t[2].data_ptr())))
    assert_close(product(), ref2, d2, 1e-5, "announced edit")
    capi.check(lib.mcsparseB200SpMatKeepConvertedValues(A.d, 0))
    t[2].div_(2)
    assert_close(product(), ref, d, 1e-5, "without the promise every product regroups")


def test_spmm_panels_forgotten_when_the_buffer_is_given_to_spmv(handle, device, monkeypatch):
    """A buffer that holds recorded panels and is then handed to mcsparseSpMV for the same matrix no longer holds
    them: the next mcsparseSpMM with that buffer must not read them (it takes the single-pass kernel)."""
    monkeypatch.setenv("MCSPARSE_B200_SPMM_PANEL_MB", "1")
    rng = np.random.default_rng(21)
    m, k, n = 1500, 9000, 64
    rp, col, val = csr_from_lengths(rng.integers(10, 30, size=m).tolist(), k, np.float32, seed=5)
    B = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B.ravel())]
    Cd = torch.zeros(m * n, dtype=torch.float32, device=device)
    A = mc.CsrMatrix(m, k, t[0], t[1], t[2])
    Bm, Cm = mc.DnMat(t[3], k, n, n), mc.DnMat(Cd, m, n, n)
    buf = torch.empty(mc.spmm_buffer_size(handle, A, Bm, Cm), dtype=torch.uint8, device=device)
    mc.spmm_preprocess(handle, A, Bm, Cm, buf)
    x = torch.from_numpy(rng.uniform(-1, 1, k).astype(np.float32)).to(device)
    y = torch.zeros(m, dtype=torch.float32, device=device)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    assert mc.spmv_buffer_size(handle, A, X, Y) <= buf.numel()
    mc.spmv(handle, A, X, Y, buf)  # writes its partition over the start of the panel data
    mc.spmm(handle, A, Bm, Cm, buf)
    torch.cuda.synchronize()
    ref, d = oracle.spmm(rp, col, val, B, n, ROW, n, 1.0, 0.0)
    assert_close(Cd.cpu().numpy().reshape(m, n), ref, d, 1e-5, "SpMM after SpMV in the same buffer")
    refv, dv = oracle.spmv(rp, col, val, x.cpu().numpy(), 1.0, 0.0, None)
    assert_close(y.cpu().numpy(), refv, dv, 1e-5, "the SpMV itself")
    # and the other way round: a partition recorded by mcsparseSpMV_preprocess is forgotten when the buffer takes panels
    mc.spmv_preprocess(handle, A, X, Y, buf)
    mc.spmm_preprocess(handle, A, Bm, Cm, buf)
    y.fill_(float("nan"))
    mc.spmv(handle, A, X, Y, buf)
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy(), refv, dv, 1e-5, "SpMV after SpMM_preprocess in the same buffer")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shared_a", [False, True])
def test_spmm_strided_batch(handle, device, dtype, shared_a):
    """Three products in one call: operands a batch stride apart; a stride of 0 shares A between them."""
    batches, k, n = 3, 60, 8
    lengths = [4, 0, 9, 17, 1, 33]
    m = len(lengths)
    mats = [csr_from_lengths(lengths, k, dtype, seed=40 + (0 if shared_a else b)) for b in range(batches)]
    nnz = mats[0][1].size  # same lengths, so every batch has the same nonzero count
    rng = np.random.default_rng(40)
    Bs = rng.uniform(-1, 1, (batches, k, n)).astype(dtype)
    C0 = rng.uniform(-1, 1, (batches, m, n)).astype(dtype)
    if shared_a:
        rp, col, val = mats[0]
        strides = (0, 0)
    else:
        rp = np.concatenate([mt[0] for mt in mats])
        col = np.concatenate([mt[1] for mt in mats])
        val = np.concatenate([mt[2] for mt in mats])
        strides = (m + 1, nnz)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, Bs.ravel(), C0.ravel().copy())]
    A = mc.CsrMatrix(m, k, t[0][:m + 1], t[1][:nnz], t[2][:nnz])
    Bm, Cm = mc.DnMat(t[3], k, n, n), mc.DnMat(t[4], m, n, n)
    capi.check(lib.mcsparseCsrSetStridedBatch(A.d, batches, strides[0], strides[1]))
    capi.check(lib.mcsparseDnMatSetStridedBatch(Bm.d, batches, k * n))
    buf = torch.empty(256, dtype=torch.uint8, device=device)
    one = (C.c_float if dtype == np.float32 else C.c_double)(1.0)
    pa = C.cast(C.pointer(one), C.c_void_p)
    dt = capi.MACA_R_32F if dtype == np.float32 else capi.MACA_R_64F
    # C without a batch setting does not match A and B
    assert lib.mcsparseSpMM(handle.h, 0, 0, pa, A.d, Bm.d, pa, Cm.d, dt, 0,
                            C.c_void_p(buf.data_ptr())) == capi.MCSPARSE_STATUS_INVALID_VALUE
    capi.check(lib.mcsparseDnMatSetStridedBatch(Cm.d, batches, m * n))
    bc, bs = C.c_int(), C.c_int64()
    capi.check(lib.mcsparseDnMatGetStridedBatch(Cm.d, C.byref(bc), C.byref(bs)))
    assert (bc.value, bs.value) == (batches, m * n)
    mc.spmm(handle, A, Bm, Cm, buf, alpha=0.5, beta=2.0)
    torch.cuda.synchronize()
    got = t[4].cpu().numpy().reshape(batches, m, n)
    for b in range(batches):
        rpb, colb, valb = mats[b]
        ref, d = oracle.spmm(rpb, colb, valb, Bs[b], n, ROW, n, 0.5, 2.0, C0[b], n, ROW)
        assert_close(got[b], ref, d, TOL[np.dtype(dtype)], f"batch {b}")
    assert lib.mcsparseCsrSetStridedBatch(A.d, 0, 0, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE


class _Descr:
    """Holder with the two attributes mc.spmm needs (descriptor and value dtype)."""

    def __init__(self, d, dtype, keep):
        self.d, self.dtype, self.keep = d, dtype, keep

    def __del__(self):
        if lib is not None and self.d is not None:
            lib.mcsparseDestroySpMat(self.d)
            self.d = None


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64])
@pytest.mark.parametrize("fmt", ["coo", "coo_shuffled", "csc"])
@pytest.mark.parametrize("n,order", [(64, ROW), (12, ROW), (5, COL)])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty"])
def test_spmm_coo_and_csc_inputs(handle, device, name, n, order, fmt, dtype):
    """A given as row-sorted COO or as CSC: converted into the external buffer, then the CSR SpMM kernels."""
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    m, k, base = lengths.size, max(int(lengths.max()), 1) + 7, 1
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=41, base=base)
    rng = np.random.default_rng(3)

    def rand(count):
        v = rng.uniform(-1, 1, count)
        return (v + 1j * rng.uniform(-1, 1, count)).astype(dtype) if np.iscomplexobj(val) else v.astype(dtype)

    ldb, ldc = (n, n) if order == ROW else (k, m)
    B, C0 = rand((k if order == ROW else n) * ldb), rand((m if order == ROW else n) * ldc)
    pad = lambda a: np.concatenate([a, np.zeros(1, a.dtype)])  # non-null device pointers for empty arrays
    up = lambda a: torch.from_numpy(pad(a)).to(device)[:a.size]
    d = C.c_void_p()
    tdtype = torch.from_numpy(val[:0]).dtype
    maca = {np.float32: capi.MACA_R_32F, np.float64: capi.MACA_R_64F, np.complex64: capi.MACA_C_32F}[dtype]
    if fmt.startswith("coo"):
        coo_rows = (np.repeat(np.arange(m), lengths) + base).astype(np.int32)
        shuffle = rng.permutation(col.size) if fmt == "coo_shuffled" else np.arange(col.size)
        t = [up(coo_rows[shuffle]), up(col[shuffle]), up(val[shuffle])]
        capi.check(lib.mcsparseCreateCoo(C.byref(d), m, k, col.size, mc.host._ptr(t[0]),
                                         mc.host._ptr(t[1]), mc.host._ptr(t[2]),
                                         capi.MCSPARSE_INDEX_32I, base, maca))
    else:
        t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, k, base)
        t = [up((t_ptr + base).astype(np.int32)), up((t_idx + base).astype(np.int32)), up(val[perm])]
        capi.check(lib.mcsparseCreateCsc(C.byref(d), m, k, col.size, mc.host._ptr(t[0]),
                                         mc.host._ptr(t[1]), mc.host._ptr(t[2]),
                                         capi.MCSPARSE_INDEX_32I, capi.MCSPARSE_INDEX_32I, base, maca))
    A = _Descr(d, tdtype, t)
    dB, dC = up(B), up(C0.copy())
    Bm, Cm = mc.DnMat(dB, k, n, ldb, order), mc.DnMat(dC, m, n, ldc, order)
    buf = torch.empty(mc.spmm_buffer_size(handle, A, Bm, Cm), dtype=torch.uint8, device=device)
    alpha, beta = (0.75, -0.5) if not np.iscomplexobj(val) else (0.75 - 0.5j, -0.5 + 0.25j)
    mc.spmm(handle, A, Bm, Cm, buf, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    ref, dd = oracle.spmm(rp, col, val, B, ldb, order, n, alpha, beta, C0, ldc, order, base=base)
    raw = dC.cpu().numpy()
    got = raw.reshape(m, ldc)[:, :n] if order == ROW else raw.reshape(n, ldc)[:, :m].T
    assert_close(got, ref, dd, TOL[np.dtype(dtype)], f"{fmt} input, n={n}")
