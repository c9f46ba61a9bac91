"""GPU tests at the benchmark's full sizes, through properties that do not need a full CPU pass
(analytic answers, linearity, sampled row blocks against the oracle) plus a full oracle comparison
where the CPU finishes in seconds."""

import numpy as np
import pytest
import torch

import mcsparse_b200 as mc
from mcsparse_b200 import workloads
from oracle import oracle
from tests.util import TOL, assert_close

pytestmark = pytest.mark.gpu


def _run(handle, device, w, x, alpha, beta, y0=None):
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    y = torch.zeros(w.rows, dtype=w.val.dtype, device=device) if y0 is None else y0.clone()
    X, Y = mc.DnVec(x), mc.DnVec(y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf)
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    return y


def _check_row_block(w, x, y, alpha, beta, y0, r0, r1, tol, what):
    """Oracle on rows [r0, r1) only: the slice of A is copied to the host, x in full."""
    a0, a1 = int(w.row_ptr[r0]), int(w.row_ptr[r1])
    rp = (w.row_ptr[r0:r1 + 1] - w.row_ptr[r0]).cpu()
    ref, d = oracle.spmv(rp, w.col[a0:a1].cpu(), w.val[a0:a1].cpu(), x.cpu(), alpha, beta,
                         None if y0 is None else y0[r0:r1].cpu())
    assert_close(y[r0:r1].cpu().numpy(), ref, d, tol, what)


def test_c1_full_against_oracle_and_row_sums(handle, device):
    w = workloads.generate("C1", device)
    assert (w.rows, w.nnz) == (1048576, 5238784)
    y = _run(handle, device, w, w.x, 1.0, 0.0)
    ref, d = oracle.spmv(w.row_ptr, w.col, w.val, w.x, 1.0, 0.0)
    assert_close(y.cpu().numpy(), ref, d, 1e-5, "C1")
    ones = torch.ones(w.cols, dtype=torch.float32, device=device)
    y1 = _run(handle, device, w, ones, 1.0, 0.0)
    lengths = torch.diff(w.row_ptr).float()
    assert torch.equal(y1, 5.0 - lengths)  # exact in fp32: small integers


def test_c2_full_against_oracle(handle, device):
    w = workloads.generate("C2", device)
    assert w.rows == 4194304 and abs(w.nnz / w.rows - 16.0) < 0.05
    y = _run(handle, device, w, w.x, w.alpha, w.beta, w.y0)
    ref, d = oracle.spmv(w.row_ptr, w.col, w.val, w.x, w.alpha, w.beta, w.y0)
    assert_close(y.cpu().numpy(), ref, d, 1e-12, "C2")


def test_c3_full_blocks_and_linearity(handle, device):
    w = workloads.generate("C3", device)
    assert w.rows == 16777216 and abs(w.nnz / 2.0e8 - 1.0) < 0.05
    lengths = torch.diff(w.row_ptr)
    assert int(lengths.max()) > 50000 and int(lengths.min()) >= 1  # the heavy tail is present
    y = _run(handle, device, w, w.x, 1.0, 0.0)
    longest = int(torch.argmax(lengths))
    for r0 in (0, max(0, longest - 1000), w.rows - 200000):
        _check_row_block(w, w.x, y, 1.0, 0.0, None, r0, min(w.rows, r0 + 200000), 1e-5, f"C3 rows from {r0}")
    # linearity: A(2x) = 2 A x exactly (powers of two commute with rounding)
    y2 = _run(handle, device, w, 2.0 * w.x, 1.0, 0.0)
    assert torch.equal(y2, 2.0 * y)
    # reproducibility at full size
    assert torch.equal(y, _run(handle, device, w, w.x, 1.0, 0.0))


def test_c5_full_row_sums_and_blocks(handle, device):
    w = workloads.generate("C5", device)
    assert (w.rows, w.nnz) == (16777216, 766 ** 3)
    ones = torch.ones(w.cols, dtype=torch.float64, device=device)
    y1 = _run(handle, device, w, ones, 1.0, 0.0)
    lengths = torch.diff(w.row_ptr).double()
    assert torch.equal(y1, 27.0 - lengths)  # 26 - (neighbours present) = missing neighbours
    y = _run(handle, device, w, w.x, 1.0, 0.0)
    for r0 in (0, 8000000, w.rows - 150000):
        _check_row_block(w, w.x, y, 1.0, 0.0, None, r0, r0 + 150000, 1e-12, f"C5 rows from {r0}")
    # y = A x - y0 with beta = -1 equals the beta = 0 result minus y0, up to one rounding of the subtraction
    y0 = workloads.dense_values(w.cfg, device, w.rows, 51)
    yb = _run(handle, device, w, w.x, 1.0, -1.0, y0)
    assert torch.allclose(yb, y - y0, rtol=0, atol=1e-12 * float((y.abs() + y0.abs()).max()))


@pytest.mark.parametrize("n", [64, 128])
def test_c4_full_sampled_rows(handle, device, n):
    w = workloads.generate("C4", device)
    assert w.rows == 1048576 and abs(w.nnz / w.rows - 32.0) < 0.1
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    Cout = torch.full((w.rows, n), float("nan"), dtype=torch.float32, device=device)
    Bm, Cm = mc.DnMat(w.B[n], w.cols, n, n), mc.DnMat(Cout, w.rows, n, n)
    buf = torch.empty(mc.spmm_buffer_size(handle, A, Bm, Cm), dtype=torch.uint8, device=device)
    mc.spmm_preprocess(handle, A, Bm, Cm, buf)
    mc.spmm(handle, A, Bm, Cm, buf)
    torch.cuda.synchronize()
    assert not torch.isnan(Cout).any()
    Bh = w.B[n].cpu()
    for r0 in (0, 524288, w.rows - 4096):
        r1 = r0 + 4096
        a0, a1 = int(w.row_ptr[r0]), int(w.row_ptr[r1])
        rp = (w.row_ptr[r0:r1 + 1] - w.row_ptr[r0]).cpu()
        ref, d = oracle.spmm(rp, w.col[a0:a1].cpu(), w.val[a0:a1].cpu(), Bh, n, 2, n, 1.0, 0.0)
        assert_close(Cout[r0:r1].cpu().numpy(), ref, d, 1e-5, f"C4 n={n} rows from {r0}")


def test_c5_full_transposed_equals_plain_product(handle, device):
    """The 27-point stencil is symmetric, so A^T x must reproduce A x: checks the conversion at full size
    (three radix passes over 449 M nonzeros, digit counts scanned in more than one 1024-chunk round) and
    the converted structure against the source (the transpose of a symmetric pattern is the pattern)."""
    from mcsparse_b200 import capi

    w = workloads.generate("C5", device)
    y_plain = _run(handle, device, w, w.x, 1.0, 0.0)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    y = torch.zeros(w.cols, dtype=w.val.dtype, device=device)
    X, Y = mc.DnVec(w.x), mc.DnVec(y)
    T = capi.MCSPARSE_OPERATION_TRANSPOSE
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y, op=T), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf, op=T)
    mc.spmv(handle, A, X, Y, buf, alpha=1.0, beta=0.0, op=T)
    torch.cuda.synchronize()
    # same rows, same columns in the same (ascending) order, same values: the very same sums
    assert torch.equal(y, y_plain)
    import ctypes as C

    rows, p_ptr, p_idx, p_val = C.c_int64(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    capi.check(capi.lib.mcsparseB200SpMVTransposedView(A.d, T, C.c_void_p(buf.data_ptr()), C.byref(rows), C.byref(p_ptr),
                                                       C.byref(p_idx), C.byref(p_val)))
    off_ptr, off_idx = p_ptr.value - buf.data_ptr(), p_idx.value - buf.data_ptr()
    assert torch.equal(buf[off_ptr:off_ptr + 4 * (w.rows + 1)].view(torch.int32), w.row_ptr)
    assert torch.equal(buf[off_idx:off_idx + 4 * w.nnz].view(torch.int32), w.col)
