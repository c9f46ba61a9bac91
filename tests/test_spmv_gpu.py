"""GPU parity tests of mcsparseSpMV and the legacy csrmv entry points, through the C ABI."""

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
DT = {np.float32: torch.float32, np.float64: torch.float64}
MACA = {np.float32: capi.MACA_R_32F, np.float64: capi.MACA_R_64F}


def run_spmv(handle, device, rp, col, val, x, y0, alpha, beta, base=0, preprocess=False, offset_elems=0,
             index_dtype=np.int32):
    """Uploads, runs mcsparseSpMV, returns (y, buffer, descriptor holder). offset_elems > 0 puts col/val at a
    misaligned address to reach the scalar-load variant; index_dtype=np.int64 passes 64-bit indices."""
    rp, col = rp.astype(index_dtype), col.astype(index_dtype)

    def up(a, off=0):
        t = torch.empty(a.size + off + 1, dtype=torch.from_numpy(a[:0]).dtype, device=device)
        t[off:off + a.size] = torch.from_numpy(a).to(device)
        return t[off:off + a.size]

    d_rp, d_col, d_val = up(rp), up(col, offset_elems), up(val, offset_elems)
    d_x, d_y = up(x), up(y0.copy())
    m = rp.size - 1
    A = mc.CsrMatrix(m, x.size, d_rp, d_col, d_val, base=base)
    X, Y = mc.DnVec(d_x), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
    if preprocess:
        mc.spmv_preprocess(handle, A, X, Y, buf)
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    return d_y.cpu().numpy(), buf, (A, X, Y)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("beta", [0.0, -0.75])
@pytest.mark.parametrize("tile", ["auto", "small", "large", "walk-small", "walk-large"])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_spmv_adversarial_shapes(handle, device, name, dtype, base, beta, tile, monkeypatch):
    if tile != "auto":  # force one of the two kernel families and one of the two tile sizes
        monkeypatch.setenv("MCSPARSE_B200_SPMV_WALK", "1" if tile.startswith("walk") else "0")
        tile = tile.replace("walk-", "")
        monkeypatch.setenv("MCSPARSE_B200_SPMV_TILE", tile)
    lengths = ADVERSARIAL_LENGTHS[name]
    ncols = max(max(lengths), 1) + 17
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=11, base=base)
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, ncols).astype(dtype)
    y0 = rng.uniform(-1, 1, len(lengths)).astype(dtype)
    y, buf, keep = run_spmv(handle, device, rp, col, val, x, y0, 1.25, beta, base)
    ref, d = oracle.spmv(rp, col, val, x, 1.25, beta, y0, base=base)
    assert_close(y, ref, d, TOL[np.dtype(dtype)], name)
    # the work partition in the buffer is bit-exact against the CPU partition
    nnz = col.size
    items, nt, p = C.c_int(), C.c_int64(), C.c_void_p()
    capi.check(lib.mcsparseB200SpMVPartitionView(keep[0].d, C.c_void_p(buf.data_ptr()), C.byref(items), C.byref(nt),
                                                 C.byref(p)))
    large, small = capi.SPMV_TILE_ITEMS[MACA[dtype]]  # the locality probe picks one of the two
    assert items.value == {"auto": items.value, "small": small, "large": large}[tile] and items.value in (large, small)
    part = oracle.merge_path_partition(rp, nnz, items.value, base)
    assert nt.value == part.shape[0] - 1
    off = p.value - buf.data_ptr()
    got = buf[off:off + part.size * 4].view(torch.int32).cpu().numpy().reshape(-1, 2)
    np.testing.assert_array_equal(got, part)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_spmv_beta_zero_does_not_read_y(handle, device, dtype):
    rp, col, val = csr_from_lengths([3, 0, 40, 5000, 1], 6000, dtype, seed=1)
    x = np.random.default_rng(0).uniform(-1, 1, 6000).astype(dtype)
    y0 = np.full(5, np.nan, dtype)
    y, _, _ = run_spmv(handle, device, rp, col, val, x, y0, 2.0, 0.0)
    ref, d = oracle.spmv(rp, col, val, x, 2.0, 0.0)
    assert_close(y, ref, d, TOL[np.dtype(dtype)], "beta=0 with NaN in y")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_spmv_alpha_zero_scales_y(handle, device, dtype):
    rp, col, val = csr_from_lengths([3, 2, 0, 9], 12, dtype, seed=1)
    x = np.ones(12, dtype)
    y0 = np.arange(4).astype(dtype)
    y, _, _ = run_spmv(handle, device, rp, col, val, x, y0, 0.0, 3.0)
    np.testing.assert_array_equal(y, 3.0 * y0)
    # alpha = beta = 0 writes zeros; nnz = 0 scales y (the reference leaves y untouched in both cases)
    y, _, _ = run_spmv(handle, device, rp, col, val, x, y0, 0.0, 0.0)
    np.testing.assert_array_equal(y, np.zeros(4, dtype))
    rp0 = np.zeros(5, np.int32)
    y, _, _ = run_spmv(handle, device, rp0, np.zeros(1, np.int32)[:0], np.zeros(0, dtype), x, y0, 1.0, 2.0)
    np.testing.assert_array_equal(y, 2.0 * y0)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("offset", [1, 2, 3])
def test_spmv_unaligned_arrays(handle, device, dtype, offset):
    lengths = ADVERSARIAL_LENGTHS["tile_straddle"] + ADVERSARIAL_LENGTHS["lengths_1_to_33"]
    ncols = 5000
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=4)
    rng = np.random.default_rng(3)
    x, y0 = rng.uniform(-1, 1, ncols).astype(dtype), rng.uniform(-1, 1, len(lengths)).astype(dtype)
    y, _, _ = run_spmv(handle, device, rp, col, val, x, y0, 1.0, 1.0, offset_elems=offset)
    ref, d = oracle.spmv(rp, col, val, x, 1.0, 1.0, y0)
    assert_close(y, ref, d, TOL[np.dtype(dtype)], f"offset {offset}")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_spmv_64bit_indices(handle, device, name, dtype, base, offset, monkeypatch):
    """MCSPARSE_INDEX_64I row offsets and column indices: same result, bit for bit, as the 32-bit
    run with the same (small) tile size, and the same work partition."""
    monkeypatch.setenv("MCSPARSE_B200_SPMV_TILE", "small")  # (8-byte values would also have the large tile)
    lengths = ADVERSARIAL_LENGTHS[name]
    ncols = max(max(lengths), 1) + 17
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=13, base=base)
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, ncols).astype(dtype)
    y0 = rng.uniform(-1, 1, len(lengths)).astype(dtype)
    y64, buf, keep = run_spmv(handle, device, rp, col, val, x, y0, 0.5, 1.5, base, offset_elems=offset,
                              index_dtype=np.int64)
    ref, d = oracle.spmv(rp, col, val, x, 0.5, 1.5, y0, base=base)
    assert_close(y64, ref, d, TOL[np.dtype(dtype)], name)
    items, nt, p = C.c_int(), C.c_int64(), C.c_void_p()
    capi.check(lib.mcsparseB200SpMVPartitionView(keep[0].d, C.c_void_p(buf.data_ptr()), C.byref(items), C.byref(nt),
                                                 C.byref(p)))
    small = capi.SPMV_TILE_ITEMS[MACA[dtype]][1]
    assert items.value == small
    part = oracle.merge_path_partition(rp, col.size, small, base)
    off = p.value - buf.data_ptr()
    got = buf[off:off + part.size * 4].view(torch.int32).cpu().numpy().reshape(-1, 2)
    np.testing.assert_array_equal(got, part)
    monkeypatch.setenv("MCSPARSE_B200_SPMV_TILE", "small")
    y32, _, _ = run_spmv(handle, device, rp, col, val, x, y0, 0.5, 1.5, base, offset_elems=offset)
    np.testing.assert_array_equal(y64, y32)


def test_spmv_64bit_indices_scaled_config(handle, device):
    cfg = workloads.scaled("C3", 64)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr.long(), w.col.long(), w.val)
    y = w.y0.clone()
    X, Y = mc.DnVec(w.x), mc.DnVec(y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf)
    mc.spmv(handle, A, X, Y, buf, alpha=w.alpha, beta=w.beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(w.row_ptr, w.col, w.val, w.x, w.alpha, w.beta, w.y0)
    assert_close(y.cpu().numpy(), ref, d, TOL[cfg.dtype], "C3 with 64-bit indices")
    # Mixed widths, 64-bit COO and the entry points that stay 32-bit only are refused, not misread.
    st = lib.mcsparseB200SpMVNoAlloc(handle.h, 0, C.byref(C.c_float(1)), A.d, X.d, C.byref(C.c_float(0)), Y.d,
                                     capi.MACA_R_32F, 0)
    assert st == capi.MCSPARSE_STATUS_NOT_SUPPORTED


@pytest.mark.parametrize("name,factor", [("C1", 16), ("C2", 64), ("C3", 64), ("C5", 64)])
def test_spmv_scaled_configs(handle, device, name, factor):
    cfg = workloads.scaled(name, factor)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    y = w.y0.clone()
    X, Y = mc.DnVec(w.x), mc.DnVec(y)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf)
    for _ in range(2):  # second call reuses the recorded analysis
        y.copy_(w.y0)
        mc.spmv(handle, A, X, Y, buf, alpha=w.alpha, beta=w.beta)
    torch.cuda.synchronize()
    ref, d = oracle.spmv(w.row_ptr, w.col, w.val, w.x, w.alpha, w.beta, w.y0)
    assert_close(y.cpu().numpy(), ref, d, TOL[cfg.dtype], name)
    status = C.c_int(-1)
    capi.check(lib.mcsparseB200SpMVGetStatus(handle.h, A.d, C.c_void_p(buf.data_ptr()), C.byref(status)))
    assert status.value == 0  # no thread block timed out waiting for its bulk copies


def test_spmv_is_reproducible(handle, device):
    cfg = workloads.scaled("C3", 64)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    ys = []
    for _ in range(3):
        y = torch.zeros(w.rows, dtype=cfg.dtype, device=device)
        X, Y = mc.DnVec(w.x), mc.DnVec(y)
        buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y), dtype=torch.uint8, device=device)
        mc.spmv(handle, A, X, Y, buf)
        ys.append(y)
    torch.cuda.synchronize()
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])


def test_spmv_device_pointer_mode_and_stream(device):
    stream = torch.cuda.Stream()
    h = mc.Handle(stream)
    s = C.c_void_p()
    capi.check(lib.mcsparseGetStream(h.h, C.byref(s)))
    assert (s.value or 0) == stream.cuda_stream
    h.set_pointer_mode(capi.MCSPARSE_POINTER_MODE_DEVICE)
    rp, col, val = csr_from_lengths(ADVERSARIAL_LENGTHS["long_then_short"], 9100, np.float64, seed=8)
    rng = np.random.default_rng(4)
    x, y0 = rng.uniform(-1, 1, 9100), rng.uniform(-1, 1, rp.size - 1)
    d_rp, d_col, d_val = (torch.from_numpy(a).to(device) for a in (rp, col, val))
    d_x, d_y = torch.from_numpy(x).to(device), torch.from_numpy(y0.copy()).to(device)
    alpha = torch.tensor([1.5], dtype=torch.float64, device=device)
    beta = torch.tensor([-2.0], dtype=torch.float64, device=device)
    A = mc.CsrMatrix(rp.size - 1, 9100, d_rp, d_col, d_val)
    X, Y = mc.DnVec(d_x), mc.DnVec(d_y)
    buf = torch.empty(mc.spmv_buffer_size(h, A, X, Y, alpha, beta), dtype=torch.uint8, device=device)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        mc.spmv(h, A, X, Y, buf, alpha=alpha, beta=beta)
    stream.synchronize()
    ref, d = oracle.spmv(rp, col, val, x, 1.5, -2.0, y0)
    assert_close(d_y.cpu().numpy(), ref, d, 1e-12, "device scalars")
    h.close()


def test_spmv_status_codes(handle, device):
    rp, col, val = csr_from_lengths([2, 3], 4, np.float32)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val)]
    x = torch.ones(4, device=device)
    y = torch.zeros(2, device=device)
    A = mc.CsrMatrix(2, 4, *t)
    X, Y, Ywrong = mc.DnVec(x), mc.DnVec(y), mc.DnVec(torch.zeros(3, device=device))
    X64 = mc.DnVec(torch.ones(4, dtype=torch.float64, device=device))
    one = C.c_float(1.0)
    pa = C.cast(C.pointer(one), C.c_void_p)
    buf = torch.empty(4096, dtype=torch.uint8, device=device)
    pb = C.c_void_p(buf.data_ptr())
    N, T, H = 0, 1, 2
    f32 = capi.MACA_R_32F
    call = lib.mcsparseSpMV
    assert call(handle.h, N, None, A.d, X.d, pa, Y.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, N, pa, None, X.d, pa, Y.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, N, pa, A.d, X.d, pa, Y.d, f32, 0, None) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, N, pa, A.d, X.d, pa, Ywrong.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, H, pa, A.d, Y.d, pa, X.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert call(handle.h, T, pa, A.d, X.d, pa, Y.d, f32, 0, pb) == capi.MCSPARSE_STATUS_INVALID_VALUE  # sizes not swapped
    assert call(handle.h, N, pa, A.d, X.d, pa, Y.d, capi.MACA_R_64F, 0, pb) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert call(handle.h, N, pa, A.d, X64.d, pa, Y.d, f32, 0, pb) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    mode = C.c_int(capi.MCSPARSE_FILL_MODE_LOWER)
    capi.check(lib.mcsparseSpMatSetAttribute(A.d, capi.MCSPARSE_SPMAT_FILL_MODE, C.byref(mode), 4))
    assert call(handle.h, N, pa, A.d, X.d, pa, Y.d, f32, 0, pb) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    mode = C.c_int(capi.MCSPARSE_FILL_MODE_FULL)
    capi.check(lib.mcsparseSpMatSetAttribute(A.d, capi.MCSPARSE_SPMAT_FILL_MODE, C.byref(mode), 4))
    assert call(handle.h, N, pa, A.d, X.d, pa, Y.d, f32, 0, pb) == 0
    sz = C.c_size_t()
    assert lib.mcsparseSpMV_bufferSize(handle.h, N, pa, A.d, X.d, pa, Y.d, f32, 0, None) == 3
    assert lib.mcsparseSpMV_bufferSize(handle.h, N, pa, A.d, X.d, pa, Y.d, f32, 0, C.byref(sz)) == 0
    assert sz.value >= 128
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "many_short", "uniform_27", "one_row_all_nnz", "all_empty"])
def test_legacy_csrmv_and_csrmvex(handle, device, dtype, name):
    lengths = ADVERSARIAL_LENGTHS[name]
    ncols = max(max(lengths), 1) + 5
    base = 1
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=6, base=base)
    rng = np.random.default_rng(9)
    x, y0 = rng.uniform(-1, 1, ncols).astype(dtype), rng.uniform(-1, 1, len(lengths)).astype(dtype)
    ref, d = oracle.spmv(rp, col, val, x, 0.5, 1.5, y0, base=base)
    pad = lambda a: np.concatenate([a, np.zeros(1, a.dtype)])  # keep device pointers non-null for empty arrays
    t = {k: torch.from_numpy(pad(v)).to(device) for k, v in dict(rp=rp, col=col, val=val, x=x).items()}
    descr = C.c_void_p()
    capi.check(lib.mcsparseCreateMatDescr(C.byref(descr)))
    capi.check(lib.mcsparseSetMatIndexBase(descr, base))
    ct = C.c_float if dtype == np.float32 else C.c_double
    a, b = ct(0.5), ct(1.5)
    pa, pb = C.cast(C.pointer(a), C.c_void_p), C.cast(C.pointer(b), C.c_void_p)
    P = lambda k: C.c_void_p(t[k].data_ptr())
    m, nnz = len(lengths), col.size

    y = torch.from_numpy(pad(y0)).to(device)
    fn = lib.mcsparseScsrmv if dtype == np.float32 else lib.mcsparseDcsrmv
    capi.check(fn(handle.h, 0, m, ncols, nnz, pa, descr, P("val"), P("rp"), P("col"), P("x"), pb,
                  C.c_void_p(y.data_ptr())))
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy()[:m], ref, d, TOL[np.dtype(dtype)], "csrmv")
    assert fn(handle.h, 1, m, ncols, nnz, pa, descr, P("val"), P("rp"), P("col"), P("x"), pb,
              C.c_void_p(y.data_ptr())) == capi.MCSPARSE_STATUS_NOT_SUPPORTED

    y = torch.from_numpy(pad(y0)).to(device)
    dt = MACA[dtype]
    sz = C.c_size_t()
    ex_args = (handle.h, capi.MCSPARSE_ALG_MERGE_PATH, 0, m, ncols, nnz, pa, dt, descr, P("val"), dt, P("rp"),
               P("col"), P("x"), dt, pb, dt, C.c_void_p(y.data_ptr()), dt, dt)
    capi.check(lib.mcsparseCsrmvEx_bufferSize(*ex_args, C.byref(sz)))
    buf = torch.empty(sz.value, dtype=torch.uint8, device=device)
    capi.check(lib.mcsparseCsrmvEx(*ex_args, C.c_void_p(buf.data_ptr())))
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy()[:m], ref, d, TOL[np.dtype(dtype)], "CsrmvEx")
    lib.mcsparseDestroyMatDescr(descr)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty",
                                  "tile_straddle"])
def test_spmv_coo_input(handle, device, name, dtype, base):
    """A row-sorted COO matrix goes through mcsparseSpMV: row offsets are derived on the device (bit-exact
    against the CPU count) and the CSR kernels run on them."""
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    ncols = max(int(lengths.max()), 1) + 11
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=31, base=base)
    coo_rows = (np.repeat(np.arange(lengths.size), lengths) + base).astype(np.int32)
    rng = np.random.default_rng(6)
    x, y0 = rng.uniform(-1, 1, ncols).astype(dtype), rng.uniform(-1, 1, lengths.size).astype(dtype)
    pad = lambda a: np.concatenate([a, np.zeros(1, a.dtype)])
    t = {k: torch.from_numpy(pad(v)).to(device) for k, v in dict(r=coo_rows, c=col, v=val, x=x, y=y0).items()}
    m, nnz = lengths.size, col.size
    d = C.c_void_p()
    P = lambda k: C.c_void_p(t[k].data_ptr())
    capi.check(lib.mcsparseCreateCoo(C.byref(d), m, ncols, nnz, P("r"), P("c"), P("v"), capi.MCSPARSE_INDEX_32I, base,
                                     MACA[dtype]))
    X, Y = mc.DnVec(t["x"][:ncols]), mc.DnVec(t["y"][:m])
    ct = C.c_float if dtype == np.float32 else C.c_double
    a, b = ct(-1.5), ct(0.25)
    pa, pb = C.cast(C.pointer(a), C.c_void_p), C.cast(C.pointer(b), C.c_void_p)
    sz = C.c_size_t()
    capi.check(lib.mcsparseSpMV_bufferSize(handle.h, 0, pa, d, X.d, pb, Y.d, MACA[dtype], 0, C.byref(sz)))
    buf = torch.empty(sz.value, dtype=torch.uint8, device=device)
    capi.check(lib.mcsparseSpMV(handle.h, 0, pa, d, X.d, pb, Y.d, MACA[dtype], 0, C.c_void_p(buf.data_ptr())))
    torch.cuda.synchronize()
    ref, dd = oracle.spmv(rp, col, val, x, -1.5, 0.25, y0, base=base)
    assert_close(t["y"].cpu().numpy()[:m], ref, dd, TOL[np.dtype(dtype)], "COO input")
    # the derived row offsets sit behind the SpMV work area
    items, nt, p = C.c_int(), C.c_int64(), C.c_void_p()
    capi.check(lib.mcsparseB200SpMVPartitionView(d, C.c_void_p(buf.data_ptr()), C.byref(items), C.byref(nt), C.byref(p)))
    csr_sz = C.c_size_t()
    A_csr = mc.CsrMatrix(m, ncols, torch.from_numpy(rp).to(device), t["c"][:max(nnz, 0)] if nnz else t["c"][:0],
                         t["v"][:nnz] if nnz else t["v"][:0], base=base)
    capi.check(lib.mcsparseSpMV_bufferSize(handle.h, 0, pa, A_csr.d, X.d, pb, Y.d, MACA[dtype], 0, C.byref(csr_sz)))
    off = (p.value - buf.data_ptr()) + (csr_sz.value - 256)
    got = buf[off:off + (m + 1) * 4].view(torch.int32).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.coo_row_offsets(coo_rows, m, base))
    # the entry points without a COO path refuse it
    assert lib.mcsparseB200SpMVNoAlloc(handle.h, 0, pa, d, X.d, pb, Y.d, MACA[dtype], 0) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    lib.mcsparseDestroySpMat(d)


@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_host_pipeline_matches_oracle(handle, device, beta):
    """HostSpmvPipeline: five products with different host vectors through two slots."""
    dtype = np.float64
    lengths = ADVERSARIAL_LENGTHS["tile_straddle"] + ADVERSARIAL_LENGTHS["lengths_1_to_33"]
    ncols = 5000
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=21)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val)]
    pipe = mc.HostSpmvPipeline(handle, len(lengths), ncols, t[0], t[1], t[2], depth=2)
    rng = np.random.default_rng(8)
    xs = [torch.from_numpy(rng.uniform(-1, 1, ncols)).pin_memory() for _ in range(5)]
    y0 = [rng.uniform(-1, 1, len(lengths)) for _ in range(5)]
    ys = [torch.from_numpy(v.copy()).pin_memory() for v in y0]
    for x, y in zip(xs, ys):
        pipe.submit(x, y, alpha=2.0, beta=beta)
    pipe.wait()
    for x, y, v in zip(xs, ys, y0):
        ref, d = oracle.spmv(rp, col, val, x.numpy(), 2.0, beta, v)
        assert_close(y.numpy(), ref, d, TOL[np.dtype(dtype)], "host pipeline")
    pipe.close()


@pytest.mark.parametrize("walk", ["0", "1"])
def test_bounded_wait_returns_error_status(device, walk, monkeypatch):
    """A tile kernel whose bulk copies never complete gives up after the handle's wait limit instead of
    spinning: with the diagnostics switch that withholds the copies (nothing is in flight), every tile
    reports through the buffer's status word and through the next call on the handle, the kernel returns
    cleanly, and the same handle computes correctly once the switch is off again."""
    monkeypatch.setenv("MCSPARSE_B200_SPMV_WALK", walk)
    h = mc.Handle()
    try:
        dtype = np.float64
        lengths = [5, 0, 300, 17] * 40
        rp, col, val = csr_from_lengths(lengths, 400, dtype, seed=21)
        x = np.random.default_rng(8).uniform(-1, 1, 400).astype(dtype)
        d_rp, d_col, d_val = (torch.from_numpy(a).to(device) for a in (rp, col, val))
        d_x = torch.from_numpy(x).to(device)
        d_y = torch.full((len(lengths),), 7.0, dtype=torch.float64, device=device)
        A = mc.CsrMatrix(len(lengths), 400, d_rp, d_col, d_val)
        X, Y = mc.DnVec(d_x), mc.DnVec(d_y)
        buf = torch.empty(mc.spmv_buffer_size(h, A, X, Y), dtype=torch.uint8, device=device)
        capi.check(lib.mcsparseB200SetDeviceWaitLimit(h.h, 100000, 1))  # 50 microseconds of SM clocks, copies withheld
        mc.spmv(h, A, X, Y, buf)  # asynchronous: the call itself succeeds
        torch.cuda.synchronize()  # ... and the kernel returns by itself
        status = C.c_int(-1)
        capi.check(lib.mcsparseB200SpMVGetStatus(h.h, A.d, C.c_void_p(buf.data_ptr()), C.byref(status)))
        assert status.value & 1
        assert torch.all(d_y == 7.0)  # the tiles that gave up wrote nothing
        capi.check(lib.mcsparseB200SetDeviceWaitLimit(h.h, 40000000, 0))
        with pytest.raises(capi.McsparseError) as err:  # reported once by the next compute call, without a sync
            mc.spmv(h, A, X, Y, buf)
        assert err.value.status == capi.MCSPARSE_STATUS_EXECUTION_FAILED
        mc.spmv_preprocess(h, A, X, Y, buf)  # a new analysis clears the buffer's status word
        mc.spmv(h, A, X, Y, buf)
        torch.cuda.synchronize()
        capi.check(lib.mcsparseB200SpMVGetStatus(h.h, A.d, C.c_void_p(buf.data_ptr()), C.byref(status)))
        assert status.value == 0
        ref, d = oracle.spmv(rp, col, val, x, 1.0, 0.0)
        assert_close(d_y.cpu().numpy(), ref, d, TOL[np.dtype(dtype)], "after the switch is off")
        assert lib.mcsparseB200SetDeviceWaitLimit(h.h, 0, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE
    finally:
        h.close()
