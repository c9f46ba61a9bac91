"""CPU tests of the C ABI: the library loads, exports what the headers declare, and the
descriptor API returns the reference's status codes. No kernel is launched."""

import ctypes as C
import os
import re

import pytest

from mcsparse_b200 import capi
from mcsparse_b200.capi import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = C.c_void_p(0x1000)  # never dereferenced by descriptor calls


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mcsparse\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 55
    dll = C.CDLL(capi.LIB_PATH)
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, missing
    assert set(names) == set(capi.PROTOTYPES), set(names) ^ set(capi.PROTOTYPES)


def test_error_names_and_strings():
    assert lib.mcsparseGetErrorName(0) == b"MCSPARSE_STATUS_SUCCESS"
    assert lib.mcsparseGetErrorName(10) == b"MCSPARSE_STATUS_NOT_SUPPORTED"
    assert lib.mcsparseGetErrorString(3) == b"invalid value"
    assert lib.mcsparseGetErrorString(6) == b"kernel launch failure"
    assert lib.mcsparseGetErrorName(99) == b"unrecognized error code"


def test_property_and_version():
    v = C.c_int()
    assert lib.mcsparseGetProperty(capi.MAJOR_VERSION, C.byref(v)) == 0 and v.value == 1
    assert lib.mcsparseGetProperty(7, C.byref(v)) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseGetVersion(None, C.byref(v)) == capi.MCSPARSE_STATUS_NOT_INITIALIZED
    assert lib.mcsparseGetVersion(FAKE, None) == capi.MCSPARSE_STATUS_INVALID_VALUE


def test_null_handle_is_not_initialized():
    s = C.c_void_p()
    assert lib.mcsparseSetStream(None, None) == capi.MCSPARSE_STATUS_NOT_INITIALIZED
    assert lib.mcsparseGetStream(None, C.byref(s)) == capi.MCSPARSE_STATUS_NOT_INITIALIZED
    assert lib.mcsparseSetPointerMode(None, 0) == capi.MCSPARSE_STATUS_NOT_INITIALIZED
    assert lib.mcsparseDestroy(None) == 0
    sz = C.c_size_t()
    assert lib.mcsparseSpMV_bufferSize(None, 0, FAKE, FAKE, FAKE, FAKE, FAKE, 0, 0, C.byref(sz)) == 1
    assert lib.mcsparseSpMV(None, 0, FAKE, FAKE, FAKE, FAKE, FAKE, 0, 0, FAKE) == 1
    assert lib.mcsparseSpMM(None, 0, 0, FAKE, FAKE, FAKE, FAKE, FAKE, 0, 0, FAKE) == 1
    assert lib.mcsparseScsrmv(None, 0, 1, 1, 1, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE) == 1


def test_csr_descriptor_roundtrip_and_errors():
    d = C.c_void_p()
    args = (FAKE, C.c_void_p(0x2000), C.c_void_p(0x3000), capi.MCSPARSE_INDEX_32I, capi.MCSPARSE_INDEX_32I, 1,
            capi.MACA_R_64F)
    assert lib.mcsparseCreateCsr(C.byref(d), -1, 4, 5, *args) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseCreateCsr(C.byref(d), 3, 4, 5, *args[:-1], capi.MACA_R_32I) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert lib.mcsparseCreateCsr(None, 3, 4, 5, *args) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseCreateCsr(C.byref(d), 3, 4, 5, *args) == 0
    rows, cols, nnz = C.c_int64(), C.c_int64(), C.c_int64()
    p0, p1, p2 = C.c_void_p(), C.c_void_p(), C.c_void_p()
    t0, t1, b, vt = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    assert lib.mcsparseCsrGet(d, C.byref(rows), C.byref(cols), C.byref(nnz), C.byref(p0), C.byref(p1), C.byref(p2),
                              C.byref(t0), C.byref(t1), C.byref(b), C.byref(vt)) == 0
    assert (rows.value, cols.value, nnz.value, p0.value, p1.value, p2.value) == (3, 4, 5, 0x1000, 0x2000, 0x3000)
    assert (t0.value, t1.value, b.value, vt.value) == (2, 2, 1, capi.MACA_R_64F)
    assert lib.mcsparseCsrGet(d, None, C.byref(cols), C.byref(nnz), C.byref(p0), C.byref(p1), C.byref(p2),
                              C.byref(t0), C.byref(t1), C.byref(b), C.byref(vt)) == capi.MCSPARSE_STATUS_INVALID_VALUE
    fmt = C.c_int()
    assert lib.mcsparseSpMatGetFormat(d, C.byref(fmt)) == 0 and fmt.value == capi.MCSPARSE_FORMAT_CSR
    assert lib.mcsparseSpMatGetIndexBase(d, C.byref(b)) == 0 and b.value == 1
    assert lib.mcsparseSpMatGetSize(d, C.byref(rows), C.byref(cols), C.byref(nnz)) == 0
    assert lib.mcsparseSpMatSetValues(d, C.c_void_p(0x4000)) == 0
    assert lib.mcsparseSpMatGetValues(d, C.byref(p2)) == 0 and p2.value == 0x4000
    assert lib.mcsparseCsrSetPointers(d, C.c_void_p(0x10), C.c_void_p(0x20), C.c_void_p(0x30)) == 0
    assert lib.mcsparseSpMatGetValues(d, C.byref(p2)) == 0 and p2.value == 0x30
    mode = C.c_int(capi.MCSPARSE_FILL_MODE_LOWER)
    assert lib.mcsparseSpMatSetAttribute(d, capi.MCSPARSE_SPMAT_FILL_MODE, C.byref(mode), 4) == 0
    got = C.c_int(-1)
    assert lib.mcsparseSpMatGetAttribute(d, capi.MCSPARSE_SPMAT_FILL_MODE, C.byref(got), 4) == 0 and got.value == 0
    assert lib.mcsparseSpMatGetAttribute(d, capi.MCSPARSE_SPMAT_FILL_MODE, None, 4) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseDestroySpMat(d) == 0
    assert lib.mcsparseDestroySpMat(None) == 0


def test_dense_descriptors():
    d = C.c_void_p()
    assert lib.mcsparseCreateDnVec(C.byref(d), -1, FAKE, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseCreateDnVec(C.byref(d), 5, None, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseCreateDnVec(C.byref(d), 5, FAKE, 26) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    assert lib.mcsparseCreateDnVec(C.byref(d), 5, FAKE, capi.MACA_R_32F) == 0
    size, p, vt = C.c_int64(), C.c_void_p(), C.c_int()
    assert lib.mcsparseDnVecGet(d, C.byref(size), C.byref(p), C.byref(vt)) == 0
    assert (size.value, p.value, vt.value) == (5, 0x1000, 0)
    assert lib.mcsparseDnVecSetValues(d, C.c_void_p(0x88)) == 0
    assert lib.mcsparseDnVecGetValues(d, C.byref(p)) == 0 and p.value == 0x88
    assert lib.mcsparseDestroyDnVec(d) == 0 and lib.mcsparseDestroyDnVec(None) == 0

    m = C.c_void_p()
    assert lib.mcsparseCreateDnMat(C.byref(m), 4, 3, -1, FAKE, 0, capi.MCSPARSE_ORDER_ROW) == 3
    assert lib.mcsparseCreateDnMat(C.byref(m), 4, 3, 3, None, 0, capi.MCSPARSE_ORDER_ROW) == 3
    assert lib.mcsparseCreateDnMat(C.byref(m), 4, 3, 3, FAKE, 27, capi.MCSPARSE_ORDER_ROW) == 10
    assert lib.mcsparseCreateDnMat(C.byref(m), 4, 3, 8, FAKE, capi.MACA_R_64F, capi.MCSPARSE_ORDER_ROW) == 0
    r, c, ld, order = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int()
    assert lib.mcsparseDnMatGet(m, C.byref(r), C.byref(c), C.byref(ld), C.byref(p), C.byref(vt), C.byref(order)) == 0
    assert (r.value, c.value, ld.value, vt.value, order.value) == (4, 3, 8, 1, 2)
    assert lib.mcsparseDnMatSetValues(m, C.c_void_p(0x99)) == 0
    assert lib.mcsparseDnMatGetValues(m, C.byref(p)) == 0 and p.value == 0x99
    assert lib.mcsparseDestroyDnMat(m) == 0 and lib.mcsparseDestroyDnMat(None) == 0


def test_mat_descr():
    d = C.c_void_p()
    assert lib.mcsparseCreateMatDescr(None) == 3
    assert lib.mcsparseCreateMatDescr(C.byref(d)) == 0
    assert lib.mcsparseGetMatIndexBase(d) == 0 and lib.mcsparseGetMatType(d) == 0
    assert lib.mcsparseGetMatFillMode(d) == capi.MCSPARSE_FILL_MODE_FULL and lib.mcsparseGetMatDiagType(d) == 0
    assert lib.mcsparseSetMatIndexBase(d, 1) == 0 and lib.mcsparseGetMatIndexBase(d) == 1
    assert lib.mcsparseSetMatIndexBase(d, 2) == 3
    assert lib.mcsparseSetMatType(d, 3) == 0 and lib.mcsparseSetMatType(d, 4) == 3
    assert lib.mcsparseSetMatFillMode(d, 0) == 0 and lib.mcsparseSetMatDiagType(d, 1) == 0
    assert lib.mcsparseSetMatIndexBase(None, 0) == 3 and lib.mcsparseGetMatIndexBase(None) == -1
    assert lib.mcsparseDestroyMatDescr(d) == 0


def test_partition_view_needs_arguments():
    ipt, nt, p = C.c_int(), C.c_int64(), C.c_void_p()
    assert lib.mcsparseB200SpMVPartitionView(None, FAKE, C.byref(ipt), C.byref(nt), C.byref(p)) == 3


def test_coo_descriptor_roundtrip():
    d = C.c_void_p()
    assert lib.mcsparseCreateCoo(C.byref(d), 3, 4, 5, FAKE, C.c_void_p(0x2000), C.c_void_p(0x3000),
                                 capi.MCSPARSE_INDEX_32I, 1, capi.MACA_R_32F) == 0
    fmt = C.c_int()
    assert lib.mcsparseSpMatGetFormat(d, C.byref(fmt)) == 0 and fmt.value == capi.MCSPARSE_FORMAT_COO
    rows, cols, nnz = C.c_int64(), C.c_int64(), C.c_int64()
    p0, p1, p2, it, b, vt = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_int(), C.c_int(), C.c_int()
    assert lib.mcsparseCooGet(d, C.byref(rows), C.byref(cols), C.byref(nnz), C.byref(p0), C.byref(p1), C.byref(p2),
                              C.byref(it), C.byref(b), C.byref(vt)) == 0
    assert (rows.value, cols.value, nnz.value, p0.value, p1.value, p2.value, it.value, b.value, vt.value) == \
        (3, 4, 5, 0x1000, 0x2000, 0x3000, 2, 1, 0)
    assert lib.mcsparseCooSetPointers(d, C.c_void_p(0x10), C.c_void_p(0x20), C.c_void_p(0x30)) == 0
    assert lib.mcsparseCooGet(d, C.byref(rows), C.byref(cols), C.byref(nnz), C.byref(p0), C.byref(p1), C.byref(p2),
                              C.byref(it), C.byref(b), None) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseCreateCoo(C.byref(d), 3, 4, -5, FAKE, FAKE, FAKE, 2, 0, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE
    assert lib.mcsparseDestroySpMat(d) == 0


def test_public_header_is_plain_c(tmp_path):
    """include/mcsparse.h is the C ABI: it must compile as C99 with nothing but the CUDA toolkit's C headers."""
    import shutil
    import subprocess

    cuda_inc = "/usr/local/cuda/include"
    if shutil.which("gcc") is None or not os.path.isdir(cuda_inc):
        pytest.skip("needs gcc and the CUDA toolkit headers")
    root = os.path.join(os.path.dirname(__file__), "..")
    src = tmp_path / "abi.c"
    src.write_text('#include "mcsparse.h"\nint main(void) { mcsparseHandle_t h = 0; (void)h; return 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(root, "include"), "-I",
                    cuda_inc, str(src)], check=True)


@pytest.mark.parametrize("env,where", [({}, "stderr"), ({"SPARSE_LOG_OUTPUT": "stdout"}, "stdout"),
                                       ({"SPARSE_LOG_OUTPUT": "file"}, "file"), ({"SPARSE_LOG_ENABLE": "0"}, None),
                                       ({"SPARSE_LOG_LEVEL": "0"}, None), ({"SPARSE_LOG_OUTPUT": "syslog"}, None)])
def test_logger_switches(tmp_path, env, where):
    """SPARSE_LOG_ENABLE / SPARSE_LOG_LEVEL / SPARSE_LOG_OUTPUT as the reference's logger reads them
    (mcsparse/src/utils/mcsp_logger.cpp:29-61), on a create-time error (mcsparse/src/common/mcsp_helper.cpp:327)."""
    import subprocess
    import sys

    code = ("import ctypes as C; from mcsparse_b200 import capi; d = C.c_void_p();"
            "st = capi.lib.mcsparseCreateDnVec(C.byref(d), -1, C.c_void_p(0x1000), capi.MACA_R_32F); print('status', st)")
    full = {k: v for k, v in os.environ.items() if not k.startswith("SPARSE_LOG")}
    full.update(env, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=full, capture_output=True, text=True, timeout=120)
    assert "status 3" in r.stdout, r.stderr
    log_file = tmp_path / "mcsparse.txt"
    seen = {"stderr": "Wrong input size" in r.stderr, "stdout": "Wrong input size" in r.stdout,
            "file": log_file.exists() and "Wrong input size" in log_file.read_text()}
    assert seen == {k: k == where for k in seen}
