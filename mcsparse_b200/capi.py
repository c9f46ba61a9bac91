"""ctypes binding of libmcsparse.so: one Python callable per C entry point, same names.

Enumerator values are the ones in ``include/mcsparse.h`` (which are the reference's,
mcsparse/include/common/mcsp_types.h.in:12-155).
"""

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# MCSPARSE_B200_LIB points the binding at another build of the library (tuning experiments).
LIB_PATH = os.environ.get("MCSPARSE_B200_LIB") or os.path.join(_HERE, "lib", "libmcsparse.so")

# status codes
MCSPARSE_STATUS_SUCCESS = 0
MCSPARSE_STATUS_NOT_INITIALIZED = 1
MCSPARSE_STATUS_ALLOC_FAILED = 2
MCSPARSE_STATUS_INVALID_VALUE = 3
MCSPARSE_STATUS_EXECUTION_FAILED = 6
MCSPARSE_STATUS_INTERNAL_ERROR = 7
MCSPARSE_STATUS_NOT_SUPPORTED = 10
MCSPARSE_STATUS_INSUFFICIENT_RESOURCES = 11
NOALLOC_SCRATCH_BYTES = 16 << 20
PEER_FLAG_INTS, PEER_FLAG_STATUS = 16, 8
# operations
MCSPARSE_OPERATION_NON_TRANSPOSE = 0
MCSPARSE_OPERATION_TRANSPOSE = 1
MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE = 2
# misc enums
MCSPARSE_INDEX_BASE_ZERO, MCSPARSE_INDEX_BASE_ONE = 0, 1
MCSPARSE_POINTER_MODE_HOST, MCSPARSE_POINTER_MODE_DEVICE = 0, 1
MCSPARSE_FORMAT_CSR = 1
MCSPARSE_FORMAT_COO = 3
MCSPARSE_ORDER_COL, MCSPARSE_ORDER_ROW = 1, 2
MCSPARSE_INDEX_16U, MCSPARSE_INDEX_32I, MCSPARSE_INDEX_64I = 1, 2, 3
MCSPARSE_MATRIX_TYPE_GENERAL, MCSPARSE_MATRIX_TYPE_SYMMETRIC = 0, 1
MCSPARSE_FILL_MODE_LOWER, MCSPARSE_FILL_MODE_UPPER, MCSPARSE_FILL_MODE_FULL = 0, 1, 2
MCSPARSE_DIAG_TYPE_NON_UNIT, MCSPARSE_DIAG_TYPE_UNIT = 0, 1
MCSPARSE_SPMAT_FILL_MODE, MCSPARSE_SPMAT_DIAG_TYPE = 0, 1
MCSPARSE_SPMV_ALG_DEFAULT = 0
MCSPARSE_SPMM_ALG_DEFAULT = 0
MCSPARSE_ALG_MERGE_PATH = 0
MACA_R_32F, MACA_R_64F, MACA_R_16F, MACA_C_32F, MACA_C_64F, MACA_R_32I = 0, 1, 2, 4, 5, 10
MACA_R_8I, MACA_R_16BF = 3, 14
MAJOR_VERSION, MINOR_VERSION, PATCH_LEVEL = 0, 1, 2

SPMV_TILE_ITEMS = {MACA_R_32F: (4096, 2048), MACA_R_64F: (2048, 1024),  # (large, small) tile per value type
                   MACA_C_32F: (2048, 1024), MACA_C_64F: (1024, 1024)}

_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_pvp = C.POINTER(C.c_void_p)
_pi, _pi64, _psz = C.POINTER(C.c_int), C.POINTER(C.c_int64), C.POINTER(C.c_size_t)

# name -> (restype, argtypes); pointers to device or host data are passed as integers/void*.
_SPMV_ARGS = [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i]
_SPMM_ARGS = [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i]
_CSRMV = [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]
_CSRMVEX = [_vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i]
_CSRMM2 = [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i]
_CSRMM = [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i]
PROTOTYPES = {
    "mcsparseCreate": (_i, [_pvp]),
    "mcsparseDestroy": (_i, [_vp]),
    "mcsparseGetVersion": (_i, [_vp, _pi]),
    "mcsparseGetProperty": (_i, [_i, _pi]),
    "mcsparseGetErrorName": (C.c_char_p, [_i]),
    "mcsparseGetErrorString": (C.c_char_p, [_i]),
    "mcsparseSetStream": (_i, [_vp, _vp]),
    "mcsparseGetStream": (_i, [_vp, _pvp]),
    "mcsparseSetPointerMode": (_i, [_vp, _i]),
    "mcsparseGetPointerMode": (_i, [_vp, _pi]),
    "mcsparseCreateMatDescr": (_i, [_pvp]),
    "mcsparseDestroyMatDescr": (_i, [_vp]),
    "mcsparseSetMatIndexBase": (_i, [_vp, _i]),
    "mcsparseGetMatIndexBase": (_i, [_vp]),
    "mcsparseSetMatType": (_i, [_vp, _i]),
    "mcsparseGetMatType": (_i, [_vp]),
    "mcsparseSetMatFillMode": (_i, [_vp, _i]),
    "mcsparseGetMatFillMode": (_i, [_vp]),
    "mcsparseSetMatDiagType": (_i, [_vp, _i]),
    "mcsparseGetMatDiagType": (_i, [_vp]),
    "mcsparseCreateDnVec": (_i, [_pvp, _i64, _vp, _i]),
    "mcsparseDestroyDnVec": (_i, [_vp]),
    "mcsparseDnVecGet": (_i, [_vp, _pi64, _pvp, _pi]),
    "mcsparseDnVecGetValues": (_i, [_vp, _pvp]),
    "mcsparseDnVecSetValues": (_i, [_vp, _vp]),
    "mcsparseCreateCsr": (_i, [_pvp, _i64, _i64, _i64, _vp, _vp, _vp, _i, _i, _i, _i]),
    "mcsparseCsrGet": (_i, [_vp, _pi64, _pi64, _pi64, _pvp, _pvp, _pvp, _pi, _pi, _pi, _pi]),
    "mcsparseCsrSetPointers": (_i, [_vp, _vp, _vp, _vp]),
    "mcsparseCreateCoo": (_i, [_pvp, _i64, _i64, _i64, _vp, _vp, _vp, _i, _i, _i]),
    "mcsparseCooGet": (_i, [_vp, _pi64, _pi64, _pi64, _pvp, _pvp, _pvp, _pi, _pi, _pi]),
    "mcsparseCooSetPointers": (_i, [_vp, _vp, _vp, _vp]),
    "mcsparseCreateCooAoS": (_i, [_pvp, _i64, _i64, _i64, _vp, _vp, _i, _i, _i]),
    "mcsparseCooAoSGet": (_i, [_vp, _pi64, _pi64, _pi64, _pvp, _pvp, _pi, _pi, _pi]),
    "mcsparseCreateCsc": (_i, [_pvp, _i64, _i64, _i64, _vp, _vp, _vp, _i, _i, _i, _i]),
    "mcsparseCscSetPointers": (_i, [_vp, _vp, _vp, _vp]),
    "mcsparseDestroySpMat": (_i, [_vp]),
    "mcsparseSpMatGetSize": (_i, [_vp, _pi64, _pi64, _pi64]),
    "mcsparseSpMatGetFormat": (_i, [_vp, _pi]),
    "mcsparseSpMatGetIndexBase": (_i, [_vp, _pi]),
    "mcsparseSpMatGetValues": (_i, [_vp, _pvp]),
    "mcsparseSpMatSetValues": (_i, [_vp, _vp]),
    "mcsparseSpMatGetAttribute": (_i, [_vp, _i, _vp, _sz]),
    "mcsparseSpMatSetAttribute": (_i, [_vp, _i, _vp, _sz]),
    "mcsparseCreateDnMat": (_i, [_pvp, _i64, _i64, _i64, _vp, _i, _i]),
    "mcsparseDestroyDnMat": (_i, [_vp]),
    "mcsparseDnMatGet": (_i, [_vp, _pi64, _pi64, _pi64, _pvp, _pi, _pi]),
    "mcsparseDnMatGetValues": (_i, [_vp, _pvp]),
    "mcsparseDnMatSetValues": (_i, [_vp, _vp]),
    "mcsparseCsrSetStridedBatch": (_i, [_vp, _i, _i64, _i64]),
    "mcsparseDnMatSetStridedBatch": (_i, [_vp, _i, _i64]),
    "mcsparseDnMatGetStridedBatch": (_i, [_vp, _pi, _pi64]),
    "mcsparseSpMV_bufferSize": (_i, _SPMV_ARGS + [_psz]),
    "mcsparseSpMV_preprocess": (_i, _SPMV_ARGS + [_vp]),
    "mcsparseSpMV": (_i, _SPMV_ARGS + [_vp]),
    "mcsparseSpMM_bufferSize": (_i, _SPMM_ARGS + [_psz]),
    "mcsparseSpMM_preprocess": (_i, _SPMM_ARGS + [_vp]),
    "mcsparseSpMM": (_i, _SPMM_ARGS + [_vp]),
    "mcsparseScsrmv": (_i, _CSRMV),
    "mcsparseCcsrmv": (_i, _CSRMV),
    "mcsparseZcsrmv": (_i, _CSRMV),
    "mcsparseDcsrmv": (_i, _CSRMV),
    "mcsparseCsrmvEx_bufferSize": (_i, _CSRMVEX + [_psz]),
    "mcsparseCsrmvEx": (_i, _CSRMVEX + [_vp]),
    "mcsparseScsrmm2": (_i, _CSRMM2),
    "mcsparseDcsrmm2": (_i, _CSRMM2),
    "mcsparseCcsrmm2": (_i, _CSRMM2),
    "mcsparseZcsrmm2": (_i, _CSRMM2),
    "mcsparseScsrmm": (_i, _CSRMM),
    "mcsparseDcsrmm": (_i, _CSRMM),
    "mcsparseCcsrmm": (_i, _CSRMM),
    "mcsparseZcsrmm": (_i, _CSRMM),
    "mcsparseB200SpMVNoAlloc": (_i, _SPMV_ARGS),
    "mcsparseB200SpMVPush": (_i, _SPMV_ARGS + [_vp, _i, _pvp, _i64]),
    "mcsparseB200SpMVPushMulticast": (_i, _SPMV_ARGS + [_vp, _vp, _i64]),
    "mcsparseB200PeerSignalWait": (_i, [_vp, _i, _pvp, _vp, _i]),
    "mcsparseB200PeerAlloc": (_i, [_pvp, _sz]),
    "mcsparseB200PeerFree": (_i, [_vp]),
    "mcsparseB200PeerExport": (_i, [_vp, _vp]),
    "mcsparseB200PeerOpen": (_i, [_vp, _pvp]),
    "mcsparseB200PeerClose": (_i, [_vp]),
    "mcsparseB200SpMVGetStatus": (_i, [_vp, _vp, _vp, _pi]),
    "mcsparseB200SetDeviceWaitLimit": (_i, [_vp, _i64, _i]),
    "mcsparseB200SpMatKeepConvertedValues": (_i, [_vp, _i]),
    "mcsparseB200GatherProbe": (_i, [_vp, _vp, _i64, _vp, _i, _vp, _i]),
    "mcsparseB200SpMVPartitionView": (_i, [_vp, _vp, _pi, _pi64, _pvp]),
    "mcsparseB200SpMVTransposedView": (_i, [_vp, _i, _vp, _pi64, _pvp, _pvp, _pvp]),
    "mcsparseB200ShardRowBounds": (_i, [_vp, _i64, _i64, _i, _vp, _i, _pi64]),
    "mcsparseB200ShardLocalRowOffsets": (_i, [_vp, _vp, _i64, _i64, _i, _vp]),
}


class McsparseError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        name = lib.mcsparseGetErrorName(status).decode() if lib is not None else str(status)
        super().__init__(f"{where}: {name} ({status})" if where else f"{name} ({status})")


def load_library(path=LIB_PATH):
    """Loads libmcsparse.so and types every entry point. Raises if it is not built:
    there is deliberately no fallback implementation behind this module."""
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `make -C mcsparse_b200/csrc` (needs nvcc)")
    dll = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(dll, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return dll


lib = None
lib = load_library()


def check(status, where=""):
    if status != MCSPARSE_STATUS_SUCCESS:
        raise McsparseError(status, where)
    return status
