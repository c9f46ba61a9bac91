"""Host-side objects over the C API: handle and descriptors that keep their torch tensors alive.

Every method is a thin call into ``capi.lib`` (the C ABI). torch is used for device memory
and streams only; all arithmetic happens in libmcsparse.so.
"""

import ctypes as C

import torch

from . import capi
from .capi import check, lib

_DTYPE = {torch.float32: capi.MACA_R_32F, torch.float64: capi.MACA_R_64F,
          torch.complex64: capi.MACA_C_32F, torch.complex128: capi.MACA_C_64F,
          # operands of the low-precision SpMV (sums in fp32 / int32)
          torch.float16: capi.MACA_R_16F, torch.bfloat16: capi.MACA_R_16BF, torch.int8: capi.MACA_R_8I,
          torch.int32: capi.MACA_R_32I}


def _ptr(t):
    """Device address of a tensor. torch reports a null data_ptr() for zero-element tensors; the
    C API (like the reference) rejects null arrays even when they are empty, so an empty view
    is given the address of its storage instead."""
    p = t.data_ptr()
    if p == 0 and t.untyped_storage().nbytes() > 0:
        p = t.untyped_storage().data_ptr() + t.storage_offset() * t.element_size()
    return C.c_void_p(p)


def _scalar(value, dtype):
    """A host scalar of the compute type, as the C API expects behind ``const void*``
    (complex types: the real and the imaginary part, interleaved)."""
    if dtype in (torch.complex64, torch.complex128):
        z = complex(value)
        return ((C.c_float if dtype == torch.complex64 else C.c_double) * 2)(z.real, z.imag)
    if dtype == torch.int32:
        return C.c_int32(int(value))
    return (C.c_double if dtype == torch.float64 else C.c_float)(value)


class Handle:
    """mcsparseHandle_t bound to the current CUDA device and (optionally) a torch stream."""

    def __init__(self, stream=None):
        h = C.c_void_p()
        check(lib.mcsparseCreate(C.byref(h)), "mcsparseCreate")
        self.h = h
        self.pointer_mode = capi.MCSPARSE_POINTER_MODE_HOST
        if stream is None:
            stream = torch.cuda.current_stream()
        self.set_stream(stream)

    def set_stream(self, stream):
        self.stream = stream
        check(lib.mcsparseSetStream(self.h, C.c_void_p(stream.cuda_stream)), "mcsparseSetStream")

    def set_pointer_mode(self, mode):
        check(lib.mcsparseSetPointerMode(self.h, mode), "mcsparseSetPointerMode")
        self.pointer_mode = mode

    def close(self):
        if self.h is not None and lib is not None:
            lib.mcsparseDestroy(self.h)
            self.h = None

    def __del__(self):
        self.close()


class CsrMatrix:
    """mcsparseSpMatDescr_t over three device tensors (borrowed by the C side, owned here)."""

    def __init__(self, rows, cols, row_offsets, col_ind, values, base=0):
        # Index types come in matched pairs: both 32-bit or both 64-bit.
        assert row_offsets.dtype == col_ind.dtype and row_offsets.dtype in (torch.int32, torch.int64)
        index_type = capi.MCSPARSE_INDEX_64I if row_offsets.dtype == torch.int64 else capi.MCSPARSE_INDEX_32I
        self.rows, self.cols, self.base = int(rows), int(cols), int(base)
        self.nnz = int(col_ind.numel())
        self.row_offsets, self.col_ind, self.values = row_offsets, col_ind, values
        d = C.c_void_p()
        check(lib.mcsparseCreateCsr(C.byref(d), self.rows, self.cols, self.nnz, _ptr(row_offsets), _ptr(col_ind),
                                    _ptr(values), index_type, index_type, self.base,
                                    _DTYPE[values.dtype]), "mcsparseCreateCsr")
        self.d = d

    @property
    def dtype(self):
        return self.values.dtype

    def __del__(self):
        if getattr(self, "d", None) is not None and lib is not None:  # lib is None at interpreter shutdown
            lib.mcsparseDestroySpMat(self.d)
            self.d = None


class CscMatrix:
    """mcsparseSpMatDescr_t in CSC form over three device tensors (column offsets, row indices, values)."""

    def __init__(self, rows, cols, col_offsets, row_ind, values, base=0):
        assert col_offsets.dtype == torch.int32 and row_ind.dtype == torch.int32
        self.rows, self.cols, self.base = int(rows), int(cols), int(base)
        self.nnz = int(row_ind.numel())
        self.col_offsets, self.row_ind, self.values = col_offsets, row_ind, values
        d = C.c_void_p()
        check(lib.mcsparseCreateCsc(C.byref(d), self.rows, self.cols, self.nnz, _ptr(col_offsets), _ptr(row_ind),
                                    _ptr(values), capi.MCSPARSE_INDEX_32I, capi.MCSPARSE_INDEX_32I, self.base,
                                    _DTYPE[values.dtype]), "mcsparseCreateCsc")
        self.d = d

    @property
    def dtype(self):
        return self.values.dtype

    def __del__(self):
        if getattr(self, "d", None) is not None and lib is not None:
            lib.mcsparseDestroySpMat(self.d)
            self.d = None


class DnVec:
    def __init__(self, values):
        self.values = values
        d = C.c_void_p()
        check(lib.mcsparseCreateDnVec(C.byref(d), values.numel(), _ptr(values), _DTYPE[values.dtype]),
              "mcsparseCreateDnVec")
        self.d = d

    def __del__(self):
        if getattr(self, "d", None) is not None and lib is not None:  # lib is None at interpreter shutdown
            lib.mcsparseDestroyDnVec(self.d)
            self.d = None


class DnMat:
    """Dense matrix descriptor. ``values`` is the backing tensor; rows/cols/ld/order describe it."""

    def __init__(self, values, rows, cols, ld, order=capi.MCSPARSE_ORDER_ROW):
        self.values, self.rows, self.cols, self.ld, self.order = values, int(rows), int(cols), int(ld), order
        d = C.c_void_p()
        check(lib.mcsparseCreateDnMat(C.byref(d), self.rows, self.cols, self.ld, _ptr(values), _DTYPE[values.dtype],
                                      order), "mcsparseCreateDnMat")
        self.d = d

    def __del__(self):
        if getattr(self, "d", None) is not None and lib is not None:  # lib is None at interpreter shutdown
            lib.mcsparseDestroyDnMat(self.d)
            self.d = None


def _scalars(handle, alpha, beta, dtype):
    """alpha/beta as C arguments: host scalars, or device tensors in device pointer mode."""
    if handle.pointer_mode == capi.MCSPARSE_POINTER_MODE_DEVICE:
        return _ptr(alpha), _ptr(beta), (alpha, beta)
    a, b = _scalar(alpha, dtype), _scalar(beta, dtype)
    return C.cast(C.byref(a), C.c_void_p), C.cast(C.byref(b), C.c_void_p), (a, b)


def spmv_buffer_size(handle, A, x, y, alpha=1.0, beta=0.0, op=capi.MCSPARSE_OPERATION_NON_TRANSPOSE, compute=None):
    compute = compute or A.dtype
    pa, pb, keep = _scalars(handle, alpha, beta, compute)
    size = C.c_size_t()
    check(lib.mcsparseSpMV_bufferSize(handle.h, op, pa, A.d, x.d, pb, y.d,
                                      _DTYPE[compute], capi.MCSPARSE_SPMV_ALG_DEFAULT, C.byref(size)),
          "mcsparseSpMV_bufferSize")
    del keep
    return size.value


def spmv_preprocess(handle, A, x, y, buffer, alpha=1.0, beta=0.0, op=capi.MCSPARSE_OPERATION_NON_TRANSPOSE, compute=None):
    compute = compute or A.dtype
    pa, pb, keep = _scalars(handle, alpha, beta, compute)
    check(lib.mcsparseSpMV_preprocess(handle.h, op, pa, A.d, x.d, pb, y.d,
                                      _DTYPE[compute], capi.MCSPARSE_SPMV_ALG_DEFAULT, _ptr(buffer)),
          "mcsparseSpMV_preprocess")
    del keep


def spmv(handle, A, x, y, buffer, alpha=1.0, beta=0.0, op=capi.MCSPARSE_OPERATION_NON_TRANSPOSE, compute=None):
    """y = alpha * op(A) @ x + beta * y through mcsparseSpMV (asynchronous on the handle's stream).
    ``compute`` is the compute type where it differs from A's (fp16 / bf16 / int8 operands: torch.float32,
    or torch.int32 for int8 -> int32)."""
    compute = compute or A.dtype
    pa, pb, keep = _scalars(handle, alpha, beta, compute)
    check(lib.mcsparseSpMV(handle.h, op, pa, A.d, x.d, pb, y.d, _DTYPE[compute],
                           capi.MCSPARSE_SPMV_ALG_DEFAULT, _ptr(buffer)), "mcsparseSpMV")
    del keep


def spmm_buffer_size(handle, A, B, Cmat, alpha=1.0, beta=0.0, op_b=capi.MCSPARSE_OPERATION_NON_TRANSPOSE):
    pa, pb, keep = _scalars(handle, alpha, beta, A.dtype)
    size = C.c_size_t()
    check(lib.mcsparseSpMM_bufferSize(handle.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, op_b, pa, A.d, B.d, pb, Cmat.d,
                                      _DTYPE[A.dtype], capi.MCSPARSE_SPMM_ALG_DEFAULT, C.byref(size)),
          "mcsparseSpMM_bufferSize")
    del keep
    return size.value


def spmm_preprocess(handle, A, B, Cmat, buffer, alpha=1.0, beta=0.0, op_b=capi.MCSPARSE_OPERATION_NON_TRANSPOSE):
    pa, pb, keep = _scalars(handle, alpha, beta, A.dtype)
    check(lib.mcsparseSpMM_preprocess(handle.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, op_b, pa, A.d, B.d, pb, Cmat.d,
                                      _DTYPE[A.dtype], capi.MCSPARSE_SPMM_ALG_DEFAULT, _ptr(buffer)),
          "mcsparseSpMM_preprocess")
    del keep


def spmm(handle, A, B, Cmat, buffer, alpha=1.0, beta=0.0, op_b=capi.MCSPARSE_OPERATION_NON_TRANSPOSE):
    """C = alpha * A @ op(B) + beta * C through mcsparseSpMM."""
    pa, pb, keep = _scalars(handle, alpha, beta, A.dtype)
    check(lib.mcsparseSpMM(handle.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, op_b, pa, A.d, B.d, pb, Cmat.d,
                           _DTYPE[A.dtype], capi.MCSPARSE_SPMM_ALG_DEFAULT, _ptr(buffer)), "mcsparseSpMM")
    del keep


class HostSpmvPipeline:
    """y_host = alpha * A @ x_host + beta * y_host for vectors that live in pinned host memory.

    The matrix stays resident on the GPU. Each `submit` runs on one of `depth` slots (own stream,
    own device x / y, own work buffer and matrix descriptor over the same three arrays), so the
    host-to-device copy of one product overlaps the device-to-host copy of the previous one: the
    two directions use different copy engines. Products submitted back to back must therefore be
    independent of one another; `wait()` returns when all submitted results are in host memory.

    With `shard=(row_offset, total_rows, group)` the matrix is this rank's row block of a
    row-sharded matrix (see sharding.ShardedSpmv): every slot then owns a peer-visible y, the
    kernel pushes finished rows to the other GPUs, and `y_host` receives this rank's rows. Each
    rank uploads only its 1/world slice of `x_host` (every rank is given the same full-length
    vector); the slices are exchanged between the GPUs by an all-gather, so the bytes crossing
    PCIe per product do not grow with the number of GPUs.
    """

    def __init__(self, handle, rows, cols, row_offsets, col_ind, values, base=0, depth=2, shard=None):
        self.h, self.depth, self.dtype = handle, int(depth), values.dtype
        self.main = handle.stream
        device = values.device
        self.slots = []
        self.submitted = 0
        for _ in range(self.depth):
            s = {"stream": torch.cuda.Stream(device=device), "done": torch.cuda.Event(),
                 "A": CsrMatrix(rows, cols, row_offsets, col_ind, values, base=base),
                 "x": torch.zeros(cols, dtype=values.dtype, device=device)}
            if shard is None:
                s["y"] = torch.zeros(rows, dtype=values.dtype, device=device)
                s["X"], s["Y"] = DnVec(s["x"]), DnVec(s["y"])
                s["buf"] = torch.empty(spmv_buffer_size(handle, s["A"], s["X"], s["Y"]), dtype=torch.uint8,
                                       device=device)
                spmv_preprocess(handle, s["A"], s["X"], s["Y"], s["buf"])
                s["sharded"] = None
            else:
                from . import sharding

                import torch.distributed as dist

                row_offset, total_rows, group = shard
                s["sharded"] = sharding.ShardedSpmv(handle, s["A"], s["x"], row_offset, total_rows, group)
                s["y"] = s["sharded"].y_local
                world, rank = dist.get_world_size(group), dist.get_rank(group)
                cut = [cols * g // world for g in range(world + 1)]
                s["x_parts"] = [s["x"][cut[g]:cut[g + 1]] for g in range(world)]
                s["x_slice"] = slice(cut[rank], cut[rank + 1])
                s["group"] = group
            self.slots.append(s)
        torch.cuda.synchronize(device)

    def submit(self, x_host, y_host, alpha=1.0, beta=0.0):
        """Queues one product; returns at once. x_host / y_host must stay untouched until wait()."""
        s = self.slots[self.submitted % self.depth]
        self.submitted += 1
        with torch.cuda.stream(s["stream"]):
            if s["sharded"] is None:
                s["x"].copy_(x_host, non_blocking=True)
            else:
                from . import sharding

                mine = s["x_slice"]
                s["x"][mine].copy_(x_host[mine], non_blocking=True)
                sharding.all_gather_ragged(s["x_parts"], s["x"][mine], s["group"])
            if beta != 0:
                s["y"].copy_(y_host, non_blocking=True)
            self.h.set_stream(s["stream"])
            try:
                if s["sharded"] is None:
                    spmv(self.h, s["A"], s["X"], s["Y"], s["buf"], alpha=alpha, beta=beta)
                else:
                    s["sharded"].step(alpha, beta)
            finally:
                self.h.set_stream(self.main)
            y_host.copy_(s["y"], non_blocking=True)
            s["done"].record(s["stream"])

    def start_after(self, stream):
        """Makes every slot's stream wait for the work queued so far on `stream`."""
        ev = torch.cuda.Event()
        ev.record(stream)
        for s in self.slots:
            s["stream"].wait_event(ev)

    def join(self, stream):
        """Makes `stream` wait for every product submitted so far (no host synchronisation)."""
        for s in self.slots:
            stream.wait_event(s["done"])

    def wait(self):
        for s in self.slots:
            s["done"].synchronize()

    def close(self):
        self.wait()
        for s in self.slots:
            if s["sharded"] is not None:
                s["sharded"].close()
        self.slots = []
