// Host side of libmcsparse.so, bookkeeping entry points: handle, matrix / vector descriptors and their
// getters and setters. Nothing here launches a kernel; the status codes are explained in api_common.h.
#include <cstring>
#include <new>

#include "api_common.h"

using namespace mcsp_b200;
using namespace mcsp_b200::api;

extern "C" {

// ----------------------------------------------------------------------------- handle

mcsparseStatus_t mcsparseCreate(mcsparseHandle_t* handle) {
    if (handle == nullptr) return pub(BAD_POINTER);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MCSPARSE_STATUS_NOT_INITIALIZED;
    mcsparseContext* ctx = new (std::nothrow) mcsparseContext();
    if (ctx == nullptr) return MCSPARSE_STATUS_ALLOC_FAILED;
    ctx->device = dev;
    cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, dev);
    // One word of pinned host memory that kernels can write: a tile kernel that gives up its bounded
    // wait says so here, and the next compute call reports it without a synchronisation. Without it
    // (allocation refused) such a failure is still recorded in the work buffer's status word.
    void* word = nullptr;
    if (cudaHostAlloc(&word, sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
        ctx->fault_word_host = static_cast<int*>(word);
        *ctx->fault_word_host = 0;
        void* dev_view = nullptr;
        if (cudaHostGetDevicePointer(&dev_view, word, 0) == cudaSuccess) ctx->fault_word_dev = static_cast<int*>(dev_view);
    } else {
        cudaGetLastError();
    }
    *handle = ctx;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDestroy(mcsparseHandle_t handle) {
    if (handle != nullptr && handle->side_stream != nullptr) {
        DeviceGuard guard(handle->device);
        cudaStreamDestroy(handle->side_stream);
        for (auto& ev : handle->events)
            if (ev != nullptr) cudaEventDestroy(ev);
        for (auto& ev : handle->fix_events)
            if (ev != nullptr) cudaEventDestroy(ev);
        for (auto& ev : handle->peer_events)
            if (ev != nullptr) cudaEventDestroy(ev);
        for (auto& st : handle->peer_streams)
            if (st != nullptr) cudaStreamDestroy(st);
        if (handle->capture_stream != nullptr) cudaStreamDestroy(handle->capture_stream);
    }
    if (handle != nullptr && handle->fault_word_host != nullptr) {
        DeviceGuard guard(handle->device);
        cudaFreeHost(handle->fault_word_host);
    }
    delete handle;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseGetVersion(mcsparseHandle_t handle, int* version) {
    if (version == nullptr) return pub(BAD_POINTER);
    if (handle == nullptr) return pub(BAD_HANDLE);
    *version = 1 * 1000000 + 0 * 1000 + 0;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseGetProperty(libraryPropertyType type, int* value) {
    if (value == nullptr) return pub(BAD_POINTER);
    switch (type) {
        case MAJOR_VERSION: *value = 1; break;
        case MINOR_VERSION: *value = 0; break;
        case PATCH_LEVEL: *value = 0; break;
        default: return pub(BAD_VALUE);
    }
    return MCSPARSE_STATUS_SUCCESS;
}

const char* mcsparseGetErrorName(mcsparseStatus_t status) {
    switch (status) {
        case MCSPARSE_STATUS_SUCCESS: return "MCSPARSE_STATUS_SUCCESS";
        case MCSPARSE_STATUS_NOT_INITIALIZED: return "MCSPARSE_STATUS_NOT_INITIALIZED";
        case MCSPARSE_STATUS_ALLOC_FAILED: return "MCSPARSE_STATUS_ALLOC_FAILED";
        case MCSPARSE_STATUS_INVALID_VALUE: return "MCSPARSE_STATUS_INVALID_VALUE";
        case MCSPARSE_STATUS_ARCH_MISMATCH: return "MCSPARSE_STATUS_ARCH_MISMATCH";
        case MCSPARSE_STATUS_MAPPING_ERROR: return "MCSPARSE_STATUS_MAPPING_ERROR";
        case MCSPARSE_STATUS_EXECUTION_FAILED: return "MCSPARSE_STATUS_EXECUTION_FAILED";
        case MCSPARSE_STATUS_INTERNAL_ERROR: return "MCSPARSE_STATUS_INTERNAL_ERROR";
        case MCSPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED: return "MCSPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED";
        case MCSPARSE_STATUS_ZERO_PIVOT: return "MCSPARSE_STATUS_ZERO_PIVOT";
        case MCSPARSE_STATUS_NOT_SUPPORTED: return "MCSPARSE_STATUS_NOT_SUPPORTED";
        case MCSPARSE_STATUS_INSUFFICIENT_RESOURCES: return "MCSPARSE_STATUS_INSUFFICIENT_RESOURCES";
        default: return "unrecognized error code";
    }
}

const char* mcsparseGetErrorString(mcsparseStatus_t status) {
    switch (status) {
        case MCSPARSE_STATUS_SUCCESS: return "success";
        case MCSPARSE_STATUS_NOT_INITIALIZED: return "initialization error";
        case MCSPARSE_STATUS_ALLOC_FAILED: return "out of memory";
        case MCSPARSE_STATUS_INVALID_VALUE: return "invalid value";
        case MCSPARSE_STATUS_ARCH_MISMATCH: return "architecture mismatch";
        case MCSPARSE_STATUS_MAPPING_ERROR: return "texture memory mapping error";
        case MCSPARSE_STATUS_EXECUTION_FAILED: return "kernel launch failure";
        case MCSPARSE_STATUS_INTERNAL_ERROR: return "internal error";
        case MCSPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED: return "matrix type not supported";
        case MCSPARSE_STATUS_ZERO_PIVOT: return "zero pivot";
        case MCSPARSE_STATUS_NOT_SUPPORTED: return "operation not supported";
        case MCSPARSE_STATUS_INSUFFICIENT_RESOURCES: return "insufficient resources";
        default: return "unrecognized error code";
    }
}

mcsparseStatus_t mcsparseSetStream(mcsparseHandle_t handle, mcStream_t sid) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    handle->stream = sid;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseGetStream(const mcsparseHandle_t handle, mcStream_t* sid) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (sid == nullptr) return pub(BAD_POINTER);
    *sid = handle->stream;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSetPointerMode(mcsparseHandle_t handle, mcsparsePointerMode_t pointer_mode) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    handle->ptr_mode = pointer_mode;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseGetPointerMode(const mcsparseHandle_t handle, mcsparsePointerMode_t* pointer_mode) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (pointer_mode == nullptr) return pub(BAD_POINTER);
    *pointer_mode = handle->ptr_mode;
    return MCSPARSE_STATUS_SUCCESS;
}

// ----------------------------------------------------------------------------- legacy matrix descriptor

mcsparseStatus_t mcsparseCreateMatDescr(mcsparseMatDescr_t* descr) {
    if (descr == nullptr) return pub(BAD_POINTER);
    *descr = new (std::nothrow) mcsparseMatDescr();
    return *descr ? MCSPARSE_STATUS_SUCCESS : MCSPARSE_STATUS_INTERNAL_ERROR;
}

mcsparseStatus_t mcsparseDestroyMatDescr(mcsparseMatDescr_t descr) {
    delete descr;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSetMatIndexBase(mcsparseMatDescr_t descr, mcsparseIndexBase_t index_base) {
    if (descr == nullptr) return pub(BAD_POINTER);
    if (index_base != MCSPARSE_INDEX_BASE_ZERO && index_base != MCSPARSE_INDEX_BASE_ONE) return pub(BAD_VALUE);
    descr->base = index_base;
    return MCSPARSE_STATUS_SUCCESS;
}
mcsparseIndexBase_t mcsparseGetMatIndexBase(const mcsparseMatDescr_t descr) {
    return descr ? descr->base : (mcsparseIndexBase_t)-1;
}

mcsparseStatus_t mcsparseSetMatType(mcsparseMatDescr_t descr, mcsparseMatrixType_t matrix_type) {
    if (descr == nullptr) return pub(BAD_POINTER);
    if ((int)matrix_type < 0 || (int)matrix_type > 3) return pub(BAD_VALUE);
    descr->type = matrix_type;
    return MCSPARSE_STATUS_SUCCESS;
}
mcsparseMatrixType_t mcsparseGetMatType(const mcsparseMatDescr_t descr) {
    return descr ? descr->type : (mcsparseMatrixType_t)-1;
}

mcsparseStatus_t mcsparseSetMatFillMode(mcsparseMatDescr_t descr, mcsparseFillMode_t mode) {
    if (descr == nullptr) return pub(BAD_POINTER);
    if ((int)mode < 0 || (int)mode > 2) return pub(BAD_VALUE);
    descr->fill_mode = mode;
    return MCSPARSE_STATUS_SUCCESS;
}
mcsparseFillMode_t mcsparseGetMatFillMode(const mcsparseMatDescr_t descr) {
    return descr ? descr->fill_mode : (mcsparseFillMode_t)-1;
}

mcsparseStatus_t mcsparseSetMatDiagType(mcsparseMatDescr_t descr, mcsparseDiagType_t diag_type) {
    if (descr == nullptr) return pub(BAD_POINTER);
    if ((int)diag_type < 0 || (int)diag_type > 1) return pub(BAD_VALUE);
    descr->diag_type = diag_type;
    return MCSPARSE_STATUS_SUCCESS;
}
mcsparseDiagType_t mcsparseGetMatDiagType(const mcsparseMatDescr_t descr) {
    return descr ? descr->diag_type : (mcsparseDiagType_t)-1;
}

// ----------------------------------------------------------------------------- dense vector

mcsparseStatus_t mcsparseCreateDnVec(mcsparseDnVecDescr_t* dnVecDescr, int64_t size, void* values,
                                     macaDataType valueType) {
    if (size < 0) {
        log_error("Wrong input size");
        return pub(BAD_SIZE);
    }
    if (dnVecDescr == nullptr || values == nullptr) return pub(BAD_POINTER);
    if (!(value_type_known(valueType) || valueType == MACA_R_32I)) return pub(NOT_IMPL);
    mcsparseDnVecDescr* d = new (std::nothrow) mcsparseDnVecDescr();
    if (d == nullptr) return MCSPARSE_STATUS_INTERNAL_ERROR;
    d->size = size;
    d->values = values;
    d->valueType = valueType;
    *dnVecDescr = d;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDestroyDnVec(mcsparseDnVecDescr_t dnVecDescr) {
    delete dnVecDescr;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnVecGet(mcsparseDnVecDescr_t d, int64_t* size, void** values, macaDataType* valueType) {
    if (d == nullptr || size == nullptr || values == nullptr || valueType == nullptr) return pub(BAD_POINTER);
    *size = d->size;
    *values = d->values;
    *valueType = d->valueType;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnVecGetValues(mcsparseDnVecDescr_t d, void** values) {
    if (d == nullptr || values == nullptr) return pub(BAD_POINTER);
    *values = d->values;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnVecSetValues(mcsparseDnVecDescr_t d, void* values) {
    if (d == nullptr) return pub(BAD_POINTER);
    d->values = values;
    return MCSPARSE_STATUS_SUCCESS;
}

// ----------------------------------------------------------------------------- CSR matrix

mcsparseStatus_t mcsparseCreateCsr(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* csrRowOffsets, void* csrColInd, void* csrValues,
                                   mcsparseIndexType_t csrRowOffsetsType, mcsparseIndexType_t csrColIndType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType) {
    if (rows < 0 || cols < 0 || nnz < 0) {
        log_error("Wrong input size");
        return pub(BAD_SIZE);
    }
    if (!value_type_known(valueType)) return pub(NOT_IMPL);
    if (spMatDescr == nullptr) return pub(BAD_POINTER);
    if (idxBase != MCSPARSE_INDEX_BASE_ZERO && idxBase != MCSPARSE_INDEX_BASE_ONE) return pub(BAD_VALUE);
    mcsparseSpMatDescr* d = new (std::nothrow) mcsparseSpMatDescr();
    mcsparseMatDescr* md = new (std::nothrow) mcsparseMatDescr();
    if (d == nullptr || md == nullptr) {
        delete d;
        delete md;
        return MCSPARSE_STATUS_INTERNAL_ERROR;
    }
    d->format = MCSPARSE_FORMAT_CSR;
    d->row_num = rows;
    d->col_num = cols;
    d->nnz = nnz;
    d->rows = csrRowOffsets;
    d->cols = csrColInd;
    d->vals = csrValues;
    d->rowIdxType = csrRowOffsetsType;
    d->colIdxType = csrColIndType;
    d->idxBase = idxBase;
    d->valueType = valueType;
    md->base = idxBase;
    d->mat_descr = md;
    *spMatDescr = d;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseCsrGet(mcsparseSpMatDescr_t d, int64_t* rows, int64_t* cols, int64_t* nnz,
                                void** csrRowOffsets, void** csrColInd, void** csrValues,
                                mcsparseIndexType_t* csrRowOffsetsType, mcsparseIndexType_t* csrColIndType,
                                mcsparseIndexBase_t* idxBase, macaDataType* valueType) {
    if (d == nullptr || rows == nullptr || cols == nullptr || nnz == nullptr || csrRowOffsets == nullptr ||
        csrColInd == nullptr || csrValues == nullptr || csrRowOffsetsType == nullptr || csrColIndType == nullptr ||
        idxBase == nullptr || valueType == nullptr)
        return pub(BAD_POINTER);
    *rows = d->row_num;
    *cols = d->col_num;
    *nnz = d->nnz;
    *csrRowOffsets = d->rows;
    *csrColInd = d->cols;
    *csrValues = d->vals;
    *csrRowOffsetsType = d->rowIdxType;
    *csrColIndType = d->colIdxType;
    *idxBase = d->idxBase;
    *valueType = d->valueType;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseCsrSetPointers(mcsparseSpMatDescr_t d, void* csrRowOffsets, void* csrColInd,
                                        void* csrValues) {
    if (d == nullptr) return pub(BAD_POINTER);
    std::lock_guard<std::mutex> g(d->lock);
    d->push_buffer = nullptr;
    d->spmm_buffer = nullptr;
    d->probed_cols = nullptr;
    d->rows = csrRowOffsets;
    d->cols = csrColInd;
    d->vals = csrValues;
    d->analysed_buffer = nullptr;
    d->analysed_rows = nullptr;
    d->trans_buffer = nullptr;
    d->trans_values_src = nullptr;
    d->spmm_values_src = nullptr;
    d->trans_probed_idx = nullptr;
    d->coo_checked_rows = nullptr;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseCreateCoo(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* cooRowInd, void* cooColInd, void* cooValues, mcsparseIndexType_t cooIdxType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType) {
    mcsparseStatus_t st = mcsparseCreateCsr(spMatDescr, rows, cols, nnz, cooRowInd, cooColInd, cooValues, cooIdxType,
                                            cooIdxType, idxBase, valueType);
    if (st == MCSPARSE_STATUS_SUCCESS) (*spMatDescr)->format = MCSPARSE_FORMAT_COO;
    return st;
}

mcsparseStatus_t mcsparseCooGet(mcsparseSpMatDescr_t d, int64_t* rows, int64_t* cols, int64_t* nnz, void** cooRowInd,
                                void** cooColInd, void** cooValues, mcsparseIndexType_t* idxType,
                                mcsparseIndexBase_t* idxBase, macaDataType* valueType) {
    if (d == nullptr || rows == nullptr || cols == nullptr || nnz == nullptr || cooRowInd == nullptr ||
        cooColInd == nullptr || cooValues == nullptr || idxType == nullptr || idxBase == nullptr ||
        valueType == nullptr)
        return pub(BAD_POINTER);
    *rows = d->row_num;
    *cols = d->col_num;
    *nnz = d->nnz;
    *cooRowInd = d->rows;
    *cooColInd = d->cols;
    *cooValues = d->vals;
    *idxType = d->rowIdxType;
    *idxBase = d->idxBase;
    *valueType = d->valueType;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseCooSetPointers(mcsparseSpMatDescr_t d, void* cooRows, void* cooColumns, void* cooValues) {
    return mcsparseCsrSetPointers(d, cooRows, cooColumns, cooValues);
}

// COO as an array of (row, column) pairs (mcsparse/src/common/mcsp_helper.cpp:486-500, :568-585): the pair
// array is kept in `rows`, `cols` stays null.
mcsparseStatus_t mcsparseCreateCooAoS(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                      void* cooInd, void* cooValues, mcsparseIndexType_t cooIdxType,
                                      mcsparseIndexBase_t idxBase, macaDataType valueType) {
    if (cooInd == nullptr) return pub(BAD_POINTER);
    mcsparseStatus_t st = mcsparseCreateCsr(spMatDescr, rows, cols, nnz, cooInd, nullptr, cooValues, cooIdxType, cooIdxType,
                                            idxBase, valueType);
    if (st == MCSPARSE_STATUS_SUCCESS) (*spMatDescr)->format = MCSPARSE_FORMAT_COO_AOS;
    return st;
}

mcsparseStatus_t mcsparseCooAoSGet(mcsparseSpMatDescr_t d, int64_t* rows, int64_t* cols, int64_t* nnz, void** cooInd,
                                   void** cooValues, mcsparseIndexType_t* idxType, mcsparseIndexBase_t* idxBase,
                                   macaDataType* valueType) {
    if (d == nullptr || rows == nullptr || cols == nullptr || nnz == nullptr || cooInd == nullptr ||
        cooValues == nullptr || idxType == nullptr || idxBase == nullptr || valueType == nullptr)
        return pub(BAD_POINTER);
    *rows = d->row_num;
    *cols = d->col_num;
    *nnz = d->nnz;
    *cooInd = d->rows;
    *cooValues = d->vals;
    *idxType = d->rowIdxType;
    *idxBase = d->idxBase;
    *valueType = d->valueType;
    return MCSPARSE_STATUS_SUCCESS;
}

// CSC: the descriptor keeps the row indices in `rows` and the column offsets in `cols`, as the
// reference does (mcsparse/src/common/mcsp_helper.cpp:447-452, :607-615).
mcsparseStatus_t mcsparseCreateCsc(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* cscColOffsets, void* cscRowInd, void* cscValues,
                                   mcsparseIndexType_t cscColOffsetsType, mcsparseIndexType_t cscRowIndType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType) {
    mcsparseStatus_t st = mcsparseCreateCsr(spMatDescr, rows, cols, nnz, cscRowInd, cscColOffsets, cscValues,
                                            cscRowIndType, cscColOffsetsType, idxBase, valueType);
    if (st == MCSPARSE_STATUS_SUCCESS) (*spMatDescr)->format = MCSPARSE_FORMAT_CSC;
    return st;
}

mcsparseStatus_t mcsparseCscSetPointers(mcsparseSpMatDescr_t d, void* cscColOffsets, void* cscRowInd, void* cscValues) {
    return mcsparseCsrSetPointers(d, cscRowInd, cscColOffsets, cscValues);
}

mcsparseStatus_t mcsparseDestroySpMat(mcsparseSpMatDescr_t d) {
    if (d == nullptr) return MCSPARSE_STATUS_SUCCESS;
    for (auto& g : d->push_graphs)
        if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
    delete d->mat_descr;
    delete d;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatGetSize(mcsparseSpMatDescr_t d, int64_t* rows, int64_t* cols, int64_t* nnz) {
    if (d == nullptr || rows == nullptr || cols == nullptr || nnz == nullptr) return pub(BAD_POINTER);
    *rows = d->row_num;
    *cols = d->col_num;
    *nnz = d->nnz;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatGetFormat(mcsparseSpMatDescr_t d, mcsparseFormat_t* format) {
    if (d == nullptr || format == nullptr) return pub(BAD_POINTER);
    *format = d->format;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatGetIndexBase(mcsparseSpMatDescr_t d, mcsparseIndexBase_t* idxBase) {
    if (d == nullptr || idxBase == nullptr) return pub(BAD_POINTER);
    *idxBase = d->idxBase;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatGetValues(mcsparseSpMatDescr_t d, void** values) {
    if (d == nullptr || values == nullptr) return pub(BAD_POINTER);
    *values = d->vals;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatSetValues(mcsparseSpMatDescr_t d, void* values) {
    if (d == nullptr) return pub(BAD_POINTER);
    d->vals = values;
    d->trans_values_src = nullptr;  // the values changed (or may have): converted copies are stale
    d->spmm_values_src = nullptr;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseB200SpMatKeepConvertedValues(mcsparseSpMatDescr_t d, int keep) {
    if (d == nullptr) return pub(BAD_POINTER);
    d->keep_converted_values = keep != 0;
    d->trans_values_src = nullptr;
    d->spmm_values_src = nullptr;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatGetAttribute(mcsparseSpMatDescr_t d, mcsparseSpMatAttribute_t attribute, void* data,
                                           size_t dataSize) {
    (void)dataSize;
    if (data == nullptr || d == nullptr || d->mat_descr == nullptr) return pub(BAD_POINTER);
    if (attribute == MCSPARSE_SPMAT_FILL_MODE)
        std::memcpy(data, &d->mat_descr->fill_mode, sizeof(d->mat_descr->fill_mode));
    else if (attribute == MCSPARSE_SPMAT_DIAG_TYPE)
        std::memcpy(data, &d->mat_descr->diag_type, sizeof(d->mat_descr->diag_type));
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMatSetAttribute(mcsparseSpMatDescr_t d, mcsparseSpMatAttribute_t attribute,
                                           const void* data, size_t dataSize) {
    (void)dataSize;
    if (data == nullptr || d == nullptr || d->mat_descr == nullptr) return pub(BAD_POINTER);
    if (attribute == MCSPARSE_SPMAT_FILL_MODE)
        std::memcpy(&d->mat_descr->fill_mode, data, sizeof(d->mat_descr->fill_mode));
    else if (attribute == MCSPARSE_SPMAT_DIAG_TYPE)
        std::memcpy(&d->mat_descr->diag_type, data, sizeof(d->mat_descr->diag_type));
    return MCSPARSE_STATUS_SUCCESS;
}

// ----------------------------------------------------------------------------- dense matrix

mcsparseStatus_t mcsparseCreateDnMat(mcsparseDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                     void* values, macaDataType valueType, mcsparseOrder_t order) {
    if (rows < 0 || cols < 0 || ld < 0) {
        log_error("Wrong input size");
        return pub(BAD_SIZE);
    }
    if (!(value_type_known(valueType) || valueType == MACA_R_32I)) {
        log_error("Dense matrix data type not supported");
        return pub(NOT_IMPL);
    }
    if (dnMatDescr == nullptr || values == nullptr) return pub(BAD_POINTER);
    if (order != MCSPARSE_ORDER_ROW && order != MCSPARSE_ORDER_COL) return pub(BAD_VALUE);
    mcsparseDnMatDescr* d = new (std::nothrow) mcsparseDnMatDescr();
    if (d == nullptr) return MCSPARSE_STATUS_INTERNAL_ERROR;
    d->row_num = rows;
    d->col_num = cols;
    d->ld = ld;
    d->values = values;
    d->valueType = valueType;
    d->order = order;
    *dnMatDescr = d;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDestroyDnMat(mcsparseDnMatDescr_t d) {
    delete d;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnMatGet(mcsparseDnMatDescr_t d, int64_t* rows, int64_t* cols, int64_t* ld, void** values,
                                  macaDataType* type, mcsparseOrder_t* order) {
    if (d == nullptr || rows == nullptr || cols == nullptr || ld == nullptr || values == nullptr ||
        type == nullptr || order == nullptr)
        return pub(BAD_POINTER);
    *rows = d->row_num;
    *cols = d->col_num;
    *ld = d->ld;
    *values = d->values;
    *type = d->valueType;
    *order = d->order;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnMatGetValues(mcsparseDnMatDescr_t d, void** values) {
    if (d == nullptr || values == nullptr) return pub(BAD_POINTER);
    *values = d->values;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnMatSetValues(mcsparseDnMatDescr_t d, void* values) {
    if (d == nullptr) return pub(BAD_POINTER);
    d->values = values;
    return MCSPARSE_STATUS_SUCCESS;
}

// ----------------------------------------------------------------------------- strided batches

mcsparseStatus_t mcsparseCsrSetStridedBatch(mcsparseSpMatDescr_t d, int batchCount, int64_t offsetsBatchStride,
                                            int64_t columnsValuesBatchStride) {
    if (d == nullptr) return pub(BAD_POINTER);
    if (batchCount <= 0 || offsetsBatchStride < 0 || columnsValuesBatchStride < 0) return pub(BAD_SIZE);
    d->batchCount = batchCount;
    d->offsetsBatchStride = offsetsBatchStride;
    d->batchStride = columnsValuesBatchStride;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnMatSetStridedBatch(mcsparseDnMatDescr_t d, int batchCount, int64_t batchStride) {
    if (d == nullptr) return pub(BAD_POINTER);
    if (batchCount <= 0 || batchStride < 0) return pub(BAD_SIZE);
    d->batchCount = batchCount;
    d->batchStride = batchStride;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseDnMatGetStridedBatch(mcsparseDnMatDescr_t d, int* batchCount, int64_t* batchStride) {
    if (d == nullptr || batchCount == nullptr || batchStride == nullptr) return pub(BAD_POINTER);
    *batchCount = (int)d->batchCount;
    *batchStride = d->batchStride;
    return MCSPARSE_STATUS_SUCCESS;
}

}  // extern "C"
