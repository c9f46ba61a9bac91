/*
 * mcsparse.h -- C ABI of libmcsparse.so (sm_100a build) for the CSR SpMV / SpMM path.
 *
 * Every name, enumerator value and argument list below is the one the mcSparse library
 * exposes for this path, so a program written against mcSparse relinks without source
 * changes. Each group cites the reference declaration it replaces (path inside the
 * mcSparse source tree : line).
 *
 * Supported compute path: MCSPARSE_FORMAT_CSR (and row-sorted MCSPARSE_FORMAT_COO or MCSPARSE_FORMAT_CSC
 * as an input of mcsparseSpMV / mcsparseSpMM), MCSPARSE_OPERATION_NON_TRANSPOSE (mcsparseSpMV: also
 * MCSPARSE_OPERATION_TRANSPOSE, through a conversion into the external buffer),
 * MACA_R_32F / MACA_R_64F / MACA_C_32F / MACA_C_64F (complex: mcsparseSpMV also takes
 * MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE), offsets and columns both MCSPARSE_INDEX_32I or both
 * MCSPARSE_INDEX_64I with extents below 2^31, index base 0 or 1.
 * Everything else that the reference accepts on these entry points returns
 * MCSPARSE_STATUS_NOT_SUPPORTED here.
 */
#ifndef MCSPARSE_B200_MCSPARSE_H_
#define MCSPARSE_B200_MCSPARSE_H_

#include <stddef.h>
#include <stdint.h>

#include <cuda_runtime_api.h> /* cudaStream_t */
#include <library_types.h>    /* libraryPropertyType: MAJOR_VERSION, MINOR_VERSION, PATCH_LEVEL */
#include <cuComplex.h>        /* interleaved (re, im) pairs behind mcComplex / mcDoubleComplex */

#ifdef __cplusplus
extern "C" {
#endif

/* Stream type. Reference: mcsparse/include/interface/mcsp_helper.h.in:21-22 (mcStream_t). */
typedef cudaStream_t mcStream_t;

/* Value types. Reference: mcsparse/include/common/internal/mcsp_datatype.h:12-41
 * (numerically equal to cudaDataType). Only the two real floating types are computed on. */
typedef enum macaDataType_t {
    MACA_R_32F = 0,
    MACA_R_64F = 1,
    MACA_R_16F = 2,
    MACA_R_8I = 3,
    MACA_C_32F = 4,
    MACA_C_64F = 5,
    MACA_C_16F = 6,
    MACA_C_8I = 7,
    MACA_R_8U = 8,
    MACA_C_8U = 9,
    MACA_R_32I = 10,
    MACA_C_32I = 11,
    MACA_R_32U = 12,
    MACA_C_32U = 13,
    MACA_R_16BF = 14,
    MACA_C_16BF = 15,
    MACA_R_4I = 16,
    MACA_C_4I = 17,
    MACA_R_4U = 18,
    MACA_C_4U = 19,
    MACA_R_16I = 20,
    MACA_C_16I = 21,
    MACA_R_16U = 22,
    MACA_C_16U = 23,
    MACA_R_64I = 24,
    MACA_C_64I = 25,
    MACA_R_64U = 26,
    MACA_C_64U = 27
} macaDataType;

/* Enumerations. Reference: mcsparse/include/common/mcsp_types.h.in:12-155. */
typedef enum {
    MCSPARSE_OPERATION_NON_TRANSPOSE = 0,
    MCSPARSE_OPERATION_TRANSPOSE = 1,
    MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE = 2
} mcsparseOperation_t;

typedef enum {
    MCSPARSE_STATUS_SUCCESS = 0,
    MCSPARSE_STATUS_NOT_INITIALIZED = 1,
    MCSPARSE_STATUS_ALLOC_FAILED = 2,
    MCSPARSE_STATUS_INVALID_VALUE = 3,
    MCSPARSE_STATUS_ARCH_MISMATCH = 4,
    MCSPARSE_STATUS_MAPPING_ERROR = 5,
    MCSPARSE_STATUS_EXECUTION_FAILED = 6,
    MCSPARSE_STATUS_INTERNAL_ERROR = 7,
    MCSPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED = 8,
    MCSPARSE_STATUS_ZERO_PIVOT = 9,
    MCSPARSE_STATUS_NOT_SUPPORTED = 10,
    MCSPARSE_STATUS_INSUFFICIENT_RESOURCES = 11
} mcsparseStatus_t;

typedef enum {
    MCSPARSE_MATRIX_TYPE_GENERAL = 0,
    MCSPARSE_MATRIX_TYPE_SYMMETRIC = 1,
    MCSPARSE_MATRIX_TYPE_HERMITIAN = 2,
    MCSPARSE_MATRIX_TYPE_TRIANGULAR = 3
} mcsparseMatrixType_t;

typedef enum { MCSPARSE_INDEX_BASE_ZERO = 0, MCSPARSE_INDEX_BASE_ONE = 1 } mcsparseIndexBase_t;

typedef enum { MCSPARSE_STORAGE_MODE_SORTED = 0, MCSPARSE_STORAGE_MODE_UNSORTED = 1 } mcsparseStorageMode_t;

typedef enum { MCSPARSE_DIAG_TYPE_NON_UNIT = 0, MCSPARSE_DIAG_TYPE_UNIT = 1 } mcsparseDiagType_t;

typedef enum {
    MCSPARSE_FILL_MODE_LOWER = 0,
    MCSPARSE_FILL_MODE_UPPER = 1,
    MCSPARSE_FILL_MODE_FULL = 2
} mcsparseFillMode_t;

typedef enum { MCSPARSE_POINTER_MODE_HOST = 0, MCSPARSE_POINTER_MODE_DEVICE = 1 } mcsparsePointerMode_t;

typedef enum { MCSPARSE_ALG_MERGE_PATH = 0 } mcsparseAlgMode_t;

typedef enum {
    MCSPARSE_FORMAT_CSR = 1,
    MCSPARSE_FORMAT_CSC = 2,
    MCSPARSE_FORMAT_COO = 3,
    MCSPARSE_FORMAT_COO_AOS = 4,
    MCSPARSE_FORMAT_BLOCKED_ELL = 5
} mcsparseFormat_t;

typedef enum { MCSPARSE_ORDER_COL = 1, MCSPARSE_ORDER_ROW = 2 } mcsparseOrder_t;

typedef enum { MCSPARSE_INDEX_16U = 1, MCSPARSE_INDEX_32I = 2, MCSPARSE_INDEX_64I = 3 } mcsparseIndexType_t;

typedef enum { MCSPARSE_SPMAT_FILL_MODE = 0, MCSPARSE_SPMAT_DIAG_TYPE = 1 } mcsparseSpMatAttribute_t;

/* The algorithm selectors are accepted and treated as hints, as in the reference, which
 * forwards them nowhere (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:686-903). */
typedef enum {
    MCSPARSE_MV_ALG_DEFAULT = 0,
    MCSPARSE_COOMV_ALG = 1,
    MCSPARSE_CSRMV_ALG1 = 2,
    MCSPARSE_CSRMV_ALG2 = 3,
    MCSPARSE_SPMV_ALG_DEFAULT = 0,
    MCSPARSE_SPMV_CSR_ALG1 = 2,
    MCSPARSE_SPMV_CSR_ALG2 = 3,
    MCSPARSE_SPMV_COO_ALG1 = 1,
    MCSPARSE_SPMV_COO_ALG2 = 4
} mcsparseSpMVAlg_t;

typedef enum {
    MCSPARSE_MM_ALG_DEFAULT = 0,
    MCSPARSE_COOMM_ALG1 = 1,
    MCSPARSE_COOMM_ALG2 = 2,
    MCSPARSE_COOMM_ALG3 = 3,
    MCSPARSE_CSRMM_ALG1 = 4,
    MCSPARSE_SPMM_ALG_DEFAULT = 0,
    MCSPARSE_SPMM_COO_ALG1 = 1,
    MCSPARSE_SPMM_COO_ALG2 = 2,
    MCSPARSE_SPMM_COO_ALG3 = 3,
    MCSPARSE_SPMM_COO_ALG4 = 5,
    MCSPARSE_SPMM_CSR_ALG1 = 4,
    MCSPARSE_SPMM_CSR_ALG2 = 6,
    MCSPARSE_SPMM_CSR_ALG3 = 12,
    MCSPARSE_SPMM_BLOCKED_ELL_ALG1 = 13
} mcsparseSpMMAlg_t;

/* Opaque objects. Reference: mcsparse/include/common/mcsp_types.h.in:196-262. */
struct mcsparseContext;
typedef struct mcsparseContext* mcsparseHandle_t;
struct mcsparseMatDescr;
typedef struct mcsparseMatDescr* mcsparseMatDescr_t;
struct mcsparseSpMatDescr;
typedef struct mcsparseSpMatDescr* mcsparseSpMatDescr_t;
struct mcsparseDnVecDescr;
typedef struct mcsparseDnVecDescr* mcsparseDnVecDescr_t;
struct mcsparseDnMatDescr;
typedef struct mcsparseDnMatDescr* mcsparseDnMatDescr_t;

/* ---- Library handle. Reference: mcsparse/include/interface/mcsp_helper.h.in:12-29,
 *      behaviour mcsparse/src/common/mcsp_helper.cpp:69-88,154-198,294-323. ----
 * The handle records the device that is current at creation, a stream (default: the
 * legacy default stream) and the pointer mode for alpha/beta. No device memory is
 * reserved by the handle. mcsparseDestroy(NULL) succeeds. */
mcsparseStatus_t mcsparseCreate(mcsparseHandle_t* handle);
mcsparseStatus_t mcsparseDestroy(mcsparseHandle_t handle);
mcsparseStatus_t mcsparseGetVersion(mcsparseHandle_t handle, int* version);
mcsparseStatus_t mcsparseGetProperty(libraryPropertyType type, int* value);
const char* mcsparseGetErrorName(mcsparseStatus_t status);
const char* mcsparseGetErrorString(mcsparseStatus_t status);
mcsparseStatus_t mcsparseSetStream(mcsparseHandle_t handle, mcStream_t sid);
mcsparseStatus_t mcsparseGetStream(const mcsparseHandle_t handle, mcStream_t* sid);
mcsparseStatus_t mcsparseSetPointerMode(mcsparseHandle_t handle, mcsparsePointerMode_t pointer_mode);
mcsparseStatus_t mcsparseGetPointerMode(const mcsparseHandle_t handle, mcsparsePointerMode_t* pointer_mode);

/* ---- Legacy matrix descriptor. Reference: mcsparse/include/interface/mcsp_helper.h.in:24-44,
 *      behaviour mcsparse/src/common/mcsp_helper.cpp:90-108,200-292. ---- */
mcsparseStatus_t mcsparseCreateMatDescr(mcsparseMatDescr_t* descr);
mcsparseStatus_t mcsparseDestroyMatDescr(mcsparseMatDescr_t descr);
mcsparseStatus_t mcsparseSetMatIndexBase(mcsparseMatDescr_t descr, mcsparseIndexBase_t index_base);
mcsparseIndexBase_t mcsparseGetMatIndexBase(const mcsparseMatDescr_t descr);
mcsparseStatus_t mcsparseSetMatType(mcsparseMatDescr_t descr, mcsparseMatrixType_t matrix_type);
mcsparseMatrixType_t mcsparseGetMatType(const mcsparseMatDescr_t descr);
mcsparseStatus_t mcsparseSetMatFillMode(mcsparseMatDescr_t descr, mcsparseFillMode_t mode);
mcsparseFillMode_t mcsparseGetMatFillMode(const mcsparseMatDescr_t descr);
mcsparseStatus_t mcsparseSetMatDiagType(mcsparseMatDescr_t descr, mcsparseDiagType_t diag_type);
mcsparseDiagType_t mcsparseGetMatDiagType(const mcsparseMatDescr_t descr);

/* ---- Dense vector descriptor. Reference: mcsp_helper.h.in:46-50, mcsp_helper.cpp:325-387.
 *      The descriptor borrows `values` (device memory); it never copies or frees it. ---- */
mcsparseStatus_t mcsparseCreateDnVec(mcsparseDnVecDescr_t* dnVecDescr, int64_t size, void* values,
                                     macaDataType valueType);
mcsparseStatus_t mcsparseDestroyDnVec(mcsparseDnVecDescr_t dnVecDescr);
mcsparseStatus_t mcsparseDnVecGet(mcsparseDnVecDescr_t dnVecDescr, int64_t* size, void** values,
                                  macaDataType* valueType);
mcsparseStatus_t mcsparseDnVecGetValues(mcsparseDnVecDescr_t dnVecDescr, void** values);
mcsparseStatus_t mcsparseDnVecSetValues(mcsparseDnVecDescr_t dnVecDescr, void* values);

/* ---- CSR sparse matrix descriptor. Reference: mcsp_helper.h.in:60-66,81-90,
 *      mcsp_helper.cpp:389-445,503-524,587-713. The three arrays are borrowed device
 *      memory. mcsparseCsrSetPointers forgets any analysis recorded by a preprocess call. ---- */
mcsparseStatus_t mcsparseCreateCsr(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* csrRowOffsets, void* csrColInd, void* csrValues,
                                   mcsparseIndexType_t csrRowOffsetsType, mcsparseIndexType_t csrColIndType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType);
mcsparseStatus_t mcsparseCsrGet(mcsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz,
                                void** csrRowOffsets, void** csrColInd, void** csrValues,
                                mcsparseIndexType_t* csrRowOffsetsType, mcsparseIndexType_t* csrColIndType,
                                mcsparseIndexBase_t* idxBase, macaDataType* valueType);
mcsparseStatus_t mcsparseCsrSetPointers(mcsparseSpMatDescr_t spMatDescr, void* csrRowOffsets, void* csrColInd,
                                        void* csrValues);
mcsparseStatus_t mcsparseDestroySpMat(mcsparseSpMatDescr_t spMatDescr);
mcsparseStatus_t mcsparseSpMatGetSize(mcsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz);
mcsparseStatus_t mcsparseSpMatGetFormat(mcsparseSpMatDescr_t spMatDescr, mcsparseFormat_t* format);
mcsparseStatus_t mcsparseSpMatGetIndexBase(mcsparseSpMatDescr_t spMatDescr, mcsparseIndexBase_t* idxBase);
mcsparseStatus_t mcsparseSpMatGetValues(mcsparseSpMatDescr_t spMatDescr, void** values);
mcsparseStatus_t mcsparseSpMatSetValues(mcsparseSpMatDescr_t spMatDescr, void* values);
mcsparseStatus_t mcsparseSpMatGetAttribute(mcsparseSpMatDescr_t spMatDescr, mcsparseSpMatAttribute_t attribute,
                                           void* data, size_t dataSize);
mcsparseStatus_t mcsparseSpMatSetAttribute(mcsparseSpMatDescr_t spMatDescr, mcsparseSpMatAttribute_t attribute,
                                           const void* data, size_t dataSize);

/* ---- COO (structure of arrays) sparse matrix descriptor, accepted by mcsparseSpMV as an input format.
 *      Reference: mcsp_helper.h.in:52-58, mcsp_helper.cpp:433-438,526-560,597-605. Entries may come
 *      in any order. For entries sorted by row, mcsparseSpMV / mcsparseSpMM derive CSR row offsets
 *      from cooRowInd into the external buffer (the reference's coo2csr step,
 *      mcsparse/src/kernels/conversion/coo2csr_device.hpp:8-24); otherwise, and for op(A) = A^T / A^H,
 *      the entries are first sorted (stable) into the external buffer. Then the CSR kernels run. ---- */
mcsparseStatus_t mcsparseCreateCoo(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* cooRowInd, void* cooColInd, void* cooValues, mcsparseIndexType_t cooIdxType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType);
mcsparseStatus_t mcsparseCooGet(mcsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz,
                                void** cooRowInd, void** cooColInd, void** cooValues, mcsparseIndexType_t* idxType,
                                mcsparseIndexBase_t* idxBase, macaDataType* valueType);
mcsparseStatus_t mcsparseCooSetPointers(mcsparseSpMatDescr_t spMatDescr, void* cooRows, void* cooColumns,
                                        void* cooValues);

/* ---- COO stored as an array of (row, column) pairs, accepted by mcsparseSpMV (32-bit indices).
 *      Reference: mcsparse/include/interface/mcsp_generic.h:188-196, mcsparse/src/common/mcsp_helper.cpp:486-500,568-585.
 *      The pairs are split into two arrays in the external buffer (as the reference does,
 *      mcsp_spmv_gpu.cpp:773-789) and the entries are sorted there; any entry order is accepted. ---- */
mcsparseStatus_t mcsparseCreateCooAoS(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                      void* cooInd, void* cooValues, mcsparseIndexType_t cooIdxType,
                                      mcsparseIndexBase_t idxBase, macaDataType valueType);
mcsparseStatus_t mcsparseCooAoSGet(mcsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz,
                                   void** cooInd, void** cooValues, mcsparseIndexType_t* idxType,
                                   mcsparseIndexBase_t* idxBase, macaDataType* valueType);

/* ---- CSC sparse matrix descriptor, accepted by mcsparseSpMV (32-bit indices).
 *      Reference: mcsp_helper.h.in:69-72, mcsparse/src/common/mcsp_helper.cpp:447-452,607-615.
 *      The CSC arrays are the CSR arrays of the transposed matrix: op(A) = A^T on a CSC matrix runs the CSR
 *      kernels directly, op(A) = A goes through the same conversion as op(A) = A^T on a CSR matrix. ---- */
mcsparseStatus_t mcsparseCreateCsc(mcsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                   void* cscColOffsets, void* cscRowInd, void* cscValues,
                                   mcsparseIndexType_t cscColOffsetsType, mcsparseIndexType_t cscRowIndType,
                                   mcsparseIndexBase_t idxBase, macaDataType valueType);
mcsparseStatus_t mcsparseCscSetPointers(mcsparseSpMatDescr_t spMatDescr, void* cscColOffsets, void* cscRowInd,
                                        void* cscValues);

/* ---- Dense matrix descriptor. Reference: mcsp_helper.h.in:92-98, mcsp_helper.cpp:715-795. ---- */
mcsparseStatus_t mcsparseCreateDnMat(mcsparseDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                     void* values, macaDataType valueType, mcsparseOrder_t order);
mcsparseStatus_t mcsparseDestroyDnMat(mcsparseDnMatDescr_t dnMatDescr);
mcsparseStatus_t mcsparseDnMatGet(mcsparseDnMatDescr_t dnMatDescr, int64_t* rows, int64_t* cols, int64_t* ld,
                                  void** values, macaDataType* type, mcsparseOrder_t* order);
mcsparseStatus_t mcsparseDnMatGetValues(mcsparseDnMatDescr_t dnMatDescr, void** values);
mcsparseStatus_t mcsparseDnMatSetValues(mcsparseDnMatDescr_t dnMatDescr, void* values);

/* ---- Strided batches for mcsparseSpMM: batchCount independent products whose operands lie batchStride
 *      elements apart (A: row offsets offsetsBatchStride apart, columns and values
 *      columnsValuesBatchStride apart; a stride of 0 shares the operand between the batches).
 *      Reference: mcsparse/include/interface/mcsp_generic.h:180-185, setters
 *      mcsparse/src/kernels/generic/mcsp_generic.cpp:701-743, batching in the kernel
 *      mcsparse/src/kernels/level3/spmm/csr_spmm_device.hpp:102-108. A, B and C must carry the same
 *      batch count (mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:96-98). ---- */
mcsparseStatus_t mcsparseCsrSetStridedBatch(mcsparseSpMatDescr_t spMatDescr, int batchCount, int64_t offsetsBatchStride,
                                            int64_t columnsValuesBatchStride);
mcsparseStatus_t mcsparseDnMatSetStridedBatch(mcsparseDnMatDescr_t dnMatDescr, int batchCount, int64_t batchStride);
mcsparseStatus_t mcsparseDnMatGetStridedBatch(mcsparseDnMatDescr_t dnMatDescr, int* batchCount, int64_t* batchStride);

/* ---- SpMV: y = alpha * A * x + beta * y.
 * Reference: mcsparse/include/interface/mcsp_generic.h:43-51; entry
 * mcsparse/src/wrapper/mcsp_interface_wrapper.cpp:1236-1249; validation order
 * mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:686-720; kernel
 * mcsparse/src/kernels/level2/spmv/csr_vector_device.hpp:22-79.
 *
 * mcsparseSpMV_bufferSize reports the bytes the merge-path work partition and the
 * per-tile carries need (the reference reports a constant 128). mcsparseSpMV launches
 * asynchronously on the handle's stream. alpha/beta are read from host or device memory
 * according to the pointer mode; in device mode they are read by the kernels, with no
 * blocking copy. y is not read when beta == 0. ---- */
mcsparseStatus_t mcsparseSpMV_bufferSize(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg, size_t* bufferSize);
mcsparseStatus_t mcsparseSpMV(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                              mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                              mcsparseDnVecDescr_t vecY, macaDataType computeType, mcsparseSpMVAlg_t alg,
                              void* externalBuffer);

/* ---- SpMM: C = alpha * A * B + beta * C.
 * Reference: mcsparse/include/interface/mcsp_generic.h:54-67; entry
 * mcsparse/src/wrapper/mcsp_interface_wrapper.cpp:1250-1272; validation
 * mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:785-807; kernel
 * mcsparse/src/kernels/level3/spmm/csr_spmm_device.hpp:91-167.
 * opA = opB = NON_TRANSPOSE; B and C may each be row- or column-major. Row-major B is
 * read in place (the reference first transposes it into a temporary allocation).
 * The call is asynchronous on the handle's stream. ---- */
mcsparseStatus_t mcsparseSpMM_bufferSize(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                                         const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                                         const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                                         mcsparseSpMMAlg_t alg, size_t* bufferSize);
mcsparseStatus_t mcsparseSpMM_preprocess(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                                         const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                                         const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                                         mcsparseSpMMAlg_t alg, void* externalBuffer);
mcsparseStatus_t mcsparseSpMM(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                              const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                              const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                              mcsparseSpMMAlg_t alg, void* externalBuffer);

/* Complex scalars and arrays of the legacy entry points: the MetaX SDK's mcComplex / mcDoubleComplex
 * (common/mcComplex.h, used by mcsparse/include/interface/mcsp_level2.h:36-44) have the layout of
 * cuComplex / cuDoubleComplex. */
typedef cuComplex mcComplex;
typedef cuComplex mcFloatComplex;
typedef cuDoubleComplex mcDoubleComplex;

/* ---- Legacy entry points onto the same kernels.
 * Reference: mcsparse/include/interface/mcsp_level2.h:10-44 and
 * mcsparse/include/interface/mcsp_level3.h:138-181; forwarding
 * mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:905-953. The S/D csrmv calls take
 * no work buffer, so they run the thread-group-per-row kernel that needs no partition. ---- */
mcsparseStatus_t mcsparseScsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const float* alpha, const mcsparseMatDescr_t descrA, const float* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const float* x, const float* beta,
                                float* y);
mcsparseStatus_t mcsparseDcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const double* alpha, const mcsparseMatDescr_t descrA, const double* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const double* x, const double* beta,
                                double* y);
mcsparseStatus_t mcsparseCcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const mcComplex* alpha, const mcsparseMatDescr_t descrA, const mcComplex* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const mcComplex* x,
                                const mcComplex* beta, mcComplex* y);
mcsparseStatus_t mcsparseZcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const mcDoubleComplex* alpha, const mcsparseMatDescr_t descrA,
                                const mcDoubleComplex* csrValA, const int* csrRowPtrA, const int* csrColIndA,
                                const mcDoubleComplex* x, const mcDoubleComplex* beta, mcDoubleComplex* y);
mcsparseStatus_t mcsparseCsrmvEx_bufferSize(mcsparseHandle_t handle, mcsparseAlgMode_t alg,
                                            mcsparseOperation_t transA, int m, int n, int nnz, const void* alpha,
                                            macaDataType alphatype, const mcsparseMatDescr_t descrA,
                                            const void* csrValA, macaDataType csrValAtype, const int* csrRowPtrA,
                                            const int* csrColIndA, const void* x, macaDataType xtype,
                                            const void* beta, macaDataType betatype, void* y, macaDataType ytype,
                                            macaDataType executiontype, size_t* bufferSizeInBytes);
mcsparseStatus_t mcsparseCsrmvEx(mcsparseHandle_t handle, mcsparseAlgMode_t alg, mcsparseOperation_t transA, int m,
                                 int n, int nnz, const void* alpha, macaDataType alphatype,
                                 const mcsparseMatDescr_t descrA, const void* csrValA, macaDataType csrValAtype,
                                 const int* csrRowPtrA, const int* csrColIndA, const void* x, macaDataType xtype,
                                 const void* beta, macaDataType betatype, void* y, macaDataType ytype,
                                 macaDataType executiontype, void* buffer);
mcsparseStatus_t mcsparseScsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const float* alpha, const mcsparseMatDescr_t descrA,
                                 const float* csrValA, const int* csrRowPtrA, const int* csrColIndA, const float* B,
                                 int ldb, const float* beta, float* C, int ldc);
mcsparseStatus_t mcsparseDcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const double* alpha,
                                 const mcsparseMatDescr_t descrA, const double* csrValA, const int* csrRowPtrA,
                                 const int* csrColIndA, const double* B, int ldb, const double* beta, double* C,
                                 int ldc);
mcsparseStatus_t mcsparseCcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const mcComplex* alpha,
                                 const mcsparseMatDescr_t descrA, const mcComplex* csrValA, const int* csrRowPtrA,
                                 const int* csrColIndA, const mcComplex* B, int ldb, const mcComplex* beta,
                                 mcComplex* C, int ldc);
mcsparseStatus_t mcsparseZcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const mcDoubleComplex* alpha,
                                 const mcsparseMatDescr_t descrA, const mcDoubleComplex* csrValA,
                                 const int* csrRowPtrA, const int* csrColIndA, const mcDoubleComplex* B, int ldb,
                                 const mcDoubleComplex* beta, mcDoubleComplex* C, int ldc);
mcsparseStatus_t mcsparseScsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const float* alpha, const mcsparseMatDescr_t descrA, const float* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const float* B, int ldb,
                                const float* beta, float* C, int ldc);
mcsparseStatus_t mcsparseDcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const double* alpha, const mcsparseMatDescr_t descrA, const double* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const double* B, int ldb,
                                const double* beta, double* C, int ldc);
mcsparseStatus_t mcsparseCcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const mcComplex* alpha, const mcsparseMatDescr_t descrA, const mcComplex* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const mcComplex* B, int ldb,
                                const mcComplex* beta, mcComplex* C, int ldc);
mcsparseStatus_t mcsparseZcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const mcDoubleComplex* alpha, const mcsparseMatDescr_t descrA,
                                const mcDoubleComplex* csrValA, const int* csrRowPtrA, const int* csrColIndA,
                                const mcDoubleComplex* B, int ldb, const mcDoubleComplex* beta, mcDoubleComplex* C,
                                int ldc);

#ifdef __cplusplus
}
#endif

#include "mcsparse_b200_ext.h"

#endif /* MCSPARSE_B200_MCSPARSE_H_ */
