// Host side of libmcsparse.so, compute entry points: argument validation, format and dtype routing for
// mcsparseSpMV / mcsparseSpMM, the legacy csrmv / csrmm calls and the added entry points. The handle and the
// descriptors are in descriptors.cpp; the status codes used here are explained in api_common.h.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "api_common.h"

using namespace mcsp_b200;
using namespace mcsp_b200::api;

namespace {


bool is_real_fp(macaDataType t) { return t == MACA_R_32F || t == MACA_R_64F; }
bool is_complex_fp(macaDataType t) { return t == MACA_C_32F || t == MACA_C_64F; }
bool is_compute_type(macaDataType t) { return is_real_fp(t) || is_complex_fp(t); }
// A real matrix applied to complex vectors with complex scalars (mcsp_spmv_gpu.cpp:852-855 routes this pair
// of types to the CSR kernel instantiated with real values and complex x, y).
bool real_matrix_complex_vectors(macaDataType a, macaDataType x, macaDataType y, macaDataType compute) {
    return ((a == MACA_R_32F && compute == MACA_C_32F) || (a == MACA_R_64F && compute == MACA_C_64F)) &&
           x == compute && y == compute;
}
// Low-precision operands with wider sums (mcsp_spmv_gpu.cpp:848-860 sends every call whose compute, matrix and
// output types are not all one type, and whose matrix is not fp32 / fp64, to mcspMixedPrecisionSpMVImpl, which
// routes by the types of x and y, :498-561). A and x share a type; the scalars and the sums are fp32, or int32
// for int8 -> int32. The half-precision complex pairs of that table are not built.
MixedKind low_precision_kind(macaDataType a, macaDataType x, macaDataType y, macaDataType compute) {
    if (a != x) return MixedKind::kNone;
    if (compute == MACA_R_32I) return (x == MACA_R_8I && y == MACA_R_32I) ? MixedKind::kInt8ToInt32 : MixedKind::kNone;
    if (compute != MACA_R_32F) return MixedKind::kNone;
    if (x == MACA_R_16F) return y == MACA_R_32F ? MixedKind::kHalfToFloat : y == MACA_R_16F ? MixedKind::kHalfToHalf : MixedKind::kNone;
    if (x == MACA_R_16BF) return y == MACA_R_32F ? MixedKind::kBf16ToFloat : y == MACA_R_16BF ? MixedKind::kBf16ToBf16 : MixedKind::kNone;
    if (x == MACA_R_8I) return y == MACA_R_32F ? MixedKind::kInt8ToFloat : MixedKind::kNone;
    return MixedKind::kNone;
}
size_t value_size(macaDataType t) { return t == MACA_C_64F ? 16 : (t == MACA_R_64F || t == MACA_C_32F) ? 8 : 4; }
bool too_big(int64_t v) { return (v >> 31) != 0; }  // int32 indices: every extent must fit

bool descr_general(const mcsparseMatDescr* d) {
    return d->type == MCSPARSE_MATRIX_TYPE_GENERAL && d->fill_mode == MCSPARSE_FILL_MODE_FULL &&
           d->diag_type == MCSPARSE_DIAG_TYPE_NON_UNIT;
}

template <typename T>
ScalarArg<T> scalar_arg(const mcsparseContext* h, const void* p) {
    ScalarArg<T> a;
    if (h->ptr_mode == MCSPARSE_POINTER_MODE_HOST) {
        a.host = *static_cast<const T*>(p);
        a.dev = nullptr;
    } else {
        a.host = T(0);
        a.dev = static_cast<const T*>(p);
    }
    return a;
}


// ----------------------------------------------------------------------------- SpMV

// Checks shared by bufferSize / preprocess / compute, in the reference's order
// (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:690-720 and :309-336).
St spmv_check(mcsparseHandle_t h, mcsparseOperation_t opA, const void* alpha, mcsparseSpMatDescr_t A,
              mcsparseDnVecDescr_t X, const void* beta, mcsparseDnVecDescr_t Y, macaDataType computeType,
              bool need_buffer, const void* buffer, bool need_size_out, const void* size_out,
              bool allow_coo = false, bool allow_wide_indices = false, bool allow_transposed = false) {
    if (h == nullptr) return BAD_HANDLE;
    if (alpha == nullptr || beta == nullptr || A == nullptr || X == nullptr || Y == nullptr) return BAD_POINTER;
    if (need_size_out && size_out == nullptr) return BAD_POINTER;
    // Index types come in matched pairs (mcsp_spmv_gpu.cpp:1112-1118); with 64-bit indices the extents
    // must still fit 31 bits.
    const bool narrow = A->rowIdxType == MCSPARSE_INDEX_32I && A->colIdxType == MCSPARSE_INDEX_32I;
    const bool wide = A->rowIdxType == MCSPARSE_INDEX_64I && A->colIdxType == MCSPARSE_INDEX_64I;
    if (!(narrow || (wide && allow_wide_indices))) return NOT_IMPL;
    if (too_big(A->row_num) || too_big(A->col_num) || too_big(A->nnz) || too_big(X->size) || too_big(Y->size) ||
        too_big(A->row_num + A->nnz) || too_big(A->col_num + A->nnz))
        return NOT_IMPL;
    if (need_buffer && buffer == nullptr) return BAD_POINTER;
    if (!(A->format == MCSPARSE_FORMAT_CSR || (allow_coo && A->format == MCSPARSE_FORMAT_COO) ||
          (allow_transposed && (A->format == MCSPARSE_FORMAT_CSC || A->format == MCSPARSE_FORMAT_COO_AOS))))
        return NOT_IMPL;
    if (A->format == MCSPARSE_FORMAT_COO_AOS && !narrow) return NOT_IMPL;  // pairs are split as 32-bit integers
    const bool n_op = opA == MCSPARSE_OPERATION_NON_TRANSPOSE;
    if (!((n_op && X->size == A->col_num && Y->size == A->row_num) ||
          (!n_op && X->size == A->row_num && Y->size == A->col_num)))
        return BAD_SIZE;
    if (is_real_fp(computeType) && opA == MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE) return BAD_VALUE;
    // op(A) = A^T / A^H and CSC inputs run through a conversion into the buffer.
    if (!n_op && !allow_transposed) return NOT_IMPL;
    // Low-precision operands: CSR, op(A) = A, 32-bit indices, through the generic entry points.
    if (low_precision_kind(A->valueType, X->valueType, Y->valueType, computeType) != MixedKind::kNone)
        return (allow_transposed && n_op && narrow && A->format == MCSPARSE_FORMAT_CSR) ? OK : NOT_IMPL;
    const bool mixed = real_matrix_complex_vectors(A->valueType, X->valueType, Y->valueType, computeType);
    if (!(computeType == A->valueType && computeType == Y->valueType && computeType == X->valueType) && !mixed)
        return NOT_IMPL;
    if (mixed && !(n_op && A->format == MCSPARSE_FORMAT_CSR)) return NOT_IMPL;
    if (!is_compute_type(computeType)) return NOT_IMPL;
    // Complex values: the generic entry points only (the same that take transposed products).
    if (is_complex_fp(computeType) && !allow_transposed) return NOT_IMPL;
    if (mixed && !narrow) return NOT_IMPL;
    return OK;
}

// Environment overrides for tuning: MCSPARSE_B200_SPMV_TILE=small|large fixes the tile size,
// MCSPARSE_B200_SPMV_WALK=0|1 the kernel family. Returns the kind with the overrides applied.
int apply_tile_overrides(int kind) {
    if (const char* e = std::getenv("MCSPARSE_B200_SPMV_TILE")) {
        if (e[0] == 's') kind |= kTileSmall;
        if (e[0] == 'l') kind &= ~kTileSmall;
    }
    if (const char* e = std::getenv("MCSPARSE_B200_SPMV_WALK")) {
        if (e[0] == '1') kind |= kTileWalk;
        if (e[0] == '0') kind &= ~kTileWalk;
    }
    return kind;
}

// Tile kind for this matrix. When neighbouring nonzeros rarely have neighbouring columns (fewer than
// a quarter of 4096 sampled pairs within 8 columns) the matrix is gather-bound and gets the walk
// kernel; otherwise the lanes-per-row kernel with the large tiles. Probed once per column array
// (one small kernel and a 4-byte copy, which synchronises the stream) and remembered on the
// descriptor. `scratch` is device memory the probe may overwrite (the start of the work buffer,
// before the analysis writes it).
int probe_tile_kind(mcsparseContext* h, const void* ptr, const void* idx, bool wide, int64_t nnz, int64_t rows,
                    size_t vsize, void* scratch) {
    int counts[2] = {4096, 0};  // {neighbouring columns, long rows}
    if (nnz >= 2) {
        int* dev = static_cast<int*>(scratch);
        const cudaError_t e =
            wide ? spmv_locality_probe(h->stream, rows, nnz, static_cast<const int64_t*>(ptr), static_cast<const int64_t*>(idx), dev, counts)
                 : spmv_locality_probe(h->stream, rows, nnz, static_cast<const int32_t*>(ptr), static_cast<const int32_t*>(idx), dev, counts);
        if (e != cudaSuccess) counts[0] = 4096, counts[1] = 0;
    }
    // Scattered columns: the half-size tile. Scattered columns and rows of very different lengths (two or more of
    // the sampled rows beyond 256 nonzeros): the walk kernel, which does not care about row lengths; rows of
    // similar, moderate length are faster with lanes per row.
    int kind = counts[0] < 1024 ? kTileSmall : kTileLarge;
    if (counts[0] < 1024 && counts[1] >= 2) kind |= kTileWalk;
    if (wide && vsize == 4) kind |= kTileSmall;  // 64-bit indices with 4-byte values: one tile size
    // A matrix so small that the large tiles would not fill the GPU four times over also gets the small ones.
    const int64_t large = spmv_workspace(rows, nnz, vsize, kTileLarge).items_per_tile;
    if ((rows + nnz) / large < 4LL * 8 * (h->sm_count > 0 ? h->sm_count : 148)) kind |= kTileSmall;
    return apply_tile_overrides(kind);
}

// `idx` / `rows`: the index array and the row count the kernels will run on (for a CSC input these
// are the row indices and the column count).
int choose_tile_kind(mcsparseContext* h, mcsparseSpMatDescr* A, const void* ptr, const void* idx, int64_t rows,
                     void* scratch) {
    std::lock_guard<std::mutex> g(A->lock);
    if (A->probed_cols == idx && A->probed_nnz == A->nnz) return A->tile_kind;
    A->tile_kind = probe_tile_kind(h, ptr, idx, A->colIdxType == MCSPARSE_INDEX_64I, A->nnz, rows,
                                   value_size(A->valueType), scratch);
    A->probed_cols = idx;
    A->probed_nnz = A->nnz;
    return A->tile_kind;
}

// The choice already made for this matrix, without probing (large tiles, lanes-per-row kernel if none was made).
int known_tile_kind(mcsparseSpMatDescr* A) {
    std::lock_guard<std::mutex> g(A->lock);
    if (A->probed_cols == A->cols && A->probed_nnz == A->nnz) return A->tile_kind;
    return apply_tile_overrides(A->colIdxType == MCSPARSE_INDEX_64I && value_size(A->valueType) == 4 ? kTileSmall : kTileLarge);
}

WaitCfg wait_cfg(const mcsparseContext* h) {
    WaitCfg w;
    w.limit_cycles = h->wait_cycles;
    w.withhold = h->withhold_copies;
    w.fault_word = h->fault_word_dev;
    return w;
}

// A tile kernel of an earlier call on this handle gave up its bounded wait: reported once, by the
// next compute call, as an execution failure (the word lives in pinned host memory the kernels can
// write, so reading it needs no synchronisation).
bool take_device_fault(mcsparseContext* h) {
    if (h->fault_word_host == nullptr || *reinterpret_cast<volatile int*>(h->fault_word_host) == 0) return false;
    *reinterpret_cast<volatile int*>(h->fault_word_host) = 0;
    log_error("an earlier SpMV on this handle gave up a bounded device-side wait; its result is incomplete");
    return true;
}

struct PushArgs {
    int count = 0;
    void* const* y = nullptr;
    int64_t row_offset = 0;
    bool multicast = false;  // y[0] is a multicast address reaching every GPU
    bool bulk = false;       // rows leave through bulk copies from shared memory
    bool crew = false;       // rows are moved by the push crew of the tile launch
};

size_t index_size(const mcsparseSpMatDescr* A) { return A->rowIdxType == MCSPARSE_INDEX_64I ? 8 : 4; }

// A product as the CSR kernels see it: an m x n CSR matrix (offsets `ptr`, indices `idx`) applied as
// it is or transposed. CSC arrays are the CSR arrays of the transposed matrix, so a CSC input swaps
// the roles (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:734-739 does the same swap).
struct CsrView {
    int64_t m = 0, n = 0;
    const void* ptr = nullptr;
    const void* idx = nullptr;
    bool transposed = false;
    bool conjugate = false;  // op(A) = A^H on complex values
    // COO entries that must be sorted first: ptr holds the index array to sort by (rows, or columns for
    // a transposed product), idx the other one, n the number of rows of the matrix the kernels will see.
    bool coo_sort = false;
    bool converted() const { return transposed || coo_sort; }
};

// Whether a COO matrix has its entries out of row order: one small kernel and a stream synchronisation the
// first time a row-index array is seen, remembered on the descriptor after that.
bool coo_unsorted(mcsparseContext* h, mcsparseSpMatDescr* A) {
    if (A->format != MCSPARSE_FORMAT_COO || A->rows == nullptr) return false;
    std::lock_guard<std::mutex> g(A->lock);
    if (A->coo_checked_rows == A->rows && A->coo_checked_nnz == A->nnz) return A->coo_unsorted;
    if (h == nullptr) return false;  // nothing to check with: the answer of the last check, if any, was given above
    DeviceGuard guard(h->device);
    int flag = 0;
    const cudaError_t e = A->rowIdxType == MCSPARSE_INDEX_64I
                              ? indices_unsorted(h->stream, A->nnz, static_cast<const int64_t*>(A->rows), &flag)
                              : indices_unsorted(h->stream, A->nnz, static_cast<const int32_t*>(A->rows), &flag);
    if (e != cudaSuccess) flag = 1;
    A->coo_unsorted = flag != 0;
    A->coo_checked_rows = A->rows;
    A->coo_checked_nnz = A->nnz;
    return A->coo_unsorted;
}

CsrView csr_view(mcsparseContext* h, mcsparseSpMatDescr* A, mcsparseOperation_t opA) {
    CsrView v;
    const bool t_op = opA != MCSPARSE_OPERATION_NON_TRANSPOSE;
    v.conjugate = opA == MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE && is_complex_fp(A->valueType);
    // (64-bit COO always goes through the sort: it leaves 32-bit arrays, which is what the kernels take when
    // the row offsets are derived rather than given.)
    if (A->format == MCSPARSE_FORMAT_COO && (t_op || A->rowIdxType == MCSPARSE_INDEX_64I || coo_unsorted(h, A))) {
        // Sorting by row gives the CSR of A, sorting by column the CSR of A^T: no further transposition.
        v.coo_sort = true;
        if (t_op)
            v.m = A->row_num, v.n = A->col_num, v.ptr = A->cols, v.idx = A->rows;
        else
            v.m = A->col_num, v.n = A->row_num, v.ptr = A->rows, v.idx = A->cols;
        return v;
    }
    if (A->format == MCSPARSE_FORMAT_CSC) {
        v.m = A->col_num, v.n = A->row_num, v.ptr = A->cols, v.idx = A->rows, v.transposed = !t_op;
    } else {
        v.m = A->row_num, v.n = A->col_num, v.ptr = A->rows, v.idx = A->cols, v.transposed = t_op;
    }
    return v;
}

// L2 residency of x for gather-bound products (opt-in: MCSPARSE_B200_L2_PERSIST_X=1). When the columns are
// scattered, every nonzero fetches its own 32-byte sector of x from L2; an x of 50-80 MB (the power-law benchmark:
// 67 MB) no longer stays in L2 beside the stream of A, and a fifth of those gathers go to HBM (measured: 3.0 GB of
// DRAM reads against 1.8 GB algorithmic). With the switch on, such a launch marks x as persisting in L2 through
// the stream's access-policy window (A's stream is already evict-first) and takes the window off again right after
// the launch; the persisting carve-out is requested once per handle, sized to x. Measured on the power-law matrix:
// 1.15 -> 1.03 ms. It is off by default because the carve-out is a setting of the whole context: every other
// kernel of the process loses that much L2 from then on (the stencil product measured 0.97 -> 1.08 ms beside it).
struct XResidency {
    cudaStream_t stream = nullptr;
    bool on = false;
    XResidency(mcsparseContext* h, const void* x, size_t bytes, int tile_kind) {
        if ((tile_kind & kTileSmall) == 0 || bytes < (size_t(40) << 20)) return;
        const char* e = std::getenv("MCSPARSE_B200_L2_PERSIST_X");
        if (e == nullptr || e[0] != '1') return;
        if (h->max_persisting_l2 < 0) {
            int v = 0;
            if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxPersistingL2CacheSize, h->device) != cudaSuccess) v = 0;
            h->max_persisting_l2 = v;
        }
        if ((long long)bytes > h->max_persisting_l2) return;
        if (!h->persisting_l2_requested) {
            if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, bytes) != cudaSuccess) {
                cudaGetLastError();
                h->max_persisting_l2 = 0;
                return;
            }
            h->persisting_l2_requested = true;
        }
        cudaStreamAttrValue attr = {};
        attr.accessPolicyWindow.base_ptr = const_cast<void*>(x);
        attr.accessPolicyWindow.num_bytes = bytes;
        attr.accessPolicyWindow.hitRatio = 1.0f;
        attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
        attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
        if (cudaStreamSetAttribute(h->stream, cudaStreamAttributeAccessPolicyWindow, &attr) != cudaSuccess) {
            cudaGetLastError();
            return;
        }
        stream = h->stream;
        on = true;
    }
    ~XResidency() {
        if (!on) return;
        cudaStreamAttrValue attr = {};  // an empty window: later launches on the stream are not affected
        cudaStreamSetAttribute(stream, cudaStreamAttributeAccessPolicyWindow, &attr);
    }
};

template <typename T, typename I>
St spmv_run(mcsparseContext* h, mcsparseSpMatDescr* A, const CsrView& v, mcsparseDnVecDescr* X, mcsparseDnVecDescr* Y,
            const void* alpha, const void* beta, void* buffer, bool analyse, bool compute, int tile_kind,
            const PushArgs& push = PushArgs(), bool scalars_on_host = false) {
    const SpmvWorkspace ws = spmv_workspace(v.m, A->nnz, sizeof(T), tile_kind, sizeof(I));
    void* buf = align_up_256(buffer);
    const int base = A->mat_descr->base;
    const I* rows = static_cast<const I*>(v.ptr);
    if (A->format == MCSPARSE_FORMAT_COO) {
        // Row offsets derived from the sorted row indices live behind the SpMV work area
        // (32-bit indices only: the argument check admits no 64-bit COO).
        int32_t* offsets = reinterpret_cast<int32_t*>(static_cast<char*>(buf) + ws.bytes);
        if (analyse) {
            cudaError_t e = coo_row_offsets(h->stream, v.m, A->nnz, base, static_cast<const int32_t*>(v.ptr), offsets);
            if (e != cudaSuccess) return from_cuda(e);
        }
        rows = reinterpret_cast<const I*>(offsets);
    }
    if (analyse) {
        cudaError_t e = spmv_analysis(h->stream, v.m, A->nnz, base, rows, ws, buf);
        if (e != cudaSuccess) return from_cuda(e);
    }
    if (!compute) return OK;
    PeerList<T> peers;
    peers.count = push.count;
    peers.row_offset = push.row_offset;
    peers.multicast = push.multicast;
    peers.bulk = push.bulk;
    // the crew copies whole 16-byte groups from the local y: it must sit at the peers' alignment
    peers.crew = push.crew && push.count > 0 &&
                 ((reinterpret_cast<uintptr_t>(Y->values) ^
                   (reinterpret_cast<uintptr_t>(push.y[0]) + size_t(push.row_offset) * sizeof(T))) & 15) == 0;
    const XResidency keep_x(h, X->values, size_t(X->size) * sizeof(T), tile_kind);
    for (int p = 0; p < push.count; ++p) peers.y[p] = static_cast<T*>(push.y[p]);
    const ScalarArg<T> sa = scalars_on_host ? ScalarArg<T>{*static_cast<const T*>(alpha), nullptr} : scalar_arg<T>(h, alpha);
    const ScalarArg<T> sb = scalars_on_host ? ScalarArg<T>{*static_cast<const T*>(beta), nullptr} : scalar_arg<T>(h, beta);
    cudaError_t e = spmv_tiled<T, I>(h->stream, v.m, A->nnz, base, rows, static_cast<const I*>(v.idx),
                                     static_cast<const T*>(A->vals), static_cast<const T*>(X->values),
                                     static_cast<T*>(Y->values), sa, sb, ws, buf, peers, wait_cfg(h));
    return from_cuda(e);
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// A^H x of a CSC matrix with complex values. The reference conjugates the values in place and runs its CSR kernel
// on the CSC arrays (mcsp_spmv_gpu.cpp:734-770). Here the values stay untouched: conj(A^T) x = conj(A^T conj(x)),
// the CSC arrays are the CSR arrays of A^T, and conj(x) (A.rows numbers) and the intermediate product (A.cols
// numbers) live behind the work area; y = alpha * conj(z) + beta * y is the last, vector-sized pass.
template <typename F, typename I>
St spmv_csc_conjugate_run(mcsparseContext* h, mcsparseSpMatDescr* A, const CsrView& v, mcsparseDnVecDescr* X,
                          mcsparseDnVecDescr* Y, const void* alpha, const void* beta, void* buffer, bool analyse,
                          bool compute, int tile_kind) {
    using T = Complex<F>;
    const SpmvWorkspace ws = spmv_workspace(v.m, A->nnz, sizeof(T), tile_kind, sizeof(I));
    char* const tail = static_cast<char*>(align_up_256(buffer)) + ws.bytes;
    T* const xc = reinterpret_cast<T*>(tail);
    T* const z = reinterpret_cast<T*>(tail + align256(size_t(v.n) * sizeof(T)));
    if (compute) {
        const cudaError_t e = complex_conj_copy<T>(h->stream, v.n, static_cast<const T*>(X->values), xc);
        if (e != cudaSuccess) return from_cuda(e);
    }
    mcsparseDnVecDescr Xc = *X, Z = *Y;
    Xc.values = xc;
    Z.values = z;
    const T one(F(1), F(0)), zero(F(0), F(0));
    const St st = spmv_run<T, I>(h, A, v, &Xc, &Z, &one, &zero, buffer, analyse, compute, tile_kind, PushArgs(), true);
    if (st != OK || !compute) return st;
    return from_cuda(complex_conj_axpby<T>(h->stream, v.m, scalar_arg<T>(h, alpha), z, scalar_arg<T>(h, beta),
                                           static_cast<T*>(Y->values)));
}

// COO as an array of (row, column) pairs: the pairs are split into two arrays behind the rest of the buffer
// (the reference does the same first, mcsp_spmv_gpu.cpp:773-789) and the entries then go through the sort.
CsrView aos_view(const mcsparseSpMatDescr* A, mcsparseOperation_t opA, int32_t* split_rows, int32_t* split_cols) {
    CsrView v;
    const bool t_op = opA != MCSPARSE_OPERATION_NON_TRANSPOSE;
    v.conjugate = opA == MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE && is_complex_fp(A->valueType);
    v.coo_sort = true;
    if (t_op)
        v.m = A->row_num, v.n = A->col_num, v.ptr = split_cols, v.idx = split_rows;
    else
        v.m = A->col_num, v.n = A->row_num, v.ptr = split_rows, v.idx = split_cols;
    return v;
}

// Layout of the external buffer of a transposed product: the SpMV work area of the n x m transposed
// matrix, then (256-byte aligned) the conversion area described by TransposePlan.
struct TransposedLayout {
    void* work = nullptr;
    void* area = nullptr;
    TransposePlan plan;
};

TransposedLayout transposed_layout(const CsrView& v, int64_t nnz, size_t vsize, void* buffer) {
    TransposedLayout L;
    L.plan = transpose_plan(v.m, v.n, nnz, vsize);
    L.work = align_up_256(buffer);
    if (buffer != nullptr) L.area = align_up_256(static_cast<char*>(L.work) + spmv_workspace(v.n, nnz, vsize).bytes);
    return L;
}

size_t transposed_buffer_bytes(const CsrView& v, int64_t nnz, size_t vsize) {
    return spmv_workspace(v.n, nnz, vsize).bytes + 256 + transpose_plan(v.m, v.n, nnz, vsize).bytes + 256;
}

// Structure of the matrix the kernels will run on, for a transposed view or a COO that needs sorting.
template <typename I>
cudaError_t convert_structure_as(cudaStream_t s, const mcsparseSpMatDescr* A, const CsrView& v, const TransposePlan& plan,
                                 void* area) {
    const int base = A->mat_descr->base;
    const I *ptr = static_cast<const I*>(v.ptr), *idx = static_cast<const I*>(v.idx);
    return v.coo_sort ? coo_sort_structure<I>(s, v.n, A->nnz, base, ptr, idx, plan, area)
                      : transpose_structure<I>(s, v.m, v.n, A->nnz, base, ptr, idx, plan, area);
}
cudaError_t convert_structure(cudaStream_t s, const mcsparseSpMatDescr* A, const CsrView& v, const TransposePlan& plan,
                              void* area) {
    return A->rowIdxType == MCSPARSE_INDEX_64I ? convert_structure_as<int64_t>(s, A, v, plan, area)
                                               : convert_structure_as<int32_t>(s, A, v, plan, area);
}

// y = alpha * V^T * x + beta * y for the CSR view V: convert (structure once per preprocess, or on
// every call without one; values on every call), then the ordinary tile kernels on the result.
template <typename T>
St spmv_transposed_run(mcsparseContext* h, mcsparseSpMatDescr* A, const CsrView& v, mcsparseDnVecDescr* X,
                       mcsparseDnVecDescr* Y, const void* alpha, const void* beta, void* buffer, bool preprocess_only) {
    const int64_t nnz = A->nnz;
    const TransposedLayout L = transposed_layout(v, nnz, sizeof(T), buffer);
    char* area = static_cast<char*>(L.area);
    const int32_t* t_ptr = reinterpret_cast<const int32_t*>(area + L.plan.off_ptr);
    const int32_t* t_idx = reinterpret_cast<const int32_t*>(area + L.plan.off_keys[L.plan.col_slot()]);
    const T* t_val = reinterpret_cast<const T*>(area + L.plan.off_val);
    bool cached = false, probed = false;
    int kind = kTileLarge;
    {
        std::lock_guard<std::mutex> g(A->lock);
        cached = A->trans_buffer == buffer && A->trans_ptr_src == v.ptr && A->trans_idx_src == v.idx && A->trans_nnz == nnz;
        probed = A->trans_probed_idx == v.idx && A->trans_probed_nnz == nnz;
        kind = A->trans_tile_kind;
    }
    if (!cached) {
        {   // this buffer is about to hold the transposed matrix's partition: forget what else was recorded in it
            std::lock_guard<std::mutex> g(A->lock);
            if (A->analysed_buffer == buffer) A->analysed_buffer = nullptr;
            if (A->push_buffer == buffer) A->push_buffer = nullptr;
            if (A->spmm_buffer == buffer) A->spmm_buffer = nullptr, A->spmm_values_src = nullptr;
        }
        cudaError_t e = convert_structure(h->stream, A, v, L.plan, L.area);
        if (e != cudaSuccess) return from_cuda(e);
        if (!probed) {  // tile size for the transposed matrix: probed once (synchronises), then remembered
            kind = probe_tile_kind(h, t_ptr, t_idx, false, nnz, v.n, sizeof(T), L.work);
            std::lock_guard<std::mutex> g(A->lock);
            A->trans_probed_idx = v.idx;
            A->trans_probed_nnz = nnz;
            A->trans_tile_kind = kind;
        }
    }
    const SpmvWorkspace ws = spmv_workspace(v.n, nnz, sizeof(T), kind);
    if (!cached) {
        cudaError_t e = spmv_analysis(h->stream, v.n, nnz, 0, t_ptr, ws, L.work);
        if (e != cudaSuccess) return from_cuda(e);
        if (preprocess_only) {
            std::lock_guard<std::mutex> g(A->lock);
            A->trans_buffer = buffer;
            A->trans_ptr_src = v.ptr;
            A->trans_idx_src = v.idx;
            A->trans_nnz = nnz;
        }
    }
    if (preprocess_only) return OK;
    // The values are gathered through the permutation on every product (they may have been edited in place), unless
    // the caller promised to announce changes (mcsparseB200SpMatKeepConvertedValues) and this buffer already holds
    // the gathered values of this array.
    bool gather = true;
    {
        std::lock_guard<std::mutex> g(A->lock);
        gather = !(cached && A->keep_converted_values && A->trans_values_src == A->vals &&
                   A->trans_values_conj == v.conjugate);
        A->trans_values_src = nullptr;
    }
    cudaError_t e = cudaSuccess;
    if (gather) {
        e = transpose_values<T>(h->stream, nnz, static_cast<const T*>(A->vals), L.plan, L.area, v.conjugate);
        if (e != cudaSuccess) return from_cuda(e);
    }
    if (cached) {  // (without a recorded conversion the buffer is rebuilt by the next call anyway)
        std::lock_guard<std::mutex> g(A->lock);
        A->trans_values_src = A->vals;
        A->trans_values_conj = v.conjugate;
    }
    e = spmv_tiled<T, int32_t>(h->stream, v.n, nnz, 0, t_ptr, t_idx, t_val, static_cast<const T*>(X->values),
                               static_cast<T*>(Y->values), scalar_arg<T>(h, alpha), scalar_arg<T>(h, beta), ws, L.work,
                               PeerList<T>(), wait_cfg(h));
    return from_cuda(e);
}

St spmv_entry(mcsparseHandle_t h, mcsparseOperation_t opA, const void* alpha, mcsparseSpMatDescr_t A,
              mcsparseDnVecDescr_t X, const void* beta, mcsparseDnVecDescr_t Y, macaDataType computeType,
              void* buffer, bool preprocess_only, const PushArgs& push = PushArgs()) {
    St st = spmv_check(h, opA, alpha, A, X, beta, Y, computeType, true, buffer, false, nullptr, push.count == 0,
                       push.count == 0, push.count == 0);
    if (st != OK) return st;
    // mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:217-225
    const bool aos = A->format == MCSPARSE_FORMAT_COO_AOS;  // one index array (kept in `rows`)
    if (A->rows == nullptr || (A->cols == nullptr && !aos) || A->vals == nullptr || X->values == nullptr ||
        Y->values == nullptr || A->mat_descr == nullptr)
        return BAD_POINTER;
    if (!descr_general(A->mat_descr)) return NOT_IMPL;
    if (!preprocess_only && take_device_fault(h)) return EXEC_FAILED;
    DeviceGuard guard(h->device);
    if (aos) {
        const int64_t out_rows = opA == MCSPARSE_OPERATION_NON_TRANSPOSE ? A->row_num : A->col_num;
        CsrView probe;
        probe.m = A->row_num + A->col_num - out_rows, probe.n = out_rows;
        char* tail = static_cast<char*>(align_up_256(buffer)) + transposed_buffer_bytes(probe, A->nnz, value_size(computeType));
        int32_t* split_rows = reinterpret_cast<int32_t*>(tail);
        int32_t* split_cols = reinterpret_cast<int32_t*>(tail + ((size_t(A->nnz) * 4 + 255) & ~size_t(255)));
        cudaError_t e = split_index_pairs(h->stream, A->nnz, static_cast<const int32_t*>(A->rows), split_rows, split_cols);
        if (e != cudaSuccess) return from_cuda(e);
        const CsrView view = aos_view(A, opA, split_rows, split_cols);
        switch (computeType) {
            case MACA_R_64F: return spmv_transposed_run<double>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            case MACA_C_32F: return spmv_transposed_run<cfloat>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            case MACA_C_64F: return spmv_transposed_run<cdouble>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            default: return spmv_transposed_run<float>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
        }
    }
    if (const MixedKind low = low_precision_kind(A->valueType, X->valueType, Y->valueType, computeType);
        low != MixedKind::kNone) {
        // Same merge-path partition as the fp32 kernels' small tile, recorded by preprocess in the same way.
        SpmvWorkspace ws = spmv_mixed_workspace(A->row_num, A->nnz);
        void* buf = align_up_256(buffer);
        // scattered columns and rows of very different lengths: every tile takes the merge walk
        ws.walk = (choose_tile_kind(h, A, A->rows, A->cols, A->row_num, buf) & kTileWalk) != 0;
        bool analyse = true;
        {
            std::lock_guard<std::mutex> g(A->lock);
            if (A->trans_buffer == buffer) A->trans_buffer = nullptr, A->trans_values_src = nullptr;
            if (A->spmm_buffer == buffer) A->spmm_buffer = nullptr, A->spmm_values_src = nullptr;  // (the panels too)
            if (preprocess_only) {
                A->analysed_buffer = buffer;
                A->analysed_rows = A->rows;
                A->analysed_items_per_tile = ws.items_per_tile;
            } else if (A->analysed_buffer == buffer && A->analysed_rows == A->rows &&
                       A->analysed_items_per_tile == ws.items_per_tile) {
                analyse = false;
            }
        }
        const int32_t* rp = static_cast<const int32_t*>(A->rows);
        if (analyse) {
            const cudaError_t e = spmv_analysis(h->stream, A->row_num, A->nnz, A->mat_descr->base, rp, ws, buf);
            if (e != cudaSuccess) return from_cuda(e);
        }
        if (preprocess_only) return OK;
        return from_cuda(spmv_mixed(h->stream, low, A->row_num, A->mat_descr->base, rp, static_cast<const int32_t*>(A->cols),
                                    A->vals, X->values, Y->values, scalar_arg<float>(h, alpha), scalar_arg<float>(h, beta),
                                    scalar_arg<int>(h, alpha), scalar_arg<int>(h, beta), ws, buf));
    }
    if (real_matrix_complex_vectors(A->valueType, X->valueType, Y->valueType, computeType)) {
        if (preprocess_only) return OK;  // nothing to record: the buffer only holds the intermediate product
        void* z = align_up_256(buffer);
        const int32_t *rp = static_cast<const int32_t*>(A->rows), *ci = static_cast<const int32_t*>(A->cols);
        if (computeType == MACA_C_64F)
            return from_cuda(spmv_real_matrix_complex_vectors<double>(
                h->stream, A->row_num, A->mat_descr->base, rp, ci, static_cast<const double*>(A->vals),
                static_cast<const cdouble*>(X->values), static_cast<cdouble*>(Y->values), scalar_arg<cdouble>(h, alpha),
                scalar_arg<cdouble>(h, beta), static_cast<cdouble*>(z)));
        return from_cuda(spmv_real_matrix_complex_vectors<float>(
            h->stream, A->row_num, A->mat_descr->base, rp, ci, static_cast<const float*>(A->vals),
            static_cast<const cfloat*>(X->values), static_cast<cfloat*>(Y->values), scalar_arg<cfloat>(h, alpha),
            scalar_arg<cfloat>(h, beta), static_cast<cfloat*>(z)));
    }
    const CsrView view = csr_view(h, A, opA);
    if (view.converted()) {
        switch (computeType) {
            case MACA_R_64F: return spmv_transposed_run<double>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            case MACA_C_32F: return spmv_transposed_run<cfloat>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            case MACA_C_64F: return spmv_transposed_run<cdouble>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
            default: return spmv_transposed_run<float>(h, A, view, X, Y, alpha, beta, buffer, preprocess_only);
        }
    }
    // (a COO matrix has row indices, not offsets, in view.ptr: its row lengths are not sampled)
    const int small = choose_tile_kind(h, A, A->format == MCSPARSE_FORMAT_COO ? nullptr : view.ptr, view.idx, view.m,
                                       align_up_256(buffer));
    const int ipt = spmv_workspace(view.m, A->nnz, value_size(computeType), small, index_size(A)).items_per_tile;
    bool analyse = true;
    {
        std::lock_guard<std::mutex> g(A->lock);
        if (A->spmm_buffer == buffer) A->spmm_buffer = nullptr, A->spmm_values_src = nullptr;  // SpMM panels recorded here are gone
        if (A->trans_buffer == buffer) {  // the buffer changes hands: a later A^T product reconverts
            A->trans_buffer = nullptr;
            A->trans_values_src = nullptr;
        }
        if (preprocess_only) {
            A->analysed_buffer = buffer;
            A->analysed_rows = view.ptr;
            A->analysed_items_per_tile = ipt;
        } else if (A->analysed_buffer == buffer && A->analysed_rows == view.ptr &&
                   A->analysed_items_per_tile == ipt) {
            analyse = false;
        }
    }
    const bool wide = index_size(A) == 8;
    if (A->format == MCSPARSE_FORMAT_CSC && view.conjugate) {  // complex values only (view.conjugate says so)
        if (computeType == MACA_C_32F)
            return wide ? spmv_csc_conjugate_run<float, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small)
                        : spmv_csc_conjugate_run<float, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small);
        return wide ? spmv_csc_conjugate_run<double, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small)
                    : spmv_csc_conjugate_run<double, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small);
    }
    if (computeType == MACA_C_32F)
        return wide ? spmv_run<cfloat, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push)
                    : spmv_run<cfloat, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push);
    if (computeType == MACA_C_64F)
        return wide ? spmv_run<cdouble, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push)
                    : spmv_run<cdouble, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push);
    if (computeType == MACA_R_64F)
        return wide ? spmv_run<double, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push)
                    : spmv_run<double, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push);
    return wide ? spmv_run<float, int64_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push)
                : spmv_run<float, int32_t>(h, A, view, X, Y, alpha, beta, buffer, analyse, !preprocess_only, small, push);
}

// Legacy csrmv family: raw arrays plus a matrix descriptor
// (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:203-259 is the shared template).
template <typename T>
St csrmv_entry(mcsparseHandle_t h, mcsparseOperation_t transA, int m, int n, int nnz, const T* alpha,
               const mcsparseMatDescr_t descr, const T* vals, const int* rows, const int* cols, const T* x,
               const T* beta, T* y, void* buffer, bool has_buffer) {
    if (h == nullptr) return BAD_HANDLE;
    if (nnz < 0 || m < 0 || n < 0) return BAD_SIZE;
    if (alpha == nullptr || beta == nullptr || rows == nullptr || cols == nullptr || vals == nullptr ||
        x == nullptr || y == nullptr || descr == nullptr)
        return BAD_POINTER;
    if (!descr_general(descr)) return NOT_IMPL;
    if (transA != MCSPARSE_OPERATION_NON_TRANSPOSE) return NOT_IMPL;
    if (too_big(int64_t(m) + nnz)) return NOT_IMPL;
    DeviceGuard guard(h->device);
    const ScalarArg<T> a = scalar_arg<T>(h, alpha), b = scalar_arg<T>(h, beta);
    if (has_buffer) {
        if (buffer == nullptr) return BAD_POINTER;
        const SpmvWorkspace ws = spmv_workspace(m, nnz, sizeof(T));
        void* buf = align_up_256(buffer);
        cudaError_t e = spmv_analysis(h->stream, m, nnz, descr->base, rows, ws, buf);
        if (e != cudaSuccess) return from_cuda(e);
        return from_cuda(spmv_tiled<T, int32_t>(h->stream, m, nnz, descr->base, rows, cols, vals, x, y, a, b, ws, buf,
                                                PeerList<T>(), wait_cfg(h)));
    }
    return from_cuda(spmv_rowgroup<T>(h->stream, m, nnz, descr->base, rows, cols, vals, x, y, a, b));
}

// ----------------------------------------------------------------------------- SpMM

// mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:789-807 (compute) and :314-331 (bufferSize).
St spmm_check(mcsparseHandle_t h, mcsparseOperation_t opA, mcsparseOperation_t opB, const void* alpha,
              mcsparseSpMatDescr_t A, mcsparseDnMatDescr_t B, const void* beta, mcsparseDnMatDescr_t C,
              macaDataType computeType, bool need_buffer, const void* buffer) {
    if (h == nullptr) return BAD_HANDLE;
    if (A == nullptr || B == nullptr || C == nullptr || alpha == nullptr || beta == nullptr) return BAD_POINTER;
    if (need_buffer && buffer == nullptr) return BAD_POINTER;
    // Matched index pairs only (mcsp_spmm_gpu.cpp:954-960); extents must fit 31 bits either way.
    if (!((A->rowIdxType == MCSPARSE_INDEX_32I && A->colIdxType == MCSPARSE_INDEX_32I) ||
          (A->rowIdxType == MCSPARSE_INDEX_64I && A->colIdxType == MCSPARSE_INDEX_64I)))
        return NOT_IMPL;
    if (too_big(A->row_num) || too_big(A->col_num) || too_big(A->nnz) || too_big(B->row_num) ||
        too_big(B->col_num) || too_big(B->ld) || too_big(C->row_num) || too_big(C->col_num) || too_big(C->ld))
        return NOT_IMPL;
    // CSR runs as it is; a row-sorted COO or a CSC matrix is converted into the external buffer on every call
    // (one product), as the reference does for CSC (mcsp_spmm_gpu.cpp:818-848).
    if (!(A->format == MCSPARSE_FORMAT_CSR || A->format == MCSPARSE_FORMAT_COO || A->format == MCSPARSE_FORMAT_CSC))
        return NOT_IMPL;
    if (A->format != MCSPARSE_FORMAT_CSR && A->batchCount != 1) return NOT_IMPL;
    if (!(computeType == A->valueType && computeType == C->valueType && computeType == B->valueType)) return NOT_IMPL;
    if (!is_compute_type(computeType)) return NOT_IMPL;
    if (opA != MCSPARSE_OPERATION_NON_TRANSPOSE) return NOT_IMPL;  // :105
    if (opB == MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE) return NOT_IMPL;
    // Shapes: op(B) is A.cols x C.cols, C is A.rows x C.cols. The reference trusts the caller
    // here; an inconsistent set would read out of bounds, so it is rejected instead.
    const bool tB = opB == MCSPARSE_OPERATION_TRANSPOSE;
    const int64_t opb_rows = tB ? B->col_num : B->row_num, opb_cols = tB ? B->row_num : B->col_num;
    if (opb_rows != A->col_num || opb_cols != C->col_num || C->row_num != A->row_num) return BAD_SIZE;
    if (!(C->batchCount == A->batchCount && C->batchCount == B->batchCount)) return BAD_SIZE;
    if (B->ld < (B->order == MCSPARSE_ORDER_ROW ? B->col_num : B->row_num)) return BAD_SIZE;
    if (C->ld < (C->order == MCSPARSE_ORDER_ROW ? C->col_num : C->row_num)) return BAD_SIZE;
    return OK;
}

// True when B (as op(B)) and C are both addressed row-major with unit column stride: the layout the
// vectorised and column-panel kernels handle.
bool spmm_row_major(mcsparseOperation_t opB, const mcsparseDnMatDescr* B, const mcsparseDnMatDescr* C) {
    const bool b_row = (B->order == MCSPARSE_ORDER_ROW) != (opB == MCSPARSE_OPERATION_TRANSPOSE);
    return b_row && C->order == MCSPARSE_ORDER_ROW;
}

SpmmPlan spmm_plan_for(mcsparseOperation_t opB, const mcsparseSpMatDescr* A, const mcsparseDnMatDescr* B,
                       const mcsparseDnMatDescr* C, macaDataType computeType) {
    if (A->format != MCSPARSE_FORMAT_CSR) return SpmmPlan();  // converted inputs run in one pass
    return spmm_plan(A->row_num, A->col_num, C->col_num, A->nnz, value_size(computeType), spmm_row_major(opB, B, C));
}

// Bytes a COO or CSC input adds to the SpMM buffer, and where that area starts.
size_t spmm_conversion_bytes(const mcsparseSpMatDescr* A, size_t vsize, bool coo_sort) {
    if (A->format == MCSPARSE_FORMAT_COO && coo_sort) return transpose_plan(A->col_num, A->row_num, A->nnz, vsize).bytes + 256;
    if (A->format == MCSPARSE_FORMAT_COO) return ((size_t(A->row_num) + 1) * 4 + 255 + 256) & ~size_t(255);
    if (A->format == MCSPARSE_FORMAT_CSC) return transpose_plan(A->col_num, A->row_num, A->nnz, vsize).bytes + 256;
    return 0;
}

template <typename T, typename I>
St spmm_run(mcsparseContext* h, mcsparseOperation_t opB, mcsparseSpMatDescr* A, mcsparseDnMatDescr* B,
            mcsparseDnMatDescr* C, const void* alpha, const void* beta, const SpmmPlan* plan, void* plan_buffer,
            void* conversion_area) {
    if (A->format != MCSPARSE_FORMAT_CSR) {
        // Convert into the buffer, then the CSR kernels on the (always 32-bit) result: a row-sorted 32-bit COO only
        // needs row offsets; any other COO is sorted by row; CSC (= CSR of the transposed matrix) is transposed.
        void* area = align_up_256(conversion_area);
        const int32_t *rows = nullptr, *cols = nullptr;
        const T* vals = static_cast<const T*>(A->vals);
        int base = A->mat_descr->base;
        cudaError_t e = cudaSuccess;
        const bool coo = A->format == MCSPARSE_FORMAT_COO;
        if (coo && sizeof(I) == 4 && !coo_unsorted(h, A)) {
            int32_t* offsets = static_cast<int32_t*>(area);
            e = coo_row_offsets(h->stream, A->row_num, A->nnz, base, static_cast<const int32_t*>(A->rows), offsets);
            rows = offsets;
            cols = static_cast<const int32_t*>(A->cols);
        } else {
            const TransposePlan plan = transpose_plan(A->col_num, A->row_num, A->nnz, sizeof(T));
            e = coo ? coo_sort_structure<I>(h->stream, A->row_num, A->nnz, base, static_cast<const I*>(A->rows),
                                            static_cast<const I*>(A->cols), plan, area)
                    : transpose_structure<I>(h->stream, A->col_num, A->row_num, A->nnz, base,
                                             static_cast<const I*>(A->cols), static_cast<const I*>(A->rows), plan, area);
            if (e == cudaSuccess) e = transpose_values<T>(h->stream, A->nnz, vals, plan, area);
            const char* a = static_cast<const char*>(area);
            rows = reinterpret_cast<const int32_t*>(a + plan.off_ptr);
            cols = reinterpret_cast<const int32_t*>(a + plan.off_keys[plan.col_slot()]);
            vals = reinterpret_cast<const T*>(a + plan.off_val);
            base = 0;
        }
        if (e != cudaSuccess) return from_cuda(e);
        int64_t b_rs = B->order == MCSPARSE_ORDER_ROW ? B->ld : 1, b_cs = B->order == MCSPARSE_ORDER_ROW ? 1 : B->ld;
        if (opB == MCSPARSE_OPERATION_TRANSPOSE) std::swap(b_rs, b_cs);
        const int64_t c_rs = C->order == MCSPARSE_ORDER_ROW ? C->ld : 1, c_cs = C->order == MCSPARSE_ORDER_ROW ? 1 : C->ld;
        return from_cuda(spmm<T, int32_t>(h->stream, A->row_num, C->col_num, base, rows, cols, vals,
                                          static_cast<const T*>(B->values), b_rs, b_cs, static_cast<T*>(C->values), c_rs,
                                          c_cs, scalar_arg<T>(h, alpha), scalar_arg<T>(h, beta)));
    }
    int64_t b_rs = B->order == MCSPARSE_ORDER_ROW ? B->ld : 1, b_cs = B->order == MCSPARSE_ORDER_ROW ? 1 : B->ld;
    if (opB == MCSPARSE_OPERATION_TRANSPOSE) std::swap(b_rs, b_cs);
    const int64_t c_rs = C->order == MCSPARSE_ORDER_ROW ? C->ld : 1, c_cs = C->order == MCSPARSE_ORDER_ROW ? 1 : C->ld;
    // Strided batch: the same product on operands batchStride elements apart, one launch sequence per batch
    // (the column panels, built for batch 0's structure, are used only for a single product).
    for (int64_t b = 0; b < C->batchCount; ++b) {
        const bool single = C->batchCount == 1;
        cudaError_t e = spmm<T, I>(h->stream, A->row_num, C->col_num, A->mat_descr->base,
                                static_cast<const I*>(A->rows) + b * A->offsetsBatchStride,
                                static_cast<const I*>(A->cols) + b * A->batchStride,
                                static_cast<const T*>(A->vals) + b * A->batchStride,
                                static_cast<const T*>(B->values) + b * B->batchStride, b_rs, b_cs,
                                static_cast<T*>(C->values) + b * C->batchStride, c_rs, c_cs, scalar_arg<T>(h, alpha),
                                scalar_arg<T>(h, beta), single ? plan : nullptr, single ? plan_buffer : nullptr);
        if (e != cudaSuccess) return from_cuda(e);
    }
    return OK;
}

// Legacy csrmm / csrmm2: column-major B and C (mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:19-80).
template <typename T>
St csrmm_entry(mcsparseHandle_t h, mcsparseOperation_t transA, mcsparseOperation_t transB, int m, int n, int k,
               int nnz, const T* alpha, const mcsparseMatDescr_t descr, const T* vals, const int* rows,
               const int* cols, const T* B, int ldb, const T* beta, T* C, int ldc) {
    if (h == nullptr) return BAD_HANDLE;
    if (m < 0 || n < 0 || k < 0 || nnz < 0) return BAD_SIZE;
    if (alpha == nullptr || beta == nullptr || vals == nullptr || rows == nullptr || cols == nullptr ||
        B == nullptr || C == nullptr || descr == nullptr)
        return BAD_POINTER;
    if (transA != MCSPARSE_OPERATION_NON_TRANSPOSE || !descr_general(descr)) return NOT_IMPL;
    if (transB == MCSPARSE_OPERATION_CONJUGATE_TRANSPOSE) return NOT_IMPL;
    DeviceGuard guard(h->device);
    int64_t b_rs = 1, b_cs = ldb;
    if (transB == MCSPARSE_OPERATION_TRANSPOSE) std::swap(b_rs, b_cs);
    return from_cuda(spmm<T, int32_t>(h->stream, m, n, descr->base, rows, cols, vals, B, b_rs, b_cs, C, 1, ldc,
                             scalar_arg<T>(h, alpha), scalar_arg<T>(h, beta)));
}

// How mcsparseB200SpMVPush moves finished rows to the peers. Measured on B200 / NVSwitch (27-point stencil,
// ms per step at 2 / 4 / 8 GPUs): with one peer, computing the tiles in 4 launches and copying each chunk's rows
// with the copy engines while the next chunk computes is fastest (0.577 against 0.625); with more peers the copy
// engines fall behind (0.418 at 4 GPUs, 0.54 at 8) and the single launch whose push crew moves the rows with bulk
// copies wins (0.339 at 4 GPUs, 0.239 at 8). MCSPARSE_B200_PUSH_CHUNKS overrides the choice (0 ... 8: 0 is the
// single launch), read on every call.
int push_chunks_setting(int num_peers) {
    const char* e = std::getenv("MCSPARSE_B200_PUSH_CHUNKS");
    const int c = e ? std::atoi(e) : (num_peers <= 1 ? 4 : 0);
    return c < 0 ? 0 : (c > kMaxPushChunks ? kMaxPushChunks : c);
}

template <typename T>
St spmv_push_pipelined(mcsparseContext* h, mcsparseSpMatDescr* A, mcsparseDnVecDescr* X,
                              mcsparseDnVecDescr* Y, const void* alpha, const void* beta, void* buffer,
                              const PushArgs& push, int chunks) {
    void* buf = align_up_256(buffer);
    const SpmvWorkspace ws = spmv_workspace(A->row_num, A->nnz, sizeof(T), choose_tile_kind(h, A, A->rows, A->cols, A->row_num, buf));
    const int base = A->mat_descr->base;
    const int32_t* rows = static_cast<const int32_t*>(A->rows);
    if (h->side_stream == nullptr) {
        // Highest priority: as CTAs of the running tile kernel retire, the block scheduler places the
        // waiting copy CTAs first, so the copy really runs beside the next chunk instead of after it.
        int least = 0, greatest = 0;
        cudaDeviceGetStreamPriorityRange(&least, &greatest);
        if (cudaStreamCreateWithPriority(&h->side_stream, cudaStreamNonBlocking, greatest) != cudaSuccess)
            return INTERNAL;
        for (auto& ev : h->events)
            if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return INTERNAL;
        for (auto& ev : h->fix_events)
            if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return INTERNAL;
        for (auto& ev : h->peer_events)
            if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return INTERNAL;
        for (auto& st : h->peer_streams)
            if (cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, greatest) != cudaSuccess) return INTERNAL;
        if (cudaStreamCreateWithFlags(&h->capture_stream, cudaStreamNonBlocking) != cudaSuccess) return INTERNAL;
    }
    {
        std::lock_guard<std::mutex> g(A->lock);
        if (!(A->push_buffer == buffer && A->push_rows_ptr == A->rows && A->push_chunks == chunks &&
              A->analysed_items_per_tile == ws.items_per_tile)) {
            // First use with this buffer: analyse, then read back where each chunk of tiles starts.
            cudaError_t e = spmv_analysis(h->stream, A->row_num, A->nnz, base, rows, ws, buf);
            if (e != cudaSuccess) return from_cuda(e);
            for (int c = 0; c <= chunks; ++c) A->push_chunk_tiles[c] = ws.num_tiles * c / chunks;
            e = spmv_read_tile_rows(h->stream, buf, chunks + 1, A->push_chunk_tiles, A->push_chunk_rows);
            if (e != cudaSuccess) return from_cuda(e);
            A->push_buffer = buffer;
            A->push_rows_ptr = A->rows;
            A->push_chunks = chunks;
            A->analysed_buffer = buffer;
            A->analysed_rows = A->rows;
            A->analysed_items_per_tile = ws.items_per_tile;
        }
    }
    PeerList<T> peers;
    peers.count = push.count;
    peers.row_offset = push.row_offset;
    for (int p = 0; p < push.count; ++p) peers.y[p] = static_cast<T*>(push.y[p]);
    PushStreams ps;
    ps.peer_streams = h->peer_streams;
    ps.fix_events = h->fix_events;
    ps.peer_events = h->peer_events;
    const ScalarArg<T> a = scalar_arg<T>(h, alpha), b = scalar_arg<T>(h, beta);
    auto enqueue = [&](cudaStream_t origin) {
        return spmv_tiled_pipelined<T>(origin, h->side_stream, h->events, ps, chunks, A->push_chunk_tiles,
                                       A->push_chunk_rows, A->row_num, A->nnz, base, rows,
                                       static_cast<const int32_t*>(A->cols), static_cast<const T*>(A->vals),
                                       static_cast<const T*>(X->values), static_cast<T*>(Y->values), a, b, ws, buf, peers,
                                       wait_cfg(h));
    };
    // A step is some forty stream operations (launches, copies, event records and waits); issued one
    // by one they cost more host time than the step takes on the GPUs. So the sequence is captured as
    // a graph the first time and replayed with one call while nothing it depends on has changed
    // (MCSPARSE_B200_PUSH_GRAPH=0 issues it directly; so does a stream that is itself being captured).
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(h->stream, &capturing);
    const char* genv = std::getenv("MCSPARSE_B200_PUSH_GRAPH");
    if (capturing != cudaStreamCaptureStatusNone || (genv != nullptr && genv[0] == '0'))
        return from_cuda(enqueue(h->stream));

    struct Key {
        const void *rows, *cols, *vals, *x, *y, *buf, *stream;
        void* peers[PeerList<T>::kMax];
        long long row_offset, m, nnz;
        double alpha_host, beta_host;
        const void *alpha_dev, *beta_dev;
        int chunks, count, items_per_tile, base, value_bytes;
    } key;
    static_assert(sizeof(Key) <= sizeof(A->push_graphs[0].key), "key buffer too small");
    std::memset(&key, 0, sizeof key);
    key.rows = rows, key.cols = A->cols, key.vals = A->vals, key.x = X->values, key.y = Y->values, key.buf = buf;
    key.stream = h->stream;
    for (int p = 0; p < push.count; ++p) key.peers[p] = push.y[p];
    key.row_offset = push.row_offset, key.m = A->row_num, key.nnz = A->nnz;
    key.alpha_host = (double)a.host, key.beta_host = (double)b.host, key.alpha_dev = a.dev, key.beta_dev = b.dev;
    key.chunks = chunks, key.count = push.count, key.items_per_tile = ws.items_per_tile, key.base = base;
    key.value_bytes = (int)sizeof(T);
    std::lock_guard<std::mutex> g(A->lock);
    mcsparseSpMatDescr::PushGraph* slot = nullptr;
    for (auto& cand : A->push_graphs)
        if (cand.exec != nullptr && cand.key_bytes == sizeof key && std::memcmp(cand.key, &key, sizeof key) == 0)
            slot = &cand;
    if (slot == nullptr) {
        slot = &A->push_graphs[0];  // an empty slot, else the least recently used one
        for (auto& cand : A->push_graphs)
            if (cand.exec == nullptr || (slot->exec != nullptr && cand.last_use < slot->last_use)) {
                slot = &cand;
                if (cand.exec == nullptr) break;
            }
        if (slot->exec != nullptr) {
            cudaGraphExecDestroy(slot->exec);
            slot->exec = nullptr;
        }
        cudaGraph_t graph = nullptr;
        // Captured from a stream of the handle's own: the caller's stream may be the legacy default
        // stream, which cannot be captured; the finished graph is launched on the caller's stream.
        cudaError_t e = cudaStreamBeginCapture(h->capture_stream, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) return from_cuda(e);
        const cudaError_t queued = enqueue(h->capture_stream);
        e = cudaStreamEndCapture(h->capture_stream, &graph);
        if (queued != cudaSuccess || e != cudaSuccess) {
            if (graph != nullptr) cudaGraphDestroy(graph);
            return from_cuda(queued != cudaSuccess ? queued : e);
        }
        e = cudaGraphInstantiate(&slot->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) {
            slot->exec = nullptr;
            return from_cuda(e);
        }
        std::memcpy(slot->key, &key, sizeof key);
        slot->key_bytes = sizeof key;
    }
    slot->last_use = ++A->push_graph_clock;
    return from_cuda(cudaGraphLaunch(slot->exec, h->stream));
}

// mcComplex / mcDoubleComplex and the kernels' complex types are both interleaved (re, im) pairs.
const cfloat* cx(const mcComplex* p) { return reinterpret_cast<const cfloat*>(p); }
cfloat* cx(mcComplex* p) { return reinterpret_cast<cfloat*>(p); }
const cdouble* cx(const mcDoubleComplex* p) { return reinterpret_cast<const cdouble*>(p); }
cdouble* cx(mcDoubleComplex* p) { return reinterpret_cast<cdouble*>(p); }

}  // namespace

extern "C" {

// ----------------------------------------------------------------------------- SpMV

mcsparseStatus_t mcsparseSpMV_bufferSize(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg, size_t* bufferSize) {
    (void)alg;
    St st = spmv_check(handle, opA, alpha, matA, vecX, beta, vecY, computeType, false, nullptr, true, bufferSize, true,
                       true, true);
    if (st != OK) return pub(st);
    // Work partition + carries, plus slack to align the caller's pointer to 256 bytes; a COO matrix
    // also needs room for the row offsets derived from its row indices.
    if (low_precision_kind(matA->valueType, vecX->valueType, vecY->valueType, computeType) != MixedKind::kNone) {
        *bufferSize = spmv_mixed_workspace(matA->row_num, matA->nnz).bytes + 256;  // (+ alignment slack)
        return MCSPARSE_STATUS_SUCCESS;
    }
    if (real_matrix_complex_vectors(matA->valueType, vecX->valueType, vecY->valueType, computeType)) {
        *bufferSize = size_t(matA->row_num) * value_size(computeType) + 512;  // the intermediate A * x
        return MCSPARSE_STATUS_SUCCESS;
    }
    if (matA->format == MCSPARSE_FORMAT_COO_AOS) {  // sort path + the two arrays the pairs are split into
        const CsrView v = aos_view(matA, opA, nullptr, nullptr);
        *bufferSize = 256 + transposed_buffer_bytes(v, matA->nnz, value_size(computeType)) +
                      2 * ((size_t(matA->nnz) * 4 + 255) & ~size_t(255)) + 256;
        return MCSPARSE_STATUS_SUCCESS;
    }
    const CsrView view = csr_view(handle, matA, opA);
    if (view.converted()) {  // work area of the converted matrix + the conversion area
        *bufferSize = transposed_buffer_bytes(view, matA->nnz, value_size(computeType));
        return MCSPARSE_STATUS_SUCCESS;
    }
    *bufferSize = spmv_workspace(view.m, matA->nnz, value_size(computeType), false, index_size(matA)).bytes + 256;
    if (matA->format == MCSPARSE_FORMAT_CSC && view.conjugate)  // conj(x) and the intermediate product
        *bufferSize += align256(size_t(view.n) * value_size(computeType)) + align256(size_t(view.m) * value_size(computeType));
    if (matA->format == MCSPARSE_FORMAT_COO) *bufferSize += ((size_t(matA->row_num) + 1) * 4 + 255) & ~size_t(255);
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMV_preprocess(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg, void* externalBuffer) {
    (void)alg;
    return pub(spmv_entry(handle, opA, alpha, matA, vecX, beta, vecY, computeType, externalBuffer, true));
}

mcsparseStatus_t mcsparseSpMV(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                              mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                              mcsparseDnVecDescr_t vecY, macaDataType computeType, mcsparseSpMVAlg_t alg,
                              void* externalBuffer) {
    (void)alg;
    return pub(spmv_entry(handle, opA, alpha, matA, vecX, beta, vecY, computeType, externalBuffer, false));
}

mcsparseStatus_t mcsparseB200SpMVPartitionView(mcsparseSpMatDescr_t matA, void* externalBuffer, int* itemsPerTile,
                                               int64_t* numTiles, const int32_t** tileStarts) {
    if (matA == nullptr || externalBuffer == nullptr || itemsPerTile == nullptr || numTiles == nullptr ||
        tileStarts == nullptr)
        return pub(BAD_POINTER);
    if (!is_compute_type(matA->valueType)) return pub(NOT_IMPL);
    const SpmvWorkspace ws =
        spmv_workspace(matA->row_num, matA->nnz, value_size(matA->valueType), known_tile_kind(matA), index_size(matA));
    *itemsPerTile = ws.items_per_tile;
    *numTiles = ws.num_tiles;
    *tileStarts = static_cast<const int32_t*>(align_up_256(externalBuffer));
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseB200SpMVGetStatus(mcsparseHandle_t handle, mcsparseSpMatDescr_t matA,
                                           void* externalBuffer, int* status) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (matA == nullptr || status == nullptr) return pub(BAD_POINTER);
    if (!is_compute_type(matA->valueType)) return pub(NOT_IMPL);
    DeviceGuard guard(handle->device);
    void* area = externalBuffer;
    if (area == nullptr) {  // the built-in work area of mcsparseB200SpMVNoAlloc
        size_t bytes = 0;
        const cudaError_t e = spmv_static_scratch(&area, &bytes);
        if (e != cudaSuccess) return pub(from_cuda(e));
    }
    const SpmvWorkspace ws =
        spmv_workspace(matA->row_num, matA->nnz, value_size(matA->valueType), known_tile_kind(matA), index_size(matA));
    const char* word = static_cast<const char*>(align_up_256(area)) + ws.off_status;
    cudaError_t e = cudaMemcpyAsync(status, word, sizeof(int), cudaMemcpyDeviceToHost, handle->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(handle->stream);
    return pub(from_cuda(e));
}

mcsparseStatus_t mcsparseB200SpMVTransposedView(mcsparseSpMatDescr_t matA, mcsparseOperation_t opA,
                                                void* externalBuffer, int64_t* rows, const int32_t** rowOffsets,
                                                const int32_t** colInd, const void** values) {
    if (matA == nullptr || externalBuffer == nullptr || rows == nullptr || rowOffsets == nullptr || colInd == nullptr ||
        values == nullptr)
        return pub(BAD_POINTER);
    if (!is_compute_type(matA->valueType)) return pub(NOT_IMPL);
    const CsrView view = csr_view(nullptr, matA, opA);  // no handle here: a COO's order as found by its last product
    if (!view.converted()) return pub(BAD_VALUE);
    const TransposedLayout L = transposed_layout(view, matA->nnz, value_size(matA->valueType), externalBuffer);
    const char* area = static_cast<const char*>(L.area);
    *rows = view.n;
    *rowOffsets = reinterpret_cast<const int32_t*>(area + L.plan.off_ptr);
    *colInd = reinterpret_cast<const int32_t*>(area + L.plan.off_keys[L.plan.col_slot()]);
    *values = area + L.plan.off_val;
    return MCSPARSE_STATUS_SUCCESS;
}

// SpMV for callers that may not allocate device memory: same arithmetic and kernels as
// mcsparseSpMV, with the work area taken from the fixed array inside the library instead of an
// external buffer. Nothing here (or below it) allocates. The analysis is redone on every call
// because the shared work area may have been used for another matrix in between.
mcsparseStatus_t mcsparseB200SpMVNoAlloc(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg) {
    (void)alg;
    St st = spmv_check(handle, opA, alpha, matA, vecX, beta, vecY, computeType, false, nullptr, false, nullptr);
    if (st != OK) return pub(st);
    if (matA->rows == nullptr || matA->cols == nullptr || matA->vals == nullptr || vecX->values == nullptr ||
        vecY->values == nullptr || matA->mat_descr == nullptr)
        return pub(BAD_POINTER);
    if (!descr_general(matA->mat_descr)) return pub(NOT_IMPL);
    if (take_device_fault(handle)) return pub(EXEC_FAILED);
    DeviceGuard guard(handle->device);
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    cudaError_t e = spmv_static_scratch(&scratch, &scratch_bytes);
    if (e != cudaSuccess) return pub(from_cuda(e));
    if (spmv_workspace(matA->row_num, matA->nnz, value_size(computeType)).bytes > scratch_bytes) {
        const SpmvWorkspace ws = spmv_workspace(matA->row_num, matA->nnz, value_size(computeType));
        char msg[200];
        std::snprintf(msg, sizeof msg,
                      "mcsparseB200SpMVNoAlloc: matrix needs %zu bytes of work area, the built-in one has %zu; "
                      "use mcsparseSpMV with an external buffer",
                      ws.bytes, scratch_bytes);
        log_error(msg);
        return MCSPARSE_STATUS_INSUFFICIENT_RESOURCES;
    }
    // No probe here: the locality probe copies a word back and synchronises the stream, which this entry
    // point must not do. A matrix that an earlier mcsparseSpMV / mcsparseSpMV_preprocess call already
    // probed keeps its choice; any other gets the default kernel and tile size.
    const SpmvWorkspace ws = spmv_workspace(matA->row_num, matA->nnz, value_size(computeType), known_tile_kind(matA));
    const int base = matA->mat_descr->base;
    const int32_t* rows = static_cast<const int32_t*>(matA->rows);
    e = spmv_analysis(handle->stream, matA->row_num, matA->nnz, base, rows, ws, scratch);
    if (e != cudaSuccess) return pub(from_cuda(e));
    if (computeType == MACA_R_64F)
        e = spmv_tiled<double, int32_t>(handle->stream, matA->row_num, matA->nnz, base, rows,
                               static_cast<const int32_t*>(matA->cols), static_cast<const double*>(matA->vals),
                               static_cast<const double*>(vecX->values), static_cast<double*>(vecY->values),
                               scalar_arg<double>(handle, alpha), scalar_arg<double>(handle, beta), ws, scratch,
                               PeerList<double>(), wait_cfg(handle));
    else
        e = spmv_tiled<float, int32_t>(handle->stream, matA->row_num, matA->nnz, base, rows,
                              static_cast<const int32_t*>(matA->cols), static_cast<const float*>(matA->vals),
                              static_cast<const float*>(vecX->values), static_cast<float*>(vecY->values),
                              scalar_arg<float>(handle, alpha), scalar_arg<float>(handle, beta), ws, scratch,
                              PeerList<float>(), wait_cfg(handle));
    return pub(from_cuda(e));
}

mcsparseStatus_t mcsparseB200GatherProbe(mcsparseHandle_t handle, const int32_t* indices, int64_t count, const void* table,
                                         int elemBytes, void* partialSums, int blocks) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (indices == nullptr || table == nullptr || partialSums == nullptr) return pub(BAD_POINTER);
    if (count < 0 || blocks < 1 || (elemBytes != 4 && elemBytes != 8)) return pub(BAD_VALUE);
    if ((reinterpret_cast<uintptr_t>(indices) & 15) != 0) return pub(BAD_VALUE);
    DeviceGuard guard(handle->device);
    return pub(from_cuda(gather_probe(handle->stream, indices, count, table, elemBytes, partialSums, blocks)));
}

mcsparseStatus_t mcsparseB200SetDeviceWaitLimit(mcsparseHandle_t handle, int64_t smClocks, int withholdCopies) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (smClocks < 1) return pub(BAD_VALUE);
    handle->wait_cycles = smClocks;
    handle->withhold_copies = withholdCopies != 0;
    return MCSPARSE_STATUS_SUCCESS;
}

// ----------------------------------------------------------------------------- SpMM

mcsparseStatus_t mcsparseSpMM_bufferSize(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                                         const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                                         const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                                         mcsparseSpMMAlg_t alg, size_t* bufferSize) {
    (void)alg;
    St st = spmm_check(handle, opA, opB, alpha, matA, matB, beta, matC, computeType, false, nullptr);
    if (st != OK) return pub(st);
    if (bufferSize == nullptr) return pub(BAD_POINTER);
    // 128 is MIN_BUFFER_SIZE of the reference (mcsparse/src/include/mcsp_config.h:11-15); a B too large
    // for L2 adds the per-row panel offsets that mcsparseSpMM_preprocess computes.
    *bufferSize = spmm_plan_for(opB, matA, matB, matC, computeType).bytes +
                  spmm_conversion_bytes(matA, value_size(computeType),
                                        index_size(matA) == 8 || coo_unsorted(handle, matA));
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMM_preprocess(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                                         const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                                         const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                                         mcsparseSpMMAlg_t alg, void* externalBuffer) {
    // The reference returns success without looking at any argument
    // (mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:965-970). Here the call is optional too and never
    // fails: when the arguments describe a row-major product whose B does not fit in L2, it computes the
    // column-panel offsets into externalBuffer and records them on matA; otherwise it does nothing.
    (void)alg;
    if (spmm_check(handle, opA, opB, alpha, matA, matB, beta, matC, computeType, true, externalBuffer) != OK)
        return MCSPARSE_STATUS_SUCCESS;
    if (matA->rows == nullptr || matA->cols == nullptr || matA->mat_descr == nullptr) return MCSPARSE_STATUS_SUCCESS;
    const SpmmPlan plan = spmm_plan_for(opB, matA, matB, matC, computeType);
    std::lock_guard<std::mutex> g(matA->lock);
    matA->spmm_buffer = nullptr;
    matA->spmm_values_src = nullptr;
    if (plan.num_panels <= 1) return MCSPARSE_STATUS_SUCCESS;
    // the buffer is about to hold the panels: what mcsparseSpMV recorded in it for this matrix is gone
    if (matA->analysed_buffer == externalBuffer) matA->analysed_buffer = nullptr;
    if (matA->push_buffer == externalBuffer) matA->push_buffer = nullptr;
    if (matA->trans_buffer == externalBuffer) matA->trans_buffer = nullptr, matA->trans_values_src = nullptr;
    DeviceGuard guard(handle->device);
    const cudaError_t e =
        matA->rowIdxType == MCSPARSE_INDEX_64I
            ? spmm_preprocess(handle->stream, matA->row_num, matA->nnz, matA->mat_descr->base,
                              static_cast<const int64_t*>(matA->rows), static_cast<const int64_t*>(matA->cols), plan,
                              align_up_256(externalBuffer))
            : spmm_preprocess(handle->stream, matA->row_num, matA->nnz, matA->mat_descr->base,
                              static_cast<const int32_t*>(matA->rows), static_cast<const int32_t*>(matA->cols), plan,
                              align_up_256(externalBuffer));
    if (e != cudaSuccess) return MCSPARSE_STATUS_SUCCESS;
    matA->spmm_buffer = externalBuffer;
    matA->spmm_rows = matA->rows;
    matA->spmm_cols = matA->cols;
    matA->spmm_panels = plan.num_panels;
    matA->spmm_lanes = plan.lanes;
    matA->spmm_n = matC->col_num;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseSpMM(mcsparseHandle_t handle, mcsparseOperation_t opA, mcsparseOperation_t opB,
                              const void* alpha, mcsparseSpMatDescr_t matA, mcsparseDnMatDescr_t matB,
                              const void* beta, mcsparseDnMatDescr_t matC, macaDataType computeType,
                              mcsparseSpMMAlg_t alg, void* externalBuffer) {
    (void)alg;
    St st = spmm_check(handle, opA, opB, alpha, matA, matB, beta, matC, computeType, true, externalBuffer);
    if (st != OK) return pub(st);
    if (matA->rows == nullptr || matA->cols == nullptr || matA->vals == nullptr || matB->values == nullptr ||
        matC->values == nullptr || matA->mat_descr == nullptr)
        return pub(BAD_POINTER);
    if (!descr_general(matA->mat_descr)) return pub(NOT_IMPL);
    DeviceGuard guard(handle->device);
    SpmmPlan plan = spmm_plan_for(opB, matA, matB, matC, computeType);
    const SpmmPlan* use_plan = nullptr;
    void* plan_buffer = nullptr;
    {
        std::lock_guard<std::mutex> g(matA->lock);
        if (matA->spmm_buffer == externalBuffer && matA->spmm_rows == matA->rows && matA->spmm_cols == matA->cols &&
            matA->spmm_n == matC->col_num && matA->spmm_panels == plan.num_panels && matA->spmm_lanes == plan.lanes &&
            plan.num_panels > 1) {
            use_plan = &plan;
            plan_buffer = align_up_256(externalBuffer);
            // The values are regrouped on every call, unless the caller promised to announce their changes and
            // the buffer holds these values from the last call (a single-matrix product; batches always regroup).
            plan.values_current = matA->keep_converted_values && matA->spmm_values_src == matA->vals && matA->batchCount <= 1;
            matA->spmm_values_src = (matA->keep_converted_values && matA->batchCount <= 1) ? matA->vals : nullptr;
        } else if (matA->spmm_buffer == externalBuffer) {
            matA->spmm_values_src = nullptr;
        }
        if (matA->format != MCSPARSE_FORMAT_CSR) {  // the conversion writes the buffer: SpMV records in it are gone
            if (matA->analysed_buffer == externalBuffer) matA->analysed_buffer = nullptr;
            if (matA->push_buffer == externalBuffer) matA->push_buffer = nullptr;
            if (matA->trans_buffer == externalBuffer) matA->trans_buffer = nullptr, matA->trans_values_src = nullptr;
        }
    }
    // A COO or CSC input is converted behind the (panel) plan's part of the buffer.
    void* conversion_area = static_cast<char*>(externalBuffer) + plan.bytes;
    const bool wide = index_size(matA) == 8;
    if (computeType == MACA_C_32F)
        return pub(wide ? spmm_run<cfloat, int64_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area)
                        : spmm_run<cfloat, int32_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area));
    if (computeType == MACA_C_64F)
        return pub(wide ? spmm_run<cdouble, int64_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area)
                        : spmm_run<cdouble, int32_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area));
    if (computeType == MACA_R_64F)
        return pub(wide ? spmm_run<double, int64_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area)
                        : spmm_run<double, int32_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area));
    return pub(wide ? spmm_run<float, int64_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area)
                    : spmm_run<float, int32_t>(handle, opB, matA, matB, matC, alpha, beta, use_plan, plan_buffer, conversion_area));
}

// ----------------------------------------------------------------------------- legacy entry points

mcsparseStatus_t mcsparseScsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const float* alpha, const mcsparseMatDescr_t descrA, const float* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const float* x, const float* beta,
                                float* y) {
    return pub(csrmv_entry<float>(handle, transA, m, n, nnz, alpha, descrA, csrValA, csrRowPtrA, csrColIndA, x, beta,
                                  y, nullptr, false));
}

mcsparseStatus_t mcsparseDcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const double* alpha, const mcsparseMatDescr_t descrA, const double* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const double* x, const double* beta,
                                double* y) {
    return pub(csrmv_entry<double>(handle, transA, m, n, nnz, alpha, descrA, csrValA, csrRowPtrA, csrColIndA, x,
                                   beta, y, nullptr, false));
}

mcsparseStatus_t mcsparseCcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const mcComplex* alpha, const mcsparseMatDescr_t descrA, const mcComplex* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const mcComplex* x,
                                const mcComplex* beta, mcComplex* y) {
    return pub(csrmv_entry<cfloat>(handle, transA, m, n, nnz, cx(alpha), descrA, cx(csrValA), csrRowPtrA, csrColIndA,
                                   cx(x), cx(beta), cx(y), nullptr, false));
}

mcsparseStatus_t mcsparseZcsrmv(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int nnz,
                                const mcDoubleComplex* alpha, const mcsparseMatDescr_t descrA,
                                const mcDoubleComplex* csrValA, const int* csrRowPtrA, const int* csrColIndA,
                                const mcDoubleComplex* x, const mcDoubleComplex* beta, mcDoubleComplex* y) {
    return pub(csrmv_entry<cdouble>(handle, transA, m, n, nnz, cx(alpha), descrA, cx(csrValA), csrRowPtrA, csrColIndA,
                                    cx(x), cx(beta), cx(y), nullptr, false));
}

static bool csrmvex_types_equal(macaDataType a, macaDataType v, macaDataType x, macaDataType b, macaDataType y,
                                macaDataType e) {
    return a == x && v == x && b == x && y == x && e == x;  // mcsp_spmv_gpu.cpp:911-914
}

mcsparseStatus_t mcsparseCsrmvEx_bufferSize(mcsparseHandle_t handle, mcsparseAlgMode_t alg,
                                            mcsparseOperation_t transA, int m, int n, int nnz, const void* alpha,
                                            macaDataType alphatype, const mcsparseMatDescr_t descrA,
                                            const void* csrValA, macaDataType csrValAtype, const int* csrRowPtrA,
                                            const int* csrColIndA, const void* x, macaDataType xtype,
                                            const void* beta, macaDataType betatype, void* y, macaDataType ytype,
                                            macaDataType executiontype, size_t* bufferSizeInBytes) {
    (void)alg; (void)transA; (void)n; (void)alpha; (void)descrA; (void)csrValA; (void)csrRowPtrA;
    (void)csrColIndA; (void)x; (void)beta; (void)y;
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (bufferSizeInBytes == nullptr) return pub(BAD_POINTER);
    if (m < 0 || nnz < 0) return pub(BAD_SIZE);
    if (!csrmvex_types_equal(alphatype, csrValAtype, xtype, betatype, ytype, executiontype) || !is_compute_type(xtype))
        return pub(NOT_IMPL);
    *bufferSizeInBytes = spmv_workspace(m, nnz, value_size(xtype)).bytes + 256;
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseCsrmvEx(mcsparseHandle_t handle, mcsparseAlgMode_t alg, mcsparseOperation_t transA, int m,
                                 int n, int nnz, const void* alpha, macaDataType alphatype,
                                 const mcsparseMatDescr_t descrA, const void* csrValA, macaDataType csrValAtype,
                                 const int* csrRowPtrA, const int* csrColIndA, const void* x, macaDataType xtype,
                                 const void* beta, macaDataType betatype, void* y, macaDataType ytype,
                                 macaDataType executiontype, void* buffer) {
    (void)alg;
    if (!csrmvex_types_equal(alphatype, csrValAtype, xtype, betatype, ytype, executiontype) || !is_compute_type(xtype))
        return pub(NOT_IMPL);
    if (xtype == MACA_C_32F)
        return pub(csrmv_entry<cfloat>(handle, transA, m, n, nnz, static_cast<const cfloat*>(alpha), descrA,
                                       static_cast<const cfloat*>(csrValA), csrRowPtrA, csrColIndA,
                                       static_cast<const cfloat*>(x), static_cast<const cfloat*>(beta),
                                       static_cast<cfloat*>(y), buffer, true));
    if (xtype == MACA_C_64F)
        return pub(csrmv_entry<cdouble>(handle, transA, m, n, nnz, static_cast<const cdouble*>(alpha), descrA,
                                        static_cast<const cdouble*>(csrValA), csrRowPtrA, csrColIndA,
                                        static_cast<const cdouble*>(x), static_cast<const cdouble*>(beta),
                                        static_cast<cdouble*>(y), buffer, true));
    if (xtype == MACA_R_64F)
        return pub(csrmv_entry<double>(handle, transA, m, n, nnz, static_cast<const double*>(alpha), descrA,
                                       static_cast<const double*>(csrValA), csrRowPtrA, csrColIndA,
                                       static_cast<const double*>(x), static_cast<const double*>(beta),
                                       static_cast<double*>(y), buffer, true));
    return pub(csrmv_entry<float>(handle, transA, m, n, nnz, static_cast<const float*>(alpha), descrA,
                                  static_cast<const float*>(csrValA), csrRowPtrA, csrColIndA,
                                  static_cast<const float*>(x), static_cast<const float*>(beta),
                                  static_cast<float*>(y), buffer, true));
}

mcsparseStatus_t mcsparseScsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const float* alpha, const mcsparseMatDescr_t descrA,
                                 const float* csrValA, const int* csrRowPtrA, const int* csrColIndA, const float* B,
                                 int ldb, const float* beta, float* C, int ldc) {
    return pub(csrmm_entry<float>(handle, transA, transB, m, n, k, nnz, alpha, descrA, csrValA, csrRowPtrA,
                                  csrColIndA, B, ldb, beta, C, ldc));
}

mcsparseStatus_t mcsparseDcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const double* alpha,
                                 const mcsparseMatDescr_t descrA, const double* csrValA, const int* csrRowPtrA,
                                 const int* csrColIndA, const double* B, int ldb, const double* beta, double* C,
                                 int ldc) {
    return pub(csrmm_entry<double>(handle, transA, transB, m, n, k, nnz, alpha, descrA, csrValA, csrRowPtrA,
                                   csrColIndA, B, ldb, beta, C, ldc));
}

mcsparseStatus_t mcsparseScsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const float* alpha, const mcsparseMatDescr_t descrA, const float* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const float* B, int ldb,
                                const float* beta, float* C, int ldc) {
    return pub(csrmm_entry<float>(handle, transA, MCSPARSE_OPERATION_NON_TRANSPOSE, m, n, k, nnz, alpha, descrA,
                                  csrValA, csrRowPtrA, csrColIndA, B, ldb, beta, C, ldc));
}

mcsparseStatus_t mcsparseDcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const double* alpha, const mcsparseMatDescr_t descrA, const double* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const double* B, int ldb,
                                const double* beta, double* C, int ldc) {
    return pub(csrmm_entry<double>(handle, transA, MCSPARSE_OPERATION_NON_TRANSPOSE, m, n, k, nnz, alpha, descrA,
                                   csrValA, csrRowPtrA, csrColIndA, B, ldb, beta, C, ldc));
}

mcsparseStatus_t mcsparseCcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const mcComplex* alpha,
                                 const mcsparseMatDescr_t descrA, const mcComplex* csrValA, const int* csrRowPtrA,
                                 const int* csrColIndA, const mcComplex* B, int ldb, const mcComplex* beta,
                                 mcComplex* C, int ldc) {
    return pub(csrmm_entry<cfloat>(handle, transA, transB, m, n, k, nnz, cx(alpha), descrA, cx(csrValA), csrRowPtrA,
                                   csrColIndA, cx(B), ldb, cx(beta), cx(C), ldc));
}

mcsparseStatus_t mcsparseZcsrmm2(mcsparseHandle_t handle, mcsparseOperation_t transA, mcsparseOperation_t transB,
                                 int m, int n, int k, int nnz, const mcDoubleComplex* alpha,
                                 const mcsparseMatDescr_t descrA, const mcDoubleComplex* csrValA,
                                 const int* csrRowPtrA, const int* csrColIndA, const mcDoubleComplex* B, int ldb,
                                 const mcDoubleComplex* beta, mcDoubleComplex* C, int ldc) {
    return pub(csrmm_entry<cdouble>(handle, transA, transB, m, n, k, nnz, cx(alpha), descrA, cx(csrValA), csrRowPtrA,
                                    csrColIndA, cx(B), ldb, cx(beta), cx(C), ldc));
}

mcsparseStatus_t mcsparseCcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const mcComplex* alpha, const mcsparseMatDescr_t descrA, const mcComplex* csrValA,
                                const int* csrRowPtrA, const int* csrColIndA, const mcComplex* B, int ldb,
                                const mcComplex* beta, mcComplex* C, int ldc) {
    return pub(csrmm_entry<cfloat>(handle, transA, MCSPARSE_OPERATION_NON_TRANSPOSE, m, n, k, nnz, cx(alpha), descrA,
                                   cx(csrValA), csrRowPtrA, csrColIndA, cx(B), ldb, cx(beta), cx(C), ldc));
}

mcsparseStatus_t mcsparseZcsrmm(mcsparseHandle_t handle, mcsparseOperation_t transA, int m, int n, int k, int nnz,
                                const mcDoubleComplex* alpha, const mcsparseMatDescr_t descrA,
                                const mcDoubleComplex* csrValA, const int* csrRowPtrA, const int* csrColIndA,
                                const mcDoubleComplex* B, int ldb, const mcDoubleComplex* beta, mcDoubleComplex* C,
                                int ldc) {
    return pub(csrmm_entry<cdouble>(handle, transA, MCSPARSE_OPERATION_NON_TRANSPOSE, m, n, k, nnz, cx(alpha), descrA,
                                    cx(csrValA), csrRowPtrA, csrColIndA, cx(B), ldb, cx(beta), cx(C), ldc));
}

// ----------------------------------------------------------------------------- sharding helpers

mcsparseStatus_t mcsparseB200SpMVPush(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                      mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                      mcsparseDnVecDescr_t vecY, macaDataType computeType, mcsparseSpMVAlg_t alg,
                                      void* externalBuffer, int numPeers, void* const* peerY, int64_t rowOffset) {
    (void)alg;
    if (numPeers < 0 || numPeers > PeerList<float>::kMax || rowOffset < 0) return pub(BAD_SIZE);
    if (numPeers > 0 && peerY == nullptr) return pub(BAD_POINTER);
    for (int p = 0; p < numPeers; ++p)
        if (peerY[p] == nullptr) return pub(BAD_POINTER);
    PushArgs push;
    push.count = numPeers;
    push.y = peerY;
    push.row_offset = rowOffset;
    // How finished rows leave (MCSPARSE_B200_PUSH_STORE): "crew" (default): thread blocks of the tile launch that
    // compute nothing copy them with bulk copies (TMA) while the tiles compute; "bulk": every tile block hands its
    // rows to the TMA unit itself; "lsu": every tile block stores them with ordinary stores. The first two need all
    // destinations at the same alignment modulo 16 bytes and fall back to "lsu" otherwise.
    {
        const char* e = std::getenv("MCSPARSE_B200_PUSH_STORE");
        bool aligned = numPeers > 0;
        for (int p = 1; p < numPeers; ++p)
            aligned = aligned && ((reinterpret_cast<uintptr_t>(peerY[p]) ^ reinterpret_cast<uintptr_t>(peerY[0])) & 15) == 0;
        const char mode = e != nullptr ? e[0] : 'c';
        push.bulk = aligned && mode != 'l';
        push.crew = aligned && mode == 'c';
    }
    const int chunks = push_chunks_setting(numPeers);
    if (chunks == 0 || numPeers == 0)
        return pub(spmv_entry(handle, opA, alpha, matA, vecX, beta, vecY, computeType, externalBuffer, false, push));
    St st = spmv_check(handle, opA, alpha, matA, vecX, beta, vecY, computeType, true, externalBuffer, false, nullptr);
    if (st != OK) return pub(st);
    if (matA->rows == nullptr || matA->cols == nullptr || matA->vals == nullptr || vecX->values == nullptr ||
        vecY->values == nullptr || matA->mat_descr == nullptr)
        return pub(BAD_POINTER);
    if (!descr_general(matA->mat_descr)) return pub(NOT_IMPL);
    DeviceGuard guard(handle->device);
    if (computeType == MACA_R_64F)
        return pub(spmv_push_pipelined<double>(handle, matA, vecX, vecY, alpha, beta, externalBuffer, push, chunks));
    return pub(spmv_push_pipelined<float>(handle, matA, vecX, vecY, alpha, beta, externalBuffer, push, chunks));
}

mcsparseStatus_t mcsparseB200SpMVPushMulticast(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                               mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                               mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                               mcsparseSpMVAlg_t alg, void* externalBuffer, void* multicastY,
                                               int64_t rowOffset) {
    (void)alg;
    if (rowOffset < 0) return pub(BAD_SIZE);
    if (multicastY == nullptr) return pub(BAD_POINTER);
    if ((reinterpret_cast<uintptr_t>(multicastY) & 15) != 0) return pub(BAD_VALUE);
    void* const dst[1] = {multicastY};
    PushArgs push;
    push.count = 1;
    push.y = dst;
    push.row_offset = rowOffset;
    push.multicast = true;
    return pub(spmv_entry(handle, opA, alpha, matA, vecX, beta, vecY, computeType, externalBuffer, false, push));
}

mcsparseStatus_t mcsparseB200PeerSignalWait(mcsparseHandle_t handle, int numPeers, void* const* remoteSlots,
                                            void* localFlags, int epoch) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (numPeers < 0 || numPeers > PeerList<float>::kMax) return pub(BAD_SIZE);
    if (numPeers == 0) return MCSPARSE_STATUS_SUCCESS;
    if (remoteSlots == nullptr || localFlags == nullptr) return pub(BAD_POINTER);
    int* slots[PeerList<float>::kMax] = {};
    for (int p = 0; p < numPeers; ++p) {
        if (remoteSlots[p] == nullptr) return pub(BAD_POINTER);
        slots[p] = static_cast<int*>(remoteSlots[p]);
    }
    if (take_device_fault(handle)) return pub(EXEC_FAILED);
    DeviceGuard guard(handle->device);
    int* local = static_cast<int*>(localFlags);
    // Peers finish their step at slightly different times: the limit is fifty times the copy-wait limit
    // (about a second of SM clocks by default).
    return pub(from_cuda(peer_signal_wait(handle->stream, numPeers, slots, local, epoch, handle->wait_cycles * 50,
                                          local + MCSPARSE_B200_PEER_FLAG_STATUS, handle->fault_word_dev)));
}

mcsparseStatus_t mcsparseB200PeerAlloc(void** devPtr, size_t bytes) {
    if (devPtr == nullptr) return pub(BAD_POINTER);
    return pub(from_cuda(cudaMalloc(devPtr, bytes)));
}

mcsparseStatus_t mcsparseB200PeerFree(void* devPtr) { return pub(from_cuda(cudaFree(devPtr))); }

mcsparseStatus_t mcsparseB200PeerExport(void* devPtr, void* handleOut) {
    static_assert(sizeof(cudaIpcMemHandle_t) == MCSPARSE_B200_PEER_HANDLE_BYTES, "handle size");
    if (devPtr == nullptr || handleOut == nullptr) return pub(BAD_POINTER);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, devPtr);
    if (e != cudaSuccess) return pub(from_cuda(e));
    std::memcpy(handleOut, &h, sizeof h);
    return MCSPARSE_STATUS_SUCCESS;
}

mcsparseStatus_t mcsparseB200PeerOpen(const void* handleIn, void** mappedPtr) {
    if (handleIn == nullptr || mappedPtr == nullptr) return pub(BAD_POINTER);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handleIn, sizeof h);
    return pub(from_cuda(cudaIpcOpenMemHandle(mappedPtr, h, cudaIpcMemLazyEnablePeerAccess)));
}

mcsparseStatus_t mcsparseB200PeerClose(void* mappedPtr) {
    if (mappedPtr == nullptr) return MCSPARSE_STATUS_SUCCESS;
    return pub(from_cuda(cudaIpcCloseMemHandle(mappedPtr)));
}

mcsparseStatus_t mcsparseB200ShardRowBounds(mcsparseHandle_t handle, int64_t rows, int64_t nnz,
                                            mcsparseIndexBase_t idxBase, const int32_t* rowOffsets, int numShards,
                                            int64_t* bounds) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (rowOffsets == nullptr || bounds == nullptr) return pub(BAD_POINTER);
    if (rows < 0 || nnz < 0 || numShards < 1 || too_big(rows) || too_big(nnz)) return pub(BAD_SIZE);
    DeviceGuard guard(handle->device);
    return pub(from_cuda(shard_row_bounds(handle->stream, rows, nnz, idxBase, rowOffsets, numShards, bounds)));
}

mcsparseStatus_t mcsparseB200ShardLocalRowOffsets(mcsparseHandle_t handle, const int32_t* rowOffsets,
                                                  int64_t firstRow, int64_t numRows, mcsparseIndexBase_t idxBase,
                                                  int32_t* localOffsets) {
    if (handle == nullptr) return pub(BAD_HANDLE);
    if (rowOffsets == nullptr || localOffsets == nullptr) return pub(BAD_POINTER);
    if (firstRow < 0 || numRows < 0) return pub(BAD_SIZE);
    DeviceGuard guard(handle->device);
    return pub(from_cuda(
        shard_local_row_offsets(handle->stream, rowOffsets, firstRow, numRows, idxBase, localOffsets)));
}

}  // extern "C"
