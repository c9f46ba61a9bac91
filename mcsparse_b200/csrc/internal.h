// Internal declarations shared by the host API (api.cpp) and the CUDA translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <mutex>

#include "mcsparse.h"
#include "value_types.h"

// Descriptor payloads. Field meaning follows the reference's structs
// (mcsparse/src/include/mcsp_internal_types.h:86-92,127-145,184-223 and
// mcsparse/src/include/mcsp_handle.h:11-27) minus everything the CSR path never reads.
constexpr int kMaxPushChunks = 8;

struct mcsparseContext {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    mcsparsePointerMode_t ptr_mode = MCSPARSE_POINTER_MODE_HOST;
    // Created on the first pipelined mcsparseB200SpMVPush: a stream for the row copies that run
    // beside the kernels, and the events that order the two streams.
    cudaStream_t side_stream = nullptr;
    cudaEvent_t events[kMaxPushChunks + 1] = {};
    // One copy stream per destination GPU, so that the copies of a chunk to different peers run on
    // different copy engines at the same time; fix_events[c]: chunk c's rows are final;
    // peer_events[p]: the last copy to peer p is done.
    static constexpr int kMaxPeers = 7;
    cudaStream_t peer_streams[kMaxPeers] = {};
    cudaEvent_t fix_events[kMaxPushChunks] = {};
    cudaEvent_t peer_events[kMaxPeers] = {};
    cudaStream_t capture_stream = nullptr;  // origin stream while the step is captured as a graph
    // Bounded device-side waits: how long a thread block waits for the bulk copies of its tile (SM clocks),
    // and a word in pinned, device-mapped host memory that a kernel sets when it gave a tile up. The next
    // compute call on the handle reads the word on the host (no synchronisation) and reports it.
    long long wait_cycles = 40000000;  // about 20 ms of SM clocks
    int withhold_copies = 0;           // diagnostics: issue no bulk copies, so that every wait runs out
    int* fault_word_host = nullptr;
    int* fault_word_dev = nullptr;
    // L2 residency of x (see XResidency in api.cpp): the device's largest persisting carve-out, read once, and
    // whether this handle has already asked for it.
    long long max_persisting_l2 = -1;
    bool persisting_l2_requested = false;
};

struct mcsparseMatDescr {
    mcsparseMatrixType_t type = MCSPARSE_MATRIX_TYPE_GENERAL;
    mcsparseFillMode_t fill_mode = MCSPARSE_FILL_MODE_FULL;
    mcsparseDiagType_t diag_type = MCSPARSE_DIAG_TYPE_NON_UNIT;
    mcsparseStorageMode_t storage_mode = MCSPARSE_STORAGE_MODE_SORTED;
    mcsparseIndexBase_t base = MCSPARSE_INDEX_BASE_ZERO;
};

struct mcsparseSpMatDescr {
    mcsparseFormat_t format = MCSPARSE_FORMAT_CSR;
    int64_t row_num = 0, col_num = 0, nnz = 0;
    void* rows = nullptr;  // CSR: row offsets; COO: row index of every entry (device)
    void* cols = nullptr;  // column indices (device)
    void* vals = nullptr;  // values (device)
    mcsparseIndexType_t rowIdxType = MCSPARSE_INDEX_32I, colIdxType = MCSPARSE_INDEX_32I;
    mcsparseIndexBase_t idxBase = MCSPARSE_INDEX_BASE_ZERO;
    macaDataType valueType = MACA_R_32F;
    mcsparseMatDescr* mat_descr = nullptr;
    int64_t batchCount = 1, batchStride = 0, offsetsBatchStride = 0;  // strided batch (SpMM)
    // Analysis recorded by mcsparseSpMV_preprocess: which buffer holds the partition of
    // which row-offset array. Guarded by `lock`; cleared by mcsparseCsrSetPointers.
    std::mutex lock;
    void* analysed_buffer = nullptr;
    const void* analysed_rows = nullptr;
    int analysed_items_per_tile = 0;
    // Tile size chosen by the locality probe for these column indices (probed once, then remembered).
    const void* probed_cols = nullptr;
    int64_t probed_nnz = -1;
    int tile_kind = 0;  // kTileSmall | kTileWalk
    // Chunk boundaries of the pipelined push (tiles and the rows they start at), read back once.
    void* push_buffer = nullptr;
    const void* push_rows_ptr = nullptr;
    int push_chunks = 0;
    int64_t push_chunk_tiles[kMaxPushChunks + 1] = {};
    int64_t push_chunk_rows[kMaxPushChunks + 1] = {};
    // Transposed products: which buffer holds the converted structure of which arrays (recorded by
    // mcsparseSpMV_preprocess), and the tile size probed for the converted matrix.
    void* trans_buffer = nullptr;
    const void* trans_ptr_src = nullptr;
    const void* trans_idx_src = nullptr;
    int64_t trans_nnz = -1;
    const void* trans_probed_idx = nullptr;
    int64_t trans_probed_nnz = -1;
    int trans_tile_kind = 0;
    // Set by mcsparseB200SpMatKeepConvertedValues: the caller promises to announce every change of the values
    // (mcsparseSpMatSetValues / SetPointers), so a transposed product may reuse the values it gathered into the
    // buffer last time (trans_values_src / _conj say which) instead of gathering them again.
    bool keep_converted_values = false;
    const void* trans_values_src = nullptr;
    bool trans_values_conj = false;
    const void* spmm_values_src = nullptr;  // the same for the values regrouped panel by panel by mcsparseSpMM
    // COO inputs: whether the row indices were found out of order (checked once per array, remembered).
    const void* coo_checked_rows = nullptr;
    int64_t coo_checked_nnz = -1;
    bool coo_unsorted = false;
    // The pipelined push of one step (tile launches, fix-ups, per-destination copies and the events
    // between them) captured once as a CUDA graph and replayed while every argument stays the same.
    // A few are kept (least recently used one replaced): a solver that alternates between two vector pairs
    // replays two graphs instead of re-capturing on every call.
    static constexpr int kPushGraphs = 4;
    struct PushGraph {
        cudaGraphExec_t exec = nullptr;
        unsigned char key[256] = {};
        size_t key_bytes = 0;
        uint64_t last_use = 0;
    };
    PushGraph push_graphs[kPushGraphs];
    uint64_t push_graph_clock = 0;
    // Column panels recorded by mcsparseSpMM_preprocess: buffer, arrays and shape they were built for.
    void* spmm_buffer = nullptr;
    const void* spmm_rows = nullptr;
    const void* spmm_cols = nullptr;
    int spmm_panels = 0;
    int spmm_lanes = 0;
    int64_t spmm_n = 0;
};

struct mcsparseDnVecDescr {
    int64_t size = 0;
    void* values = nullptr;
    macaDataType valueType = MACA_R_32F;
};

struct mcsparseDnMatDescr {
    int64_t row_num = 0, col_num = 0, ld = 0;
    void* values = nullptr;
    macaDataType valueType = MACA_R_32F;
    mcsparseOrder_t order = MCSPARSE_ORDER_COL;
    int64_t batchCount = 1, batchStride = 0;
};

namespace mcsp_b200 {

// alpha / beta as the kernels receive them: a host value, or a device address to read.
template <typename T>
struct ScalarArg {
    T host;
    const T* dev;
#ifdef __CUDACC__
    __device__ __forceinline__ T get() const { return dev ? *dev : host; }
#endif
};

// Destinations of the fused row push of a row-sharded SpMV: the full-length y vectors of the
// other GPUs (addresses valid on this device) and the global index of this shard's first row.
// With `multicast`, count is 1 and y[0] is the vector's address in an NVSwitch multicast mapping
// that covers every GPU of the run; the kernels then store with multimem.st.
template <typename T>
struct PeerList {
    static constexpr int kMax = 7;
    int count = 0;
    bool multicast = false;
    bool bulk = false;  // finished rows leave through bulk copies from shared memory (all y[p] congruent modulo 16)
    bool crew = false;  // finished rows are moved by the launch's push crew (all y[p] and the local y congruent modulo 16)
    long long row_offset = 0;
    T* y[kMax] = {};
};

// Streams and events of the per-destination row copies of the pipelined push (owned by the handle).
struct PushStreams {
    cudaStream_t* peer_streams = nullptr;
    cudaEvent_t* fix_events = nullptr;
    cudaEvent_t* peer_events = nullptr;
};

// How the tile kernels wait for their bulk copies: the limit in SM clocks, the diagnostics switch that
// withholds the copies, and the device address of the handle's host-visible fault word (may be null).
struct WaitCfg {
    long long limit_cycles = 40000000;
    int withhold = 0;
    int* fault_word = nullptr;
};

// The push crew of a sharded tile launch: the first `pushers` thread blocks compute no tile; they wait for
// chunks of `tiles_per_chunk` consecutive tiles to finish (done[c] counts them; zeroed before the launch) and
// copy the rows that ended in a finished chunk from the local y to every peer with bulk copies.
struct CrewCfg {
    int pushers = 0;
    int tiles_per_chunk = 64;
    int num_chunks = 0;
    int* done = nullptr;
};
constexpr int kCrewTilesPerChunk = 64;

// Layout of the SpMV work buffer (all offsets from the 256-byte aligned start):
//   int32 pairs tile_starts[num_tiles + 1] | int32 carry_row[num_tiles] | T carry_val[num_tiles] | int32 status |
//   int32 chunk_done[ceil(num_tiles / kCrewTilesPerChunk)]
// status stays 0 unless a kernel gave up a bounded wait (zeroed by the analysis kernel).
struct SpmvWorkspace {
    int items_per_tile = 0;
    bool walk = false;  // scattered columns: every tile takes the thread-per-merge-segment walk kernel
    int64_t num_tiles = 0;
    size_t off_carry_row = 0, off_carry_val = 0, off_status = 0, off_done = 0, bytes = 0;
};
// Layout for the chosen tile size; `bytes` is always the size the small tiles would need, so that
// mcsparseSpMV_bufferSize does not depend on the choice.
// tile_kind: kTileSmall for the half-size tile, kTileWalk for the walk kernel (they combine).
enum : int { kTileLarge = 0, kTileSmall = 1, kTileWalk = 2 };
SpmvWorkspace spmv_workspace(int64_t m, int64_t nnz, size_t value_size, int tile_kind = kTileLarge,
                             size_t index_size = 4);
// host_count[0]: over 4096 evenly spaced positions j, how often |col[j + 1] - col[j]| <= 8; host_count[1]: how many
// of 4096 evenly spaced rows hold more than 256 nonzeros. The counts are left in device_count[0..1] and copied
// to host_count (synchronises the stream).
template <typename I>
cudaError_t spmv_locality_probe(cudaStream_t s, int64_t m, int64_t nnz, const I* row_ptr, const I* col, int* device_count,
                                int* host_count);
// Launches the gather-rate probe: `blocks` thread blocks of 256 threads gather table[idx[i]] for i < count and
// leave one partial sum per thread in `out` (blocks * 256 elements of elem_bytes = 4 or 8).
cudaError_t gather_probe(cudaStream_t s, const int32_t* idx, int64_t count, const void* table, int elem_bytes, void* out,
                         int blocks);
inline void* align_up_256(void* p) {
    return reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(p) + 255) & ~uintptr_t(255));
}

// I: type of the row offsets and column indices (int32_t or int64_t; extents must fit 31 bits either way).
template <typename I>
cudaError_t spmv_analysis(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const SpmvWorkspace& ws,
                          void* buf);
template <typename T, typename I>
cudaError_t spmv_tiled(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const I* col, const T* val,
                       const T* x, T* y, ScalarArg<T> alpha, ScalarArg<T> beta, const SpmvWorkspace& ws, void* buf,
                       const PeerList<T>& peers = PeerList<T>(), const WaitCfg& wait = WaitCfg());
// Rows at which the given tiles start, copied to the host (synchronises the stream).
cudaError_t spmv_read_tile_rows(cudaStream_t s, const void* buf, int count, const int64_t* tiles, int64_t* rows);
// The tiles in `chunks` launches; after each, a copy kernel on `side` pushes the rows that ended in
// it to the peers while the next chunk computes; the carry fix-up (with its own pushes) comes last.
template <typename T>
cudaError_t spmv_tiled_pipelined(cudaStream_t s, cudaStream_t side, cudaEvent_t* events, const PushStreams& ps,
                                 int chunks,
                                 const int64_t* chunk_tiles, const int64_t* chunk_rows, int64_t m, int64_t nnz,
                                 int base, const int32_t* row_ptr, const int32_t* col, const T* val, const T* x, T* y,
                                 ScalarArg<T> alpha, ScalarArg<T> beta, const SpmvWorkspace& ws, void* buf,
                                 const PeerList<T>& peers, const WaitCfg& wait = WaitCfg());
template <typename T>
cudaError_t spmv_rowgroup(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                          const int32_t* col, const T* val, const T* x, T* y, ScalarArg<T> alpha,
                          ScalarArg<T> beta);

// Fixed device work area behind mcsparseB200SpMVNoAlloc (address on the current device).
cudaError_t spmv_static_scratch(void** ptr, size_t* bytes);

// Column-panel plan of an SpMM whose B does not fit in L2 (num_panels == 1: no panels). The work
// buffer then holds int32 panel_ptr[(num_panels + 1) * m]: where each panel starts inside each row.
// With panels the work buffer holds (256-byte aligned pieces, in this order)
//   int32 panel_ptr[(num_panels + 1) * m]   where each panel starts inside each row of A
//   int32 piece_pos[num_panels * m + 1]     panel-major prefix sums of the piece lengths: the piece of row r in
//                                           panel p occupies [piece_pos[p * m + r], piece_pos[p * m + r + 1]) below
//   int32 ccol[nnz], value cval[nnz]        A's column indices (0-based) and values regrouped panel by panel, so
//                                           that one pass streams a contiguous range instead of a piece per row
//   uint32 scan scratch
struct SpmmPlan {
    int num_panels = 1;
    int panel_cols = 0;  // rows of B (columns of A) per panel
    int lanes = 0;       // lanes per row of the panel kernel: the slab is lanes x 16 bytes wide
    size_t off_pos = 0, off_ccol = 0, off_cval = 0, off_dst = 0, off_scan = 0;
    size_t bytes = 128;
    int64_t nnz = 0;              // nonzeros of the matrix the plan was made for
    bool values_current = false;  // the buffer already holds these values regrouped (the caller vouches for it)
};
long long scan_scratch_elems(long long count);
cudaError_t exclusive_scan_u32(cudaStream_t s, unsigned* data, long long count, unsigned* sums);
SpmmPlan spmm_plan(int64_t m, int64_t k, int64_t n, int64_t nnz, size_t value_size, bool row_major_operands);
template <typename I>
cudaError_t spmm_preprocess(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const I* col,
                            const SpmmPlan& plan, void* buf);

// Dense operand addressed as element(r, c) = ptr[r * row_stride + c * col_stride].
template <typename T, typename I>
cudaError_t spmm(cudaStream_t s, int64_t m, int64_t n, int base, const I* row_ptr, const I* col, const T* val,
                 const T* B, int64_t b_row_stride, int64_t b_col_stride, T* C, int64_t c_row_stride,
                 int64_t c_col_stride, ScalarArg<T> alpha, ScalarArg<T> beta, const SpmmPlan* plan = nullptr,
                 void* plan_buffer = nullptr);

// y = alpha * A * x + beta * y with a real CSR matrix and complex x, y, alpha, beta; scratch: m complex numbers.
template <typename F>
cudaError_t spmv_real_matrix_complex_vectors(cudaStream_t s, int64_t m, int base, const int32_t* row_ptr,
                                             const int32_t* col, const F* val, const Complex<F>* x, Complex<F>* y,
                                             ScalarArg<Complex<F>> alpha, ScalarArg<Complex<F>> beta,
                                             Complex<F>* scratch);

// dst = conj(src); y = alpha * conj(z) + beta * y (complex vectors).
template <typename T>
cudaError_t complex_conj_copy(cudaStream_t s, int64_t n, const T* src, T* dst);
template <typename T>
cudaError_t complex_conj_axpby(cudaStream_t s, int64_t m, ScalarArg<T> alpha, const T* z, ScalarArg<T> beta, T* y);

// Low-precision operands (A and x of one type) with fp32 or int32 sums: operand type -> type of y.
enum class MixedKind { kNone, kHalfToFloat, kBf16ToFloat, kInt8ToFloat, kHalfToHalf, kBf16ToBf16, kInt8ToInt32 };

// y = alpha * A * x + beta * y for a CSR matrix (32-bit indices) of one of the kinds above. alpha and beta are
// floats, for kInt8ToInt32 32-bit integers (the other pair is not read). `buf` holds spmv_mixed_workspace(m, nnz)
// with the partition written by spmv_analysis for that workspace.
SpmvWorkspace spmv_mixed_workspace(int64_t m, int64_t nnz);
cudaError_t spmv_mixed(cudaStream_t s, MixedKind kind, int64_t m, int base, const int32_t* row_ptr, const int32_t* col,
                       const void* val, const void* x, void* y, ScalarArg<float> alpha_f, ScalarArg<float> beta_f,
                       ScalarArg<int> alpha_i, ScalarArg<int> beta_i, const SpmvWorkspace& ws, void* buf);

cudaError_t coo_row_offsets(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* coo_rows,
                            int32_t* offsets);

// Where the CSR arrays of the transposed matrix and the scratch of the conversion live inside a
// buffer (byte offsets from a 256-byte aligned start). The transposed matrix is n x m, 0-based:
// row offsets at off_ptr, column indices in keys[col_slot()], values at off_val.
struct TransposePlan {
    int passes = 1;          // radix-sort passes (8 bits of the column index each)
    int64_t tiles = 0;       // thread blocks of one pass
    int64_t hist_count = 0;  // 256 digit counts per tile
    int64_t scan_chunks = 0;
    size_t off_ptr = 0, off_keys[2] = {0, 0}, off_perm[2] = {0, 0}, off_val = 0, off_hist = 0, off_sums = 0;
    size_t bytes = 0;
    int final_slot() const { return (passes - 1) & 1; }  // where the last pass leaves sorted keys and permutation
    int col_slot() const { return final_slot() ^ 1; }
};
TransposePlan transpose_plan(int64_t m, int64_t n, int64_t nnz, size_t value_size);
// Structure of the transposed matrix (row offsets, column indices, permutation) of an m x n CSR matrix.
// (I: the caller's index type; the converted arrays are always 32-bit, extents fit 31 bits.)
template <typename I>
cudaError_t transpose_structure(cudaStream_t s, int64_t m, int64_t n, int64_t nnz, int base, const I* row_ptr,
                                const I* col, const TransposePlan& plan, void* buf);
// CSR structure of a COO matrix whose entries come in any order, by the same stable sort: sorted by
// `key_idx` (the row indices; or the column indices, which yields the transposed matrix), row
// offsets over [0, key_range], and the other index of every entry gathered into keys[col_slot()],
// 0-based. The plan is transpose_plan(any, key_range, nnz, value_size).
template <typename I>
cudaError_t coo_sort_structure(cudaStream_t s, int64_t key_range, int64_t nnz, int base, const I* key_idx,
                               const I* other_idx, const TransposePlan& plan, void* buf);
// Array-of-pairs COO indices (row0, col0, row1, col1, ...; 8-byte aligned) -> two arrays.
cudaError_t split_index_pairs(cudaStream_t s, int64_t nnz, const int32_t* pairs, int32_t* rows, int32_t* cols);
// *host_flag = 1 if idx[0 .. count) is not ascending (one kernel, a 4-byte copy, a stream synchronisation).
template <typename I>
cudaError_t indices_unsorted(cudaStream_t s, int64_t count, const I* idx, int* host_flag);
// Values of the transposed matrix, gathered through the permutation left by transpose_structure
// (conjugated on the way for op(A) = A^H).
template <typename T>
cudaError_t transpose_values(cudaStream_t s, int64_t nnz, const T* val, const TransposePlan& plan, void* buf,
                             bool conjugate = false);
// Signals `epoch` into remote_slots[p] (p < count <= 7) and waits, for at most `limit` SM clocks per peer, until
// local_slots[p] has reached it; a wait that runs out sets bit 0 of *status and the fault word.
cudaError_t peer_signal_wait(cudaStream_t s, int count, int* const* remote_slots, const int* local_slots, int epoch,
                             long long limit, int* status, int* fault_word);
cudaError_t shard_row_bounds(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                             int num_shards, int64_t* bounds_host);
cudaError_t shard_local_row_offsets(cudaStream_t s, const int32_t* row_ptr, int64_t first_row, int64_t num_rows,
                                    int base, int32_t* local);

}  // namespace mcsp_b200
