/*
 * mcsparse_b200_ext.h -- entry points this build adds next to the mcSparse API.
 *
 * None of these exists in the mcSparse reference; each comment says which reference
 * behaviour it complements. They share the handle and descriptor objects of mcsparse.h.
 */
#ifndef MCSPARSE_B200_EXT_H_
#define MCSPARSE_B200_EXT_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Merge items (rows + nonzeros) one thread block of the tiled SpMV kernel consumes. Two sizes exist
 * per value type: the large one for matrices whose neighbouring nonzeros have neighbouring columns
 * (stencils, banded matrices: x is reused through L1 and per-tile overhead matters), half of it for
 * matrices with scattered columns (gather-latency bound: shorter tiles measured 20-40 % faster). The
 * choice is made once per matrix from a 4096-sample probe of the column indices. */
#define MCSPARSE_B200_SPMV_TILE_ITEMS_F32 4096
#define MCSPARSE_B200_SPMV_TILE_ITEMS_F64 2048
#define MCSPARSE_B200_SPMV_SMALL_TILE_ITEMS_F32 2048
#define MCSPARSE_B200_SPMV_TILE_ITEMS_C64 1024 /* 16-byte values (complex double): one tile size */
#define MCSPARSE_B200_SPMV_SMALL_TILE_ITEMS_F64 1024

/* L2 bytes (MiB) that one column panel of B may occupy in the panelled SpMM (mcsparseSpMM_preprocess);
 * the environment variable MCSPARSE_B200_SPMM_PANEL_MB overrides it, 0 turns the panels off. */
#define MCSPARSE_B200_SPMM_PANEL_MB_DEFAULT 48

/*
 * mcsparseSpMV_preprocess: same argument list as mcsparseSpMV. Runs the merge-path
 * analysis for matA into externalBuffer and records on matA that this buffer holds it, so
 * later mcsparseSpMV calls with the same matA, buffer and row-offset array skip the
 * analysis. The reference has no such call: its analysis hook is an empty stub
 * (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:129-158) and mcsparseSpMV needs
 * none. Without it, mcsparseSpMV re-runs the (cheap) analysis on every call, which is
 * always safe when the caller edits the row offsets in place. Between the preprocess call
 * and the products that rely on it, externalBuffer must not be handed to a call on another
 * matrix (the same matrix may alternate between op(A) = A and op(A) = A^T on one buffer:
 * each switch redoes the analysis or the conversion). With op(A) = A^T / A^H or a CSC
 * matrix the preprocess call also records the converted structure in externalBuffer.
 */
mcsparseStatus_t mcsparseSpMV_preprocess(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg, void* externalBuffer);

/*
 * View of the work partition a preprocess (or compute) call wrote into externalBuffer:
 * tileStarts points at (numTiles + 1) pairs {row, nonzero} of int32 in device memory;
 * tile t covers merge-path diagonals [t * itemsPerTile, (t + 1) * itemsPerTile) of the
 * (rows + nnz) long merge of row ends and nonzero indices. Used to check the device
 * analysis bit for bit against a CPU partition. No reference counterpart.
 */
mcsparseStatus_t mcsparseB200SpMVPartitionView(mcsparseSpMatDescr_t matA, void* externalBuffer,
                                               int* itemsPerTile, int64_t* numTiles,
                                               const int32_t** tileStarts);

/*
 * View of the converted matrix that a transposed product (op(A) = A^T on CSR, op(A) = A on CSC)
 * left in externalBuffer: the CSR arrays of the transposed matrix, 0-based, `rows` row offsets + 1
 * entries, nonzeros of a row in the order of the source (stable), values as of the last product.
 * Used to check the device conversion bit for bit against a CPU one. Returns INVALID_VALUE when
 * (matA, opA) is not a transposed product. No reference counterpart.
 */
mcsparseStatus_t mcsparseB200SpMVTransposedView(mcsparseSpMatDescr_t matA, mcsparseOperation_t opA,
                                                void* externalBuffer, int64_t* rows, const int32_t** rowOffsets,
                                                const int32_t** colInd, const void** values);

/*
 * A promise about the values of matA, for transposed products (op(A) = A^T / A^H on CSR, op(A) = A on CSC) that run
 * from a structure recorded by mcsparseSpMV_preprocess: with keep != 0 the caller will announce every change of the
 * value array through mcsparseSpMatSetValues or the SetPointers call of its format (passing the same pointer again
 * is enough after an in-place edit). A product may then reuse the values it gathered into the external buffer the
 * last time instead of gathering all nonzeros again (on the 27-point stencil the gather costs twice the product
 * itself). Without the promise (the default) every product gathers, which is always right. The reference converts
 * on every call (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:797-846); it has no such switch.
 * The same promise lets mcsparseSpMM, running from the panels recorded by mcsparseSpMM_preprocess, skip the pass that
 * regroups the values panel by panel when the buffer holds them from the last call (single matrices, not batches).
 */
mcsparseStatus_t mcsparseB200SpMatKeepConvertedValues(mcsparseSpMatDescr_t matA, int keep);

/*
 * Device-side status of the SpMV calls that used externalBuffer since its last analysis (pass
 * NULL for the built-in work area of mcsparseB200SpMVNoAlloc): 0; bit 0 set if a thread block gave
 * up its bounded wait for the bulk copies of its tile and left its rows unwritten; bit 1 set if a
 * wait exceeded the limit but the copies then arrived and the tile was computed (a warning).
 * Synchronises the handle's stream. A tile that was given up is also reported without any
 * synchronisation: the kernel sets a word in pinned host memory owned by the handle, and the next
 * mcsparseSpMV / mcsparseB200SpMVPush / mcsparseB200SpMVNoAlloc call on that handle returns
 * MCSPARSE_STATUS_EXECUTION_FAILED once (and clears the word) before doing anything else.
 * The reference has no device-side waits and no such query.
 */
mcsparseStatus_t mcsparseB200SpMVGetStatus(mcsparseHandle_t handle, mcsparseSpMatDescr_t matA,
                                           void* externalBuffer, int* status);

/*
 * How long a thread block of the tiled SpMV kernels waits for the bulk copies of its tile before
 * it reports a failure instead of spinning: smClocks SM clock cycles (default 40,000,000, about
 * 20 ms; a healthy copy takes microseconds). After the limit the block sets the status words
 * described above, stays resident for 256 times the limit in case its copies still land, and
 * returns. withholdCopies != 0 is a diagnostics switch for tests of that path: the kernels then
 * issue no bulk copy at all, so every wait runs out with nothing in flight and every tile is
 * given up. No reference counterpart.
 */
mcsparseStatus_t mcsparseB200SetDeviceWaitLimit(mcsparseHandle_t handle, int64_t smClocks, int withholdCopies);

/*
 * Measures the second roofline of CSR SpMV on this GPU: the rate at which the SMs can gather unrelated
 * elements. `blocks` thread blocks of 256 threads read indices[0 .. count) (device, 16-byte aligned, values
 * below the table's length) with coalesced loads, gather table[indices[i]] (elements of elemBytes = 4 or 8)
 * and leave one partial sum per thread in partialSums (blocks * 256 elements). A gather of an element whose
 * neighbours are not wanted costs one 32-byte sector request to L2, and an SM issues about one such request
 * per clock, whatever the element size and however the load is written; an SpMV with scattered columns makes
 * one per nonzero, so nnz / (gathers per second) bounds its time from below beside bytes / HBM bandwidth.
 * The caller times the launch (bench.py does). Asynchronous on the handle's stream. No reference counterpart.
 */
mcsparseStatus_t mcsparseB200GatherProbe(mcsparseHandle_t handle, const int32_t* indices, int64_t count,
                                         const void* table, int elemBytes, void* partialSums, int blocks);

/*
 * Row-block sharding of one CSR matrix over numShards GPUs, balanced by nonzeros:
 * bounds[g] = first row r with rowOffsets[r] - base >= floor(g * nnz / numShards),
 * bounds[0] = 0, bounds[numShards] = rows. rowOffsets is device memory; bounds is host
 * memory of numShards + 1 entries; the call synchronises the handle's stream.
 * The reference is single-device (mcsparse/src/common/mcsp_handle.cpp:5-8).
 */
mcsparseStatus_t mcsparseB200ShardRowBounds(mcsparseHandle_t handle, int64_t rows, int64_t nnz,
                                            mcsparseIndexBase_t idxBase, const int32_t* rowOffsets,
                                            int numShards, int64_t* bounds);

/*
 * localOffsets[i] = rowOffsets[firstRow + i] - rowOffsets[firstRow] + base for
 * i in [0, numRows]: the row offsets of a shard as a stand-alone CSR matrix whose column
 * and value arrays start at nonzero rowOffsets[firstRow] - base. Asynchronous.
 */
mcsparseStatus_t mcsparseB200ShardLocalRowOffsets(mcsparseHandle_t handle, const int32_t* rowOffsets,
                                                  int64_t firstRow, int64_t numRows,
                                                  mcsparseIndexBase_t idxBase, int32_t* localOffsets);

/*
 * Row-sharded SpMV with the assembly of y fused into the kernel. Same arguments as
 * mcsparseSpMV for this GPU's row block (matA: the block with local row offsets; vecX: the
 * full x; vecY: this block's slice of the local full-length y), plus the destinations of the
 * push: peerY[p] is the full-length y of another GPU as an address valid on this device
 * (see mcsparseB200PeerOpen), rowOffset the global index of the block's first row. Every
 * finished y value ends up in vecY and in peerY[p][rowOffset + row] for all p, moved over
 * NVLink while the SpMV is still running: either the tile kernel stores each finished row to
 * all peers itself, or the tiles are computed in a few launches and each chunk's rows are copied
 * by the copy engines on a second, higher-priority stream while the next chunk computes (chosen
 * from the number of peers; MCSPARSE_B200_PUSH_CHUNKS=0..8 overrides). No separate all-gather
 * of y is needed. The first call with a given buffer analyses the matrix and synchronises once.
 * The caller orders the GPUs afterwards (any collective or barrier on the same streams)
 * before x is overwritten or y is read. numPeers <= 7. The reference is single-device
 * (mcsparse/src/common/mcsp_handle.cpp:5-8); this call has no counterpart there.
 */
mcsparseStatus_t mcsparseB200SpMVPush(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                      mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                      mcsparseDnVecDescr_t vecY, macaDataType computeType, mcsparseSpMVAlg_t alg,
                                      void* externalBuffer, int numPeers, void* const* peerY, int64_t rowOffset);

/*
 * Same product as mcsparseB200SpMVPush, with the finished rows stored once into an NVSwitch
 * multicast mapping instead of once per peer: multicastY is the address of the full-length y in a
 * multicast address range bound to the same-sized, same-offset allocation on every GPU of the run
 * (this one included), 16-byte aligned; the kernels use multimem.st, the switch replicates the
 * store to all GPUs. vecY must be this GPU's rows inside its own unicast mapping of that
 * allocation. Creating the mapping is the caller's job (CUDA virtual-memory multicast objects;
 * the Python harness takes it from torch's symmetric-memory allocator). As with the peer-store
 * variant, order the GPUs with any collective before y is read. No reference counterpart.
 */
mcsparseStatus_t mcsparseB200SpMVPushMulticast(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                               mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                               mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                               mcsparseSpMVAlg_t alg, void* externalBuffer, void* multicastY,
                                               int64_t rowOffset);

/*
 * Orders the GPUs of a row-sharded step on the device, without a collective. Every rank owns a flag area of
 * MCSPARSE_B200_PEER_FLAG_INTS 32-bit integers in peer-mapped memory, zeroed once: slot p (p < numPeers)
 * belongs to the rank's p-th peer, integer MCSPARSE_B200_PEER_FLAG_STATUS is a status word. The call
 * enqueues one small kernel on the handle's stream, after whatever moved this rank's rows (in stream
 * order): it stores `epoch` into remoteSlots[p], this rank's slot inside peer p's flag area, with release
 * semantics at system scope, and then waits until every slot of localFlags has reached `epoch` (acquire),
 * i.e. until every peer's rows of that step are in this GPU's memory. Epochs must grow from step to step
 * (compared modulo 2^32). The wait is bounded (fifty times the handle's device wait limit, about a second):
 * when it runs out the kernel sets bit 0 of the status word and the handle's fault word and returns, and the
 * next compute call on the handle reports MCSPARSE_STATUS_EXECUTION_FAILED. The waiting kernels of the ranks
 * run on different GPUs; never run two ranks of one job on the same GPU. No reference counterpart.
 */
#define MCSPARSE_B200_PEER_FLAG_INTS 16
#define MCSPARSE_B200_PEER_FLAG_STATUS 8
mcsparseStatus_t mcsparseB200PeerSignalWait(mcsparseHandle_t handle, int numPeers, void* const* remoteSlots,
                                            void* localFlags, int epoch);

/*
 * Device buffers that other processes on the same node can map (one process per GPU):
 * PeerAlloc/PeerFree allocate with the plain CUDA allocator; PeerExport fills a 64-byte
 * handle that another process passes to PeerOpen to obtain an address valid on its current
 * device (peer access is enabled on first use); PeerClose unmaps it. No reference counterpart.
 */
#define MCSPARSE_B200_PEER_HANDLE_BYTES 64
mcsparseStatus_t mcsparseB200PeerAlloc(void** devPtr, size_t bytes);
mcsparseStatus_t mcsparseB200PeerFree(void* devPtr);
mcsparseStatus_t mcsparseB200PeerExport(void* devPtr, void* handleOut);
mcsparseStatus_t mcsparseB200PeerOpen(const void* handleIn, void** mappedPtr);
mcsparseStatus_t mcsparseB200PeerClose(void* mappedPtr);

/*
 * mcsparseB200SpMVNoAlloc: y = alpha * A * x + beta * y like mcsparseSpMV, for callers that
 * are not allowed to allocate device memory and therefore have no external buffer to pass:
 * code running inside a memory-budgeted plugin or solver callback whose host hands it x and y
 * but forbids cudaMalloc, code that must not trigger the implicit synchronisation of an
 * allocation, or a late stage of a job whose memory is already fully committed. It has no
 * counterpart in the reference, whose SpMV always takes a caller-allocated buffer.
 *
 * The merge-path partition and the per-tile carries are kept in a fixed array compiled into
 * the library (MCSPARSE_B200_NOALLOC_SCRATCH_BYTES per GPU that loads it, held until the
 * process exits). The call allocates nothing, on the host side of CUDA or through any library.
 *   - Limit: the work area must hold the partition of (rows + nnz) merge items; larger
 *     matrices are refused with MCSPARSE_STATUS_INSUFFICIENT_RESOURCES and a message on stderr
 *     (about 8.5e8 items for fp64 values, 2.1e9 for fp32). Use mcsparseSpMV for those.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call outside any stream capture. No call copies anything back to the host or waits for the
 *     stream: the kernel family and tile size are the ones an earlier mcsparseSpMV / mcsparseSpMV_preprocess
 *     call chose for this matrix, or the defaults if there was none (mcsparseSpMV's choice involves a small
 *     probe kernel and a stream synchronisation, which this entry point must not do; results then agree with
 *     mcsparseSpMV to rounding, not bit for bit).
 *   - All calls on a device share the one array and it keeps what the previous call left.
 *     Every entry a call reads is written earlier in the same call, so nothing needs clearing,
 *     but two calls that overlap on the GPU (different streams, or threads) would overwrite each
 *     other's partition: run them one after the other.
 *   - A thread block that gives up its bounded wait reports through the handle (the next call returns
 *     MCSPARSE_STATUS_EXECUTION_FAILED) and through the work area's status word, which
 *     mcsparseB200SpMVGetStatus reads when its externalBuffer argument is NULL.
 * Arguments and status codes are those of mcsparseSpMV without the buffer.
 */
#define MCSPARSE_B200_NOALLOC_SCRATCH_BYTES (16u << 20)
mcsparseStatus_t mcsparseB200SpMVNoAlloc(mcsparseHandle_t handle, mcsparseOperation_t opA, const void* alpha,
                                         mcsparseSpMatDescr_t matA, mcsparseDnVecDescr_t vecX, const void* beta,
                                         mcsparseDnVecDescr_t vecY, macaDataType computeType,
                                         mcsparseSpMVAlg_t alg);

#ifdef __cplusplus
}
#endif

#endif /* MCSPARSE_B200_EXT_H_ */
