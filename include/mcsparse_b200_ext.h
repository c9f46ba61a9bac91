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

/* Merge items (rows + nonzeros) one thread block of the tiled SpMV kernel consumes. */
#define MCSPARSE_B200_SPMV_TILE_ITEMS_F32 4096
#define MCSPARSE_B200_SPMV_TILE_ITEMS_F64 2048

/*
 * mcsparseSpMV_preprocess: same argument list as mcsparseSpMV. Runs the merge-path
 * analysis for matA into externalBuffer and records on matA that this buffer holds it, so
 * later mcsparseSpMV calls with the same matA, buffer and row-offset array skip the
 * analysis. The reference has no such call: its analysis hook is an empty stub
 * (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:129-158) and mcsparseSpMV needs
 * none. Without it, mcsparseSpMV re-runs the (cheap) analysis on every call, which is
 * always safe when the caller edits the row offsets in place.
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

#ifdef __cplusplus
}
#endif

#endif /* MCSPARSE_B200_EXT_H_ */
