// CSR of the transposed matrix (equivalently: CSC of the matrix), built on the device so that
// y = alpha * A^T * x + beta * y and products with CSC inputs run on the same CSR kernels.
//
// The reference reaches its CSR kernel the same way: it converts with csr2csc into the external
// buffer and multiplies with the converted arrays (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:797-846,
// mcsparse/src/common/mcsp_internal_transpose_sparse.hpp:237-341).
//
// The conversion is a stable sort of the nonzeros by column:
//   1. least-significant-digit radix sort (8-bit digits, as many passes as the column count needs)
//      of the pairs (column, position), each pass = tile histograms -> exclusive scan -> stable
//      scatter; stable means that within a column the nonzeros keep their order (ascending rows),
//      so the transposed matrix, and with it every later product, is the same on every run;
//   2. row offsets of the transposed matrix = lower bounds of 0 .. cols in the sorted columns;
//   3. column indices of the transposed matrix = the row that owns each source position (upper
//      bound in the source row offsets, evaluated for all positions in order and then gathered
//      through the permutation);
//   4. values gathered through the permutation (repeated on every product: values may have changed).
#include <cstdint>
#include <mutex>

#include "internal.h"

namespace mcsp_b200 {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItemsPerWarp = 1024;                         // 32 rounds of one item per lane
constexpr int kSortTile = kSortWarps * kSortItemsPerWarp;       // items per thread block
constexpr int kScanThreads = 1024;
constexpr int kScanItems = 8;                                   // consecutive items per thread
constexpr int kScanChunk = kScanThreads * kScanItems;

// K: type of the keys a pass reads (the caller's 32- or 64-bit indices in the first pass, the
// 32-bit keys of the previous pass after that; sorted keys always fit 31 bits).
template <typename K>
__device__ __forceinline__ unsigned sort_key(const K* __restrict__ keys, long long i, int sub) {
    return (unsigned)(__ldg(keys + i) - sub);
}

// hist[d * tiles + t] = number of items of tile t whose digit is d.
template <typename K>
__global__ void __launch_bounds__(kSortThreads)
    radix_hist_kernel(const K* __restrict__ keys, int sub, long long count, int shift, unsigned* __restrict__ hist,
                      long long tiles) {
    __shared__ unsigned s_cnt[256];
    const long long t = blockIdx.x;
    s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const long long begin = t * kSortTile;
    const int lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < kSortTile; i += kSortThreads) {  // block-uniform trip count
        const long long idx = begin + i;
        const unsigned d = idx < count ? (sort_key(keys, idx, sub) >> shift) & 255u : 256u;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (d < 256u && lane == __ffs(peers) - 1) atomicAdd(&s_cnt[d], __popc(peers));
    }
    __syncthreads();
    hist[(long long)threadIdx.x * tiles + t] = s_cnt[threadIdx.x];
}

// Stable scatter of one tile: item idx goes to offsets[digit][tile] + (number of earlier items of
// the tile with the same digit). Warps own consecutive 1024-item pieces of the tile and walk them
// 32 items at a time, so "earlier" is decided by (warp, round, lane) = ascending idx.
template <typename K>
__global__ void __launch_bounds__(kSortThreads)
    radix_scatter_kernel(const K* __restrict__ keys_in, int sub, const unsigned* __restrict__ perm_in,
                         int* __restrict__ keys_out, unsigned* __restrict__ perm_out, long long count, int shift,
                         const unsigned* __restrict__ offsets, long long tiles) {
    __shared__ unsigned s_cnt[kSortWarps][256];
    const long long t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long begin = t * kSortTile + (long long)warp * kSortItemsPerWarp;
    for (int w = 0; w < kSortWarps; ++w) s_cnt[w][threadIdx.x] = 0;
    __syncthreads();
    // pass 1: digit counts of each warp's piece
    for (int r = 0; r < kSortItemsPerWarp / 32; ++r) {
        const long long idx = begin + r * 32 + lane;
        const unsigned d = idx < count ? (sort_key(keys_in, idx, sub) >> shift) & 255u : 256u;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (d < 256u && lane == __ffs(peers) - 1) s_cnt[warp][d] += __popc(peers);  // one writer per digit and round
        __syncwarp();
    }
    __syncthreads();
    // counts -> first output position of every (warp, digit)
    {
        const int d = threadIdx.x;
        unsigned running = offsets[(long long)d * tiles + t];
        for (int w = 0; w < kSortWarps; ++w) {
            const unsigned c = s_cnt[w][d];
            s_cnt[w][d] = running;
            running += c;
        }
    }
    __syncthreads();
    // pass 2: positions, in the same order as pass 1 counted
    for (int r = 0; r < kSortItemsPerWarp / 32; ++r) {
        const long long idx = begin + r * 32 + lane;
        const bool live = idx < count;
        const unsigned key = live ? sort_key(keys_in, idx, sub) : 0u;
        const unsigned d = live ? (key >> shift) & 255u : 256u;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(peers) - 1;
        unsigned base = 0;
        if (live && lane == leader) {
            base = s_cnt[warp][d];
            s_cnt[warp][d] = base + __popc(peers);
        }
        base = __shfl_sync(0xffffffffu, base, leader);
        if (live) {
            const unsigned pos = base + __popc(peers & ((1u << lane) - 1u));
            keys_out[pos] = (int)key;
            perm_out[pos] = perm_in ? __ldg(perm_in + idx) : (unsigned)idx;
        }
        __syncwarp();
    }
}

// ---- exclusive scan of a long array of counts, in place (three kernels)

__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* s_warp, unsigned* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inc = v;
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned w = s_warp[lane];  // kScanThreads / 32 == 32 warps
        unsigned winc = w;
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned o = __shfl_up_sync(0xffffffffu, winc, d);
            if (lane >= d) winc += o;
        }
        s_warp[lane] = winc - w;  // exclusive prefix of the warp totals
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return s_warp[warp] + inc - v;
}

__global__ void __launch_bounds__(kScanThreads)
    scan_chunk_sums_kernel(const unsigned* __restrict__ data, long long count, unsigned* __restrict__ sums) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_total;
    const long long first = (long long)blockIdx.x * kScanChunk + (long long)threadIdx.x * kScanItems;
    unsigned v = 0;
    for (int i = 0; i < kScanItems; ++i)
        if (first + i < count) v += data[first + i];
    block_exclusive_scan(v, s_warp, &s_total);
    if (threadIdx.x == 0) sums[blockIdx.x] = s_total;
}

// One thread block: exclusive scan of the chunk sums, 1024 at a time with a running carry.
__global__ void __launch_bounds__(kScanThreads) scan_sums_kernel(unsigned* __restrict__ sums, long long chunks) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_total;
    unsigned carry = 0;
    for (long long first = 0; first < chunks; first += kScanThreads) {  // block-uniform trip count
        const long long i = first + threadIdx.x;
        const unsigned v = i < chunks ? sums[i] : 0u;
        const unsigned ex = block_exclusive_scan(v, s_warp, &s_total);
        if (i < chunks) sums[i] = carry + ex;
        carry += s_total;
        __syncthreads();  // s_warp / s_total are reused by the next round
    }
}

__global__ void __launch_bounds__(kScanThreads)
    scan_apply_kernel(unsigned* __restrict__ data, long long count, const unsigned* __restrict__ sums) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_total;
    const long long first = (long long)blockIdx.x * kScanChunk + (long long)threadIdx.x * kScanItems;
    unsigned item[kScanItems];
    unsigned v = 0;
    for (int i = 0; i < kScanItems; ++i) {
        item[i] = first + i < count ? data[first + i] : 0u;
        v += item[i];
    }
    unsigned run = sums[blockIdx.x] + block_exclusive_scan(v, s_warp, &s_total);
    for (int i = 0; i < kScanItems; ++i) {
        if (first + i < count) data[first + i] = run;
        run += item[i];
    }
}

// row_of[j] = the row that holds source position j (0-based): eight lanes per row write the row's
// number over the row's positions. (One binary search in row_ptr per position, in order or through
// the permutation, cost 1.1 ms where this costs well under a tenth of that.)
template <typename I>
__global__ void __launch_bounds__(256)
    expand_rows_kernel(long long m, int base, const I* __restrict__ row_ptr, int* __restrict__ row_of) {
    const long long r = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 3;
    const int lane = threadIdx.x & 7;
    if (r >= m) return;
    const int j1 = (int)__ldg(row_ptr + r + 1) - base;
    for (int j = (int)__ldg(row_ptr + r) - base + lane; j < j1; j += 8) row_of[j] = (int)r;
}

// out[k] = row_of[perm[k]]: the column index of the k-th nonzero of the transposed matrix.
// (`sub` is taken off every gathered index: the index base when the source is a caller's array.)
template <typename I>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(long long nnz, const I* __restrict__ row_of, const unsigned* __restrict__ perm,
                       int* __restrict__ out, int sub) {
    const long long k = 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x);
    if (k + 3 < nnz) {
        const uint4 p = __ldcs(reinterpret_cast<const uint4*>(perm + k));
        const int4 r = make_int4((int)__ldg(row_of + p.x) - sub, (int)__ldg(row_of + p.y) - sub,
                                 (int)__ldg(row_of + p.z) - sub, (int)__ldg(row_of + p.w) - sub);
        *reinterpret_cast<int4*>(out + k) = r;
    } else {
        for (long long i = k; i < nnz; ++i) out[i] = (int)__ldg(row_of + perm[i]) - sub;
    }
}

// COO stored as an array of (row, column) pairs -> separate row and column arrays.
__global__ void split_index_pairs_kernel(long long nnz, const int2* __restrict__ pairs, int* __restrict__ rows,
                                         int* __restrict__ cols) {
    const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (j >= nnz) return;
    const int2 p = __ldcs(pairs + j);
    rows[j] = p.x;
    cols[j] = p.y;
}

// flag[0] = 1 if the indices are not in ascending order somewhere.
template <typename I>
__global__ void unsorted_flag_kernel(long long count, const I* __restrict__ idx, int* __restrict__ flag) {
    const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (j + 1 < count && __ldg(idx + j) > __ldg(idx + j + 1)) *flag = 1;
}

// out[k] = val[perm[k]]. Four consecutive k per thread: one 128-bit load of the permutation, four
// gathers in flight, 128-bit stores (perm and out start on 256-byte boundaries of the buffer).
// A separate pass on purpose: gathering inside the SpMV tile kernel was measured at 6.1 ms against
// 2.8 ms for the 27-point stencil, because that kernel's shared-memory footprint leaves too little
// L1 for the four values of a 32-byte sector to be picked up by neighbouring rows before eviction.
template <typename T>
__global__ void __launch_bounds__(256)
    permute_values_kernel(long long nnz, const T* __restrict__ val, const unsigned* __restrict__ perm,
                          T* __restrict__ out, bool conjugate) {
    const long long k = 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x);
    if (k + 3 < nnz) {
        const uint4 p = __ldcs(reinterpret_cast<const uint4*>(perm + k));
        alignas(16) T v[4] = {ldg(val + p.x), ldg(val + p.y), ldg(val + p.z), ldg(val + p.w)};
        if (conjugate) {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = conj_value(v[i]);
        }
        const uint4* src = reinterpret_cast<const uint4*>(v);
        uint4* dst = reinterpret_cast<uint4*>(out + k);
#pragma unroll
        for (int i = 0; i < (int)(4 * sizeof(T) / 16); ++i) __stcs(dst + i, src[i]);
    } else {
        for (long long i = k; i < nnz; ++i) {
            const T v = ldg(val + perm[i]);
            out[i] = conjugate ? conj_value(v) : v;
        }
    }
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

// In-place exclusive prefix sum of `count` unsigned values; `sums` is scratch of scan_scratch_elems(count) words.
long long scan_scratch_elems(long long count) { return (count + kScanChunk - 1) / kScanChunk; }
cudaError_t exclusive_scan_u32(cudaStream_t s, unsigned* data, long long count, unsigned* sums) {
    if (count <= 0) return cudaSuccess;
    const long long chunks = scan_scratch_elems(count);
    scan_chunk_sums_kernel<<<(unsigned)chunks, kScanThreads, 0, s>>>(data, count, sums);
    scan_sums_kernel<<<1, kScanThreads, 0, s>>>(sums, chunks);
    scan_apply_kernel<<<(unsigned)chunks, kScanThreads, 0, s>>>(data, count, sums);
    return cudaGetLastError();
}

TransposePlan transpose_plan(int64_t m, int64_t n, int64_t nnz, size_t value_size) {
    (void)m;
    TransposePlan p;
    int bits = 1;
    while (bits < 31 && (int64_t(1) << bits) < n) ++bits;
    p.passes = (bits + 7) / 8;
    p.tiles = (nnz + kSortTile - 1) / kSortTile;
    p.hist_count = 256 * p.tiles;
    p.scan_chunks = (p.hist_count + kScanChunk - 1) / kScanChunk;
    size_t off = 0;
    p.off_ptr = off;
    off += align256(size_t(n + 1) * 4);
    for (int i = 0; i < 2; ++i) {
        p.off_keys[i] = off;
        off += align256(size_t(nnz) * 4);
    }
    for (int i = 0; i < 2; ++i) {
        p.off_perm[i] = off;
        off += align256(size_t(nnz) * 4);
    }
    p.off_val = off;
    off += align256(size_t(nnz) * value_size);
    p.off_hist = off;
    off += align256(size_t(p.hist_count) * 4);
    p.off_sums = off;
    off += align256(size_t(p.scan_chunks) * 4);
    p.bytes = off;
    return p;
}

// Stable sort of the positions 0 .. nnz-1 by key (key - base in [0, 2^(8 passes))): leaves the sorted
// 0-based keys in keys[final_slot()] and the permutation in perm[final_slot()].
template <typename I>
static cudaError_t radix_sort_positions(cudaStream_t s, int64_t nnz, int base, const I* key_src,
                                        const TransposePlan& p, void* buf) {
    char* b = static_cast<char*>(buf);
    int* keys[2] = {reinterpret_cast<int*>(b + p.off_keys[0]), reinterpret_cast<int*>(b + p.off_keys[1])};
    unsigned* perm[2] = {reinterpret_cast<unsigned*>(b + p.off_perm[0]), reinterpret_cast<unsigned*>(b + p.off_perm[1])};
    unsigned* hist = reinterpret_cast<unsigned*>(b + p.off_hist);
    unsigned* sums = reinterpret_cast<unsigned*>(b + p.off_sums);
    cudaError_t e = cudaSuccess;
    for (int pass = 0; pass < p.passes && nnz > 0; ++pass) {
        const int dst = pass & 1;
        const int shift = 8 * pass;
        if (pass == 0)  // the caller's indices, with their base, and the identity permutation
            radix_hist_kernel<I><<<(unsigned)p.tiles, kSortThreads, 0, s>>>(key_src, base, nnz, shift, hist, p.tiles);
        else
            radix_hist_kernel<int><<<(unsigned)p.tiles, kSortThreads, 0, s>>>(keys[dst ^ 1], 0, nnz, shift, hist, p.tiles);
        scan_chunk_sums_kernel<<<(unsigned)p.scan_chunks, kScanThreads, 0, s>>>(hist, p.hist_count, sums);
        scan_sums_kernel<<<1, kScanThreads, 0, s>>>(sums, p.scan_chunks);
        scan_apply_kernel<<<(unsigned)p.scan_chunks, kScanThreads, 0, s>>>(hist, p.hist_count, sums);
        if (pass == 0)
            radix_scatter_kernel<I><<<(unsigned)p.tiles, kSortThreads, 0, s>>>(key_src, base, nullptr, keys[dst], perm[dst],
                                                                                nnz, shift, hist, p.tiles);
        else
            radix_scatter_kernel<int><<<(unsigned)p.tiles, kSortThreads, 0, s>>>(keys[dst ^ 1], 0, perm[dst ^ 1], keys[dst],
                                                                                  perm[dst], nnz, shift, hist, p.tiles);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    return e;
}

template <typename I>
cudaError_t coo_sort_structure(cudaStream_t s, int64_t key_range, int64_t nnz, int base, const I* key_idx,
                               const I* other_idx, const TransposePlan& p, void* buf) {
    char* b = static_cast<char*>(buf);
    int32_t* ptr = reinterpret_cast<int32_t*>(b + p.off_ptr);
    int* keys[2] = {reinterpret_cast<int*>(b + p.off_keys[0]), reinterpret_cast<int*>(b + p.off_keys[1])};
    unsigned* perm[2] = {reinterpret_cast<unsigned*>(b + p.off_perm[0]), reinterpret_cast<unsigned*>(b + p.off_perm[1])};
    cudaError_t e = radix_sort_positions(s, nnz, base, key_idx, p, buf);
    if (e != cudaSuccess) return e;
    const int fin = p.final_slot();
    if ((e = coo_row_offsets(s, key_range, nnz, 0, keys[fin], ptr)) != cudaSuccess) return e;
    if (nnz > 0) {
        gather_rows_kernel<I><<<(unsigned)((nnz + 1023) / 1024), 256, 0, s>>>(nnz, other_idx, perm[fin], keys[fin ^ 1], base);
        e = cudaGetLastError();
    }
    return e;
}

__device__ int g_unsorted_flag;  // result word of indices_unsorted (one check at a time per process)
static std::mutex g_unsorted_lock;  // one lock for every index type: the instantiations share the word above

cudaError_t split_index_pairs(cudaStream_t s, int64_t nnz, const int32_t* pairs, int32_t* rows, int32_t* cols) {
    if (nnz == 0) return cudaSuccess;
    split_index_pairs_kernel<<<(unsigned)((nnz + 255) / 256), 256, 0, s>>>(nnz, reinterpret_cast<const int2*>(pairs), rows,
                                                                         cols);
    return cudaGetLastError();
}

template <typename I>
cudaError_t indices_unsorted(cudaStream_t s, int64_t count, const I* idx, int* host_flag) {
    std::lock_guard<std::mutex> g(g_unsorted_lock);
    int* device_flag = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&device_flag), g_unsorted_flag);
    if (e == cudaSuccess) e = cudaMemsetAsync(device_flag, 0, sizeof(int), s);
    if (e == cudaSuccess && count > 1) {
        unsorted_flag_kernel<I><<<(unsigned)((count + 255) / 256), 256, 0, s>>>(count, idx, device_flag);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_flag, device_flag, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e;
}

template <typename I>
cudaError_t transpose_structure(cudaStream_t s, int64_t m, int64_t n, int64_t nnz, int base, const I* row_ptr,
                                const I* col, const TransposePlan& p, void* buf) {
    char* b = static_cast<char*>(buf);
    int32_t* ptr = reinterpret_cast<int32_t*>(b + p.off_ptr);
    int* keys[2] = {reinterpret_cast<int*>(b + p.off_keys[0]), reinterpret_cast<int*>(b + p.off_keys[1])};
    unsigned* perm[2] = {reinterpret_cast<unsigned*>(b + p.off_perm[0]), reinterpret_cast<unsigned*>(b + p.off_perm[1])};
    cudaError_t e = radix_sort_positions(s, nnz, base, col, p, buf);
    if (e != cudaSuccess) return e;
    const int fin = p.final_slot();
    // Row offsets of the transposed matrix from the sorted (0-based) columns; with no nonzeros they are all zero.
    if ((e = coo_row_offsets(s, n, nnz, 0, keys[fin], ptr)) != cudaSuccess) return e;
    if (nnz > 0) {
        // Both buffers the last pass did not write are free now: one takes the row of every source
        // position, the other the column indices of the transposed matrix.
        int* row_of = reinterpret_cast<int*>(perm[fin ^ 1]);
        expand_rows_kernel<I><<<(unsigned)((m * 8 + 255) / 256), 256, 0, s>>>(m, base, row_ptr, row_of);
        gather_rows_kernel<int><<<(unsigned)((nnz + 1023) / 1024), 256, 0, s>>>(nnz, row_of, perm[fin], keys[fin ^ 1], 0);
        e = cudaGetLastError();
    }
    return e;
}

template <typename T>
cudaError_t transpose_values(cudaStream_t s, int64_t nnz, const T* val, const TransposePlan& p, void* buf,
                             bool conjugate) {
    if (nnz == 0) return cudaSuccess;
    char* b = static_cast<char*>(buf);
    permute_values_kernel<T><<<(unsigned)((nnz + 1023) / 1024), 256, 0, s>>>(
        nnz, val, reinterpret_cast<const unsigned*>(b + p.off_perm[p.final_slot()]), reinterpret_cast<T*>(b + p.off_val),
        conjugate);
    return cudaGetLastError();
}

#define INSTANTIATE_INDEX(I)                                                                                  \
    template cudaError_t transpose_structure<I>(cudaStream_t, int64_t, int64_t, int64_t, int, const I*, const I*, \
                                                const TransposePlan&, void*);                                   \
    template cudaError_t coo_sort_structure<I>(cudaStream_t, int64_t, int64_t, int, const I*, const I*,          \
                                               const TransposePlan&, void*);                                    \
    template cudaError_t indices_unsorted<I>(cudaStream_t, int64_t, const I*, int*);
INSTANTIATE_INDEX(int32_t)
INSTANTIATE_INDEX(int64_t)
#undef INSTANTIATE_INDEX

template cudaError_t transpose_values<float>(cudaStream_t, int64_t, const float*, const TransposePlan&, void*, bool);
template cudaError_t transpose_values<double>(cudaStream_t, int64_t, const double*, const TransposePlan&, void*, bool);
template cudaError_t transpose_values<cfloat>(cudaStream_t, int64_t, const cfloat*, const TransposePlan&, void*, bool);
template cudaError_t transpose_values<cdouble>(cudaStream_t, int64_t, const cdouble*, const TransposePlan&, void*,
                                               bool);

}  // namespace mcsp_b200
