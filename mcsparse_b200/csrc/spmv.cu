// CSR SpMV for sm_100a: merge-path analysis, tiled kernel, carry fix-up, row-group kernel.
//
// Replaces the reference's one-warp-per-row kernel
// (mcsparse/src/kernels/level2/spmv/csr_vector_device.hpp:22-79, launched from
// mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:203-259) with the same arithmetic
// y[r] = beta * y[r] + alpha * sum_j val[j] * x[col[j] - base].
//
// The path is HBM-bound: each nonzero moves sizeof(T) + 4 bytes once, so the kernels are
// organised around wide, coalesced, streaming loads of col/val with many bytes in flight
// per SM, while x is gathered through L1/L2 with default caching.
#include <cstdio>

#include "internal.h"

namespace mcsp_b200 {

namespace {

constexpr int kThreads = 256;

template <typename T>
struct TileCfg;
template <>
struct TileCfg<float> {
    static constexpr int kItemsPerThread = MCSPARSE_B200_SPMV_TILE_ITEMS_F32 / kThreads;
};
template <>
struct TileCfg<double> {
    static constexpr int kItemsPerThread = MCSPARSE_B200_SPMV_TILE_ITEMS_F64 / kThreads;
};

// ---------------------------------------------------------------------------------------
// K0: merge-path analysis. Thread t finds where diagonal min(t * items_per_tile, m + nnz)
// crosses the merge of row ends and nonzero indices. Same search, same tie-break (a row end
// equal to a nonzero index is taken first) as the CPU partition it is checked against.
// ---------------------------------------------------------------------------------------
__global__ void merge_path_partition_kernel(int m, int nnz, int base, const int* __restrict__ row_ptr,
                                            int items_per_tile, long long num_tiles, int2* __restrict__ starts) {
    long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t > num_tiles) return;
    long long items = (long long)m + nnz;
    long long diag = t * items_per_tile;
    if (diag > items) diag = items;
    long long lo = diag > nnz ? diag - nnz : 0;
    long long hi = diag < m ? diag : m;
    while (lo < hi) {
        long long mid = (lo + hi) >> 1;
        if ((long long)__ldg(row_ptr + mid + 1) - base <= diag - mid - 1)
            lo = mid + 1;
        else
            hi = mid;
    }
    starts[t] = make_int2((int)lo, (int)(diag - lo));
}

// ---------------------------------------------------------------------------------------
// Streaming 4-element loads of the matrix arrays (evict-first: A is read exactly once and
// must not push x out of L2).
// ---------------------------------------------------------------------------------------
template <typename T>
struct Quad;
template <>
struct Quad<float> {
    float4 v;
    __device__ __forceinline__ void load(const float* p) { v = __ldcs(reinterpret_cast<const float4*>(p)); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Quad<double> {
    double2 lo, hi;
    __device__ __forceinline__ void load(const double* p) {
        lo = __ldcs(reinterpret_cast<const double2*>(p));
        hi = __ldcs(reinterpret_cast<const double2*>(p) + 1);
    }
    __device__ __forceinline__ void store(double* p) const {
        reinterpret_cast<double2*>(p)[0] = lo;
        reinterpret_cast<double2*>(p)[1] = hi;
    }
};

// ---------------------------------------------------------------------------------------
// K1: tiled SpMV. Block t owns merge items [t * TILE, (t + 1) * TILE): `nrows` row ends and
// `nnz_tile` nonzeros (nrows + nnz_tile = TILE except in the last tile).
//
//   phase 1  the tile's slice of col/val is staged in shared memory with 128-bit coalesced
//            streaming loads (all of a thread's loads are issued before the first use), together
//            with the row ends of the tile's rows.
//   phase 2  one of two block-uniform paths, chosen from the longest row piece in the tile:
//     short rows  G lanes per row (G = 1, 2, ... 32), each lane walking its share of the row in
//                 shared memory: sum += val * x[col]. With one or two lanes per row the lanes of a
//                 warp are consecutive rows, so for banded / stencil matrices one gather
//                 instruction touches a handful of L1 sectors instead of one per lane. Results are
//                 written to y straight from registers.
//     long rows   products are formed in place (lane-consecutive gathers), then each thread walks
//                 WALK consecutive merge items (balanced whatever the row lengths); thread carries
//                 (a row open at a thread boundary) are combined with a warp-shuffle segmented scan
//                 and across the 8 warps in a fixed order; coalesced epilogue from shared memory.
//   Both paths leave the sum of the row still open at the tile's end in carry_{row,val}[t].
//
// On B200 the L1 data pipe (wavefronts of the x gathers plus shared-memory traffic) saturates
// before HBM does, so the kernel is organised to spend few L1 wavefronts per nonzero.
// No atomics: every addition has a fixed place, so results are reproducible run to run.
// VEC = false is the same kernel with scalar loads for arrays that are not 16-byte aligned.
// ---------------------------------------------------------------------------------------
template <typename T, int THREADS, int IPT, bool VEC>
__global__ void __launch_bounds__(THREADS)
    spmv_tile_kernel(int m, int base, const int* __restrict__ row_ptr, const int* __restrict__ col,
                     const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y, ScalarArg<T> alpha_arg,
                     ScalarArg<T> beta_arg, const int2* __restrict__ tile_starts, int* __restrict__ carry_row,
                     T* __restrict__ carry_val) {
    constexpr int TILE = THREADS * IPT;
    constexpr int NWARPS = THREADS / 32;
    constexpr int CPT = IPT / 4;     // 4-element chunks per thread in the unrolled staging pass
    constexpr int WALK = IPT + 1;    // merge items per thread in the long-row walk: odd, so that the
                                     // stride-WALK shared reads of a warp fall in distinct banks
    static_assert(IPT % 4 == 0, "items per thread must be a multiple of 4");

    __shared__ __align__(32) T s_val[TILE + 8];  // values (then products); long-row path: row sums behind them
    __shared__ __align__(16) int s_col[TILE + 8];  // column indices, then the tile's row ends behind them
    __shared__ int s_warp_row[NWARPS];  // long-row path: last carry of each warp
    __shared__ T s_warp_sum[NWARPS];
    __shared__ int s_warp_maxlen[NWARPS];

    const int tid = threadIdx.x;
    const int t = blockIdx.x;
    const int2 s0 = tile_starts[t];
    const int2 s1 = tile_starts[t + 1];
    const int row_s = s0.x, nz_s = s0.y;
    const int nrows = s1.x - s0.x;
    const int nz_e = s1.y;
    const int nnz_tile = nz_e - nz_s;
    const int tile_items = nrows + nnz_tile;

    const int a0 = VEC ? (nz_s & ~3) : nz_s;  // nonzero a0 + k is staged at index k
    const int head = nz_s - a0;
    const int* const colv = s_col + head;  // colv[k], valv[k]: k-th nonzero of the tile
    T* const valv = s_val + head;
    int* const s_row_end = s_col + head + nnz_tile;  // nrows + 1 entries; nrows + nnz_tile <= TILE

    // ---- phase 1: stage col / val
    if (VEC) {
        const int nchunks = (head + nnz_tile + 3) >> 2;
        int4 cc[CPT];
        Quad<T> vv[CPT];
        bool full[CPT];
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = tid + k * THREADS;
            const int g = a0 + 4 * c;
            full[k] = (c < nchunks) && (g >= nz_s) && (g + 4 <= nz_e);
            if (full[k]) {
                cc[k] = __ldcs(reinterpret_cast<const int4*>(col + g));
                vv[k].load(val + g);
            }
        }
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            if (full[k]) {
                *reinterpret_cast<int4*>(s_col + 4 * (tid + k * THREADS)) = cc[k];
                vv[k].store(s_val + 4 * (tid + k * THREADS));
            }
        }
        // Ragged chunks (the tile's first and last) and the one chunk beyond the unrolled pass.
        for (int c = tid; c < nchunks; c += THREADS) {
            const int g = a0 + 4 * c;
            const bool done = (c < CPT * THREADS) && (g >= nz_s) && (g + 4 <= nz_e);
            if (!done) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int gi = g + e;
                    if (gi >= nz_s && gi < nz_e) {
                        s_col[4 * c + e] = __ldcs(col + gi);
                        s_val[4 * c + e] = __ldcs(val + gi);
                    }
                }
            }
        }
    } else {
        for (int k = tid; k < nnz_tile; k += THREADS) {
            s_col[k] = __ldcs(col + nz_s + k);
            s_val[k] = __ldcs(val + nz_s + k);
        }
    }

    // Row ends in tile-local nonzero coordinates; entry nrows is the row left open.
    // Alongside: the longest piece of a row inside this tile, which selects the phase-2 path.
    int maxlen = 0;
    for (int i = tid; i <= nrows; i += THREADS) {
        const int r = row_s + i;
        int e = (r < m) ? __ldg(row_ptr + r + 1) - base : nz_e;
        e = min(e, nz_e);
        const int b = (r < m) ? max(__ldg(row_ptr + r) - base, nz_s) : nz_e;
        maxlen = max(maxlen, e - b);
        s_row_end[i] = e - nz_s;
    }
    maxlen = __reduce_max_sync(0xffffffffu, maxlen);
    if ((tid & 31) == 0) s_warp_maxlen[tid >> 5] = maxlen;
    __syncthreads();

    // ---- phase 2
    maxlen = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) maxlen = max(maxlen, s_warp_maxlen[w]);
    int lgG = 0;
    while ((32 << lgG) < maxlen) ++lgG;  // lanes per row so that each lane sums <= 32 products ...
    while (lgG < 2 && ((nrows + 1) << (lgG + 1)) <= THREADS) ++lgG;  // ... and idle threads are put to use
    const bool short_rows = lgG <= 5 && (((nrows + 1) << lgG) <= 8 * THREADS);
    const T* const xb = x - base;
    const T alpha = alpha_arg.get();
    const T beta = beta_arg.get();

    if (short_rows) {
        const int G = 1 << lgG;
        const int ngroups = THREADS >> lgG;
        const int gidx = tid >> lgG, glane = tid & (G - 1);
        for (int i0 = 0; i0 <= nrows; i0 += ngroups) {  // block-uniform trip count
            const int i = i0 + gidx;
            int b = 0, e = 0;
            if (i <= nrows) {
                b = (i == 0) ? 0 : s_row_end[i - 1];
                e = s_row_end[i];
            }
            T sum = T(0);
            int k = b + glane;
            for (; k + 3 * G < e; k += 4 * G) {  // four independent gathers in flight per lane
                const T x0 = __ldg(xb + colv[k]), x1 = __ldg(xb + colv[k + G]);
                const T x2 = __ldg(xb + colv[k + 2 * G]), x3 = __ldg(xb + colv[k + 3 * G]);
                sum += valv[k] * x0;
                sum += valv[k + G] * x1;
                sum += valv[k + 2 * G] * x2;
                sum += valv[k + 3 * G] * x3;
            }
            for (; k < e; k += G) sum += valv[k] * __ldg(xb + colv[k]);
            for (int d = G >> 1; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
            if (glane == 0 && i <= nrows) {
                if (i < nrows) {
                    T v = alpha * sum;
                    if (beta != T(0)) v += beta * y[row_s + i];
                    y[row_s + i] = v;
                } else {
                    carry_row[t] = row_s + nrows;
                    carry_val[t] = sum;
                }
            }
        }
        return;
    }

    // ---- long rows: products in place, merge walk, segmented reduction of the carries
    T* const s_y = valv + nnz_tile;  // s_y[i]: row row_s + i, i in [0, nrows]
    for (int k = tid; k < nnz_tile; k += THREADS) valv[k] *= __ldg(xb + colv[k]);
    for (int i = tid; i <= nrows; i += THREADS) s_y[i] = T(0);
    __syncthreads();

    const int d0 = min(tid * WALK, tile_items);
    const int d1 = min(d0 + WALK, tile_items);
    int lo = max(d0 - nnz_tile, 0), hi = min(d0, nrows);
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_row_end[mid] <= d0 - mid - 1)
            lo = mid + 1;
        else
            hi = mid;
    }
    int r = lo;       // tile-local row
    int k = d0 - lo;  // tile-local nonzero
    int end = s_row_end[r];
    T sum = T(0);
#pragma unroll
    for (int it = 0; it < WALK; ++it) {
        if (d0 + it < d1) {
            if (k < end) {
                sum += valv[k];
                ++k;
            } else {
                s_y[r] = sum;
                sum = T(0);
                ++r;
                end = s_row_end[r];
            }
        }
    }

    // segmented reduction of the per-thread carries (key = r, value = sum)
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const T up = __shfl_up_sync(0xffffffffu, sum, d);
        const int ru = __shfl_up_sync(0xffffffffu, r, d);
        if (lane >= d && ru == r) sum += up;
    }
    const int rn = __shfl_down_sync(0xffffffffu, r, 1);
    __syncthreads();  // all direct row sums are in s_y
    if (lane == 31) {
        s_warp_row[warp] = r;
        s_warp_sum[warp] = sum;
    } else if (rn != r) {
        s_y[r] += sum;  // the run of threads holding row r ends inside this warp: single writer
    }
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) s_y[s_warp_row[w]] += s_warp_sum[w];
    }
    __syncthreads();

    for (int i = tid; i < nrows; i += THREADS) {
        T v = alpha * s_y[i];
        if (beta != T(0)) v += beta * y[row_s + i];
        y[row_s + i] = v;
    }
    if (tid == 0) {
        carry_row[t] = row_s + nrows;
        carry_val[t] = s_y[nrows];
    }
}

// Adds the carries of rows that cross tile boundaries. The first tile of each run of equal
// carry rows sums the run in tile order, so the result does not depend on scheduling.
template <typename T>
__global__ void spmv_carry_fixup_kernel(int m, long long num_tiles, const int* __restrict__ carry_row,
                                        const T* __restrict__ carry_val, T* __restrict__ y, ScalarArg<T> alpha_arg) {
    long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= num_tiles) return;
    const int r = carry_row[t];
    if (r >= m) return;
    if (t > 0 && carry_row[t - 1] == r) return;
    T sum = carry_val[t];
    for (long long u = t + 1; u < num_tiles && carry_row[u] == r; ++u) sum += carry_val[u];
    y[r] += alpha_arg.get() * sum;
}

// ---------------------------------------------------------------------------------------
// K2: row-group SpMV. G lanes share a row (G chosen from the mean row length), lane-strided
// loads, xor-shuffle reduction. Needs no analysis and no work buffer: the kernel behind the
// legacy csrmv calls, which have neither.
// ---------------------------------------------------------------------------------------
template <typename T, int G>
__global__ void __launch_bounds__(kThreads)
    spmv_rowgroup_kernel(int m, int base, const int* __restrict__ row_ptr, const int* __restrict__ col,
                         const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y,
                         ScalarArg<T> alpha_arg, ScalarArg<T> beta_arg) {
    const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) / G;
    const int lane = threadIdx.x & (G - 1);
    const bool active = gid < m;
    T sum = T(0);
    if (active) {
        const int j0 = __ldg(row_ptr + gid) - base, j1 = __ldg(row_ptr + gid + 1) - base;
        const T* xb = x - base;
        for (int j = j0 + lane; j < j1; j += G) sum += __ldcs(val + j) * __ldg(xb + __ldcs(col + j));
    }
#pragma unroll
    for (int d = G >> 1; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d, G);
    if (active && lane == 0) {
        const T alpha = alpha_arg.get(), beta = beta_arg.get();
        T v = alpha * sum;
        if (beta != T(0)) v += beta * y[gid];
        y[gid] = v;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
SpmvWorkspace spmv_workspace(int64_t m, int64_t nnz, size_t value_size) {
    SpmvWorkspace ws;
    ws.items_per_tile = value_size == 8 ? MCSPARSE_B200_SPMV_TILE_ITEMS_F64 : MCSPARSE_B200_SPMV_TILE_ITEMS_F32;
    const int64_t items = m + nnz;
    ws.num_tiles = (items + ws.items_per_tile - 1) / ws.items_per_tile;
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    ws.off_carry_row = up(size_t(ws.num_tiles + 1) * 8);
    ws.off_carry_val = ws.off_carry_row + up(size_t(ws.num_tiles) * 4);
    ws.bytes = ws.off_carry_val + up(size_t(ws.num_tiles) * value_size);
    return ws;
}

cudaError_t spmv_analysis(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                          const SpmvWorkspace& ws, void* buf) {
    const long long n = ws.num_tiles + 1;
    const int threads = 128;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    merge_path_partition_kernel<<<blocks, threads, 0, s>>>((int)m, (int)nnz, base, row_ptr, ws.items_per_tile,
                                                           ws.num_tiles, reinterpret_cast<int2*>(buf));
    return cudaGetLastError();
}

template <typename T>
cudaError_t spmv_tiled(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                       const int32_t* col, const T* val, const T* x, T* y, ScalarArg<T> alpha, ScalarArg<T> beta,
                       const SpmvWorkspace& ws, void* buf) {
    (void)nnz;
    if (ws.num_tiles == 0) return cudaSuccess;
    char* base_ptr = static_cast<char*>(buf);
    const int2* starts = reinterpret_cast<const int2*>(base_ptr);
    int* carry_row = reinterpret_cast<int*>(base_ptr + ws.off_carry_row);
    T* carry_val = reinterpret_cast<T*>(base_ptr + ws.off_carry_val);
    constexpr int IPT = TileCfg<T>::kItemsPerThread;
    const bool aligned =
        ((reinterpret_cast<uintptr_t>(col) | reinterpret_cast<uintptr_t>(val)) & 15) == 0;
    const unsigned grid = (unsigned)ws.num_tiles;
    if (aligned)
        spmv_tile_kernel<T, kThreads, IPT, true><<<grid, kThreads, 0, s>>>(
            (int)m, base, row_ptr, col, val, x, y, alpha, beta, starts, carry_row, carry_val);
    else
        spmv_tile_kernel<T, kThreads, IPT, false><<<grid, kThreads, 0, s>>>(
            (int)m, base, row_ptr, col, val, x, y, alpha, beta, starts, carry_row, carry_val);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int threads = 256;
    spmv_carry_fixup_kernel<T><<<(unsigned)((ws.num_tiles + threads - 1) / threads), threads, 0, s>>>(
        (int)m, ws.num_tiles, carry_row, carry_val, y, alpha);
    return cudaGetLastError();
}

template <typename T, int G>
static cudaError_t launch_rowgroup(cudaStream_t s, int64_t m, int base, const int32_t* row_ptr, const int32_t* col,
                                   const T* val, const T* x, T* y, ScalarArg<T> alpha, ScalarArg<T> beta) {
    const long long threads_total = m * G;
    const unsigned grid = (unsigned)((threads_total + kThreads - 1) / kThreads);
    spmv_rowgroup_kernel<T, G><<<grid, kThreads, 0, s>>>((int)m, base, row_ptr, col, val, x, y, alpha, beta);
    return cudaGetLastError();
}

template <typename T>
cudaError_t spmv_rowgroup(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                          const int32_t* col, const T* val, const T* x, T* y, ScalarArg<T> alpha,
                          ScalarArg<T> beta) {
    if (m == 0) return cudaSuccess;
    const double mean = double(nnz) / double(m);
    if (mean <= 3.0) return launch_rowgroup<T, 2>(s, m, base, row_ptr, col, val, x, y, alpha, beta);
    if (mean <= 6.0) return launch_rowgroup<T, 4>(s, m, base, row_ptr, col, val, x, y, alpha, beta);
    if (mean <= 12.0) return launch_rowgroup<T, 8>(s, m, base, row_ptr, col, val, x, y, alpha, beta);
    if (mean <= 24.0) return launch_rowgroup<T, 16>(s, m, base, row_ptr, col, val, x, y, alpha, beta);
    return launch_rowgroup<T, 32>(s, m, base, row_ptr, col, val, x, y, alpha, beta);
}

// ---------------------------------------------------------------------------------------
// Built-in work area for mcsparseB200SpMVNoAlloc: callers that must not allocate device
// memory (and so cannot size and provide the external buffer) get the partition and carry
// arrays from this fixed array instead. It is part of the loaded module, so every GPU that
// loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_spmv_static_scratch[MCSPARSE_B200_NOALLOC_SCRATCH_BYTES];

// Device address of the array above on the current device. The array's name is only a
// host-side handle for the symbol; kernels need the address cudaGetSymbolAddress reports for
// the device that is current. Looked up once per device and remembered.
cudaError_t spmv_static_scratch(void** ptr, size_t* bytes) {
    constexpr int kMaxDevices = 64;
    static std::mutex lock;
    static void* cached[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(lock);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_spmv_static_scratch);
        if (e != cudaSuccess) return e;
        cached[dev] = p;
    }
    *ptr = cached[dev];
    *bytes = sizeof(g_spmv_static_scratch);
    return cudaSuccess;
}

#define INSTANTIATE(T)                                                                                         \
    template cudaError_t spmv_tiled<T>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*,    \
                                       const T*, const T*, T*, ScalarArg<T>, ScalarArg<T>,                     \
                                       const SpmvWorkspace&, void*);                                           \
    template cudaError_t spmv_rowgroup<T>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*, \
                                          const T*, const T*, T*, ScalarArg<T>, ScalarArg<T>);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace mcsp_b200
