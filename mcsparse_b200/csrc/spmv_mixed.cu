// CSR SpMV with low-precision operands: A and x in fp16, bf16 or int8, sums in fp32 (int32 for the
// all-integer case), y in fp32, in the operands' own type, or in int32.
//
// Replaces the instantiations of mcspSpmvCsrVectorKernel with differing input / compute / output types
// (mcsparse/src/kernels/level2/spmv/csr_vector_device.hpp:22-79, routed by mcspMixedPrecisionSpMVImpl,
// mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:492-561; the reference compiles these cases only for
// MetaX hardware). Same arithmetic: every product is formed from the operands converted to the compute
// type, the row sum is kept in the compute type, y[r] = beta * compute(y[r]) + alpha * sum is converted to
// y's type (round to nearest even) once.
//
// The matrix moves 4 + 2 (or 4 + 1) bytes per nonzero, so what matters is bytes in flight and work balance, as for
// the fp32 / fp64 kernels; the kernel uses the same merge-path partition (2048 merge items per tile, 256 threads)
// and the same two in-tile paths (lanes per row for short rows, the merge walk for long ones). Differences:
//   - the tile's column indices and values are loaded lane-consecutively into registers (sixteen independent loads
//     per thread before the first use) instead of by bulk copies;
//   - sums and products are in the compute type;
//   - a row that continues from an earlier tile is not added into y piecewise (y may be a 16-bit type, and the
//     result is to be rounded once): the tile leaves the row's local part in head_val[t] and a second kernel adds the
//     carries of the tiles before it and writes y.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace mcsp_b200 {

namespace {

constexpr int kThreads = 256;

// head_val (one sum per tile) is the last array of the work area, behind what the fp32 kernels use for the
// same partition.
size_t head_bytes(const SpmvWorkspace& ws) { return (size_t(ws.num_tiles) * 4 + 255) & ~size_t(255); }
size_t head_offset(const SpmvWorkspace& ws) { return ws.bytes - head_bytes(ws); }

template <typename C, typename V>
__device__ __forceinline__ C widen(V v);
template <>
__device__ __forceinline__ float widen<float, __half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float widen<float, int8_t>(int8_t v) { return (float)v; }
template <>
__device__ __forceinline__ float widen<float, float>(float v) { return v; }
template <>
__device__ __forceinline__ int widen<int, int8_t>(int8_t v) { return (int)v; }
template <>
__device__ __forceinline__ int widen<int, int>(int v) { return v; }

template <typename Y, typename C>
__device__ __forceinline__ Y narrow(C v);
template <>
__device__ __forceinline__ float narrow<float, float>(float v) { return v; }
template <>
__device__ __forceinline__ __half narrow<__half, float>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ int narrow<int, int>(int v) { return v; }

__device__ __forceinline__ float times(float a, float b) { return a * b; }
__device__ __forceinline__ int times(int a, int b) { return a * b; }

// Six resident blocks per SM (40 registers): what the default shared-memory carve-out admits. Asking for the
// largest carve-out to fit eight shrinks L1 and doubles the time of the scattered-column matrices.
constexpr int kMinBlocks = 6;
constexpr int kItemsPerThread = 8;
constexpr int kTile = kThreads * kItemsPerThread;  // merge items per tile: the fp32 kernels' small tile

// V: type of A's values and of x; C: compute type (float or int); Y: type of y.
// Block t owns merge items [t * kTile, (t + 1) * kTile): nrows row ends and nnz_tile nonzeros.
// WALK_ONLY: every tile takes the merge walk (no shared memory for the short-row path: more of it is left to L1).
template <typename V, typename C, typename Y, bool WALK_ONLY>
__global__ void __launch_bounds__(kThreads, kMinBlocks)
    spmv_mixed_tile_kernel(int m, int base, const int* __restrict__ row_ptr, const int* __restrict__ col,
                           const V* __restrict__ val, const V* __restrict__ x, Y* __restrict__ y, ScalarArg<C> alpha_arg,
                           ScalarArg<C> beta_arg, const int2* __restrict__ tile_starts, int* __restrict__ carry_row,
                           C* __restrict__ carry_val, C* __restrict__ head_val) {
    constexpr int IPT = kItemsPerThread, NWARPS = kThreads / 32;
    constexpr int WALK = IPT + 1;  // odd: the stride-WALK shared reads of a warp fall in distinct banks
    __shared__ C s_prod[kTile + 2];       // long rows: products, behind them the sums of the tile's rows (nrows + 1);
                                          // short rows: the tile's column indices
    __shared__ int s_row_end[kTile + 2];  // row ends in tile-local nonzero coordinates; entry nrows: the open row
    __shared__ V s_val[WALK_ONLY ? 1 : kTile];  // short rows: the tile's values
    __shared__ int s_warp_row[NWARPS];
    __shared__ C s_warp_sum[NWARPS];
    __shared__ int s_warp_maxlen[NWARPS];
    static_assert(sizeof(C) == sizeof(int), "the column indices share s_prod");

    const int tid = threadIdx.x, t = blockIdx.x;
    const int2 s0 = tile_starts[t], s1 = tile_starts[t + 1];
    const int row_s = s0.x, nz_s = s0.y, nz_e = s1.y;
    const int nrows = s1.x - s0.x, nnz_tile = nz_e - nz_s, tile_items = nrows + nnz_tile;

    // ---- loads: lane-consecutive nonzeros, all issued before the first use
    int c[IPT];
    V a[IPT];
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
        const int k = tid + j * kThreads;
        const bool in = k < nnz_tile;
        c[j] = in ? __ldcs(col + nz_s + k) : base;
        a[j] = in ? val[nz_s + k] : V(0);
    }
    int maxlen = 0;  // the longest piece of a row inside this tile selects the path below
    for (int i = tid; i <= nrows; i += kThreads) {
        const int r = row_s + i;
        const int e = min((r < m) ? __ldg(row_ptr + r + 1) - base : nz_e, nz_e);
        if constexpr (!WALK_ONLY) {
            const int b = (r < m) ? max(__ldg(row_ptr + r) - base, nz_s) : nz_e;
            maxlen = max(maxlen, e - b);
        }
        s_row_end[i] = e - nz_s;
    }
    bool short_rows = false;
    int lgG = 0;
    if constexpr (!WALK_ONLY) {
        maxlen = __reduce_max_sync(0xffffffffu, maxlen);
        if ((tid & 31) == 0) s_warp_maxlen[tid >> 5] = maxlen;
        __syncthreads();
        maxlen = 0;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) maxlen = max(maxlen, s_warp_maxlen[w]);
        while ((32 << lgG) < maxlen) ++lgG;  // lanes per row so that each lane sums <= 32 products ...
        while (lgG < 2 && ((nrows + 1) << (lgG + 1)) <= kThreads) ++lgG;  // ... and idle threads are put to use
        short_rows = lgG <= 5 && (((nrows + 1) << lgG) <= 8 * kThreads);
    }
    const bool continued = nrows > 0 && __ldg(row_ptr + row_s) - base < nz_s;  // the first row began in an earlier tile
    const V* const xb = x - base;
    const C alpha = alpha_arg.get(), beta = beta_arg.get();

    if (short_rows) {
        // G lanes per row, each walking its share of the row in shared memory. With one or two lanes per row the
        // lanes of a warp are consecutive rows: for banded / stencil matrices one gather instruction then touches
        // a few sectors of x instead of one per lane.
        int* const s_col = reinterpret_cast<int*>(s_prod);
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            const int k = tid + j * kThreads;
            if (k < nnz_tile) {
                s_col[k] = c[j];
                s_val[k] = a[j];
            }
        }
        __syncthreads();
        const int G = 1 << lgG, ngroups = kThreads >> lgG;
        const int gidx = tid >> lgG, glane = tid & (G - 1);
        for (int i0 = 0; i0 <= nrows; i0 += ngroups) {  // block-uniform trip count
            const int i = i0 + gidx;
            int b = 0, e = 0;
            if (i <= nrows) {
                b = (i == 0) ? 0 : s_row_end[i - 1];
                e = s_row_end[i];
            }
            C sum = C(0);
            int k = b + glane;
            for (; k + 3 * G < e; k += 4 * G) {  // four independent gathers in flight per lane
                const V x0 = xb[s_col[k]], x1 = xb[s_col[k + G]], x2 = xb[s_col[k + 2 * G]], x3 = xb[s_col[k + 3 * G]];
                sum += times(widen<C, V>(s_val[k]), widen<C, V>(x0));
                sum += times(widen<C, V>(s_val[k + G]), widen<C, V>(x1));
                sum += times(widen<C, V>(s_val[k + 2 * G]), widen<C, V>(x2));
                sum += times(widen<C, V>(s_val[k + 3 * G]), widen<C, V>(x3));
            }
            if (k < e) {  // up to three left: gathered together as well
                const int k1 = min(k + G, e - 1), k2 = min(k + 2 * G, e - 1);
                const V x0 = xb[s_col[k]], x1 = xb[s_col[k1]], x2 = xb[s_col[k2]];
                sum += times(widen<C, V>(s_val[k]), widen<C, V>(x0));
                if (k + G < e) sum += times(widen<C, V>(s_val[k + G]), widen<C, V>(x1));
                if (k + 2 * G < e) sum += times(widen<C, V>(s_val[k + 2 * G]), widen<C, V>(x2));
            }
            for (int d = G >> 1; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
            if (glane == 0 && i <= nrows) {
                if (i == nrows) {
                    carry_row[t] = row_s + nrows;
                    carry_val[t] = sum;
                } else if (i == 0 && continued) {
                    head_val[t] = sum;
                } else {
                    C v = times(alpha, sum);
                    if (beta != C(0)) v += times(beta, widen<C, Y>(y[row_s + i]));
                    y[row_s + i] = narrow<Y, C>(v);
                }
            }
        }
        return;
    }

    // ---- long rows: products to shared memory, then each thread walks WALK consecutive merge items
    V xv[IPT];
#pragma unroll
    for (int j = 0; j < IPT; ++j) xv[j] = (tid + j * kThreads < nnz_tile) ? xb[c[j]] : V(0);
#pragma unroll
    for (int j = 0; j < IPT; ++j) {
        const int k = tid + j * kThreads;
        if (k < nnz_tile) s_prod[k] = times(widen<C, V>(a[j]), widen<C, V>(xv[j]));
    }
    C* const s_y = s_prod + nnz_tile;  // s_y[i]: row row_s + i, i in [0, nrows]
    for (int i = tid; i <= nrows; i += kThreads) s_y[i] = C(0);
    __syncthreads();

    const int d0 = min(tid * WALK, tile_items), d1 = min(d0 + WALK, tile_items);
    int lo = max(d0 - nnz_tile, 0), hi = min(d0, nrows);
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_row_end[mid] <= d0 - mid - 1)
            lo = mid + 1;
        else
            hi = mid;
    }
    int r = lo, k = d0 - lo, end = s_row_end[r];
    C sum = C(0);
#pragma unroll
    for (int it = 0; it < WALK; ++it) {
        if (d0 + it < d1) {
            if (k < end) {
                sum += s_prod[k];
                ++k;
            } else {
                s_y[r] = sum;  // the row ends in this thread's span: its part from this thread on
                sum = C(0);
                ++r;
                end = s_row_end[r];
            }
        }
    }
    // ---- segmented reduction of what the threads still hold (key r, value sum): warp scan, then the warps in order
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const C up = __shfl_up_sync(0xffffffffu, sum, d);
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

    // ---- results. A first row that began in an earlier tile is finished by the second kernel.
    for (int i = tid; i < nrows; i += kThreads) {
        if (i == 0 && continued) {
            head_val[t] = s_y[0];
        } else {
            C v = times(alpha, s_y[i]);
            if (beta != C(0)) v += times(beta, widen<C, Y>(y[row_s + i]));
            y[row_s + i] = narrow<Y, C>(v);
        }
    }
    if (tid == 0) {
        carry_row[t] = row_s + nrows;
        carry_val[t] = s_y[nrows];
    }
}

// One thread per tile whose first row began in an earlier tile: the row's sum is the tile's local part plus the
// open-row sums of the tiles before it back to the one the row began in (fixed order: nearest tile first).
template <typename C, typename Y>
__global__ void spmv_mixed_finish_kernel(long long num_tiles, int base, const int* __restrict__ row_ptr,
                                         const int2* __restrict__ tile_starts, const int* __restrict__ carry_row,
                                         const C* __restrict__ carry_val, const C* __restrict__ head_val,
                                         Y* __restrict__ y, ScalarArg<C> alpha_arg, ScalarArg<C> beta_arg) {
    const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= num_tiles || t == 0) return;
    const int2 s0 = tile_starts[t], s1 = tile_starts[t + 1];
    const int row = s0.x;
    if (s1.x == s0.x || __ldg(row_ptr + row) - base >= s0.y) return;
    C sum = head_val[t];
    for (long long u = t - 1; u >= 0 && carry_row[u] == row; --u) sum += carry_val[u];
    const C alpha = alpha_arg.get(), beta = beta_arg.get();
    C v = times(alpha, sum);
    if (beta != C(0)) v += times(beta, widen<C, Y>(y[row]));
    y[row] = narrow<Y, C>(v);
}

template <typename V, typename C, typename Y>
cudaError_t run(cudaStream_t s, int64_t m, int base, const int32_t* row_ptr, const int32_t* col, const void* val,
                const void* x, void* y, ScalarArg<C> alpha, ScalarArg<C> beta, const SpmvWorkspace& ws, void* buf) {
    if (ws.num_tiles == 0) return cudaSuccess;
    char* const b = static_cast<char*>(buf);
    const int2* starts = reinterpret_cast<const int2*>(b);
    int* carry_row = reinterpret_cast<int*>(b + ws.off_carry_row);
    C* carry_val = reinterpret_cast<C*>(b + ws.off_carry_val);
    C* head_val = reinterpret_cast<C*>(b + head_offset(ws));
    if (ws.walk)
        spmv_mixed_tile_kernel<V, C, Y, true><<<(unsigned)ws.num_tiles, kThreads, 0, s>>>(
            (int)m, base, row_ptr, col, static_cast<const V*>(val), static_cast<const V*>(x), static_cast<Y*>(y), alpha,
            beta, starts, carry_row, carry_val, head_val);
    else
        spmv_mixed_tile_kernel<V, C, Y, false><<<(unsigned)ws.num_tiles, kThreads, 0, s>>>(
            (int)m, base, row_ptr, col, static_cast<const V*>(val), static_cast<const V*>(x), static_cast<Y*>(y), alpha,
            beta, starts, carry_row, carry_val, head_val);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || ws.num_tiles < 2) return e;
    spmv_mixed_finish_kernel<C, Y><<<(unsigned)((ws.num_tiles + 255) / 256), 256, 0, s>>>(
        ws.num_tiles, base, row_ptr, starts, carry_row, carry_val, head_val, static_cast<Y*>(y), alpha, beta);
    return cudaGetLastError();
}

}  // namespace

SpmvWorkspace spmv_mixed_workspace(int64_t m, int64_t nnz) {
    SpmvWorkspace ws = spmv_workspace(m, nnz, 4, kTileSmall);  // 4-byte sums; kTile merge items per tile
    ws.bytes += head_bytes(ws);
    return ws;
}

cudaError_t spmv_mixed(cudaStream_t s, MixedKind kind, int64_t m, int base, const int32_t* row_ptr, const int32_t* col,
                       const void* val, const void* x, void* y, ScalarArg<float> alpha_f, ScalarArg<float> beta_f,
                       ScalarArg<int> alpha_i, ScalarArg<int> beta_i, const SpmvWorkspace& ws, void* buf) {
    if (ws.items_per_tile != kTile) return cudaErrorInvalidValue;
    switch (kind) {
        case MixedKind::kHalfToFloat:
            return run<__half, float, float>(s, m, base, row_ptr, col, val, x, y, alpha_f, beta_f, ws, buf);
        case MixedKind::kBf16ToFloat:
            return run<__nv_bfloat16, float, float>(s, m, base, row_ptr, col, val, x, y, alpha_f, beta_f, ws, buf);
        case MixedKind::kInt8ToFloat:
            return run<int8_t, float, float>(s, m, base, row_ptr, col, val, x, y, alpha_f, beta_f, ws, buf);
        case MixedKind::kHalfToHalf:
            return run<__half, float, __half>(s, m, base, row_ptr, col, val, x, y, alpha_f, beta_f, ws, buf);
        case MixedKind::kBf16ToBf16:
            return run<__nv_bfloat16, float, __nv_bfloat16>(s, m, base, row_ptr, col, val, x, y, alpha_f, beta_f, ws, buf);
        case MixedKind::kInt8ToInt32:
            return run<int8_t, int, int>(s, m, base, row_ptr, col, val, x, y, alpha_i, beta_i, ws, buf);
        default:
            return cudaErrorInvalidValue;
    }
}

}  // namespace mcsp_b200
