// CSR SpMM for sm_100a: C = alpha * A * B + beta * C.
//
// Replaces mcspBatchedSpmmCsrNnKernel (mcsparse/src/kernels/level3/spmm/csr_spmm_device.hpp:91-167,
// launched from mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:82-162). The reference runs one
// warp per (row, C column), re-reading A's row for every column, and needs B column-major, so a
// row-major B is first transposed into a temporary allocation. Here a row of A is read once
// and every nonzero is applied to a whole row of B with 128-bit loads; row-major B and C are
// used in place. No temporary memory, no stream synchronisation.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "internal.h"

namespace mcsp_b200 {

namespace {

constexpr int kThreads = 256;
#ifndef MCSP_PANEL_MIN_BLOCKS
#define MCSP_PANEL_MIN_BLOCKS 4  // at most 64 registers: measured best (5 blocks of 48 registers ran 15 % slower)
#endif

template <typename T>
struct VecOf;
template <>
struct VecOf<float> {
    using type = float4;
    static constexpr int W = 4;
};
template <>
struct VecOf<double> {
    using type = double2;
    static constexpr int W = 2;
};

template <>
struct VecOf<cfloat> {  // two complex numbers per 128-bit access
    using type = float4;
    static constexpr int W = 2;
};
template <>
struct VecOf<cdouble> {
    using type = double2;
    static constexpr int W = 1;
};

__device__ __forceinline__ void fma_vec(float4& acc, cfloat a, const float4& b) {
    const cfloat lo = mad(a, cfloat(b.x, b.y), cfloat(acc.x, acc.y)), hi = mad(a, cfloat(b.z, b.w), cfloat(acc.z, acc.w));
    acc = make_float4(lo.re, lo.im, hi.re, hi.im);
}
__device__ __forceinline__ void fma_vec(double2& acc, cdouble a, const double2& b) {
    const cdouble r = mad(a, cdouble(b.x, b.y), cdouble(acc.x, acc.y));
    acc = make_double2(r.re, r.im);
}
__device__ __forceinline__ float4 scale(cfloat alpha, const float4& a) {
    const cfloat lo = alpha * cfloat(a.x, a.y), hi = alpha * cfloat(a.z, a.w);
    return make_float4(lo.re, lo.im, hi.re, hi.im);
}
__device__ __forceinline__ double2 scale(cdouble alpha, const double2& a) {
    const cdouble r = alpha * cdouble(a.x, a.y);
    return make_double2(r.re, r.im);
}
__device__ __forceinline__ float4 axpby(cfloat alpha, const float4& a, cfloat beta, const float4& c) {
    const float4 p = scale(alpha, a), q = scale(beta, c);
    return make_float4(p.x + q.x, p.y + q.y, p.z + q.z, p.w + q.w);
}
__device__ __forceinline__ double2 axpby(cdouble alpha, const double2& a, cdouble beta, const double2& c) {
    const double2 p = scale(alpha, a), q = scale(beta, c);
    return make_double2(p.x + q.x, p.y + q.y);
}

__device__ __forceinline__ void fma_vec(float4& acc, float a, const float4& b) {
    acc.x = fmaf(a, b.x, acc.x);
    acc.y = fmaf(a, b.y, acc.y);
    acc.z = fmaf(a, b.z, acc.z);
    acc.w = fmaf(a, b.w, acc.w);
}
__device__ __forceinline__ void fma_vec(double2& acc, double a, const double2& b) {
    acc.x = fma(a, b.x, acc.x);
    acc.y = fma(a, b.y, acc.y);
}
__device__ __forceinline__ float4 axpby(float alpha, const float4& a, float beta, const float4& c) {
    return make_float4(alpha * a.x + beta * c.x, alpha * a.y + beta * c.y, alpha * a.z + beta * c.z,
                       alpha * a.w + beta * c.w);
}
__device__ __forceinline__ double2 axpby(double alpha, const double2& a, double beta, const double2& c) {
    return make_double2(alpha * a.x + beta * c.x, alpha * a.y + beta * c.y);
}
__device__ __forceinline__ float4 scale(float alpha, const float4& a) {
    return make_float4(alpha * a.x, alpha * a.y, alpha * a.z, alpha * a.w);
}
__device__ __forceinline__ double2 scale(double alpha, const double2& a) {
    return make_double2(alpha * a.x, alpha * a.y);
}
template <typename V>
__device__ __forceinline__ V zero_vec();
template <>
__device__ __forceinline__ float4 zero_vec<float4>() {
    return make_float4(0.f, 0.f, 0.f, 0.f);
}
template <>
__device__ __forceinline__ double2 zero_vec<double2>() {
    return make_double2(0.0, 0.0);
}

// ---------------------------------------------------------------------------------------
// K3: row-major SpMM. G lanes form a group that owns one row of A and a slab of G * W
// consecutive columns of C (W = 4 floats or 2 doubles per lane: one 128-bit access). The
// group loads G (col, val) pairs of the row with one coalesced access, then broadcasts them
// lane by lane with shuffles; each broadcast nonzero costs one 128-bit load of B per lane
// and W FMAs. The loop over the G nonzeros is unrolled so several B rows are in flight.
// B rows are fetched with default caching: B is the operand with reuse (through L2).
// ---------------------------------------------------------------------------------------
//
// PANEL variant: B is too large for L2, so the product is done in column panels of A whose slice of
// B fits; the launch for panel p covers, in each row, only the nonzeros between panel_lo[row] and
// panel_hi[row] (found once by spmm_panel_ptr_kernel; columns sorted within a row) and adds into
// C. Successive rows hit the same L2-resident slice of B instead of all of B, which trades the
// random re-reads of B from HBM for streaming re-reads of C. Rows with nothing in a later panel
// are skipped entirely.
template <typename T, int G, bool PANEL, typename I>
__global__ void __launch_bounds__(kThreads)
    spmm_rowmajor_kernel(int m, int n, int base, const I* __restrict__ row_ptr, const I* __restrict__ col,
                         const T* __restrict__ val, const T* __restrict__ B, long long ldb, T* __restrict__ C,
                         long long ldc, ScalarArg<T> alpha_arg, ScalarArg<T> beta_arg,
                         const int* __restrict__ panel_lo, const int* __restrict__ panel_hi, int first_panel) {
    using V = typename VecOf<T>::type;
    constexpr int W = VecOf<T>::W;
    const int lane = threadIdx.x & (G - 1);
    const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) / G;
    const int c0 = (blockIdx.y * G + lane) * W;  // first column of this lane
    const bool row_ok = row < m;                 // uniform within a group
    const bool col_ok = c0 < n;
    // Shuffles below use the full-warp mask with width G: all 32 lanes always execute them.
    int j0 = 0, j1 = 0;
    if (row_ok) {
        if (PANEL) {
            j0 = __ldg(panel_lo + row);
            j1 = __ldg(panel_hi + row);
        } else {
            j0 = (int)__ldg(row_ptr + row) - base;
            j1 = (int)__ldg(row_ptr + row + 1) - base;
        }
    }
    V acc = zero_vec<V>();
    const T* const Bc = B + c0 - (long long)base * ldb;
    // The groups of a warp own different rows, with different lengths. Both loops run to the
    // largest count among them with the work predicated per group: sub-warp branches would make the
    // hardware run the groups one after the other.
    for (int j = j0; __any_sync(0xffffffffu, j < j1); j += G) {
        int cj = 0;
        T vj = T(0);
        if (j + lane < j1) {
            cj = (int)__ldcs(col + j + lane);
            vj = ldcs(val + j + lane);
        }
        const int cnt = max(0, min(G, j1 - j));
        const int maxcnt = __reduce_max_sync(0xffffffffu, cnt);
        // chunks of four B rows requested together, predicated; no remainder loop (its loads would go one by one)
        for (int q0 = 0; q0 < maxcnt; q0 += 4) {
            V b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int cq = __shfl_sync(0xffffffffu, cj, (q0 + u) & (G - 1), G);
                b[u] = (q0 + u < cnt && col_ok) ? *reinterpret_cast<const V*>(Bc + (long long)cq * ldb) : zero_vec<V>();
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) fma_vec(acc, shfl_idx(0xffffffffu, vj, (q0 + u) & (G - 1), G), b[u]);
        }
    }
    if (row_ok && col_ok) {
        const T alpha = alpha_arg.get(), beta = beta_arg.get();
        V* out = reinterpret_cast<V*>(C + row * ldc + c0);
        if (!PANEL || first_panel) {
            *out = (beta != T(0)) ? axpby(alpha, acc, beta, *out) : scale(alpha, acc);
        } else if (j1 > j0) {  // later panels add to what the earlier ones left; C streams through L2
            __stcs(out, axpby(alpha, acc, T(1), __ldcs(out)));
        }
    }
}

// ---------------------------------------------------------------------------------------
// K3p: one pass of the column-panel SpMM: the nonzeros of A whose column lies in one panel of
// rows of B, applied to one slab of G * W consecutive columns of B and C.
//
// Why panels and slabs. With uniform columns and a B larger than L2, the single-pass kernel
// above fetches most B rows from HBM once per nonzero. A panel of B rows small enough to stay
// in L2 is fetched from HBM once and then hit by every row of A; the price is that C is read and
// rewritten once per extra panel. A narrower slab makes the same L2 bytes cover more rows of B,
// so a slab needs fewer panels; the price is that A is read once per slab. The plan picks the
// slab width and panel count with the least modelled HBM traffic.
//
// The pass reads A regrouped panel by panel (ccol / cval, built by the preprocess call): the pieces
// of consecutive rows are adjacent, so the lane groups of a warp load one contiguous range, where
// pieces left in place inside their rows cost a DRAM burst of 64 bytes or two per 40-byte piece.
// G lanes own one row and the slab's G * W columns; a thread block loops over rows (grid-stride)
// with a software pipeline, because a row piece is short (nnz / rows / panels) and one row at a time
// would leave every load latency exposed: while the B rows of the current row are in flight, the
// piece of the group's next row (two elements per lane) and the bounds of the row after that are
// already being fetched, and C's old value (later panels add to it) is requested before the B rows.
// The piece is broadcast lane by lane with shuffles; each nonzero costs one 128-bit load of B per
// lane and W multiply-adds. Loop bounds are those of the longest piece among the warp's groups, with
// the work predicated per group: sub-warp branches would make the hardware run the groups in turn.
// B rows are loaded with default caching (they are the L2-resident operand); A, the bounds and C
// are streamed (evict-first).
// ---------------------------------------------------------------------------------------
constexpr int kPanelRound = 8;  // B rows a lane group has in flight in one round (divides every lane-group width above 4)
// 16 bytes global -> shared, asynchronously (L2 only: the B rows are the L2-resident operand), and the wait for
// all of this thread's copies.
__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copies_wait() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <typename T, int G, bool FIRST>
__global__ void __launch_bounds__(kThreads, MCSP_PANEL_MIN_BLOCKS)
    spmm_panel_kernel(int m, int n, const int* __restrict__ pos, const int* __restrict__ ccol,
                      const T* __restrict__ cval, const T* __restrict__ B, long long ldb, T* __restrict__ C,
                      long long ldc, ScalarArg<T> alpha_arg, ScalarArg<T> beta_arg, int slab_c0) {
    using V = typename VecOf<T>::type;
    constexpr int W = VecOf<T>::W;
    const int lane = threadIdx.x & (G - 1);
    const long long ngroups = (long long)gridDim.x * (kThreads / G);
    long long row0 = (blockIdx.x * (long long)kThreads + threadIdx.x) / G;
    const int c0 = slab_c0 + lane * W;  // first column of this lane
    const bool col_ok = c0 < n;
    const T* const Bc = B + c0;
    const unsigned ldb32 = (unsigned)ldb;  // the launcher checks that every element offset into B fits 32 bits
    __shared__ __align__(16) V s_rows[kThreads / G][kPanelRound < G ? kPanelRound : G][G];
    V* const mine = &s_rows[threadIdx.x / G][0][lane];  // row u of the round: mine[u * G]
    const T alpha = alpha_arg.get(), beta = beta_arg.get();

    // bounds of the group's rows i, i + 1, i + 2; the first 2 G elements of the pieces of rows i, i + 1
    int lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
    long long row1 = row0 + ngroups;
    if (row0 < m) lo0 = __ldcs(pos + row0), hi0 = __ldcs(pos + row0 + 1);
    if (row1 < m) lo1 = __ldcs(pos + row1), hi1 = __ldcs(pos + row1 + 1);
    int ca0 = 0, cb0 = 0;
    T va0 = T(0), vb0 = T(0);
    if (lo0 + lane < hi0) ca0 = __ldcs(ccol + lo0 + lane), va0 = ldcs(cval + lo0 + lane);
    if (lo0 + G + lane < hi0) cb0 = __ldcs(ccol + lo0 + G + lane), vb0 = ldcs(cval + lo0 + G + lane);
    while (__any_sync(0xffffffffu, row0 < m)) {
        const bool row_ok = row0 < m;
        const long long row2 = row1 + ngroups;
        int lo2 = 0, hi2 = 0;
        if (row2 < m) lo2 = __ldcs(pos + row2), hi2 = __ldcs(pos + row2 + 1);
        int ca1 = 0, cb1 = 0;
        T va1 = T(0), vb1 = T(0);
        if (lo1 + lane < hi1) ca1 = __ldcs(ccol + lo1 + lane), va1 = ldcs(cval + lo1 + lane);
        if (lo1 + G + lane < hi1) cb1 = __ldcs(ccol + lo1 + G + lane), vb1 = ldcs(cval + lo1 + G + lane);
        V* const out = reinterpret_cast<V*>(C + row0 * ldc + c0);
        const bool write_c = row_ok && col_ok && (FIRST || hi0 > lo0);
        V old = zero_vec<V>();
        if (write_c && (FIRST ? beta != T(0) : true)) old = __ldcs(out);

        V acc = zero_vec<V>();
        for (int j = lo0; __any_sync(0xffffffffu, j < hi0); j += 2 * G) {
            if (j != lo0) {  // a piece longer than 2 G: the rest is fetched as it is needed
                ca0 = cb0 = 0, va0 = vb0 = T(0);
                if (j + lane < hi0) ca0 = __ldcs(ccol + j + lane), va0 = ldcs(cval + j + lane);
                if (j + G + lane < hi0) cb0 = __ldcs(ccol + j + G + lane), vb0 = ldcs(cval + j + G + lane);
            }
            const int cnt = max(0, min(2 * G, hi0 - j));
            const int maxcnt = __reduce_max_sync(0xffffffffu, cnt);
            // Rounds of R nonzeros: the lanes copy their 16 bytes of each of the round's B rows into shared memory
            // asynchronously (cp.async: no destination registers are held while the rows are in flight, so a round
            // can be twice as deep as a register-staged one), wait once, and multiply from shared memory; every lane
            // reads back only what it copied itself. No remainder loop (it would fetch its B rows one after the
            // other, an L2 round trip each): rows past a group's piece are predicated off.
            // Measured at 64 columns: register-staged chunks of 4 with a remainder loop 1.105 ms, without 1.004 ms,
            // chunks of 8 1.04 ms; these rounds of 8 0.955 ms; one round of 16 (three blocks per SM) 0.98 ms.
            constexpr int R = kPanelRound < G ? kPanelRound : G;
            auto round = [&](int creg, T vreg, int q0, int before) {
                // slots are issued in groups of four, only as many groups as the longest piece of the warp needs
                // (a predicated-off slot still costs its issue slots)
                const int need = maxcnt - before - q0;  // warp-uniform
#pragma unroll
                for (int u0 = 0; u0 < R; u0 += 4) {
                    if (u0 < need) {
#pragma unroll
                        for (int u = u0; u < u0 + 4; ++u) {
                            const int cq = __shfl_sync(0xffffffffu, creg, q0 + u, G);
                            if (before + q0 + u < cnt && col_ok) copy16_async(mine + u * G, Bc + (unsigned)cq * ldb32);
                        }
                    }
                }
                copies_wait();
#pragma unroll
                for (int u0 = 0; u0 < R; u0 += 4) {
                    if (u0 < need) {
#pragma unroll
                        for (int u = u0; u < u0 + 4; ++u) {
                            const T vq = shfl_idx(0xffffffffu, vreg, q0 + u, G);
                            if (before + q0 + u < cnt && col_ok) fma_vec(acc, vq, mine[u * G]);
                        }
                    }
                }
            };
            const int first_half = min(maxcnt, G);
            for (int q0 = 0; q0 < first_half; q0 += R) round(ca0, va0, q0, 0);
            for (int q0 = G; q0 < maxcnt; q0 += R) round(cb0, vb0, q0 - G, G);
        }
        if (write_c) {
            if (FIRST)
                __stcs(out, beta != T(0) ? axpby(alpha, acc, beta, old) : scale(alpha, acc));
            else
                __stcs(out, axpby(alpha, acc, T(1), old));
        }
        row0 = row1, row1 = row2;
        lo0 = lo1, hi0 = hi1, lo1 = lo2, hi1 = hi2;
        ca0 = ca1, cb0 = cb1, va0 = va1, vb0 = vb1;
    }
}

// One thread per row: where each column panel starts inside the row (lower bound of the panel's first
// column among the row's sorted columns). A row whose columns are not sorted is given to panel 0 whole.
template <typename I>
__global__ void spmm_panel_ptr_kernel(int m, int base, const I* __restrict__ row_ptr, const I* __restrict__ col,
                                      int num_panels, int panel_cols, int* __restrict__ panel_ptr) {
    const long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (r >= m) return;
    const int j0 = (int)row_ptr[r] - base, j1 = (int)row_ptr[r + 1] - base;
    bool sorted = true;
    for (int j = j0 + 1; j < j1; ++j) sorted &= col[j - 1] <= col[j];
    panel_ptr[r] = j0;
    for (int p = 1; p < num_panels; ++p) {
        int lo = j0, hi = j1;
        if (sorted) {
            const long long first_col = (long long)p * panel_cols + base;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (col[mid] < first_col)
                    lo = mid + 1;
                else
                    hi = mid;
            }
        } else {
            lo = j1;
        }
        panel_ptr[(long long)p * m + r] = lo;
    }
    panel_ptr[(long long)num_panels * m + r] = j1;
}

// piece_len[p * m + r] = nonzeros of row r in panel p (panel-major; one extra zero at the end so that the
// exclusive scan leaves the total there).
__global__ void spmm_piece_len_kernel(long long m, int num_panels, const int* __restrict__ panel_ptr,
                                      unsigned* __restrict__ piece_len) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long count = (long long)num_panels * m;
    if (i < count) piece_len[i] = (unsigned)(panel_ptr[i + m] - panel_ptr[i]);
    if (i == count) piece_len[i] = 0u;
}

// Regroups one array of A (column indices made 0-based, or values; without a source: for every entry of A the
// position it is regrouped to) panel by panel: eight lanes copy the piece of one (panel, row) from its place inside the row to
// piece_pos[p * m + r].
template <typename S, typename D>
__global__ void __launch_bounds__(256)
    spmm_regroup_kernel(long long pieces, const int* __restrict__ panel_ptr, long long m, int num_panels,
                        const int* __restrict__ piece_pos, const S* __restrict__ src, D* __restrict__ dst, int sub) {
    // Lane groups are numbered row by row (the pieces of one row are neighbours in a warp), so that a warp reads a
    // contiguous stretch of the source and every sector of it once; piece (panel p, row r) has index p * m + r.
    const long long g = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 3;
    const int lane = threadIdx.x & 7;
    if (g >= pieces) return;
    const long long r = g / num_panels;
    const long long i = (g - r * num_panels) * m + r;
    const int from = panel_ptr[i], len = panel_ptr[i + m] - from, to = piece_pos[i];
    for (int e = lane; e < len; e += 8) {
        if constexpr (std::is_integral<D>::value) {
            if (src == nullptr)
                dst[from + e] = (D)(to + e);  // where the entry goes (indexed by where it comes from)
            else
                dst[to + e] = (D)src[from + e] - (D)sub;
        } else {
            dst[to + e] = src[from + e];
        }
    }
}

// cval[dst[j]] = val[j]: the per-call regrouping of the values through the destinations recorded by the preprocess
// call. In source order on purpose: val and dst are read once, fully coalesced (four consecutive j per thread, 128-bit
// loads where the value type allows), and the stores of a piece (a run of consecutive destinations) meet those of the
// same piece of the neighbouring rows in L2 before the lines are written back. In destination order every 40-byte
// piece re-read its 64-byte bursts of val: 534 MB of reads instead of 2 x 134.
template <typename T>
__global__ void __launch_bounds__(256)
    spmm_scatter_values_kernel(long long nnz, const T* __restrict__ val, const int* __restrict__ dst, T* __restrict__ cval) {
    const long long k = 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x);
    if (k + 3 < nnz && (reinterpret_cast<uintptr_t>(val) & 15) == 0) {
        const int4 p = __ldcs(reinterpret_cast<const int4*>(dst + k));
        alignas(16) T v[4];
        const uint4* from = reinterpret_cast<const uint4*>(val + k);
        uint4* to = reinterpret_cast<uint4*>(v);
#pragma unroll
        for (int i = 0; i < (int)(4 * sizeof(T) / 16); ++i) to[i] = __ldcs(from + i);
        cval[p.x] = v[0], cval[p.y] = v[1], cval[p.z] = v[2], cval[p.w] = v[3];
    } else {
        for (long long i = k; i < nnz && i < k + 4; ++i) cval[dst[i]] = val[i];
    }
}

// Any layout, any n: one thread per C element, addressed through (row, col) strides.
// Consecutive threads run along C's contiguous dimension.
template <typename T, typename I>
__global__ void __launch_bounds__(kThreads)
    spmm_strided_kernel(long long m, long long n, int base, const I* __restrict__ row_ptr,
                        const I* __restrict__ col, const T* __restrict__ val, const T* __restrict__ B,
                        long long b_rs, long long b_cs, T* __restrict__ C, long long c_rs, long long c_cs,
                        ScalarArg<T> alpha_arg, ScalarArg<T> beta_arg) {
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= m * n) return;
    long long r, c;
    if (c_cs == 1) {
        r = idx / n;
        c = idx - r * n;
    } else {
        c = idx / m;
        r = idx - c * m;
    }
    const int j0 = (int)__ldg(row_ptr + r) - base, j1 = (int)__ldg(row_ptr + r + 1) - base;
    T sum = T(0);
    for (int j = j0; j < j1; ++j)
        sum += ldg(val + j) * ldg(B + ((long long)__ldg(col + j) - base) * b_rs + c * b_cs);
    const T alpha = alpha_arg.get(), beta = beta_arg.get();
    T* out = C + r * c_rs + c * c_cs;
    T v = alpha * sum;
    if (beta != T(0)) v += beta * *out;
    *out = v;
}

template <typename T, int G, typename I>
cudaError_t launch_rowmajor(cudaStream_t s, int64_t m, int64_t n, int base, const I* row_ptr, const I* col, const T* val, const T* B, int64_t ldb, T* C, int64_t ldc,
                            ScalarArg<T> alpha, ScalarArg<T> beta) {
    constexpr int W = VecOf<T>::W;
    const long long threads_total = m * G;
    dim3 grid((unsigned)((threads_total + kThreads - 1) / kThreads), (unsigned)((n + G * W - 1) / (G * W)));
    spmm_rowmajor_kernel<T, G, false, I><<<grid, kThreads, 0, s>>>((int)m, (int)n, base, row_ptr, col, val, B, ldb, C,
                                                                ldc, alpha, beta, nullptr, nullptr, 1);
    return cudaGetLastError();
}

// All passes of the column-panel product: the values are regrouped panel by panel first (on every call: the
// caller may have edited them in place since the preprocess call; the column indices were regrouped there),
// then, for every slab of G * W columns, panel 0 writes C and the later panels add to it. One launch per
// (slab, panel), in that order, so that at any time the resident thread blocks work on one panel of one slab of B.
template <typename T, int G>
cudaError_t launch_panels(cudaStream_t s, int64_t m, int64_t n, const T* val, const T* B, int64_t ldb, T* C,
                          int64_t ldc, ScalarArg<T> alpha, ScalarArg<T> beta, const SpmmPlan& plan, void* buf) {
    constexpr int W = VecOf<T>::W;
    static int blocks_per_sm = 0, sm_count = 0;
    if (blocks_per_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, spmm_panel_kernel<T, G, false>, kThreads, 0);
        if (blocks_per_sm < 1) blocks_per_sm = 1;
        if (sm_count < 1) sm_count = 148;
        // Tuning: MCSPARSE_B200_SPMM_PANEL_BLOCKS caps the resident thread blocks per SM of a pass.
        if (const char* v = std::getenv("MCSPARSE_B200_SPMM_PANEL_BLOCKS"))
            blocks_per_sm = std::max(1, std::min(blocks_per_sm, std::atoi(v)));
    }
    char* base_ptr = static_cast<char*>(buf);
    const int* pos = reinterpret_cast<const int*>(base_ptr + plan.off_pos);
    const int* ccol = reinterpret_cast<const int*>(base_ptr + plan.off_ccol);
    T* cval = reinterpret_cast<T*>(base_ptr + plan.off_cval);
    cudaError_t e = cudaSuccess;
    const long long nnz = plan.nnz;
    if (!plan.values_current && nnz > 0) {
        const int* dst = reinterpret_cast<const int*>(base_ptr + plan.off_dst);
        spmm_scatter_values_kernel<T><<<(unsigned)((nnz + 1023) / 1024), 256, 0, s>>>(nnz, val, dst, cval);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const long long groups_per_block = kThreads / G;
    const long long want = (m + groups_per_block - 1) / groups_per_block;
    const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>(want, (long long)sm_count * blocks_per_sm));
    for (int c0 = 0; c0 < n; c0 += G * W) {
        for (int p = 0; p < plan.num_panels; ++p) {
            const int* pos_p = pos + (size_t)p * m;
            if (p == 0)
                spmm_panel_kernel<T, G, true><<<grid, kThreads, 0, s>>>((int)m, (int)n, pos_p, ccol, cval, B, ldb, C, ldc,
                                                                       alpha, beta, c0);
            else
                spmm_panel_kernel<T, G, false><<<grid, kThreads, 0, s>>>((int)m, (int)n, pos_p, ccol, cval, B, ldb, C, ldc,
                                                                        alpha, beta, c0);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

}  // namespace

// L2 bytes one panel of B may occupy, in MiB: MCSPARSE_B200_SPMM_PANEL_MB (0 turns the panels off).
// The default is what a B200 keeps resident beside the streams of A and C (measured: see the plan below).
static long long spmm_panel_budget_bytes() {
    const char* e = std::getenv("MCSPARSE_B200_SPMM_PANEL_MB");
    const long long mb = e ? std::atoll(e) : MCSPARSE_B200_SPMM_PANEL_MB_DEFAULT;
    return mb <= 0 ? 0 : mb << 20;
}
// Lanes per row forced for tuning runs (MCSPARSE_B200_SPMM_PANEL_LANES = 4, 8, 16 or 32); 0: modelled choice.
static int spmm_forced_lanes() {
    const char* e = std::getenv("MCSPARSE_B200_SPMM_PANEL_LANES");
    return e ? std::atoi(e) : 0;
}

// Slab width and panel count with the least modelled HBM traffic:
//   single pass      A + C + B * (1 + (nnz / k - 1) * miss),  miss = 1 - budget / |B|  (uniform columns: a B row is
//                    needed nnz / k times and found in L2 with the probability that L2 holds it)
//   slabs x panels   B + slabs * A + slabs * (2 * panels - 1) * |C slab|
// where a slab is G lanes x 16 bytes wide, a panel holds budget / max(128, 16 G) rows of B (L2 keeps
// whole 128-byte lines) and C's slab is written by the first panel and read and rewritten by the others.
SpmmPlan spmm_plan(int64_t m, int64_t k, int64_t n, int64_t nnz, size_t value_size, bool row_major_operands) {
    SpmmPlan plan;
    const long long budget = spmm_panel_budget_bytes();
    const double b_bytes = (double)k * n * value_size;
    if (!row_major_operands || budget == 0 || m == 0 || n == 0 || k == 0 || b_bytes <= 1.25 * budget) return plan;
    const double a_bytes = (double)nnz * (value_size + 4), c_bytes = (double)m * n * value_size;
    const double reuse = std::max(1.0, (double)nnz / (double)k);
    const double miss = 1.0 - (double)budget / b_bytes;
    const double single = a_bytes + c_bytes + b_bytes * (1.0 + (reuse - 1.0) * miss);
    const int w = 16 / (int)value_size;
    double best = single / 1.25;  // panels must save a quarter of the traffic to be worth their extra launches
    const int forced = spmm_forced_lanes();
    for (int g = 4; g <= 32; g *= 2) {
        if (forced != 0 && g != forced) continue;
        const long long slab_cols = (long long)g * w;
        if (slab_cols > n && g > 4) continue;
        const long long slabs = (n + slab_cols - 1) / slab_cols;
        const long long panel_rows = std::max<long long>(1, budget / std::max(128, 16 * g));
        const long long panels = (k + panel_rows - 1) / panel_rows;
        if (panels > 32) continue;
        const double traffic = b_bytes + slabs * a_bytes + slabs * (2.0 * panels - 1.0) * (double)m * 16.0 * g;
        if (traffic < best || forced != 0) {
            best = traffic;
            plan.num_panels = (int)panels;
            plan.panel_cols = (int)panel_rows;
            plan.lanes = g;
        }
    }
    if (plan.num_panels > 1) {
        auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
        const size_t pieces = size_t(plan.num_panels) * size_t(m);
        plan.off_pos = up(size_t(plan.num_panels + 1) * size_t(m) * 4);
        plan.off_ccol = plan.off_pos + up((pieces + 1) * 4);
        plan.off_cval = plan.off_ccol + up(size_t(nnz) * 4);
        plan.nnz = nnz;
        plan.off_dst = plan.off_cval + up(size_t(nnz) * value_size);
        plan.off_scan = plan.off_dst + up(size_t(nnz) * 4);
        plan.bytes = 256 + plan.off_scan + up(size_t(scan_scratch_elems((long long)pieces + 1)) * 4);
    }
    return plan;
}

template <typename I>
cudaError_t spmm_preprocess(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const I* col,
                            const SpmmPlan& plan, void* buf) {
    if (plan.num_panels <= 1) return cudaSuccess;
    (void)nnz;
    char* base_ptr = static_cast<char*>(buf);
    int* panel_ptr = reinterpret_cast<int*>(base_ptr);
    unsigned* pos = reinterpret_cast<unsigned*>(base_ptr + plan.off_pos);
    int* ccol = reinterpret_cast<int*>(base_ptr + plan.off_ccol);
    unsigned* scratch = reinterpret_cast<unsigned*>(base_ptr + plan.off_scan);
    spmm_panel_ptr_kernel<I><<<(unsigned)((m + 127) / 128), 128, 0, s>>>((int)m, base, row_ptr, col, plan.num_panels,
                                                                    plan.panel_cols, panel_ptr);
    const long long pieces = (long long)plan.num_panels * m;
    spmm_piece_len_kernel<<<(unsigned)((pieces + 1 + 255) / 256), 256, 0, s>>>(m, plan.num_panels, panel_ptr, pos);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = exclusive_scan_u32(s, pos, pieces + 1, scratch);
    if (e != cudaSuccess) return e;
    spmm_regroup_kernel<I, int><<<(unsigned)((pieces * 8 + 255) / 256), 256, 0, s>>>(
        pieces, panel_ptr, m, plan.num_panels, reinterpret_cast<const int*>(pos), col, ccol, base);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // where every entry of A is regrouped to: the values follow through these positions on every product
    spmm_regroup_kernel<int, int><<<(unsigned)((pieces * 8 + 255) / 256), 256, 0, s>>>(
        pieces, panel_ptr, m, plan.num_panels, reinterpret_cast<const int*>(pos), nullptr,
        reinterpret_cast<int*>(base_ptr + plan.off_dst), 0);
    return cudaGetLastError();
}

template <typename T, typename I>
cudaError_t spmm(cudaStream_t s, int64_t m, int64_t n, int base, const I* row_ptr, const I* col, const T* val, const T* B, int64_t b_rs, int64_t b_cs, T* C, int64_t c_rs, int64_t c_cs,
                 ScalarArg<T> alpha, ScalarArg<T> beta, const SpmmPlan* plan, void* plan_buffer) {
    if (m == 0 || n == 0) return cudaSuccess;
    constexpr int W = VecOf<T>::W;
    const bool vec_ok = b_cs == 1 && c_cs == 1 && n % W == 0 && b_rs % W == 0 && c_rs % W == 0 &&
                        ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
    // (the pass kernel addresses B with 32-bit element offsets: rows of B x leading dimension must fit)
    const bool fits32 = plan != nullptr && (unsigned long long)plan->num_panels * plan->panel_cols * (unsigned long long)b_rs < (1ull << 32);
    if (vec_ok && fits32 && plan->num_panels > 1 && plan_buffer != nullptr) {
        switch (plan->lanes) {
            case 4: return launch_panels<T, 4>(s, m, n, val, B, b_rs, C, c_rs, alpha, beta, *plan, plan_buffer);
            case 8: return launch_panels<T, 8>(s, m, n, val, B, b_rs, C, c_rs, alpha, beta, *plan, plan_buffer);
            case 16: return launch_panels<T, 16>(s, m, n, val, B, b_rs, C, c_rs, alpha, beta, *plan, plan_buffer);
            default: return launch_panels<T, 32>(s, m, n, val, B, b_rs, C, c_rs, alpha, beta, *plan, plan_buffer);
        }
    }
    if (vec_ok) {
        const int64_t lanes = n / W;
        if (lanes <= 2) return launch_rowmajor<T, 2, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta);
        if (lanes <= 4) return launch_rowmajor<T, 4, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta);
        if (lanes <= 8) return launch_rowmajor<T, 8, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta);
        if (lanes <= 16) return launch_rowmajor<T, 16, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta);
        return launch_rowmajor<T, 32, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta);
    }
    const long long total = m * n;
    spmm_strided_kernel<T, I><<<(unsigned)((total + kThreads - 1) / kThreads), kThreads, 0, s>>>(
        m, n, base, row_ptr, col, val, B, b_rs, b_cs, C, c_rs, c_cs, alpha, beta);
    return cudaGetLastError();
}

// y = alpha * z + beta * y on complex vectors (y is not read when beta == 0).
template <typename T>
__global__ void complex_axpby_kernel(long long m, ScalarArg<T> alpha_arg, const T* __restrict__ z,
                                     ScalarArg<T> beta_arg, T* __restrict__ y) {
    const long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (r >= m) return;
    const T alpha = alpha_arg.get(), beta = beta_arg.get();
    T v = alpha * ldcs(z + r);
    if (beta != T(0)) v = mad(beta, y[r], v);
    y[r] = v;
}

// dst = conj(src), and y = alpha * conj(z) + beta * y (y is not read when beta == 0): the two vector passes
// around a product with conj(A), which is conj(A * conj(x)).
template <typename T>
__global__ void complex_conj_copy_kernel(long long n, const T* __restrict__ src, T* __restrict__ dst) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) dst[i] = conj_value(src[i]);
}
template <typename T>
__global__ void complex_conj_axpby_kernel(long long m, ScalarArg<T> alpha_arg, const T* __restrict__ z,
                                          ScalarArg<T> beta_arg, T* __restrict__ y) {
    const long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (r >= m) return;
    const T alpha = alpha_arg.get(), beta = beta_arg.get();
    T v = alpha * conj_value(ldcs(z + r));
    if (beta != T(0)) v = mad(beta, y[r], v);
    y[r] = v;
}
template <typename T>
cudaError_t complex_conj_copy(cudaStream_t s, int64_t n, const T* src, T* dst) {
    if (n == 0) return cudaSuccess;
    complex_conj_copy_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(n, src, dst);
    return cudaGetLastError();
}
template <typename T>
cudaError_t complex_conj_axpby(cudaStream_t s, int64_t m, ScalarArg<T> alpha, const T* z, ScalarArg<T> beta, T* y) {
    if (m == 0) return cudaSuccess;
    complex_conj_axpby_kernel<T><<<(unsigned)((m + 255) / 256), 256, 0, s>>>(m, alpha, z, beta, y);
    return cudaGetLastError();
}
template cudaError_t complex_conj_copy<cfloat>(cudaStream_t, int64_t, const cfloat*, cfloat*);
template cudaError_t complex_conj_copy<cdouble>(cudaStream_t, int64_t, const cdouble*, cdouble*);
template cudaError_t complex_conj_axpby<cfloat>(cudaStream_t, int64_t, ScalarArg<cfloat>, const cfloat*,
                                                ScalarArg<cfloat>, cfloat*);
template cudaError_t complex_conj_axpby<cdouble>(cudaStream_t, int64_t, ScalarArg<cdouble>, const cdouble*,
                                                 ScalarArg<cdouble>, cdouble*);

// Real matrix, complex vectors (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:633-658 instantiates its
// CSR kernel with real values and complex x, y, alpha, beta). A complex vector is a two-column row-major real
// matrix, so z = A * x is the real SpMM with n = 2 into `scratch` (m complex numbers), and the complex
// scaling follows in a second small kernel.
template <typename F>
cudaError_t spmv_real_matrix_complex_vectors(cudaStream_t s, int64_t m, int base, const int32_t* row_ptr,
                                             const int32_t* col, const F* val, const Complex<F>* x, Complex<F>* y,
                                             ScalarArg<Complex<F>> alpha, ScalarArg<Complex<F>> beta,
                                             Complex<F>* scratch) {
    if (m == 0) return cudaSuccess;
    const ScalarArg<F> one{F(1), nullptr}, zero{F(0), nullptr};
    cudaError_t e = spmm<F, int32_t>(s, m, 2, base, row_ptr, col, val, reinterpret_cast<const F*>(x), 2, 1,
                                     reinterpret_cast<F*>(scratch), 2, 1, one, zero, nullptr, nullptr);
    if (e != cudaSuccess) return e;
    complex_axpby_kernel<Complex<F>><<<(unsigned)((m + 255) / 256), 256, 0, s>>>(m, alpha, scratch, beta, y);
    return cudaGetLastError();
}
template cudaError_t spmv_real_matrix_complex_vectors<float>(cudaStream_t, int64_t, int, const int32_t*,
                                                             const int32_t*, const float*, const cfloat*, cfloat*,
                                                             ScalarArg<cfloat>, ScalarArg<cfloat>, cfloat*);
template cudaError_t spmv_real_matrix_complex_vectors<double>(cudaStream_t, int64_t, int, const int32_t*,
                                                              const int32_t*, const double*, const cdouble*, cdouble*,
                                                              ScalarArg<cdouble>, ScalarArg<cdouble>, cdouble*);

#define INSTANTIATE(T, I)                                                                                     \
    template cudaError_t spmm<T, I>(cudaStream_t, int64_t, int64_t, int, const I*, const I*, const T*, const T*, \
                                    int64_t, int64_t, T*, int64_t, int64_t, ScalarArg<T>, ScalarArg<T>,        \
                                    const SpmmPlan*, void*);
INSTANTIATE(float, int32_t)
INSTANTIATE(double, int32_t)
INSTANTIATE(float, int64_t)
INSTANTIATE(double, int64_t)
INSTANTIATE(cfloat, int32_t)
INSTANTIATE(cdouble, int32_t)
INSTANTIATE(cfloat, int64_t)
INSTANTIATE(cdouble, int64_t)
#undef INSTANTIATE
template cudaError_t spmm_preprocess<int32_t>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*,
                                              const SpmmPlan&, void*);
template cudaError_t spmm_preprocess<int64_t>(cudaStream_t, int64_t, int64_t, int, const int64_t*, const int64_t*,
                                              const SpmmPlan&, void*);

}  // namespace mcsp_b200
