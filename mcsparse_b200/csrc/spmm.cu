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

#include "internal.h"

namespace mcsp_b200 {

namespace {

constexpr int kThreads = 256;

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
    // Groups of one warp may have different trip counts; width-G shuffles only need the
    // lanes of the same group to be converged, which the group-uniform bounds guarantee.
    for (int j = j0; j < j1; j += G) {
        int cj = 0;
        T vj = T(0);
        if (j + lane < j1) {
            cj = (int)__ldcs(col + j + lane);
            vj = ldcs(val + j + lane);
        }
        const int cnt = min(G, j1 - j);
        const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
#pragma unroll 8
        for (int q = 0; q < cnt; ++q) {
            const int cq = __shfl_sync(gmask, cj, q, G);
            const T vq = shfl_idx(gmask, vj, q, G);
            if (col_ok) {
                const V b = *reinterpret_cast<const V*>(Bc + (long long)cq * ldb);
                fma_vec(acc, vq, b);
            }
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
                            ScalarArg<T> alpha, ScalarArg<T> beta, int num_panels, const int* panel_ptr) {
    constexpr int W = VecOf<T>::W;
    const long long threads_total = m * G;
    dim3 grid((unsigned)((threads_total + kThreads - 1) / kThreads), (unsigned)((n + G * W - 1) / (G * W)));
    if (num_panels <= 1 || panel_ptr == nullptr) {
        spmm_rowmajor_kernel<T, G, false, I><<<grid, kThreads, 0, s>>>((int)m, (int)n, base, row_ptr, col, val, B, ldb, C,
                                                                    ldc, alpha, beta, nullptr, nullptr, 1);
        return cudaGetLastError();
    }
    for (int p = 0; p < num_panels; ++p) {
        spmm_rowmajor_kernel<T, G, true, I><<<grid, kThreads, 0, s>>>(
            (int)m, (int)n, base, row_ptr, col, val, B, ldb, C, ldc, alpha, beta, panel_ptr + (size_t)p * m,
            panel_ptr + (size_t)(p + 1) * m, p == 0);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace

// L2 budget for one panel of B in MiB: MCSPARSE_B200_SPMM_PANEL_MB. Panels are off unless it is set:
// on the 1M x 1M, 32 nonzeros per row benchmark they cut DRAM traffic from 6.9 GB to 3.4 GB (n = 64,
// four panels) but each pass is latency-bound on its short row pieces and the total was slower
// (1.74 ms against 1.46 ms), so the single-pass kernel stays the default.
static long long spmm_panel_budget_bytes() {
    const char* e = std::getenv("MCSPARSE_B200_SPMM_PANEL_MB");
    const long long mb = e ? std::atoll(e) : 0;
    return mb <= 0 ? 0 : mb << 20;
}

SpmmPlan spmm_plan(int64_t m, int64_t k, int64_t n, int64_t nnz, size_t value_size, bool row_major_operands) {
    SpmmPlan plan;
    const long long budget = spmm_panel_budget_bytes();
    const long long b_bytes = (long long)k * n * (long long)value_size;
    if (!row_major_operands || budget == 0 || m == 0 || n == 0 || b_bytes <= 2 * budget) return plan;
    const long long panel_cols = std::max<long long>(1, budget / (n * (long long)value_size));
    const long long panels = (k + panel_cols - 1) / panel_cols;
    // Each extra panel re-reads and re-writes C once; worth it only while a row still brings a few
    // nonzeros to every panel (the re-reads of B it saves are proportional to nnz).
    if (panels < 2 || panels > 16 || nnz < 4 * (panels - 1) * m) return plan;
    plan.num_panels = (int)panels;
    plan.panel_cols = (int)panel_cols;
    plan.bytes = 256 + size_t(panels + 1) * size_t(m) * 4;
    return plan;
}

template <typename I>
cudaError_t spmm_preprocess(cudaStream_t s, int64_t m, int base, const I* row_ptr, const I* col, const SpmmPlan& plan,
                            void* buf) {
    if (plan.num_panels <= 1) return cudaSuccess;
    spmm_panel_ptr_kernel<I><<<(unsigned)((m + 127) / 128), 128, 0, s>>>((int)m, base, row_ptr, col, plan.num_panels,
                                                                    plan.panel_cols, static_cast<int*>(buf));
    return cudaGetLastError();
}

template <typename T, typename I>
cudaError_t spmm(cudaStream_t s, int64_t m, int64_t n, int base, const I* row_ptr, const I* col, const T* val, const T* B, int64_t b_rs, int64_t b_cs, T* C, int64_t c_rs, int64_t c_cs,
                 ScalarArg<T> alpha, ScalarArg<T> beta, int num_panels, const int* panel_ptr) {
    if (m == 0 || n == 0) return cudaSuccess;
    constexpr int W = VecOf<T>::W;
    const bool vec_ok = b_cs == 1 && c_cs == 1 && n % W == 0 && b_rs % W == 0 && c_rs % W == 0 &&
                        ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
    if (vec_ok) {
        const int64_t lanes = n / W;
        if (lanes <= 2) return launch_rowmajor<T, 2, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta, num_panels, panel_ptr);
        if (lanes <= 4) return launch_rowmajor<T, 4, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta, num_panels, panel_ptr);
        if (lanes <= 8) return launch_rowmajor<T, 8, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta, num_panels, panel_ptr);
        if (lanes <= 16)
            return launch_rowmajor<T, 16, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta, num_panels, panel_ptr);
        return launch_rowmajor<T, 32, I>(s, m, n, base, row_ptr, col, val, B, b_rs, C, c_rs, alpha, beta, num_panels, panel_ptr);
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
                                     reinterpret_cast<F*>(scratch), 2, 1, one, zero, 1, nullptr);
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
                                    int64_t, int64_t, T*, int64_t, int64_t, ScalarArg<T>, ScalarArg<T>, int,   \
                                    const int*);
INSTANTIATE(float, int32_t)
INSTANTIATE(double, int32_t)
INSTANTIATE(float, int64_t)
INSTANTIATE(double, int64_t)
INSTANTIATE(cfloat, int32_t)
INSTANTIATE(cdouble, int32_t)
INSTANTIATE(cfloat, int64_t)
INSTANTIATE(cdouble, int64_t)
#undef INSTANTIATE
template cudaError_t spmm_preprocess<int32_t>(cudaStream_t, int64_t, int, const int32_t*, const int32_t*,
                                              const SpmmPlan&, void*);
template cudaError_t spmm_preprocess<int64_t>(cudaStream_t, int64_t, int, const int64_t*, const int64_t*,
                                              const SpmmPlan&, void*);

}  // namespace mcsp_b200
