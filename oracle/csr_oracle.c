/*
 * csr_oracle.c -- CPU restatement of the mcSparse CSR SpMV / SpMM path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library and the timed
 * CPU baseline of the benchmark; the library itself never links, loads or calls it.
 *
 * PARITY UNPINNED BY THE REFERENCE: mcSparse ships no tests, golden vectors or fixtures
 * for this path and has no CPU implementation, so there is nothing of the reference's to
 * check these loops against on a CPU. They are pinned instead by (1) scipy.sparse on
 * random cases, (2) analytically known answers (stencil times the ones vector, diagonal
 * matrices, alpha = 0, beta in {0, 1}) and (3) where the reference's own device kernels
 * could be compiled from its sources, their output on a GPU (oracle/ref_kernels.cu).
 *
 * Reference lines restated here (paths inside the mcSparse tree):
 *   row loop and index-base handling   mcsparse/src/kernels/level2/spmv/csr_vector_device.hpp:35-57
 *   SpMV epilogue y = beta*y + alpha*s mcsparse/src/kernels/level2/spmv/csr_vector_device.hpp:66-77
 *   SpMM indexing of B and C           mcsparse/src/kernels/level3/spmm/csr_spmm_device.hpp:116-137,149-165
 *   meaning of B's order               mcsparse/src/kernels/level3/spmm/mcsp_spmm_gpu.cpp:119-133
 *
 * The oracle_* functions accumulate in a wider type than the inputs (double for fp32
 * data, long double for fp64 data) and also return d_i = |alpha| * sum_j |a_ij||x_j| +
 * |beta||y0_i|, the scale the tolerance is stated against. y (or C) is not read when
 * beta == 0, as in the CUDA path. The baseline_* functions are the same arithmetic in
 * native precision with OpenMP over nnz-balanced row chunks: the reported CPU baseline.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORDER_COL 1
#define ORDER_ROW 2

/* ------------------------------------------------------------------ SpMV oracle */

#define DEFINE_ORACLE_SPMV(NAME, VT, ACC)                                                              \
    void NAME(int64_t m, int base, const int32_t* row_ptr, const int32_t* col, const VT* val,          \
              const VT* x, double alpha, double beta, const VT* y_in, double* y_out, double* d_out) {  \
        _Pragma("omp parallel for schedule(dynamic, 4096)") for (int64_t r = 0; r < m; ++r) {          \
            ACC s = 0, d = 0;                                                                          \
            for (int64_t j = (int64_t)row_ptr[r] - base; j < (int64_t)row_ptr[r + 1] - base; ++j) {    \
                ACC a = (ACC)val[j], xv = (ACC)x[(int64_t)col[j] - base];                              \
                s += a * xv;                                                                           \
                d += fabsl((long double)a) * fabsl((long double)xv);                                   \
            }                                                                                          \
            ACC out = (ACC)alpha * s;                                                                  \
            ACC dd = (ACC)fabs(alpha) * d;                                                             \
            if (beta != 0.0) {                                                                         \
                out += (ACC)beta * (ACC)y_in[r];                                                       \
                dd += (ACC)fabs(beta) * (ACC)fabsl((long double)y_in[r]);                              \
            }                                                                                          \
            y_out[r] = (double)out;                                                                    \
            if (d_out) d_out[r] = (double)dd;                                                          \
        }                                                                                              \
    }

DEFINE_ORACLE_SPMV(oracle_csr_spmv_f32, float, double)
DEFINE_ORACLE_SPMV(oracle_csr_spmv_f64, double, long double)

/* ------------------------------------------------------------------ SpMM oracle */

static inline int64_t dn_index(int64_t r, int64_t c, int64_t ld, int order) {
    return order == ORDER_ROW ? r * ld + c : c * ld + r;
}

/* C_out and d_out are dense m x n, row-major with leading dimension n, whatever C's order. */
#define DEFINE_ORACLE_SPMM(NAME, VT, ACC)                                                              \
    void NAME(int64_t m, int64_t n, int base, const int32_t* row_ptr, const int32_t* col,              \
              const VT* val, const VT* B, int64_t ldb, int orderB, double alpha, double beta,          \
              const VT* C_in, int64_t ldc, int orderC, double* C_out, double* d_out) {                 \
        _Pragma("omp parallel for schedule(dynamic, 256)") for (int64_t r = 0; r < m; ++r) {           \
            for (int64_t c = 0; c < n; ++c) {                                                          \
                ACC s = 0, d = 0;                                                                      \
                for (int64_t j = (int64_t)row_ptr[r] - base; j < (int64_t)row_ptr[r + 1] - base; ++j) { \
                    ACC a = (ACC)val[j];                                                               \
                    ACC b = (ACC)B[dn_index((int64_t)col[j] - base, c, ldb, orderB)];                  \
                    s += a * b;                                                                        \
                    d += fabsl((long double)a) * fabsl((long double)b);                                \
                }                                                                                      \
                ACC out = (ACC)alpha * s;                                                              \
                ACC dd = (ACC)fabs(alpha) * d;                                                         \
                if (beta != 0.0) {                                                                     \
                    VT c0 = C_in[dn_index(r, c, ldc, orderC)];                                         \
                    out += (ACC)beta * (ACC)c0;                                                        \
                    dd += (ACC)fabs(beta) * (ACC)fabsl((long double)c0);                               \
                }                                                                                      \
                C_out[r * n + c] = (double)out;                                                        \
                if (d_out) d_out[r * n + c] = (double)dd;                                              \
            }                                                                                          \
        }                                                                                              \
    }

DEFINE_ORACLE_SPMM(oracle_csr_spmm_f32, float, double)
DEFINE_ORACLE_SPMM(oracle_csr_spmm_f64, double, long double)

/* ------------------------------------------------------------------ complex oracles
 *
 * Values, x, y, B and C are interleaved (re, im) pairs, as MACA_C_32F / MACA_C_64F lay them out
 * (mcspComplexFloat / mcspComplexDouble, mcsparse/src/include/mcsp_internal_types.h); the row loop
 * and the epilogue are those of the real kernels above (csr_vector_device.hpp:35-57,66-77), on
 * complex numbers. `conj_a` multiplies with conj(a) (what op(A) = A^H does after transposition).
 * Outputs: y_out interleaved in double, d_out = |alpha| sum |a||x| + |beta||y0| with complex moduli. */
#define DEFINE_ORACLE_SPMV_C(NAME, VT, ACC)                                                             \
    void NAME(int64_t m, int base, const int32_t* row_ptr, const int32_t* col, const VT* val, const VT* x, \
              const double* alpha, const double* beta, int conj_a, const VT* y_in, double* y_out,        \
              double* d_out) {                                                                           \
        const double abs_alpha = hypot(alpha[0], alpha[1]), abs_beta = hypot(beta[0], beta[1]);          \
        _Pragma("omp parallel for schedule(dynamic, 4096)") for (int64_t r = 0; r < m; ++r) {            \
            ACC sr = 0, si = 0, d = 0;                                                                   \
            for (int64_t j = (int64_t)row_ptr[r] - base; j < (int64_t)row_ptr[r + 1] - base; ++j) {      \
                const int64_t c = (int64_t)col[j] - base;                                                \
                const ACC ar = val[2 * j], ai = conj_a ? -(ACC)val[2 * j + 1] : (ACC)val[2 * j + 1];     \
                const ACC xr = x[2 * c], xi = x[2 * c + 1];                                              \
                sr += ar * xr - ai * xi;                                                                 \
                si += ar * xi + ai * xr;                                                                 \
                d += (ACC)hypotl((long double)ar, (long double)ai) * (ACC)hypotl((long double)xr, (long double)xi); \
            }                                                                                            \
            ACC outr = (ACC)alpha[0] * sr - (ACC)alpha[1] * si, outi = (ACC)alpha[0] * si + (ACC)alpha[1] * sr; \
            ACC dd = (ACC)abs_alpha * d;                                                                 \
            if (abs_beta != 0.0) {                                                                       \
                const ACC yr = y_in[2 * r], yi = y_in[2 * r + 1];                                        \
                outr += (ACC)beta[0] * yr - (ACC)beta[1] * yi;                                           \
                outi += (ACC)beta[0] * yi + (ACC)beta[1] * yr;                                           \
                dd += (ACC)abs_beta * (ACC)hypotl((long double)yr, (long double)yi);                     \
            }                                                                                            \
            y_out[2 * r] = (double)outr;                                                                 \
            y_out[2 * r + 1] = (double)outi;                                                             \
            if (d_out) d_out[r] = (double)dd;                                                            \
        }                                                                                                \
    }

DEFINE_ORACLE_SPMV_C(oracle_csr_spmv_c32, float, double)
DEFINE_ORACLE_SPMV_C(oracle_csr_spmv_c64, double, long double)

/* C_out (interleaved) and d_out are dense m x n row-major with leading dimension n, whatever C's order
 * (mcsparse/src/kernels/level3/spmm/csr_spmm_device.hpp:116-137,149-165 on complex numbers). */
#define DEFINE_ORACLE_SPMM_C(NAME, VT, ACC)                                                             \
    void NAME(int64_t m, int64_t n, int base, const int32_t* row_ptr, const int32_t* col, const VT* val, \
              const VT* B, int64_t ldb, int orderB, const double* alpha, const double* beta, const VT* C_in, \
              int64_t ldc, int orderC, double* C_out, double* d_out) {                                   \
        const double abs_alpha = hypot(alpha[0], alpha[1]), abs_beta = hypot(beta[0], beta[1]);          \
        _Pragma("omp parallel for schedule(dynamic, 256)") for (int64_t r = 0; r < m; ++r) {             \
            for (int64_t c = 0; c < n; ++c) {                                                            \
                ACC sr = 0, si = 0, d = 0;                                                               \
                for (int64_t j = (int64_t)row_ptr[r] - base; j < (int64_t)row_ptr[r + 1] - base; ++j) {  \
                    const int64_t bi = dn_index((int64_t)col[j] - base, c, ldb, orderB);                 \
                    const ACC ar = val[2 * j], ai = val[2 * j + 1], br = B[2 * bi], bim = B[2 * bi + 1]; \
                    sr += ar * br - ai * bim;                                                            \
                    si += ar * bim + ai * br;                                                            \
                    d += (ACC)hypotl((long double)ar, (long double)ai) * (ACC)hypotl((long double)br, (long double)bim); \
                }                                                                                        \
                ACC outr = (ACC)alpha[0] * sr - (ACC)alpha[1] * si, outi = (ACC)alpha[0] * si + (ACC)alpha[1] * sr; \
                ACC dd = (ACC)abs_alpha * d;                                                             \
                if (abs_beta != 0.0) {                                                                   \
                    const int64_t ci = dn_index(r, c, ldc, orderC);                                      \
                    const ACC cr = C_in[2 * ci], cim = C_in[2 * ci + 1];                                 \
                    outr += (ACC)beta[0] * cr - (ACC)beta[1] * cim;                                      \
                    outi += (ACC)beta[0] * cim + (ACC)beta[1] * cr;                                      \
                    dd += (ACC)abs_beta * (ACC)hypotl((long double)cr, (long double)cim);                \
                }                                                                                        \
                C_out[2 * (r * n + c)] = (double)outr;                                                   \
                C_out[2 * (r * n + c) + 1] = (double)outi;                                               \
                if (d_out) d_out[r * n + c] = (double)dd;                                                \
            }                                                                                            \
        }                                                                                                \
    }

DEFINE_ORACLE_SPMM_C(oracle_csr_spmm_c32, float, double)
DEFINE_ORACLE_SPMM_C(oracle_csr_spmm_c64, double, long double)

/* ------------------------------------------------------------------ analysis oracle
 *
 * Merge-path work partition. The reference's analysis hook is an empty stub
 * (mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:129-158), so this specification
 * belongs to this build and the device kernel must reproduce it bit for bit.
 *
 * The merge list has m + nnz items: the m row ends e_r = row_ptr[r + 1] - base and the
 * nnz nonzero indices 0..nnz-1; a row end is taken before a nonzero index when
 * e_r <= index. Diagonal d splits the list after d items into (i rows, d - i nonzeros)
 * where i is the smallest value with e_i > d - i - 1. Tile t starts on diagonal
 * min(t * items_per_tile, m + nnz). Output: (num_tiles + 1) int32 pairs {row, nonzero}.
 * Returns num_tiles = ceil((m + nnz) / items_per_tile).
 */
int64_t oracle_merge_path_partition(int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                                    int items_per_tile, int32_t* tile_starts) {
    int64_t items = m + nnz;
    int64_t num_tiles = (items + items_per_tile - 1) / items_per_tile;
    for (int64_t t = 0; t <= num_tiles; ++t) {
        int64_t diag = t * (int64_t)items_per_tile;
        if (diag > items) diag = items;
        int64_t lo = diag > nnz ? diag - nnz : 0;
        int64_t hi = diag < m ? diag : m;
        while (lo < hi) {
            int64_t mid = (lo + hi) >> 1;
            if ((int64_t)row_ptr[mid + 1] - base <= diag - mid - 1)
                lo = mid + 1;
            else
                hi = mid;
        }
        tile_starts[2 * t] = (int32_t)lo;
        tile_starts[2 * t + 1] = (int32_t)(diag - lo);
    }
    return num_tiles;
}

/* Shard g starts at the first row r with row_ptr[r] - base >= floor(g * nnz / G);
 * bounds[0] = 0 and bounds[G] = m. */
void oracle_shard_row_bounds(int64_t m, int64_t nnz, int base, const int32_t* row_ptr, int num_shards,
                             int64_t* bounds) {
    bounds[0] = 0;
    for (int g = 1; g < num_shards; ++g) {
        int64_t target = (int64_t)(((__int128)g * nnz) / num_shards);
        int64_t lo = 0, hi = m;
        while (lo < hi) {
            int64_t mid = (lo + hi) >> 1;
            if ((int64_t)row_ptr[mid] - base < target)
                lo = mid + 1;
            else
                hi = mid;
        }
        bounds[g] = lo;
    }
    bounds[num_shards] = m;
}

void oracle_shard_local_row_offsets(const int32_t* row_ptr, int64_t first_row, int64_t num_rows, int base,
                                    int32_t* local) {
    for (int64_t i = 0; i <= num_rows; ++i) local[i] = row_ptr[first_row + i] - row_ptr[first_row] + base;
}

/* CSR row offsets of a COO matrix sorted by row, by counting (the reference's coo2csr step,
 * mcsparse/src/kernels/conversion/coo2csr_device.hpp:8-24, states the same mapping as a scatter). */
void oracle_coo_row_offsets(int64_t m, int64_t nnz, int base, const int32_t* coo_rows, int32_t* offsets) {
    for (int64_t r = 0; r <= m; ++r) offsets[r] = 0;
    for (int64_t j = 0; j < nnz; ++j) offsets[(int64_t)coo_rows[j] - base + 1] += 1;
    offsets[0] = base;
    for (int64_t r = 0; r < m; ++r) offsets[r + 1] += offsets[r];
}

/* CSR arrays of the transposed matrix (equivalently the CSC arrays of the matrix), 0-based, by a
 * stable counting sort on the column: within a row of the transpose the nonzeros keep the order of
 * the source, i.e. ascending source rows. The reference reaches its transposed products through the
 * same conversion (csr2csc, mcsparse/src/common/mcsp_internal_transpose_sparse.hpp:237-341, called from
 * mcsparse/src/kernels/level2/spmv/mcsp_spmv_gpu.cpp:797-846); the order inside a row is this build's
 * choice and is what the device conversion is checked against bit for bit.
 * t_ptr: n + 1 entries; t_idx, perm: nnz entries; perm[k] = source position of transposed nonzero k. */
void oracle_csr_transpose(int64_t m, int64_t n, int64_t nnz, int base, const int32_t* row_ptr, const int32_t* col,
                          int32_t* t_ptr, int32_t* t_idx, int32_t* perm) {
    for (int64_t c = 0; c <= n; ++c) t_ptr[c] = 0;
    for (int64_t j = 0; j < nnz; ++j) t_ptr[(int64_t)col[j] - base + 1] += 1;
    for (int64_t c = 0; c < n; ++c) t_ptr[c + 1] += t_ptr[c];
    int32_t* next = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
    for (int64_t c = 0; c < n; ++c) next[c] = t_ptr[c];
    for (int64_t r = 0; r < m; ++r) {
        for (int64_t j = (int64_t)row_ptr[r] - base; j < (int64_t)row_ptr[r + 1] - base; ++j) {
            const int32_t k = next[(int64_t)col[j] - base]++;
            t_idx[k] = (int32_t)r;
            perm[k] = (int32_t)j;
        }
    }
    free(next);
}

/* Host-side structural check of a CSR matrix: 0 when valid, else the number of the first
 * rule broken (1 first offset, 2 monotone offsets, 3 last offset, 4 column range). */
int oracle_csr_validate(int64_t m, int64_t cols, int64_t nnz, int base, const int32_t* row_ptr,
                        const int32_t* col) {
    if (row_ptr[0] != base) return 1;
    for (int64_t r = 0; r < m; ++r)
        if (row_ptr[r + 1] < row_ptr[r]) return 2;
    if ((int64_t)row_ptr[m] - base != nnz) return 3;
    for (int64_t j = 0; j < nnz; ++j)
        if (col[j] < base || (int64_t)col[j] - base >= cols) return 4;
    return 0;
}

/* ------------------------------------------------------------------ OpenMP baseline */

int baseline_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Size of the OpenMP team of the baseline kernels (a launcher may have exported OMP_NUM_THREADS=1). */
void baseline_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline int baseline_threads_in_region(void) {
#ifdef _OPENMP
    return omp_get_num_threads();
#else
    return 1;
#endif
}
static inline int baseline_thread_id(void) {
#ifdef _OPENMP
    return omp_get_thread_num();
#else
    return 0;
#endif
}

/* Row range of thread t out of T, balanced by nonzeros. */
static void nnz_chunk(int64_t m, const int32_t* row_ptr, int t, int T, int64_t* r0, int64_t* r1) {
    int64_t first = row_ptr[0], nnz = (int64_t)row_ptr[m] - first;
    int64_t bounds[2];
    for (int k = 0; k < 2; ++k) {
        int g = t + k;
        if (g <= 0) {
            bounds[k] = 0;
        } else if (g >= T) {
            bounds[k] = m;
        } else {
            int64_t target = first + (int64_t)(((__int128)g * nnz) / T);
            int64_t lo = 0, hi = m;
            while (lo < hi) {
                int64_t mid = (lo + hi) >> 1;
                if (row_ptr[mid] < target)
                    lo = mid + 1;
                else
                    hi = mid;
            }
            bounds[k] = lo;
        }
    }
    *r0 = bounds[0];
    *r1 = bounds[1];
}

#define DEFINE_BASELINE_SPMV(NAME, VT)                                                                 \
    void NAME(int64_t m, int base, const int32_t* row_ptr, const int32_t* col, const VT* val,          \
              const VT* x, VT alpha, VT beta, VT* y) {                                                 \
        const VT* xb = x - base;                                                                       \
        _Pragma("omp parallel") {                                                                      \
            int T = baseline_threads_in_region(), t = baseline_thread_id();                            \
            int64_t r0, r1;                                                                            \
            nnz_chunk(m, row_ptr, t, T, &r0, &r1);                                                     \
            for (int64_t r = r0; r < r1; ++r) {                                                        \
                VT s = 0;                                                                              \
                int64_t j0 = (int64_t)row_ptr[r] - base, j1 = (int64_t)row_ptr[r + 1] - base;          \
                for (int64_t j = j0; j < j1; ++j) s += val[j] * xb[col[j]];                            \
                y[r] = (beta == (VT)0) ? alpha * s : alpha * s + beta * y[r];                          \
            }                                                                                          \
        }                                                                                              \
    }

DEFINE_BASELINE_SPMV(baseline_csr_spmv_f32, float)
DEFINE_BASELINE_SPMV(baseline_csr_spmv_f64, double)

/* B and C row-major (the benchmark's layout): the inner loop runs along a B row. */
#define DEFINE_BASELINE_SPMM(NAME, VT)                                                                 \
    void NAME(int64_t m, int64_t n, int base, const int32_t* row_ptr, const int32_t* col,              \
              const VT* val, const VT* B, int64_t ldb, VT alpha, VT beta, VT* C, int64_t ldc) {        \
        _Pragma("omp parallel") {                                                                      \
            int T = baseline_threads_in_region(), t = baseline_thread_id();                            \
            int64_t r0, r1;                                                                            \
            nnz_chunk(m, row_ptr, t, T, &r0, &r1);                                                     \
            VT* acc = (VT*)malloc((size_t)(n > 0 ? n : 1) * sizeof(VT));                               \
            for (int64_t r = r0; r < r1; ++r) {                                                        \
                for (int64_t c = 0; c < n; ++c) acc[c] = 0;                                            \
                int64_t j0 = (int64_t)row_ptr[r] - base, j1 = (int64_t)row_ptr[r + 1] - base;          \
                for (int64_t j = j0; j < j1; ++j) {                                                    \
                    const VT a = val[j];                                                               \
                    const VT* brow = B + ((int64_t)col[j] - base) * ldb;                               \
                    for (int64_t c = 0; c < n; ++c) acc[c] += a * brow[c];                             \
                }                                                                                      \
                VT* crow = C + r * ldc;                                                                \
                if (beta == (VT)0)                                                                     \
                    for (int64_t c = 0; c < n; ++c) crow[c] = alpha * acc[c];                          \
                else                                                                                   \
                    for (int64_t c = 0; c < n; ++c) crow[c] = alpha * acc[c] + beta * crow[c];         \
            }                                                                                          \
            free(acc);                                                                                 \
        }                                                                                              \
    }

DEFINE_BASELINE_SPMM(baseline_csr_spmm_f32, float)
DEFINE_BASELINE_SPMM(baseline_csr_spmm_f64, double)
