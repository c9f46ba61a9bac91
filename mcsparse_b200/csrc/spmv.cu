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
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include <type_traits>

#include "internal.h"

namespace mcsp_b200 {

namespace {

constexpr int kThreads = 256;

// Items per thread of the two tile sizes. With 64-bit column indices the staged columns take twice the shared
// memory: 8-byte values keep both sizes (the large tile is then 33 KB), 4-byte values only the small one
// (their large tile would need 49 KB, over the 48 KB of static shared memory).
// The sizes go by the bytes of a value: 4 (float), 8 (double, complex float), 16 (complex double, one size).
constexpr int tile_items(size_t value_size, bool small) {
    return value_size == 4   ? (small ? MCSPARSE_B200_SPMV_SMALL_TILE_ITEMS_F32 : MCSPARSE_B200_SPMV_TILE_ITEMS_F32)
           : value_size == 8 ? (small ? MCSPARSE_B200_SPMV_SMALL_TILE_ITEMS_F64 : MCSPARSE_B200_SPMV_TILE_ITEMS_F64)
                             : MCSPARSE_B200_SPMV_TILE_ITEMS_C64;
}
constexpr bool wide_index_one_size(size_t value_size, size_t index_size) { return index_size == 8 && value_size == 4; }
// Thread blocks per SM the tile kernels are compiled for: as many as their shared memory admits, at most 8
// (256 threads x 8 = all the SM's threads). Without it the push variants, which keep the peer list live, take
// 40 registers and lose a quarter of the resident blocks.
constexpr int tile_min_blocks(size_t value_size, size_t index_size, int threads, int ipt) {
    const size_t smem = size_t(threads) * ipt * (value_size + index_size) + 6144;
    const size_t fit = (227u * 1024u) / smem;
    return fit >= 8 ? 8 : (fit < 1 ? 1 : (int)fit);
}
template <typename T, typename I>
struct TileCfg {
    static constexpr int kSmall = tile_items(sizeof(T), true) / kThreads;
    static constexpr int kLarge = wide_index_one_size(sizeof(T), sizeof(I)) ? kSmall : tile_items(sizeof(T), false) / kThreads;
};

// Structure probe: 1024 threads x 4 samples. count[0]: how many of 4096 evenly spaced pairs of neighbouring
// nonzeros have columns within 8 of each other; count[1]: how many of 4096 evenly spaced rows are longer
// than 256 nonzeros.
template <typename I>
__global__ void locality_probe_kernel(long long m, long long nnz, const I* __restrict__ row_ptr,
                                      const I* __restrict__ col, int* __restrict__ count) {
    __shared__ int s_near, s_long;
    if (threadIdx.x == 0) s_near = s_long = 0;
    __syncthreads();
    int near = 0, longer = 0;
    for (int q = 0; q < 4; ++q) {
        const long long u = threadIdx.x * 4 + q;
        const long long j = (u * (nnz - 1)) / 4096;
        if (nnz >= 2 && j + 1 < nnz) {
            const long long d = (long long)__ldg(col + j + 1) - (long long)__ldg(col + j);
            near += (d <= 8 && d >= -8);
        }
        const long long r = (u * m) / 4096;
        if (row_ptr != nullptr && r < m && (m >= 4096 || (u * m) % 4096 < m))  // each row at most once
            longer += ((long long)__ldg(row_ptr + r + 1) - (long long)__ldg(row_ptr + r)) > 256;
    }
    atomicAdd(&s_near, near);
    atomicAdd(&s_long, longer);
    __syncthreads();
    if (threadIdx.x == 0) count[0] = s_near, count[1] = s_long;
}

// Gather-rate probe: every thread loads 8 indices (two coalesced 128-bit loads), gathers the 8 table
// elements they name and adds them up. With indices that are spread over a table larger than L1 this
// measures how many independent 32-byte sectors per second the SMs can request from L2, which is the
// bound of an SpMV whose columns are scattered (one x gather per nonzero, one sector each).
template <typename T>
__global__ void __launch_bounds__(256) gather_probe_kernel(const int* __restrict__ idx, long long count,
                                                           const T* __restrict__ table, T* __restrict__ out) {
    const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    T acc = T(0);
    for (long long b = t * 4; b + 4 * nthreads + 3 < count; b += nthreads * 8) {
        const int4 a = __ldcs(reinterpret_cast<const int4*>(idx + b));
        const int4 c = __ldcs(reinterpret_cast<const int4*>(idx + b + 4 * nthreads));
        const T v0 = ldg(table + a.x), v1 = ldg(table + a.y), v2 = ldg(table + a.z), v3 = ldg(table + a.w);
        const T v4 = ldg(table + c.x), v5 = ldg(table + c.y), v6 = ldg(table + c.z), v7 = ldg(table + c.w);
        acc += ((v0 + v1) + (v2 + v3)) + ((v4 + v5) + (v6 + v7));
    }
    out[t] = acc;
}

// ---------------------------------------------------------------------------------------
// K0: merge-path analysis. Thread t finds where diagonal min(t * items_per_tile, m + nnz)
// crosses the merge of row ends and nonzero indices. Same search, same tie-break (a row end
// equal to a nonzero index is taken first) as the CPU partition it is checked against.
// ---------------------------------------------------------------------------------------
template <typename I>
__global__ void merge_path_partition_kernel(int m, int nnz, int base, const I* __restrict__ row_ptr,
                                            int items_per_tile, long long num_tiles, int2* __restrict__ starts,
                                            int* __restrict__ status) {
    long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t == 0) *status = 0;
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
// Bulk asynchronous copies (TMA, untiled form) and the mbarrier they complete on.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Global -> this CTA's shared memory; src, dst and bytes are multiples of 16. The data is read
// exactly once, so it is marked evict-first in L2 to leave the cache to x.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar,
                                              unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// Waits for phase `parity` of the barrier for at most `limit` SM clocks. Returns false on timeout,
// which the kernel reports in the status words instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, uint32_t parity, long long limit) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit) return false;
    }
    return true;
}


// PUSH variants: a finished y value is also stored, with ordinary global stores through
// peer-mapped pointers, into the full-length y of every other GPU of a row-sharded run, at
// the row's global position. The NVLink traffic thus overlaps the kernel instead of
// following it as a separate all-gather. A row that continues from an earlier tile is the
// exception: its value is final only after the carry fix-up, which pushes it then.
//
// Multicast mode (peers.multicast): y[0] is the address of the full-length y inside an NVSwitch
// multicast mapping that spans all GPUs of the run; one multimem.st then reaches every GPU's copy
// (this one included), so a row costs one store instruction instead of one per peer and the
// replication happens in the switch.
__device__ __forceinline__ void multicast_store(float* p, float v) {
    asm volatile("multimem.st.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void multicast_store(double* p, double v) {
    asm volatile("multimem.st.global.f64 [%0], %1;" ::"l"(p), "d"(v) : "memory");
}
// 16 bytes at a 16-byte aligned multicast address (the bit patterns travel unchanged).
__device__ __forceinline__ void multicast_store_vec16(float* dst, const float* v) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]),
                 "f"(v[3])
                 : "memory");
}
__device__ __forceinline__ void multicast_store_vec16(double* dst, const double* v) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__int_as_float(__double2loint(v[0]))),
                 "f"(__int_as_float(__double2hiint(v[0]))), "f"(__int_as_float(__double2loint(v[1]))),
                 "f"(__int_as_float(__double2hiint(v[1])))
                 : "memory");
}

// peers.y[p] for a p that is not a compile-time constant. Indexing the array directly would make the compiler
// copy the whole kernel parameter to local memory at the start of every thread (80 bytes x every thread of every
// tile block: measured a quarter of the kernel's time); a chain of selects keeps it in the constant bank.
template <typename T>
__device__ __forceinline__ T* peer_ptr(const PeerList<T>& peers, int p) {
    T* q = peers.y[0];
#pragma unroll
    for (int i = 1; i < PeerList<T>::kMax; ++i)
        if (p == i) q = peers.y[i];
    return q;
}

// (Write-through and streaming cache operators on the peer stores were measured and change
// nothing: 0.645 ms per step at two GPUs with any of them.)
template <typename T>
__device__ __forceinline__ void push_to_peers(const PeerList<T>& peers, long long row, T v) {
    if (peers.multicast) {
        multicast_store(peers.y[0] + peers.row_offset + row, v);
        return;
    }
#pragma unroll 1
    for (int p = 0; p < peers.count; ++p) peer_ptr(peers, p)[peers.row_offset + row] = v;  // a loop: this path is rare
}

__device__ __forceinline__ void store_vec16(float* dst, const float* v) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_vec16(double* dst, const double* v) {
    *reinterpret_cast<double2*>(dst) = make_double2(v[0], v[1]);
}

// Stores the n finished values vals[0..n) (shared memory) of local rows row0.. to every peer, with
// 128-bit stores aligned on the destination address: one warp instruction then moves 512
// contiguous bytes, and NVLink carries a few large writes much better than many 8-byte ones.
template <typename T, int THREADS>
__device__ __forceinline__ void push_tile_rows(const PeerList<T>& peers, const T* vals, long long row0, int n,
                                               int tid) {
    constexpr int VW = 16 / (int)sizeof(T);
#pragma unroll
    for (int p = 0; p < PeerList<T>::kMax; ++p) {
        if (p < peers.count) {
            T* const dst = peers.y[p] + peers.row_offset + row0;
            const int mis = (int)((reinterpret_cast<uintptr_t>(dst) / sizeof(T)) & (VW - 1));
            const int head = min(n, (VW - mis) & (VW - 1));
            const int nvec = (n - head) / VW;
            for (int c = tid; c < nvec; c += THREADS) {
                T v[VW];
#pragma unroll
                for (int e = 0; e < VW; ++e) v[e] = vals[head + c * VW + e];
                if (peers.multicast)
                    multicast_store_vec16(dst + head + c * VW, v);
                else
                    store_vec16(dst + head + c * VW, v);
            }
            const int tail0 = head + nvec * VW;
            const int u = THREADS - 1 - tid;  // the scalar edges go to the last threads, idle above
            if (peers.multicast) {
                if (u < head) multicast_store(dst + u, vals[u]);
                if (u >= VW && u - VW < n - tail0) multicast_store(dst + tail0 + (u - VW), vals[tail0 + (u - VW)]);
            } else {
                if (u < head) dst[u] = vals[u];
                if (u >= VW && u - VW < n - tail0) dst[tail0 + (u - VW)] = vals[tail0 + (u - VW)];
            }
        }
    }
}

// Misalignment, in elements, of the peers' address of local row `row0` against 16 bytes (the same for every
// peer when the bulk push is on): rows staged for the bulk push start at this offset of a 16-byte aligned area.
template <typename T>
__device__ __forceinline__ int push_misalign(const PeerList<T>& peers, long long row0) {
    constexpr int VW = 16 / (int)sizeof(T);
    if (!peers.bulk) return 0;
    return (int)((reinterpret_cast<uintptr_t>(peers.y[0] + peers.row_offset + row0) / sizeof(T)) & (VW - 1));
}

// Same job as push_tile_rows with the bulk of the bytes moved by the TMA unit instead of the load/store
// unit: the finished rows sit in shared memory, placed so that the value bound for the first 16-byte
// aligned destination address is itself 16-byte aligned (vals[i] = row row0 + i; the caller offsets its
// staging area by the destination's misalignment), and one thread starts one bulk copy shared -> global
// per peer. Peer stores issued by the load/store unit queue behind NVLink in the same path as the x
// gathers and stall the SM's other thread blocks; bulk stores wait in the TMA unit instead, so the tiles
// that are still computing keep their loads flowing and the transfer overlaps the computation.
// All destinations must share their alignment modulo 16 bytes (the host checks). Every thread of the
// block calls this after writing its rows; the block may not touch the staged rows until it returns.
template <typename T, int THREADS>
__device__ __forceinline__ void push_tile_rows_bulk(const PeerList<T>& peers, const T* vals, long long row0, int n,
                                                    int tid) {
    constexpr int VW = 16 / (int)sizeof(T);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // this thread's rows, for the bulk copies
    __syncthreads();
    T* const dst0 = peers.y[0] + peers.row_offset + row0;
    const int mis = (int)((reinterpret_cast<uintptr_t>(dst0) / sizeof(T)) & (VW - 1));
    const int head = min(n, (VW - mis) & (VW - 1));
    const int nvec = (n - head) / VW;
    const int tail0 = head + nvec * VW;
    if (tid == 0 && nvec > 0) {
        const uint32_t src = smem_addr(vals + head);
        const uint32_t bytes = (uint32_t)nvec * 16u;
        for (int p = 0; p < peers.count; ++p)
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                             peer_ptr(peers, p) + peers.row_offset + row0 + head),
                         "r"(src), "r"(bytes)
                         : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    // the few rows before the first and after the last aligned group: ordinary stores by the last warp
    // (the other warps have nothing left to do here: the peer loop is kept out of their instruction stream)
    if (tid >= THREADS - 32 && (head > 0 || tail0 < n)) {
        const int u = THREADS - 1 - tid;
        for (int p = 0; p < peers.count; ++p) {
            T* const dst = peer_ptr(peers, p) + peers.row_offset + row0;
            if (u < head) dst[u] = vals[u];
            if (u >= VW && u - VW < n - tail0) dst[tail0 + (u - VW)] = vals[tail0 + (u - VW)];
        }
    }
    if (tid == 0 && nvec > 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staged rows were read
}

// ---------------------------------------------------------------------------------------
// Staging of one tile's slice of col / val in shared memory, shared by the tile kernels.
//
// issue   one thread starts two bulk asynchronous copies (TMA) of the 16-byte aligned part of the
//         slice that lies inside the arrays; they complete on the mbarrier. The few elements such
//         a boundary would push outside the arrays (at most 3 at either end of an array, or all
//         of a tile of at most 6 elements) are fetched with ordinary loads by warp 0.
// finish  thread 0 waits for the barrier, for at most wait.limit_cycles SM clocks. If the limit
//         runs out the tile is not computed: the status word of the work buffer and the handle's
//         host-visible fault word are set and the function returns false to every thread. Copies
//         that were issued may still land in this block's shared memory, so the block stays
//         resident for a second, far longer limit before it gives the tile up; with the diagnostics
//         switch wait.withhold no copy was issued and it leaves at once. A copy that completes
//         during the second wait is used normally and only leaves a warning (status 2).
// ---------------------------------------------------------------------------------------
template <typename T, typename I>
struct TileSlice {
    int head_c, head_v;  // element nz_s + k of col / val is staged at s_col[head_c + k] / s_val[head_v + k]
    int span_c;          // staged extent of s_col in elements (the row ends live behind it)
    bool copies;         // a bulk copy was asked for
};

template <typename T, typename I>
__device__ __forceinline__ TileSlice<T, I> stage_issue(int tid, int nnz, int nz_s, int nz_e, const I* __restrict__ col,
                                                       const T* __restrict__ val, T* s_val, I* s_col,
                                                       unsigned long long* s_mbar, const WaitCfg& wait) {
    constexpr int GV = 16 / (int)sizeof(T);  // values per 16 bytes
    constexpr int GC = 16 / (int)sizeof(I);  // column indices per 16 bytes
    const int nnz_tile = nz_e - nz_s;
    TileSlice<T, I> ts;
    // head_c is chosen so that the element at index 0 of s_col sits on a 16-byte boundary in global
    // memory. Likewise for val.
    ts.head_c = (int)((reinterpret_cast<uintptr_t>(col) / sizeof(I)) + (unsigned)nz_s) & (GC - 1);
    ts.head_v = (int)((reinterpret_cast<uintptr_t>(val) / sizeof(T)) + (unsigned)nz_s) & (GV - 1);
    ts.span_c = (ts.head_c + nnz_tile + GC - 1) & ~(GC - 1);
    int lo_c = nz_s - ts.head_c, hi_c = lo_c + ts.span_c;  // global element range of the col copy
    if (lo_c < 0) lo_c += GC;
    if (hi_c > nnz) hi_c -= GC;
    int lo_v = nz_s - ts.head_v, hi_v = lo_v + ((ts.head_v + nnz_tile + GV - 1) & ~(GV - 1));
    if (lo_v < 0) lo_v += GV;
    if (hi_v > nnz) hi_v -= GV;
    const bool copy_c = hi_c > lo_c, copy_v = hi_v > lo_v;
    ts.copies = copy_c || copy_v;
    if (tid == 0) mbar_init(s_mbar, 1);
    __syncthreads();
    if (tid == 0 && ts.copies) {
        const unsigned long long policy = l2_evict_first_policy();
        const uint32_t bytes_c = copy_c ? (uint32_t)(hi_c - lo_c) * (uint32_t)sizeof(I) : 0u;
        const uint32_t bytes_v = copy_v ? (uint32_t)(hi_v - lo_v) * (uint32_t)sizeof(T) : 0u;
        mbar_expect_tx(s_mbar, bytes_c + bytes_v);
        if (!wait.withhold) {
            if (copy_c) bulk_copy_g2s(s_col + (lo_c - (nz_s - ts.head_c)), col + lo_c, bytes_c, s_mbar, policy);
            if (copy_v) bulk_copy_g2s(s_val + (lo_v - (nz_s - ts.head_v)), val + lo_v, bytes_v, s_mbar, policy);
        }
    }
    // Lanes 0-15 of warp 0 handle col, lanes 16-31 val; sub-lanes 0-7 the front part, 8-15 the back.
    if (tid < 32) {
        const bool is_val = tid >= 16;
        const int u = tid & 15;
        const bool cp = is_val ? copy_v : copy_c;
        const int lo = is_val ? lo_v : lo_c, hi = is_val ? hi_v : hi_c;
        const int front = cp ? max(0, min(lo, nz_e) - nz_s) : nnz_tile;
        const int back0 = cp ? max(hi, nz_s) : nz_e;
        const int g = u < 8 ? nz_s + u : back0 + (u - 8);
        const bool mine = u < 8 ? (u < front) : (g < nz_e);
        if (mine) {
            if (is_val)
                s_val[ts.head_v + (g - nz_s)] = ldcs(val + g);
            else
                s_col[ts.head_c + (g - nz_s)] = __ldcs(col + g);
        }
    }
    return ts;
}

// One thread polls the barrier (a whole CTA polling would crowd the shared-memory pipe that the
// other resident CTAs need); the block barrier then publishes the copied data to everyone.
__device__ __forceinline__ bool stage_finish(int tid, bool copies, unsigned long long* s_mbar, int* s_failed,
                                             int* __restrict__ status, const WaitCfg& wait) {
    if (tid == 0) {
        int failed = 0;
        if (copies && !mbar_wait_bounded(s_mbar, 0, wait.limit_cycles)) {  // never expected; reported, not spun on
            failed = 1;
            if (!wait.withhold && mbar_wait_bounded(s_mbar, 0, wait.limit_cycles * 256)) {
                failed = 0;  // the copies did arrive: the tile is computed, the delay is only noted
                atomicOr(status, 2);
            }
            if (failed) {
                atomicOr(status, 1);
                if (wait.fault_word != nullptr) {
                    *reinterpret_cast<volatile int*>(wait.fault_word) = 1;
                    __threadfence_system();
                }
            }
        }
        *s_failed = failed;
    }
    __syncthreads();
    return *s_failed == 0;
}

// ---------------------------------------------------------------------------------------
// Push crew: the thread blocks of a sharded tile launch that move finished rows to the peers.
//
// The tile blocks of such a launch compute exactly as on one GPU and only count themselves off
// (done[chunk] += 1 after their rows are written). A crew block takes the chunks c = blockIdx.x,
// blockIdx.x + pushers, ...: it waits (bounded) until all tiles of the chunk have counted off, then
// copies the rows that ended in the chunk from the local y to the same global rows of every peer's y:
// one thread runs a two-stage pipeline of bulk copies (TMA) global -> shared -> the peers' global
// memory, a second warp stores the few rows before and after the 16-byte aligned middle. The copies use
// neither registers nor the load/store unit, and a crew block holds one of the SM's block slots, not
// the SM: the NVLink transfer runs beside the computation instead of stretching every tile block.
// Rows that take a carry from an earlier tile are final only after the fix-up kernel, which pushes them again.
// `vals` is shared memory of at least 2 * piece_elems elements, 16-byte aligned; the local y and all
// peers' y share their alignment modulo 16 bytes (checked on the host).
// ---------------------------------------------------------------------------------------
constexpr int kCrewStages = 4;  // pieces of a crew block in flight
// Polls with relaxed loads that bypass L1. An acquire at GPU scope would invalidate the SM's L1 on every poll,
// and with it the x lines that the tile blocks sharing the SM live on; nothing the crew reads afterwards can be
// stale in L1 instead: the rows are fetched by bulk copies and by ld.global.cg, both served by L2, where the
// tile blocks' stores were before their release of the counter.
__device__ __forceinline__ bool chunk_wait_bounded(const int* counter, int want, long long limit) {
    const long long t0 = clock64();
    for (;;) {
        int seen;
        asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
        if (seen >= want) return true;
        if (clock64() - t0 > limit) return false;
        __nanosleep(500);
    }
}

template <typename T>
__device__ __forceinline__ void crew_report_failure(int* status, const WaitCfg& wait) {
    atomicOr(status, 1);
    if (wait.fault_word != nullptr) {
        *reinterpret_cast<volatile int*>(wait.fault_word) = 1;
        __threadfence_system();
    }
}

template <typename T>
__device__ void push_crew(const CrewCfg& crew, const PeerList<T>& peers, const int2* __restrict__ tile_starts,
                          long long num_tiles, T* __restrict__ y, const int* __restrict__ carry_row,
                          const T* __restrict__ carry_val, T alpha, T* vals, int piece_elems,
                          unsigned long long* bars, int* __restrict__ status, const WaitCfg& wait) {
    constexpr int VW = 16 / (int)sizeof(T);
    const int tid = threadIdx.x;
    if (tid >= 32) return;  // one warp: all lanes finish the chunk's rows, lane 0 runs the bulk copies
    const long long limit = wait.limit_cycles * 50;  // a chunk is ready when the tiles ahead of it have run
    if (tid == 0)
        for (int st = 0; st < kCrewStages; ++st) mbar_init(bars + st, 1);
    constexpr int NS = kCrewStages;
    uint32_t parity = 0u;  // bit s: phase of stage s's barrier
    bool dead = false;     // lane 0: a bulk load never arrived; the block stops at the next chunk
    for (int c = blockIdx.x; c < crew.num_chunks; c += crew.pushers) {
        const long long t0 = (long long)c * crew.tiles_per_chunk;
        const long long t1 = min(t0 + crew.tiles_per_chunk, num_tiles);
        // this chunk's tiles, and the chunk before (its last tiles hold the carries of this chunk's first rows)
        int give_up = 0;
        if (tid == 0) {
            give_up = dead || !chunk_wait_bounded(crew.done + c, (int)(t1 - t0), limit) ||
                      (c > 0 && !chunk_wait_bounded(crew.done + c - 1, crew.tiles_per_chunk, limit));
            if (give_up && !dead) crew_report_failure<T>(status, wait);  // never finished: reported, not waited for
        }
        if (__shfl_sync(0xffffffffu, give_up, 0)) return;  // nothing of this block is in flight here
        // Carries: a tile's first row, if it ends in the tile, also takes what earlier tiles left for it, summed in
        // tile order exactly as spmv_carry_fixup_range_kernel does (same bits). Everything is read through L2
        // (ld.global.cg): L1 may hold lines of these arrays from before their tiles had written them.
        long long oldest = c > 0 ? t0 - crew.tiles_per_chunk : 0;  // first tile known to have finished
        for (long long tt = t0 + tid; tt < t1; tt += 32) {
            if (tt == 0) continue;
            const int r = tile_starts[tt].x;
            if (tile_starts[tt + 1].x <= r) continue;  // no row ends in this tile
            long long u = tt - 1;                      // carry_row[tt - 1] == r by construction
            bool ok = true;
            while (u > 0) {
                if (u - 1 < oldest) {  // the run reaches into a still older chunk: it must have finished too
                    const long long q = (u - 1) / crew.tiles_per_chunk;
                    if (!chunk_wait_bounded(crew.done + q, crew.tiles_per_chunk, limit)) {
                        ok = false;
                        break;
                    }
                    oldest = q * crew.tiles_per_chunk;
                }
                if (__ldcg(carry_row + u - 1) != r) break;
                --u;
            }
            if (!ok) {
                crew_report_failure<T>(status, wait);
                continue;
            }
            T sum = __ldcg(carry_val + u);
            for (++u; u < tt; ++u) sum += __ldcg(carry_val + u);
            y[r] = mad(alpha, sum, __ldcg(y + r));
        }
        asm volatile("fence.proxy.async;" ::: "memory");  // this lane's stores, and the tiles', before the bulk loads
        __syncwarp();
        const long long r0 = tile_starts[t0].x, r1 = tile_starts[t1].x;  // rows that ended in the chunk
        if (r1 <= r0) continue;
        const T* const src = y + r0;
        const int n = (int)(r1 - r0);
        const int mis = (int)((reinterpret_cast<uintptr_t>(src) / sizeof(T)) & (VW - 1));
        const int head = min(n, (VW - mis) & (VW - 1));
        const int nvec = (n - head) / VW;
        const int tail0 = head + nvec * VW;
        if (tid >= 1 && tid <= 2 * VW) {  // edges: at most VW - 1 rows at either end, by lanes 1 ... 2 VW
            const int u = tid - 1;
            for (int p = 0; p < peers.count; ++p) {
                T* const dst = peer_ptr(peers, p) + peers.row_offset + r0;
                if (u < head) dst[u] = __ldcg(src + u);
                if (u >= VW && u - VW < n - tail0) dst[tail0 + (u - VW)] = __ldcg(src + tail0 + (u - VW));
            }
        }
        if (tid != 0 || nvec == 0) continue;
        // lane 0: pieces of the aligned middle through NS stages: up to NS - 1 loads in flight while one piece leaves
        asm volatile("fence.proxy.async;" ::: "memory");  // the tiles' ordinary stores, before the bulk loads
        const unsigned long long policy = l2_evict_first_policy();
        const int total = nvec * VW;
        const int pieces = (total + piece_elems - 1) / piece_elems;
        auto load = [&](int k) {
            const int st = k % NS, e0 = k * piece_elems, cnt = min(piece_elems, total - e0);
            mbar_expect_tx(bars + st, (uint32_t)cnt * (uint32_t)sizeof(T));
            bulk_copy_g2s(vals + st * piece_elems, src + head + e0, (uint32_t)cnt * (uint32_t)sizeof(T), bars + st, policy);
        };
        for (int k = 0; k < min(pieces, NS - 1); ++k) load(k);
        bool failed = false;
        for (int k = 0; k < pieces; ++k) {
            const int st = k % NS;
            const uint32_t ph = (parity >> st) & 1u;
            if (!mbar_wait_bounded(bars + st, ph, wait.limit_cycles) &&
                !mbar_wait_bounded(bars + st, ph, wait.limit_cycles * 256)) {
                failed = true;
                break;
            }
            parity ^= 1u << st;
            const int e0 = k * piece_elems, cnt = min(piece_elems, total - e0);
            const uint32_t sm = smem_addr(vals + st * piece_elems);
            for (int p = 0; p < peers.count; ++p)
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                                 peer_ptr(peers, p) + peers.row_offset + r0 + head + e0),
                             "r"(sm), "r"((uint32_t)cnt * (uint32_t)sizeof(T))
                             : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            if (k + NS - 1 < pieces) {
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // piece k - 1 has left its stage
                load(k + NS - 1);
            }
        }
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (failed) {  // a bulk load that never arrived
            crew_report_failure<T>(status, wait);
            dead = true;
        }
        // (lanes 1 ... 31 wait for lane 0 at the shuffle of the next chunk, and leave with it)
    }
}

// A tile block of a launch with a push crew counts itself off once its rows are in global memory.
template <bool CREW>
__device__ __forceinline__ void tile_count_off(const CrewCfg& crew, int t, int tid) {
    if constexpr (CREW) {
        __syncthreads();  // every thread's stores to y are issued
        // A release without the acquire half: a full fence here would invalidate the SM's L1 at the end of every
        // tile and take the x lines of the other resident tiles with it.
        if (tid == 0)
            asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(crew.done + t / crew.tiles_per_chunk) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// K1: tiled SpMV. Block t owns merge items [t * TILE, (t + 1) * TILE): `nrows` row ends and
// `nnz_tile` nonzeros (nrows + nnz_tile = TILE except in the last tile).
//
//   phase 1  one thread issues two bulk asynchronous copies (TMA) that bring the tile's slice
//            of col and val into shared memory, widened to 16-byte boundaries; the few elements
//            such a boundary would push outside the arrays are fetched with ordinary loads.
//            Meanwhile all threads stage the row ends of the tile's rows. The copies complete on
//            an mbarrier. They cost no registers and no load/store-unit traffic, and a resident
//            CTA keeps up to 24 KB in flight, which is what hides HBM latency here.
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
// No atomics on the data path: every addition has a fixed place, so results are reproducible.
// ---------------------------------------------------------------------------------------
template <typename T, int THREADS, int IPT, bool PUSH, typename I, bool CREW = false>
__global__ void __launch_bounds__(THREADS, (PUSH || CREW) ? tile_min_blocks(sizeof(T), sizeof(I), THREADS, IPT) : 0)
    spmv_tile_kernel(int m, int nnz, int base, const I* __restrict__ row_ptr, const I* __restrict__ col,
                     const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y, ScalarArg<T> alpha_arg,
                     ScalarArg<T> beta_arg, const int2* __restrict__ tile_starts, int* __restrict__ carry_row,
                     T* __restrict__ carry_val, int* __restrict__ status, PeerList<T> peers, int tile_offset,
                     WaitCfg wait, CrewCfg crew) {
    constexpr int TILE = THREADS * IPT;
    constexpr int NWARPS = THREADS / 32;
    constexpr int WALK = IPT + 1;  // merge items per thread in the long-row walk: odd, so that the
                                   // stride-WALK shared reads of a warp fall in distinct banks

    __shared__ __align__(128) T s_val[TILE + 16];   // values (then products); long-row path: row sums behind them
    __shared__ __align__(128) I s_col[TILE + 16];  // column indices, then the tile's row ends (int) behind them
    __shared__ __align__(8) unsigned long long s_mbar;
    __shared__ __align__(8) unsigned long long s_mbar_crew[CREW ? kCrewStages : 1];
    __shared__ int s_warp_row[NWARPS];  // long-row path: last carry of each warp
    __shared__ T s_warp_sum[NWARPS];
    __shared__ int s_warp_maxlen[NWARPS];
    __shared__ int s_failed;
    constexpr int PUSHCAP = PUSH ? 128 : 1;  // finished rows of a short-row tile staged for the push
    __shared__ __align__(16) T s_push[PUSHCAP + 4];

    const int tid = threadIdx.x;
    if constexpr (CREW) {
        if ((int)blockIdx.x < crew.pushers) {  // this block belongs to the push crew: it computes no tile
            push_crew<T>(crew, peers, tile_starts, (long long)gridDim.x - crew.pushers, y, carry_row, carry_val,
                         alpha_arg.get(), s_val, (TILE / kCrewStages) & ~3, &s_mbar_crew[0], status, wait);
            return;
        }
    }
    const int t = (int)blockIdx.x - (CREW ? crew.pushers : 0) + tile_offset;  // a launch may cover a sub-range of the tiles
    const int2 s0 = tile_starts[t];
    const int2 s1 = tile_starts[t + 1];
    const int row_s = s0.x, nz_s = s0.y;
    const int nrows = s1.x - s0.x;
    const int nz_e = s1.y;
    const int nnz_tile = nz_e - nz_s;
    const int tile_items = nrows + nnz_tile;

    // ---- phase 1: bulk copies of the tile's slice of col / val, edge elements by ordinary loads
    const TileSlice<T, I> ts = stage_issue<T, I>(tid, nnz, nz_s, nz_e, col, val, s_val, s_col, &s_mbar, wait);
    const I* const colv = s_col + ts.head_c;  // colv[k], valv[k]: k-th nonzero of the tile
    T* const valv = s_val + ts.head_v;
    int* const s_row_end = reinterpret_cast<int*>(s_col + ts.span_c);  // nrows + 1 ints; nrows + nnz_tile <= TILE

    // Row ends in tile-local nonzero coordinates; entry nrows is the row left open.
    // Alongside: the longest piece of a row inside this tile, which selects the phase-2 path.
    int maxlen = 0;
    for (int i = tid; i <= nrows; i += THREADS) {
        const int r = row_s + i;
        int e = (r < m) ? (int)__ldg(row_ptr + r + 1) - base : nz_e;
        e = min(e, nz_e);
        const int b = (r < m) ? max((int)__ldg(row_ptr + r) - base, nz_s) : nz_e;
        maxlen = max(maxlen, e - b);
        s_row_end[i] = e - nz_s;
    }
    maxlen = __reduce_max_sync(0xffffffffu, maxlen);
    if ((tid & 31) == 0) s_warp_maxlen[tid >> 5] = maxlen;
    if (!stage_finish(tid, ts.copies, &s_mbar, &s_failed, status, wait)) {
        if (tid == 0) carry_row[t] = m;  // a tile that was given up leaves no carry for the fix-up
        tile_count_off<CREW>(crew, t, tid);  // (the crew must not wait for it; the failure is already reported)
        return;
    }

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

    const int push_mis = PUSH ? push_misalign(peers, row_s) : 0;
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
                const T x0 = ldg(xb + colv[k]), x1 = ldg(xb + colv[k + G]);
                const T x2 = ldg(xb + colv[k + 2 * G]), x3 = ldg(xb + colv[k + 3 * G]);
                sum = mad(valv[k], x0, sum);
                sum = mad(valv[k + G], x1, sum);
                sum = mad(valv[k + 2 * G], x2, sum);
                sum = mad(valv[k + 3 * G], x3, sum);
            }
            if constexpr (sizeof(T) <= 8 && IPT <= 8) {
                if (k < e) {  // up to three left: gathered together as well (one after the other, each would wait for the last)
                    const int k1 = min(k + G, e - 1), k2 = min(k + 2 * G, e - 1);
                    const T x0 = ldg(xb + colv[k]), x1 = ldg(xb + colv[k1]), x2 = ldg(xb + colv[k2]);
                    sum = mad(valv[k], x0, sum);
                    if (k + G < e) sum = mad(valv[k + G], x1, sum);
                    if (k + 2 * G < e) sum = mad(valv[k + 2 * G], x2, sum);
                }
            } else {  // (complex double and the 16-item tiles would pay for it with a resident block less per SM)
                for (; k < e; k += G) sum = mad(valv[k], ldg(xb + colv[k]), sum);
            }
            for (int d = G >> 1; d > 0; d >>= 1) sum += shfl_xor(sum, d);
            if (glane == 0 && i <= nrows) {
                if (i < nrows) {
                    T v = alpha * sum;
                    if (beta != T(0)) v = mad(beta, y[row_s + i], v);
                    y[row_s + i] = v;
                    if constexpr (PUSH) {
                        if (nrows <= PUSHCAP)
                            s_push[push_mis + i] = v;
                        else
                            push_to_peers(peers, row_s + i, v);
                    }
                } else {
                    carry_row[t] = row_s + nrows;
                    carry_val[t] = sum;
                }
            }
        }
        if constexpr (PUSH) {
            if (nrows <= PUSHCAP) {  // block-uniform
                if (peers.bulk) {
                    push_tile_rows_bulk<T, THREADS>(peers, s_push + push_mis, row_s, nrows, tid);
                } else {
                    __syncthreads();
                    push_tile_rows<T, THREADS>(peers, s_push, row_s, nrows, tid);
                }
            }
        }
        tile_count_off<CREW>(crew, t, tid);
        return;
    }

    // ---- long rows: products in place, merge walk, segmented reduction of the carries
    // s_y[i]: row row_s + i, i in [0, nrows]; with the bulk push, placed for 16-byte aligned copies
    T* const s_y = (PUSH && peers.bulk) ? s_val + ((ts.head_v + nnz_tile + 3) & ~3) + push_mis : valv + nnz_tile;
    {
        // Lane-consecutive nonzeros; all of a thread's gathers are issued before the first product.
        T xv[IPT];
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            const int k = tid + j * THREADS;
            xv[j] = (k < nnz_tile) ? ldg(xb + colv[k]) : T(0);
        }
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            const int k = tid + j * THREADS;
            if (k < nnz_tile) valv[k] *= xv[j];
        }
    }
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
        const T up = shfl_up(sum, d);
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
        if (beta != T(0)) v = mad(beta, y[row_s + i], v);
        y[row_s + i] = v;
        if constexpr (PUSH) s_y[i] = v;  // only this thread touches s_y[i] here
    }
    if constexpr (PUSH) {
        const T open_sum = s_y[nrows];
        if (peers.bulk) {
            push_tile_rows_bulk<T, THREADS>(peers, s_y, row_s, nrows, tid);
        } else {
            __syncthreads();
            push_tile_rows<T, THREADS>(peers, s_y, row_s, nrows, tid);
        }
        if (tid == 0) {
            carry_row[t] = row_s + nrows;
            carry_val[t] = open_sum;
        }
        return;
    }
    if (tid == 0) {
        carry_row[t] = row_s + nrows;
        carry_val[t] = s_y[nrows];
    }
    tile_count_off<CREW>(crew, t, tid);
}

// ---------------------------------------------------------------------------------------
// K1w: tiled SpMV for matrices with scattered columns (every x gather is its own 32-byte sector).
//
// On such matrices the limit is not HBM but the one request per clock that an SM can send to L2:
// a random gather is one request, so the kernel is built to keep that port busy and to spend as
// little else of the L1 data pipe as it can. Same tiles, staging and carries as K1, but one path
// for every tile and no products written back to shared memory:
//   - each thread owns WALK consecutive merge items of the tile (found by a merge-path search over
//     the staged row ends; WALK is odd, so the stride-WALK shared reads of a warp hit distinct banks);
//   - it reads its nonzeros' columns, issues all its x gathers at once, multiplies by the staged
//     values in registers, and then walks its items: a product adds to the running sum, a row end
//     stores the sum of the row piece seen by this thread;
//   - the piece of a row that was still open at the end of a thread is carried to the thread where
//     the row ends by a warp-shuffle segmented scan and, across the warps, in a fixed order.
// Per nonzero that is two conflict-free shared loads, one gather and one multiply-add; empty rows,
// rows of one nonzero and rows of a hundred thousand go through the same code.
// ---------------------------------------------------------------------------------------
template <typename T, int THREADS, int IPT, bool PUSH, typename I, bool CREW = false>
__global__ void __launch_bounds__(THREADS, (PUSH || CREW) ? tile_min_blocks(sizeof(T), sizeof(I), THREADS, IPT) : 0)
    spmv_walk_kernel(int m, int nnz, int base, const I* __restrict__ row_ptr, const I* __restrict__ col,
                     const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y, ScalarArg<T> alpha_arg,
                     ScalarArg<T> beta_arg, const int2* __restrict__ tile_starts, int* __restrict__ carry_row,
                     T* __restrict__ carry_val, int* __restrict__ status, PeerList<T> peers, int tile_offset,
                     WaitCfg wait, CrewCfg crew) {
    constexpr int TILE = THREADS * IPT;
    constexpr int NWARPS = THREADS / 32;
    constexpr int WALK = IPT + 1;
    static_assert(WALK % 2 == 1, "the walk stride must be odd");

    __shared__ __align__(128) T s_val[TILE + 16];  // values; the row sums behind them
    __shared__ __align__(128) I s_col[TILE + 16];  // column indices, then the tile's row ends (int) behind them
    __shared__ __align__(8) unsigned long long s_mbar;
    __shared__ __align__(8) unsigned long long s_mbar_crew[CREW ? kCrewStages : 1];
    __shared__ int s_k0[THREADS];  // first nonzero of every thread's segment
    __shared__ int s_warp_row[NWARPS];
    __shared__ T s_warp_sum[NWARPS];
    __shared__ int s_failed;

    const int tid = threadIdx.x;
    if constexpr (CREW) {
        if ((int)blockIdx.x < crew.pushers) {  // this block belongs to the push crew: it computes no tile
            push_crew<T>(crew, peers, tile_starts, (long long)gridDim.x - crew.pushers, y, carry_row, carry_val,
                         alpha_arg.get(), s_val, (TILE / kCrewStages) & ~3, &s_mbar_crew[0], status, wait);
            return;
        }
    }
    const int t = (int)blockIdx.x - (CREW ? crew.pushers : 0) + tile_offset;
    const int2 s0 = tile_starts[t];
    const int2 s1 = tile_starts[t + 1];
    const int row_s = s0.x, nz_s = s0.y;
    const int nrows = s1.x - s0.x;
    const int nz_e = s1.y;
    const int nnz_tile = nz_e - nz_s;
    const int tile_items = nrows + nnz_tile;

    const TileSlice<T, I> ts = stage_issue<T, I>(tid, nnz, nz_s, nz_e, col, val, s_val, s_col, &s_mbar, wait);
    const I* const colv = s_col + ts.head_c;
    const T* const valv = s_val + ts.head_v;
    int* const s_row_end = reinterpret_cast<int*>(s_col + ts.span_c);  // nrows + 1 ints; nrows + nnz_tile <= TILE
    // s_y[i]: row row_s + i, i in [0, nrows]; with the bulk push, placed for 16-byte aligned copies
    T* const s_y = (PUSH && peers.bulk) ? s_val + ((ts.head_v + nnz_tile + 3) & ~3) + push_misalign(peers, row_s)
                                        : s_val + ts.head_v + nnz_tile;

    // Row ends in tile-local nonzero coordinates; entry nrows belongs to the row left open.
    for (int i = tid; i <= nrows; i += THREADS) {
        const int r = row_s + i;
        const int e = (r < m) ? (int)__ldg(row_ptr + r + 1) - base : nz_e;
        s_row_end[i] = min(e, nz_e) - nz_s;
    }
    if (!stage_finish(tid, ts.copies, &s_mbar, &s_failed, status, wait)) {
        if (tid == 0) carry_row[t] = m;  // a tile that was given up leaves no carry for the fix-up
        tile_count_off<CREW>(crew, t, tid);  // (the crew must not wait for it; the failure is already reported)
        return;
    }

    // Where this thread's segment starts: diagonal d0 of the merge of row ends and nonzeros
    // (a row end equal to a nonzero index comes first, as in the tile partition).
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
    int r = lo;              // tile-local row the segment starts in
    const int k0 = d0 - lo;  // tile-local nonzero it starts at
    s_k0[tid] = k0;
    if (tid == 0) s_y[nrows] = T(0);  // the open row only ever receives carries
    __syncthreads();
    const int k1 = (tid + 1 < THREADS) ? s_k0[tid + 1] : nnz_tile;
    const int cnt = k1 - k0;      // nonzeros of this thread, 0 ... WALK
    const int r1 = d1 - k1;       // row its segment ends in (that row stays open)

    // All gathers of the thread are in flight before the first product is formed.
    const T* const xb = x - base;
    T p[WALK];
#pragma unroll
    for (int j = 0; j < WALK; ++j) {
        p[j] = T(0);
        if (j < cnt) p[j] = ldg(xb + colv[k0 + j]);
    }
#pragma unroll
    for (int j = 0; j < WALK; ++j)
        if (j < cnt) p[j] = valv[k0 + j] * p[j];

    int end = s_row_end[r];
    T sum = T(0);
#pragma unroll
    for (int j = 0; j < WALK; ++j) {
        if (j < cnt) {
            while (k0 + j >= end) {  // rows that end before this nonzero (empty rows included)
                s_y[r] = sum;
                sum = T(0);
                ++r;
                end = s_row_end[r];
            }
            sum += p[j];
        }
    }
    while (r < r1) {  // row ends behind the thread's last nonzero
        s_y[r] = sum;
        sum = T(0);
        ++r;
    }

    // Segmented reduction of the per-thread carries (key = r, value = sum): the carry of a thread
    // belongs to the row that is open at its end.
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const T up = shfl_up(sum, d);
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

    const T alpha = alpha_arg.get();
    const T beta = beta_arg.get();
    for (int i = tid; i < nrows; i += THREADS) {
        T v = alpha * s_y[i];
        if (beta != T(0)) v = mad(beta, y[row_s + i], v);
        y[row_s + i] = v;
        if constexpr (PUSH) s_y[i] = v;  // only this thread touches s_y[i] here
    }
    if constexpr (PUSH) {
        const T open_sum = s_y[nrows];
        if (peers.bulk) {
            push_tile_rows_bulk<T, THREADS>(peers, s_y, row_s, nrows, tid);
        } else {
            __syncthreads();
            push_tile_rows<T, THREADS>(peers, s_y, row_s, nrows, tid);
        }
        if (tid == 0) {
            carry_row[t] = row_s + nrows;
            carry_val[t] = open_sum;
        }
        return;
    }
    if (tid == 0) {
        carry_row[t] = row_s + nrows;
        carry_val[t] = s_y[nrows];
    }
    tile_count_off<CREW>(crew, t, tid);
}

// Copies local rows [r0, r1) of y to the same global rows of every peer's y with 128-bit stores
// aligned on the destination (NVLink carries large aligned writes near its peak; scattered 8-byte
// stores reach about half of it). Runs on a side stream while later tiles are still computing.
template <typename T>
__global__ void __launch_bounds__(512) push_rows_kernel(PeerList<T> peers, const T* __restrict__ y, long long r0,
                                                        long long r1) {
    constexpr int VW = 16 / (int)sizeof(T);
    constexpr int UNROLL = 4;
    const int p = blockIdx.y;  // one grid row of CTAs per destination: all peers are written concurrently
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    T* const dst = peer_ptr(peers, p) + peers.row_offset;
    const long long mis = (long long)((reinterpret_cast<uintptr_t>(dst + r0) / sizeof(T)) & (VW - 1));
    long long v0 = r0 + ((VW - mis) & (VW - 1));  // first row whose destination is 16-byte aligned
    if (v0 > r1) v0 = r1;
    const long long nvec = (r1 - v0) / VW;
    for (long long c = tid; c < nvec; c += nthreads * UNROLL) {
        T v[UNROLL][VW];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const long long cc = c + u * nthreads;
            if (cc < nvec) {
#pragma unroll
                for (int e = 0; e < VW; ++e) v[u][e] = y[v0 + cc * VW + e];
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const long long cc = c + u * nthreads;
            if (cc < nvec) store_vec16(dst + v0 + cc * VW, v[u]);
        }
    }
    const long long tail0 = v0 + nvec * VW;  // fewer than VW rows before v0 and after tail0
    if (tid < VW && r0 + tid < v0) dst[r0 + tid] = y[r0 + tid];
    if (tid >= 32 && tid < 32 + VW && tail0 + (tid - 32) < r1) dst[tail0 + (tid - 32)] = y[tail0 + (tid - 32)];
}

// Adds the carries of rows that cross tile boundaries. The first tile of each run of equal
// carry rows sums the run in tile order, so the result does not depend on scheduling.
template <typename T, bool PUSH>
__global__ void spmv_carry_fixup_kernel(int m, long long num_tiles, const int* __restrict__ carry_row,
                                        const T* __restrict__ carry_val, T* __restrict__ y, ScalarArg<T> alpha_arg,
                                        PeerList<T> peers) {
    long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= num_tiles) return;
    const int r = carry_row[t];
    if (r < 0 || r >= m) return;
    if (t > 0 && carry_row[t - 1] == r) return;
    T sum = carry_val[t];
    for (long long u = t + 1; u < num_tiles && carry_row[u] == r; ++u) sum += carry_val[u];
    const T v = mad(alpha_arg.get(), sum, y[r]);
    y[r] = v;
    if constexpr (PUSH) push_to_peers(peers, r, v);
}

// The same correction for the tiles [t0, t1) only, looking backwards: tile t finishes its first
// row if at least one row ends in it, and then adds the carries that earlier tiles left for that
// row, summed in tile order exactly as above (so both kernels produce the same bits). It needs
// nothing from later tiles, so it can run right after a sub-range of the tiles has been computed.
template <typename T>
__global__ void spmv_carry_fixup_range_kernel(long long t0, long long t1, const int2* __restrict__ tile_starts,
                                              const int* __restrict__ carry_row, const T* __restrict__ carry_val,
                                              T* __restrict__ y, ScalarArg<T> alpha_arg) {
    const long long t = t0 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= t1 || t == 0) return;
    const int r = tile_starts[t].x;
    if (tile_starts[t + 1].x <= r) return;  // no row ends in this tile
    long long u = t - 1;                    // carry_row[t - 1] == r by construction
    while (u > 0 && carry_row[u - 1] == r) --u;
    T sum = carry_val[u];
    for (++u; u < t; ++u) sum += carry_val[u];
    y[r] = mad(alpha_arg.get(), sum, y[r]);
}

// ---------------------------------------------------------------------------------------
// K2: row-group SpMV. G lanes share a row (G chosen from the mean row length), lane-strided
// loads, xor-shuffle reduction. Needs no analysis and no work buffer: the kernel behind the
// legacy csrmv calls, which have neither.
// ---------------------------------------------------------------------------------------
template <typename T, int G, typename I>
__global__ void __launch_bounds__(kThreads)
    spmv_rowgroup_kernel(int m, int base, const I* __restrict__ row_ptr, const I* __restrict__ col,
                         const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y,
                         ScalarArg<T> alpha_arg, ScalarArg<T> beta_arg) {
    const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) / G;
    const int lane = threadIdx.x & (G - 1);
    const bool active = gid < m;
    T sum = T(0);
    if (active) {
        const int j0 = (int)__ldg(row_ptr + gid) - base, j1 = (int)__ldg(row_ptr + gid + 1) - base;
        const T* xb = x - base;
        for (int j = j0 + lane; j < j1; j += G) sum = mad(ldcs(val + j), ldg(xb + __ldcs(col + j)), sum);
    }
#pragma unroll
    for (int d = G >> 1; d > 0; d >>= 1) sum += shfl_xor(sum, d, G);
    if (active && lane == 0) {
        const T alpha = alpha_arg.get(), beta = beta_arg.get();
        T v = alpha * sum;
        if (beta != T(0)) v = mad(beta, y[gid], v);
        y[gid] = v;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static SpmvWorkspace spmv_layout(int64_t m, int64_t nnz, size_t value_size, int items_per_tile) {
    SpmvWorkspace ws;
    ws.items_per_tile = items_per_tile;
    const int64_t items = m + nnz;
    ws.num_tiles = (items + ws.items_per_tile - 1) / ws.items_per_tile;
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    ws.off_carry_row = up(size_t(ws.num_tiles + 1) * 8);
    ws.off_carry_val = ws.off_carry_row + up(size_t(ws.num_tiles) * 4);
    ws.off_status = ws.off_carry_val + up(size_t(ws.num_tiles) * value_size);
    ws.off_done = ws.off_status + 256;
    ws.bytes = ws.off_done + up(size_t(ws.num_tiles / kCrewTilesPerChunk + 1) * 4);
    return ws;
}

SpmvWorkspace spmv_workspace(int64_t m, int64_t nnz, size_t value_size, int tile_kind, size_t index_size) {
    const int small = tile_items(value_size, true);
    const int large = wide_index_one_size(value_size, index_size) ? small : tile_items(value_size, false);
    SpmvWorkspace ws = spmv_layout(m, nnz, value_size, (tile_kind & kTileSmall) ? small : large);
    ws.walk = (tile_kind & kTileWalk) != 0;
    ws.bytes = spmv_layout(m, nnz, value_size, small).bytes;
    return ws;
}

template <typename I>
cudaError_t spmv_locality_probe(cudaStream_t s, int64_t m, int64_t nnz, const I* row_ptr, const I* col, int* device_count,
                                int* host_count) {
    locality_probe_kernel<I><<<1, 1024, 0, s>>>(m, nnz, row_ptr, col, device_count);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_count, device_count, 2 * sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e;
}

cudaError_t gather_probe(cudaStream_t s, const int32_t* idx, int64_t count, const void* table, int elem_bytes, void* out,
                         int blocks) {
    if (elem_bytes == 8)
        gather_probe_kernel<double><<<blocks, 256, 0, s>>>(idx, count, static_cast<const double*>(table),
                                                           static_cast<double*>(out));
    else
        gather_probe_kernel<float><<<blocks, 256, 0, s>>>(idx, count, static_cast<const float*>(table),
                                                          static_cast<float*>(out));
    return cudaGetLastError();
}

template <typename I>
cudaError_t spmv_analysis(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const SpmvWorkspace& ws,
                          void* buf) {
    const long long n = ws.num_tiles + 1;
    const int threads = 128;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    merge_path_partition_kernel<I><<<blocks, threads, 0, s>>>(
        (int)m, (int)nnz, base, row_ptr, ws.items_per_tile, ws.num_tiles, reinterpret_cast<int2*>(buf),
        reinterpret_cast<int*>(static_cast<char*>(buf) + ws.off_status));
    return cudaGetLastError();
}

// Extra dynamic shared memory per CTA (bytes), read once from MCSPARSE_B200_SPMV_PAD_SMEM: lowers
// the number of resident CTAs per SM for tuning experiments. 0 (the default) in normal use.
static size_t tuning_pad_smem() {
    static const size_t pad = [] {
        const char* v = std::getenv("MCSPARSE_B200_SPMV_PAD_SMEM");
        return v ? (size_t)std::strtoul(v, nullptr, 10) : (size_t)0;
    }();
    return pad;
}

// One launch of the tile kernel over tiles [tile0, tile0 + count), for the tile size of `ws`.
template <typename T, bool PUSH, typename I, bool CREW = false>
static cudaError_t launch_tiles(cudaStream_t s, int64_t tile0, int64_t count, int64_t m, int64_t nnz, int base,
                                const I* row_ptr, const I* col, const T* val, const T* x, T* y,
                                ScalarArg<T> alpha, ScalarArg<T> beta, const SpmvWorkspace& ws, void* buf,
                                const PeerList<T>& peers, const WaitCfg& wait, const CrewCfg& crew = CrewCfg()) {
    char* base_ptr = static_cast<char*>(buf);
    const int2* starts = reinterpret_cast<const int2*>(base_ptr);
    int* carry_row = reinterpret_cast<int*>(base_ptr + ws.off_carry_row);
    T* carry_val = reinterpret_cast<T*>(base_ptr + ws.off_carry_val);
    int* status = reinterpret_cast<int*>(base_ptr + ws.off_status);
    constexpr int kL = TileCfg<T, I>::kLarge, kS = TileCfg<T, I>::kSmall;
    const bool large = ws.items_per_tile == kThreads * kL;
    const unsigned grid = (unsigned)(count + (CREW ? crew.pushers : 0));
    const size_t pad = tuning_pad_smem();
#define MCSP_LAUNCH_TILES(KERNEL, IPT)                                                                                   \
    KERNEL<T, kThreads, IPT, PUSH, I, CREW><<<grid, kThreads, pad, s>>>((int)m, (int)nnz, base, row_ptr, col, val, x, y, \
                                                                        alpha, beta, starts, carry_row, carry_val,       \
                                                                        status, peers, (int)tile0, wait, crew)
    if (ws.walk) {
        if (large)
            MCSP_LAUNCH_TILES(spmv_walk_kernel, kL);
        else
            MCSP_LAUNCH_TILES(spmv_walk_kernel, kS);
    } else {
        if (large)
            MCSP_LAUNCH_TILES(spmv_tile_kernel, kL);
        else
            MCSP_LAUNCH_TILES(spmv_tile_kernel, kS);
    }
#undef MCSP_LAUNCH_TILES
    return cudaGetLastError();
}

// Thread blocks of the push crew of a sharded tile launch: MCSPARSE_B200_PUSH_CREW, default 96 (two thirds of the SMs
// lend one of their eight block slots; each block keeps up to four pieces of 2-4 KB in flight).
static int push_crew_blocks() {
    const char* e = std::getenv("MCSPARSE_B200_PUSH_CREW");
    const int v = e ? std::atoi(e) : 96;
    return v < 1 ? 1 : (v > 592 ? 592 : v);
}

template <typename T, typename I>
cudaError_t spmv_tiled(cudaStream_t s, int64_t m, int64_t nnz, int base, const I* row_ptr, const I* col, const T* val,
                       const T* x, T* y, ScalarArg<T> alpha, ScalarArg<T> beta, const SpmvWorkspace& ws, void* buf,
                       const PeerList<T>& peers, const WaitCfg& wait) {
    if (ws.num_tiles == 0) return cudaSuccess;
    char* base_ptr = static_cast<char*>(buf);
    int* carry_row = reinterpret_cast<int*>(base_ptr + ws.off_carry_row);
    T* carry_val = reinterpret_cast<T*>(base_ptr + ws.off_carry_val);
    const unsigned fix_grid = (unsigned)((ws.num_tiles + 255) / 256);
    if constexpr (std::is_floating_point<T>::value && sizeof(I) == 4) {
        if (peers.count > 0 && peers.crew && !peers.multicast) {
            // the tiles compute as on one GPU; a crew of thread blocks in the same launch moves the finished rows
            CrewCfg crew;
            crew.pushers = push_crew_blocks();
            crew.tiles_per_chunk = kCrewTilesPerChunk;
            crew.num_chunks = (int)((ws.num_tiles + kCrewTilesPerChunk - 1) / kCrewTilesPerChunk);
            crew.done = reinterpret_cast<int*>(base_ptr + ws.off_done);
            cudaError_t e = cudaMemsetAsync(crew.done, 0, size_t(crew.num_chunks) * 4, s);
            if (e != cudaSuccess) return e;
            // (no fix-up kernel: the crew adds the carries of a chunk's rows before it copies them)
            return launch_tiles<T, false, I, true>(s, 0, ws.num_tiles, m, nnz, base, row_ptr, col, val, x, y, alpha, beta,
                                                   ws, buf, peers, wait, crew);
        }
    }
    if constexpr (std::is_floating_point<T>::value) {  // the row push exists for the real types only
        if (peers.count > 0) {
            cudaError_t e = launch_tiles<T, true, I>(s, 0, ws.num_tiles, m, nnz, base, row_ptr, col, val, x, y, alpha,
                                                     beta, ws, buf, peers, wait);
            if (e != cudaSuccess) return e;
            spmv_carry_fixup_kernel<T, true><<<fix_grid, 256, 0, s>>>((int)m, ws.num_tiles, carry_row, carry_val, y,
                                                                      alpha, peers);
            return cudaGetLastError();
        }
    } else if (peers.count > 0) {
        return cudaErrorInvalidValue;
    }
    cudaError_t e = launch_tiles<T, false, I>(s, 0, ws.num_tiles, m, nnz, base, row_ptr, col, val, x, y, alpha, beta, ws,
                                              buf, peers, wait);
    if (e != cudaSuccess) return e;
    spmv_carry_fixup_kernel<T, false><<<fix_grid, 256, 0, s>>>((int)m, ws.num_tiles, carry_row, carry_val, y, alpha,
                                                               peers);
    return cudaGetLastError();
}

// CTAs (of 512 threads, over all peers) of one row-copy kernel: MCSPARSE_B200_PUSH_CTAS, default 112.
// Enough to keep NVLink busy, few enough to leave most SM slots to the tile kernel running beside it.
static long long push_copy_ctas() {
    const char* e = std::getenv("MCSPARSE_B200_PUSH_CTAS");
    const long long v = e ? std::atoll(e) : 112;
    return v < 1 ? 1 : (v > 1184 ? 1184 : v);
}

// MCSPARSE_B200_PUSH_ENGINE=sm selects the copy kernel; the default is the copy engines.
static bool push_with_copy_engines() {
    const char* e = std::getenv("MCSPARSE_B200_PUSH_ENGINE");
    return !(e && e[0] == 's');
}

cudaError_t spmv_read_tile_rows(cudaStream_t s, const void* buf, int count, const int64_t* tiles, int64_t* rows) {
    const int2* starts = static_cast<const int2*>(buf);
    int2 v;
    for (int c = 0; c < count; ++c) {
        cudaError_t e = cudaMemcpyAsync(&v, starts + tiles[c], sizeof v, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return e;
        rows[c] = v.x;
    }
    return cudaSuccess;
}

template <typename T>
cudaError_t spmv_tiled_pipelined(cudaStream_t s, cudaStream_t side, cudaEvent_t* events, const PushStreams& ps,
                                 int chunks, const int64_t* chunk_tiles, const int64_t* chunk_rows, int64_t m, int64_t nnz,
                                 int base, const int32_t* row_ptr, const int32_t* col, const T* val, const T* x, T* y,
                                 ScalarArg<T> alpha, ScalarArg<T> beta, const SpmvWorkspace& ws, void* buf,
                                 const PeerList<T>& peers, const WaitCfg& wait) {
    if (ws.num_tiles == 0) return cudaSuccess;
    char* base_ptr = static_cast<char*>(buf);
    const int2* starts = reinterpret_cast<const int2*>(base_ptr);
    int* carry_row = reinterpret_cast<int*>(base_ptr + ws.off_carry_row);
    T* carry_val = reinterpret_cast<T*>(base_ptr + ws.off_carry_val);
    const PeerList<T> none;
    cudaError_t e = cudaSuccess;
    for (int c = 0; c < chunks && e == cudaSuccess; ++c) {
        const int64_t t0 = chunk_tiles[c], t1 = chunk_tiles[c + 1];
        if (t1 > t0)
            e = launch_tiles<T, false, int32_t>(s, t0, t1 - t0, m, nnz, base, row_ptr, col, val, x, y, alpha, beta, ws, buf,
                                                none, wait);
        if (e == cudaSuccess) e = cudaEventRecord(events[c], s);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(side, events[c], 0);
        if (e == cudaSuccess && t1 > t0) {
            // On the side stream, so that the tile kernels run back to back on the main one: rows that
            // end in this chunk get their carries, and the copy below then sends final values.
            spmv_carry_fixup_range_kernel<T><<<(unsigned)((t1 - t0 + 255) / 256), 256, 0, side>>>(
                t0, t1, starts, carry_row, carry_val, y, alpha);
            e = cudaGetLastError();
        }
        const int64_t r0 = chunk_rows[c], r1 = chunk_rows[c + 1];
        if (e == cudaSuccess && r1 > r0) {
            if (push_with_copy_engines()) {
                // one peer-to-peer copy per destination, each on that destination's own stream: the
                // copy engines drive NVLink at its full rate, take no SM away from the tile kernel
                // running beside them, and copies to different GPUs proceed at the same time
                e = cudaEventRecord(ps.fix_events[c], side);
                for (int p = 0; p < peers.count && e == cudaSuccess; ++p) {
                    e = cudaStreamWaitEvent(ps.peer_streams[p], ps.fix_events[c], 0);
                    if (e == cudaSuccess)
                        e = cudaMemcpyAsync(peers.y[p] + peers.row_offset + r0, y + r0, size_t(r1 - r0) * sizeof(T),
                                            cudaMemcpyDeviceToDevice, ps.peer_streams[p]);
                }
            } else {
                const long long vecs = (r1 - r0) * (long long)sizeof(T) / 16 + 1;
                const unsigned gx = (unsigned)std::max<long long>(
                    1, std::min<long long>((vecs + 2047) / 2048, push_copy_ctas() / peers.count));
                push_rows_kernel<T><<<dim3(gx, (unsigned)peers.count), 512, 0, side>>>(peers, y, r0, r1);
                e = cudaGetLastError();
            }
        }
    }
    // Whatever the caller enqueues next on its stream comes after the last fix-up and the last row copy.
    if (e == cudaSuccess) e = cudaEventRecord(events[chunks], side);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, events[chunks], 0);
    if (push_with_copy_engines()) {
        for (int p = 0; p < peers.count && e == cudaSuccess; ++p) {
            e = cudaEventRecord(ps.peer_events[p], ps.peer_streams[p]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s, ps.peer_events[p], 0);
        }
    }
    return e;
}

template <typename T, int G>
static cudaError_t launch_rowgroup(cudaStream_t s, int64_t m, int base, const int32_t* row_ptr, const int32_t* col,
                                   const T* val, const T* x, T* y, ScalarArg<T> alpha, ScalarArg<T> beta) {
    const long long threads_total = m * G;
    const unsigned grid = (unsigned)((threads_total + kThreads - 1) / kThreads);
    spmv_rowgroup_kernel<T, G, int32_t><<<grid, kThreads, 0, s>>>((int)m, base, row_ptr, col, val, x, y, alpha, beta);
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

#define INSTANTIATE_TI(T, I)                                                                                  \
    template cudaError_t spmv_tiled<T, I>(cudaStream_t, int64_t, int64_t, int, const I*, const I*, const T*,    \
                                          const T*, T*, ScalarArg<T>, ScalarArg<T>, const SpmvWorkspace&,      \
                                          void*, const PeerList<T>&, const WaitCfg&);
#define INSTANTIATE(T)                                                                                         \
    INSTANTIATE_TI(T, int32_t)                                                                                 \
    INSTANTIATE_TI(T, int64_t)                                                                                 \
    template cudaError_t spmv_rowgroup<T>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*, \
                                          const T*, const T*, T*, ScalarArg<T>, ScalarArg<T>);                 \
    template cudaError_t spmv_tiled_pipelined<T>(cudaStream_t, cudaStream_t, cudaEvent_t*, const PushStreams&, \
                                                 int, const int64_t*,                                          \
                                                 const int64_t*, int64_t, int64_t, int, const int32_t*,        \
                                                 const int32_t*, const T*, const T*, T*, ScalarArg<T>,         \
                                                 ScalarArg<T>, const SpmvWorkspace&, void*, const PeerList<T>&, \
                                                 const WaitCfg&);
INSTANTIATE(float)
INSTANTIATE(double)
INSTANTIATE_TI(cfloat, int32_t)
INSTANTIATE_TI(cdouble, int32_t)
INSTANTIATE_TI(cfloat, int64_t)
INSTANTIATE_TI(cdouble, int64_t)
template cudaError_t spmv_rowgroup<cfloat>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*,
                                           const cfloat*, const cfloat*, cfloat*, ScalarArg<cfloat>, ScalarArg<cfloat>);
template cudaError_t spmv_rowgroup<cdouble>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const int32_t*,
                                            const cdouble*, const cdouble*, cdouble*, ScalarArg<cdouble>,
                                            ScalarArg<cdouble>);
template cudaError_t spmv_analysis<int32_t>(cudaStream_t, int64_t, int64_t, int, const int32_t*, const SpmvWorkspace&,
                                            void*);
template cudaError_t spmv_analysis<int64_t>(cudaStream_t, int64_t, int64_t, int, const int64_t*, const SpmvWorkspace&,
                                            void*);
template cudaError_t spmv_locality_probe<int32_t>(cudaStream_t, int64_t, int64_t, const int32_t*, const int32_t*, int*,
                                                  int*);
template cudaError_t spmv_locality_probe<int64_t>(cudaStream_t, int64_t, int64_t, const int64_t*, const int64_t*, int*,
                                                  int*);
#undef INSTANTIATE
#undef INSTANTIATE_TI

}  // namespace mcsp_b200
