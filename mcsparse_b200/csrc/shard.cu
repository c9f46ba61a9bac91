// Row-block sharding helpers for running one CSR matrix on several GPUs.
// The reference is single-device (mcsparse/src/common/mcsp_handle.cpp:5-8); these kernels
// have no counterpart there. Their CPU restatement is the bit-exact check.
#include "internal.h"

namespace mcsp_b200 {

namespace {

// bounds[g] = first row r with row_ptr[r] - base >= floor(g * nnz / G); bounds[0] = 0, bounds[G] = m.
__global__ void shard_row_bounds_kernel(long long m, long long nnz, int base, const int* __restrict__ row_ptr,
                                        int num_shards, long long* __restrict__ bounds) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > num_shards) return;
    if (g == 0) {
        bounds[0] = 0;
        return;
    }
    if (g == num_shards) {
        bounds[g] = m;
        return;
    }
    // g * nnz < 2^31 * 2^31: fits in 64 bits.
    const long long target = (long long)(((unsigned long long)g * (unsigned long long)nnz) / (unsigned)num_shards);
    long long lo = 0, hi = m;
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)__ldg(row_ptr + mid) - base < target)
            lo = mid + 1;
        else
            hi = mid;
    }
    bounds[g] = lo;
}

__global__ void shard_local_row_offsets_kernel(const int* __restrict__ row_ptr, long long first_row,
                                               long long num_rows, int base, int* __restrict__ local) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i > num_rows) return;
    local[i] = __ldg(row_ptr + first_row + i) - __ldg(row_ptr + first_row) + base;
}

// CSR row offsets of a COO matrix sorted by row: offsets[r] = base + number of entries whose row is
// smaller than r, found by a lower bound over the sorted row indices (one thread per offset).
// Same result as the reference's scatter formulation (mcsparse/src/kernels/conversion/coo2csr_device.hpp:8-24).
__global__ void coo_row_offsets_kernel(long long m, long long nnz, int base, const int* __restrict__ coo_rows,
                                       int* __restrict__ offsets) {
    const long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (r > m) return;
    long long lo = 0, hi = nnz;
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)__ldg(coo_rows + mid) - base < r)
            lo = mid + 1;
        else
            hi = mid;
    }
    offsets[r] = (int)lo + base;
}

// Orders the GPUs of a row-sharded step without a collective: lane p tells peer p "my rows of step `epoch`
// are in your memory" by storing the epoch into that peer's flag slot for this rank (a release at system
// scope: the kernel runs after the kernels and copies that moved the rows, in stream order), then lane q
// waits until peer q's epoch has arrived in this GPU's own slots (acquire at system scope). The wait is
// bounded: when `limit` SM clocks pass without the flag, the lane records it in the status word (and in the
// handle's host-visible fault word) and the kernel returns. Epochs only grow; slots are never reset.
struct PeerFlags {
    int* remote[7];  // remote[p]: peer p's slot for this rank
};
__global__ void peer_signal_wait_kernel(int count, PeerFlags flags, const int* local_slots, int epoch, long long limit,
                                        int* status, int* fault_word) {
    const int p = threadIdx.x;
    if (p >= count) return;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.remote[p]), "r"(epoch) : "memory");
    const long long t0 = clock64();
    for (;;) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(local_slots + p) : "memory");
        if (seen - epoch >= 0) break;
        if (clock64() - t0 > limit) {
            atomicOr(status, 1);
            if (fault_word != nullptr) {
                *reinterpret_cast<volatile int*>(fault_word) = 1;
                __threadfence_system();
            }
            break;
        }
    }
}

}  // namespace

cudaError_t coo_row_offsets(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* coo_rows,
                            int32_t* offsets) {
    coo_row_offsets_kernel<<<(unsigned)((m + 1 + 255) / 256), 256, 0, s>>>(m, nnz, base, coo_rows, offsets);
    return cudaGetLastError();
}

cudaError_t shard_row_bounds(cudaStream_t s, int64_t m, int64_t nnz, int base, const int32_t* row_ptr,
                             int num_shards, int64_t* bounds_host) {
    long long* d = nullptr;
    cudaError_t e = cudaMalloc(&d, sizeof(long long) * (num_shards + 1));
    if (e != cudaSuccess) return e;
    shard_row_bounds_kernel<<<(num_shards + 1 + 63) / 64, 64, 0, s>>>(m, nnz, base, row_ptr, num_shards, d);
    e = cudaGetLastError();
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(bounds_host, d, sizeof(long long) * (num_shards + 1), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(d);
    return e;
}

cudaError_t shard_local_row_offsets(cudaStream_t s, const int32_t* row_ptr, int64_t first_row, int64_t num_rows,
                                    int base, int32_t* local) {
    const int threads = 256;
    shard_local_row_offsets_kernel<<<(unsigned)((num_rows + 1 + threads - 1) / threads), threads, 0, s>>>(
        row_ptr, first_row, num_rows, base, local);
    return cudaGetLastError();
}

cudaError_t peer_signal_wait(cudaStream_t s, int count, int* const* remote_slots, const int* local_slots, int epoch,
                             long long limit, int* status, int* fault_word) {
    if (count <= 0) return cudaSuccess;
    if (count > 7) return cudaErrorInvalidValue;
    PeerFlags f;
    for (int p = 0; p < 7; ++p) f.remote[p] = p < count ? remote_slots[p] : nullptr;
    peer_signal_wait_kernel<<<1, 32, 0, s>>>(count, f, local_slots, epoch, limit, status, fault_word);
    return cudaGetLastError();
}

}  // namespace mcsp_b200
