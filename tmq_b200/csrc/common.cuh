// Shared host/device helpers for the tmq_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <utility>

#include "tmq_b200.h"

namespace tmq {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// cudaError_t of the last failed runtime call made by this library on the calling thread
extern thread_local int g_last_cuda_error;

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return TMQ_ERR_LAUNCH;
    }
    return TMQ_OK;
}

inline int cuda_status(cudaError_t e) {
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        (void)cudaGetLastError();
        return TMQ_ERR_LAUNCH;
    }
    return TMQ_OK;
}

// Row-major prepacked weights: a row holds the K/16 packed words of one output channel (K rounded up to 64, zeros
// beyond K) followed by padding that places consecutive rows 32 bytes (bf16-ready words, kind 0) or 64 bytes (int8-ready
// words, kind 1) apart modulo 128.  A run of rows copied verbatim into shared memory is then read without bank
// conflicts by the warp-fragment access pattern of the skinny kernels (8-byte / 16-byte reads, 8 rows per warp), and a
// CTA's rows stay one contiguous byte range, i.e. one bulk copy.  The stride stays a multiple of 16 bytes (TMA).
inline long long prepack_valid_words(long long K) { return ((K + 63) / 64) * 4; }
inline long long prepack_row_words(long long K, int kind) {
    const long long bytes = prepack_valid_words(K) * 4;
    const long long want = kind ? 64 : 32;
    return (bytes + ((want - bytes % 128) + 128) % 128) / 4;
}

// Opt-in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device) pair, so it is set
// once per kernel on every device the library is used on; the calling thread's current device is the one that launches.
template <typename K>
inline int ensure_dynamic_smem(K kernel, int bytes, bool max_carveout = false) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, bool> done;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cuda_status(cudaGetLastError());
    const std::pair<const void *, int> key(reinterpret_cast<const void *>(kernel), dev);
    std::lock_guard<std::mutex> lock(mu);
    if (done.count(key)) return TMQ_OK;
    int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (rc == TMQ_OK && max_carveout)
        rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    if (rc == TMQ_OK) done[key] = true;
    return rc;
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Resident blocks per SM for a kernel, cached by the caller in a function-local static.
template <typename K>
inline int blocks_per_sm(K kernel, int threads, size_t smem = 0) {
    int b = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kernel, threads, smem) != cudaSuccess || b < 1) {
        (void)cudaGetLastError();
        b = 1;
    }
    return b;
}

// Deterministic two-stage reduction scratch: [0] arrival counter, [256..] one fp64 partial per block.
constexpr int kMaxPartials = 65536;
constexpr size_t kScratchHeader = 256;
constexpr size_t kScratchBytes = kScratchHeader + sizeof(double) * kMaxPartials;

#ifdef __CUDACC__
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a 256-thread block, result valid in thread 0. Fixed order -> bitwise reproducible.
__device__ __forceinline__ double block_sum_256(double v, double *smem8) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem8[warp] = v;
    __syncthreads();
    double s = 0.0;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; i++) s += smem8[i];
    }
    __syncthreads();
    return s;
}

// Publishes this block's partial; the last block to arrive folds all partials in index order into *out
// and re-arms the counter, so the scratch is zero again when the kernel ends.
__device__ __forceinline__ void grid_sum_finish(double block_total, void *scratch, double *out, double *smem8) {
    unsigned *counter = reinterpret_cast<unsigned *>(scratch);
    double *partials = reinterpret_cast<double *>(reinterpret_cast<char *>(scratch) + kScratchHeader);
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block_total;
        __threadfence();
        unsigned ticket = atomicAdd(counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        double s = 0.0;
        for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) s += __ldcg(partials + i);
        s = block_sum_256(s, smem8);
        if (threadIdx.x == 0) {
            *out = s;
            *counter = 0u;
        }
    }
}
#endif

}  // namespace tmq
