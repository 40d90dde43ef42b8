// Bit-exact 2-bit packing of ternary weights and its inverse.
//
// Contract (tmq/tmq_native.cpp:152-171, :185-208, transpose at :303-319): W[N][K] -> P[K][ceil(N/16)];
// word q of row k carries W[16q+i][k] for i = 0..15, element i in bits [31-2i : 30-2i]; fp32 inputs are rounded
// half away from zero and clamped to [-1, 1]; codes 0 -> 00, +1 -> 01, -1 -> 10; tail elements are zero.
//
// Both kernels are transposes (the packed matrix is K-major, the weight N-major), so each block stages a
// 32 x 32 tile of words in shared memory: global reads run along k, global writes along q (or the reverse),
// both coalesced.  Integer/byte work, HBM-bound: 4 B read per element, 0.25 B written.
#include <initializer_list>

#include "common.cuh"

namespace tmq {

// float -> {-1,0,+1} exactly as `(int)roundf(v)` + clamp behaves in the reference's x86-64 build, where
// out-of-range and non-finite values convert to INT_MIN and therefore clamp to -1.
__device__ __forceinline__ int ternary_of(float v) {
    const float r = roundf(v);
    if (!(r >= -2147483648.0f && r < 2147483648.0f)) return -1;
    return r > 1.0f ? 1 : (r < -1.0f ? -1 : (int)r);
}
__device__ __forceinline__ int ternary_of(int v) { return v > 1 ? 1 : (v < -1 ? -1 : v); }
__device__ __forceinline__ int ternary_of(signed char v) { return ternary_of((int)v); }

__device__ __forceinline__ unsigned code_of(int t) { return t == 0 ? 0u : (t == 1 ? 1u : 2u); }

template <typename T>
__global__ void __launch_bounds__(256) pack2b_kernel(const T *__restrict__ W, uint32_t *__restrict__ P, int64_t N,
                                                      int64_t K, int64_t Q) {
    __shared__ uint32_t tile[32][33];
    const int lane = threadIdx.x, wy = threadIdx.y;  // 32 x 8
    const int64_t k0 = (int64_t)blockIdx.x * 32, q0 = (int64_t)blockIdx.y * 32;
    const int64_t k = k0 + lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int ql = wy + 8 * j;
        const int64_t q = q0 + ql;
        uint32_t word = 0;
        if (k < K && q < Q) {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int64_t n = q * 16 + i;
                const int t = (n < N) ? ternary_of(W[n * K + k]) : 0;
                word = (word << 2) | code_of(t);
            }
        }
        tile[ql][lane] = word;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int kl = wy + 8 * j;
        const int64_t kk = k0 + kl, q = q0 + lane;
        if (kk < K && q < Q) P[kk * Q + q] = tile[lane][kl];
    }
}

__global__ void __launch_bounds__(256) unpack2b_kernel(const uint32_t *__restrict__ P, float *__restrict__ W, int64_t N,
                                                        int64_t K, int64_t Q) {
    __shared__ uint32_t tile[32][33];
    const int lane = threadIdx.x, wy = threadIdx.y;
    const int64_t k0 = (int64_t)blockIdx.x * 32, q0 = (int64_t)blockIdx.y * 32;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int kl = wy + 8 * j;
        const int64_t kk = k0 + kl, q = q0 + lane;
        tile[kl][lane] = (kk < K && q < Q) ? P[kk * Q + q] : 0u;
    }
    __syncthreads();
    const int64_t k = k0 + lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int ql = wy + 8 * j;
        const int64_t q = q0 + ql;
        if (k < K && q < Q) {
            const uint32_t word = tile[lane][ql];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int64_t n = q * 16 + i;
                const unsigned c = (word >> (2 * (15 - i))) & 3u;
                if (n < N) W[n * K + k] = (c == 1u) ? 1.0f : ((c == 2u) ? -1.0f : 0.0f);
            }
        }
    }
}

template <typename T>
static int launch_pack(const T *W, uint32_t *P, int64_t N, int64_t K, cudaStream_t st) {
    if (N == 0 || K == 0) return TMQ_OK;
    if (!W || !P || N < 0 || K < 0) return TMQ_ERR_ARG;
    const int64_t Q = (N + 15) / 16;
    const int64_t gx = (K + 31) / 32, gy = (Q + 31) / 32;
    if (gx > 0x7FFFFFFF || gy > 65535) return TMQ_ERR_UNSUPPORTED;
    pack2b_kernel<T><<<dim3((unsigned)gx, (unsigned)gy), dim3(32, 8), 0, st>>>(W, P, N, K, Q);
    return launch_status();
}

}  // namespace tmq

using namespace tmq;

extern "C" int tmq_pack2b_f32(const float *W, uint32_t *P, int64_t N, int64_t K, void *stream) {
    return launch_pack<float>(W, P, N, K, (cudaStream_t)stream);
}
extern "C" int tmq_pack2b_i32(const int32_t *W, uint32_t *P, int64_t N, int64_t K, void *stream) {
    return launch_pack<int>(W, P, N, K, (cudaStream_t)stream);
}
extern "C" int tmq_pack2b_i8(const int8_t *W, uint32_t *P, int64_t N, int64_t K, void *stream) {
    return launch_pack<signed char>(reinterpret_cast<const signed char *>(W), P, N, K, (cudaStream_t)stream);
}
extern "C" int tmq_unpack2b_f32(const uint32_t *P, float *W, int64_t N, int64_t K, void *stream) {
    if (N == 0 || K == 0) return TMQ_OK;
    if (!P || !W || N < 0 || K < 0) return TMQ_ERR_ARG;
    const int64_t Q = (N + 15) / 16;
    const int64_t gx = (K + 31) / 32, gy = (Q + 31) / 32;
    if (gx > 0x7FFFFFFF || gy > 65535) return TMQ_ERR_UNSUPPORTED;
    unpack2b_kernel<<<dim3((unsigned)gx, (unsigned)gy), dim3(32, 8), 0, (cudaStream_t)stream>>>(P, W, N, K, Q);
    return launch_status();
}
