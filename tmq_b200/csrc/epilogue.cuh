// Warp-level epilogue shared by the tcgen05 GEMM and convolution kernels: one tcgen05.ld chunk (32 accumulator rows =
// output channels, one per lane, x 16 accumulator columns = output rows / pixels) is scaled, transposed through a
// small shared-memory stage and written as 16-byte bf16 vectors (8 channels of one output row per lane), with an
// optional residual read the same way and an optional ReLU.  Against one 2-byte store per element this cuts the
// global instructions eight-fold.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace tmq {

// Further destinations of the same output block: buffers of the same shape and row stride in OTHER GPUs' memory (peer
// mappings), written with plain stores over NVLink next to the local store, so that an all-gather of column blocks
// needs no separate pass: the block is in every rank's buffer when the kernel completes.
constexpr int kMaxPeers = 7;
struct PeerList {
    __nv_bfloat16 *y[kMaxPeers];
    int n;
};

// stage: this warp's private 16 x 32 fp32 area (2 KB, 16-byte aligned).  n_base: first channel of the warp's 32.
__device__ __forceinline__ void epilogue_chunk_bf16(const uint32_t (&v)[16], float sc, float bi, float *stage,
                                                    __nv_bfloat16 *Y, const __nv_bfloat16 *residual, long long m_base,
                                                    long long M, long long ldy, long long n_base, long long N, int relu,
                                                    int lane, const PeerList *peers = nullptr) {
#pragma unroll
    for (int j = 0; j < 16; j++) stage[j * 32 + lane] = fmaf(__uint_as_float(v[j]), sc, bi);
    __syncwarp();
    const int cg = (lane & 3) * 8;  // channel offset of this lane's 8-channel vector
    const long long n = n_base + cg;
    // 16-byte vectors only when every row's vector is 16-byte aligned: row stride and both base pointers (a caller may
    // hand in a column block of a wider output, Y = base + n0 with any n0); anything else takes the scalar stores
    bool vec_ok = ((ldy & 7) == 0) && (n + 8 <= N) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(residual) & 15) == 0);
    const int npeers = peers ? peers->n : 0;
    for (int q = 0; q < npeers; q++) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(peers->y[q]) & 15) == 0);
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int p = it * 8 + (lane >> 2);
        const long long m = m_base + p;
        if (m < M && n < N) {
            const float4 lo = *reinterpret_cast<const float4 *>(stage + p * 32 + cg);
            const float4 hi = *reinterpret_cast<const float4 *>(stage + p * 32 + cg + 4);
            float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            if (vec_ok) {
                if (residual) {
                    const uint4 rv = *reinterpret_cast<const uint4 *>(residual + m * ldy + n);
                    const __nv_bfloat16 *rb = reinterpret_cast<const __nv_bfloat16 *>(&rv);
#pragma unroll
                    for (int e = 0; e < 8; e++) f[e] += __bfloat162float(rb[e]);
                }
                __align__(16) __nv_bfloat16 o[8];
#pragma unroll
                for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(relu ? fmaxf(f[e], 0.0f) : f[e]);
                const uint4 ov = *reinterpret_cast<const uint4 *>(o);
                *reinterpret_cast<uint4 *>(Y + m * ldy + n) = ov;
                for (int q = 0; q < npeers; q++) *reinterpret_cast<uint4 *>(peers->y[q] + m * ldy + n) = ov;
            } else {
                for (int e = 0; e < 8 && n + e < N; e++) {
                    float x = f[e];
                    if (residual) x += __bfloat162float(residual[m * ldy + n + e]);
                    const __nv_bfloat16 ob = __float2bfloat16_rn(relu ? fmaxf(x, 0.0f) : x);
                    Y[m * ldy + n + e] = ob;
                    for (int q = 0; q < npeers; q++) peers->y[q][m * ldy + n + e] = ob;
                }
            }
        }
    }
    __syncwarp();
}

}  // namespace tmq
