// Activation-side layout kernels around the packed inference path: everything that would otherwise be a chain of eager
// elementwise tensor operations between two tensor-core launches.
//
//   * split of fp32 activations into bf16 terms.  x = hi + mid + lo with hi = bf16(x), mid = bf16(x - hi),
//     lo = bf16(x - hi - mid) is EXACT for every finite fp32 x whose low term is not subnormal in bf16 (8 + 8 + 8
//     significant bits), so a product with a weight in {-1, 0, +1} is exact per term and the tensor core's fp32
//     accumulation reproduces an fp32 GEMM / convolution.  The three terms ride along K (GEMM: [M][3*Kp]) or along the
//     channels (convolution: NHWC [B][H][W][3*C]) against three stacked copies of the weights, SMALLEST TERM FIRST
//     (lo, mid, hi): the tensor core aligns every product to its running fp32 sum and drops the bits below it, so the
//     tiny terms are added while the sum is still tiny (measured at K = 4096: relative error 6e-5 with the large terms
//     first, fp32-GEMM level with them last).
//   * NCHW fp32 -> NHWC bf16 (one or three terms) in one pass, for convolutions fed with torch's default layout.
//   * global average pooling on NHWC bf16.
#include <cuda_bf16.h>

#include "common.cuh"

namespace tmq {

__device__ __forceinline__ void split3(float x, __nv_bfloat16 &hi, __nv_bfloat16 &mid, __nv_bfloat16 &lo) {
    hi = __float2bfloat16_rn(x);
    const float r1 = __fsub_rn(x, __bfloat162float(hi));
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(__fsub_rn(r1, __bfloat162float(mid)));
}

// X fp32 [M][K] -> out bf16 [M][terms * Kp]; term t of element (m, k) at out[m][t * Kp + k]; k in [K, Kp) is zero.
__global__ void __launch_bounds__(256) split_rows_kernel(const float *__restrict__ X, __nv_bfloat16 *__restrict__ out,
                                                          long long M, long long K, long long Kp, int terms) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * Kp) return;
    const long long m = idx / Kp, k = idx - m * Kp;
    const float x = k < K ? __ldg(X + m * K + k) : 0.0f;
    __nv_bfloat16 *o = out + m * terms * Kp + k;
    if (terms == 1) {
        o[0] = __float2bfloat16_rn(x);
    } else {
        __nv_bfloat16 hi, mid, lo;
        split3(x, hi, mid, lo);
        o[0] = lo;                 // smallest term first: see the note on the accumulation order above
        o[Kp] = mid;
        o[2 * Kp] = hi;
    }
}

// X fp32 [B][C][P] (P = H*W) -> Y bf16 [B][P][terms * C], through a 32 x 32 shared tile so that both sides are coalesced
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const float *__restrict__ X, __nv_bfloat16 *__restrict__ Y, int C,
                                                            long long P, int terms) {
    __shared__ float tile[32][33];
    const long long p0 = (long long)blockIdx.x * 32;
    const int c0 = blockIdx.y * 32, b = blockIdx.z;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    const float *src = X + ((long long)b * C) * P;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int c = c0 + ty + 8 * i;
        const long long p = p0 + tx;
        tile[ty + 8 * i][tx] = (c < C && p < P) ? __ldg(src + (long long)c * P + p) : 0.0f;
    }
    __syncthreads();
    __nv_bfloat16 *dst = Y + ((long long)b * P) * terms * C;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const long long p = p0 + ty + 8 * i;
        const int c = c0 + tx;
        if (c < C && p < P) {
            const float x = tile[tx][ty + 8 * i];
            __nv_bfloat16 *o = dst + p * terms * C + c;
            if (terms == 1) {
                o[0] = __float2bfloat16_rn(x);
            } else {
                __nv_bfloat16 hi, mid, lo;
                split3(x, hi, mid, lo);
                o[0] = lo;
                o[C] = mid;
                o[2 * C] = hi;
            }
        }
    }
}

// X bf16 [B][P][C] -> Y bf16 [B][C] = mean over P (fp32 accumulation in pixel order); one thread per (b, 2 channels)
__global__ void __launch_bounds__(128) avgpool_nhwc_kernel(const __nv_bfloat162 *__restrict__ X, __nv_bfloat162 *__restrict__ Y,
                                                            int B, int P, int C2) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C2) return;
    const int b = idx / C2, c = idx - b * C2;
    const __nv_bfloat162 *src = X + (long long)b * P * C2 + c;
    float s0 = 0.0f, s1 = 0.0f;
    for (int p = 0; p < P; p++) {
        const float2 v = __bfloat1622float2(src[(long long)p * C2]);
        s0 += v.x;
        s1 += v.y;
    }
    const float inv = 1.0f / (float)P;
    Y[idx] = __floats2bfloat162_rn(s0 * inv, s1 * inv);
}

}  // namespace tmq

using namespace tmq;

// Max pooling for TRAINING on fp32 NHWC activations (the pooling behind the stem of a ResNet under quantisation-aware
// training): the forward pass also records, per output element, which window position won (first maximum in (ky, kx)
// scan order, NaN wins: torch's rule), and the backward pass GATHERS - every input element adds the gradients of the
// windows it won - so it needs neither atomics nor a zero-fill pass and is deterministic.  Four channels per thread.
__global__ void __launch_bounds__(256) maxpool_f32_fwd_kernel(const float4 *__restrict__ X, float4 *__restrict__ Y,
                                                              char4 *__restrict__ idx, int B, int H, int W, int C4, int OH,
                                                              int OW, int k, int s, int p) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * OH * OW * C4) return;
    const int c = (int)(i % C4);
    long long r = i / C4;
    const int ox = (int)(r % OW); r /= OW;
    const int oy = (int)(r % OH);
    const int b = (int)(r / OH);
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    int w[4] = {-1, -1, -1, -1};
    for (int fy = 0; fy < k; fy++) {
        const int y = oy * s - p + fy;
        if (y < 0 || y >= H) continue;
        for (int fx = 0; fx < k; fx++) {
            const int x = ox * s - p + fx;
            if (x < 0 || x >= W) continue;
            const float4 v = X[(((long long)b * H + y) * W + x) * C4 + c];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (w[q] < 0 || e[q] > m[q] || e[q] != e[q]) {     // first element of the window, a larger one, or a NaN
                    m[q] = e[q];
                    w[q] = fy * k + fx;
                }
        }
    }
    Y[i] = make_float4(m[0], m[1], m[2], m[3]);
    idx[i] = make_char4((signed char)w[0], (signed char)w[1], (signed char)w[2], (signed char)w[3]);
}

__global__ void __launch_bounds__(256) maxpool_f32_bwd_kernel(const float4 *__restrict__ gY, const char4 *__restrict__ idx,
                                                              float4 *__restrict__ gX, int B, int H, int W, int C4, int OH,
                                                              int OW, int k, int s, int p) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * H * W * C4) return;
    const int c = (int)(i % C4);
    long long r = i / C4;
    const int x = (int)(r % W); r /= W;
    const int y = (int)(r % H);
    const int b = (int)(r / H);
    float g[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // windows that contain (y, x): oy * s - p <= y < oy * s - p + k
    int oy0 = y + p - k + 1;
    oy0 = oy0 <= 0 ? 0 : (oy0 + s - 1) / s;
    int ox0 = x + p - k + 1;
    ox0 = ox0 <= 0 ? 0 : (ox0 + s - 1) / s;
    const int oy1 = min((y + p) / s, OH - 1), ox1 = min((x + p) / s, OW - 1);
    for (int oy = oy0; oy <= oy1; oy++)
        for (int ox = ox0; ox <= ox1; ox++) {
            const int off = (y - (oy * s - p)) * k + (x - (ox * s - p));
            const long long o = (((long long)b * OH + oy) * OW + ox) * C4 + c;
            const char4 w = idx[o];
            const float4 v = gY[o];
            if (w.x == off) g[0] += v.x;
            if (w.y == off) g[1] += v.y;
            if (w.z == off) g[2] += v.z;
            if (w.w == off) g[3] += v.w;
        }
    gX[i] = make_float4(g[0], g[1], g[2], g[3]);
}

extern "C" int tmq_split_f32_bf16(const float *X, void *out, int64_t M, int64_t K, int64_t Kp, int terms, void *stream) {
    if (!X || !out || M <= 0 || K <= 0 || Kp < K || (terms != 1 && terms != 3)) return TMQ_ERR_ARG;
    if (!aligned(X, 4) || !aligned(out, 2)) return TMQ_ERR_ALIGN;
    const long long blocks = (M * Kp + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    split_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(X, reinterpret_cast<__nv_bfloat16 *>(out), M, K, Kp,
                                                                         terms);
    return launch_status();
}

extern "C" int tmq_nchw_f32_to_nhwc_bf16(const float *X, void *Y, int B, int C, int H, int W, int terms, void *stream) {
    if (!X || !Y || B <= 0 || C <= 0 || H <= 0 || W <= 0 || (terms != 1 && terms != 3)) return TMQ_ERR_ARG;
    if (!aligned(X, 4) || !aligned(Y, 2)) return TMQ_ERR_ALIGN;
    const long long P = (long long)H * W;
    const long long gx = (P + 31) / 32;
    if (gx > 0x7FFFFFFF || (C + 31) / 32 > 65535 || B > 65535) return TMQ_ERR_UNSUPPORTED;
    dim3 grid((unsigned)gx, (unsigned)((C + 31) / 32), (unsigned)B);
    nchw_to_nhwc_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(X, reinterpret_cast<__nv_bfloat16 *>(Y), C, P, terms);
    return launch_status();
}

extern "C" int tmq_avgpool_nhwc_bf16(const void *X, void *Y, int B, int P, int C, void *stream) {
    if (!X || !Y || B <= 0 || P <= 0 || C <= 0) return TMQ_ERR_ARG;
    if (C % 2 != 0) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 4) || !aligned(Y, 4)) return TMQ_ERR_ALIGN;
    const long long total = (long long)B * (C / 2);
    if (total > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    avgpool_nhwc_kernel<<<(unsigned)((total + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat162 *>(X), reinterpret_cast<__nv_bfloat162 *>(Y), B, P, C / 2);
    return launch_status();
}

static int maxpool_train_check(const void *a, const void *b, const void *c, int B, int H, int W, int C, int k, int s, int p) {
    if (!a || !b || !c) return TMQ_ERR_ARG;
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || k <= 0 || s <= 0 || p < 0) return TMQ_ERR_ARG;
    if (C % 4 != 0 || k > 11 || 2 * p > k) return TMQ_ERR_UNSUPPORTED;        // window positions fit a signed byte
    if (H + 2 * p < k || W + 2 * p < k) return TMQ_ERR_ARG;
    if (!aligned(a, 16) || !aligned(b, 16) || !aligned(c, 4)) return TMQ_ERR_ALIGN;
    return TMQ_OK;
}

extern "C" int tmq_maxpool2d_nhwc_f32_fwd(const float *X, float *Y, signed char *idx, int B, int H, int W, int C, int k, int s,
                                          int p, void *stream) {
    int rc = maxpool_train_check(X, Y, idx, B, H, W, C, k, s, p);
    if (rc != TMQ_OK) return rc;
    const int OH = (H + 2 * p - k) / s + 1, OW = (W + 2 * p - k) / s + 1;
    const long long total = (long long)B * OH * OW * (C / 4);
    if ((total + 255) / 256 > 0x7FFFFFFFll) return TMQ_ERR_UNSUPPORTED;
    maxpool_f32_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4 *>(X), reinterpret_cast<float4 *>(Y), reinterpret_cast<char4 *>(idx), B, H, W, C / 4, OH, OW,
        k, s, p);
    return launch_status();
}

extern "C" int tmq_maxpool2d_nhwc_f32_bwd(const float *gY, const signed char *idx, float *gX, int B, int H, int W, int C, int k,
                                          int s, int p, void *stream) {
    int rc = maxpool_train_check(gY, gX, idx, B, H, W, C, k, s, p);
    if (rc != TMQ_OK) return rc;
    const int OH = (H + 2 * p - k) / s + 1, OW = (W + 2 * p - k) / s + 1;
    const long long total = (long long)B * H * W * (C / 4);
    if ((total + 255) / 256 > 0x7FFFFFFFll) return TMQ_ERR_UNSUPPORTED;
    maxpool_f32_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4 *>(gY), reinterpret_cast<const char4 *>(idx), reinterpret_cast<float4 *>(gX), B, H, W, C / 4,
        OH, OW, k, s, p);
    return launch_status();
}
