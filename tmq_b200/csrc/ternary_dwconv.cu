// Depthwise ternary convolutions from 2-bit packed weights (groups == channels): forward and transposed, fp32.
//
// Replaces the reference's depthwise kernels and the Python glue around them:
//   * ternaryDWConvFP32 (tmq/tmq_cuda.cu:163-238, launcher :607-644) works on an UNFOLDED input
//     [batch][pixels][ky*kx*C] that Conv2d.compact_forward materialises with F.unfold + permute
//     (tmq/tmq.py:849-854): ky*kx times the input in extra traffic, and only batch element 0 is processed.
//   * ternaryDWConvTransFP32 (tmq/tmq_cuda.cu:118-159, launcher :647-686) writes [batch][C*ky*kx][pixels] columns
//     that ConvTranspose2d.compact_forward sums with F.fold (tmq/tmq.py:1025-1029).
// Both are memory-bound: a tap costs one multiply-add with a weight in {-1, 0, +1}.  Here each comes in two forms:
//   * the operator-level form on the same unfolded / column layouts as the reference operators (all batch elements), and
//   * a direct NCHW form that reads the image itself and writes the final output: 4 bytes in + 4 bytes out per
//     element, no unfold, no fold, per-channel scale and bias applied in the same pass.
//
// Arithmetic contract: fp32, taps accumulated in (ky, kx) order starting from +0, every tap contributes
// fma(x, t, acc) with x = 0 outside the image (so signed zeros follow one rule), then y = acc * scale + bias with two
// roundings, as the reference's `final *= post_scale; bias + final` does.  The file is compiled without contraction.
//
// Packed weights: the reference layout of a [C][1][ky][kx] (or transposed [C][1][ky][kx]) kernel tensor, i.e. int32
// [ky*kx][ceil(C/16)], 16 channels per word, most significant pair first, 01 = +1, 10 = -1.
#include <cstdint>

#include "common.cuh"

namespace tmq {

constexpr int kMaxTaps = 128;  // up to 11 x 11 kernels

__device__ __forceinline__ float tap_value(const uint32_t *__restrict__ W, int Q, int tap, int c) {
    const uint32_t code = (W[(size_t)tap * Q + (c >> 4)] >> (2 * (15 - (c & 15)))) & 3u;
    return code == 1u ? 1.0f : (code == 2u ? -1.0f : 0.0f);
}

struct DwArgs {
    const float *X;
    const uint32_t *W;
    const float *scale, *bias;
    float *Y;
    int B, C, H, Wd, OH, OW, ky, kx, sy, sx, py, px, dy, dx;
};

__device__ __forceinline__ float finish(float acc, const float *scale, const float *bias, int c) {
    if (scale) acc = __fmul_rn(acc, scale[c]);
    if (bias) acc = __fadd_rn(acc, bias[c]);
    return acc;
}

// One block works on one (batch, channel) plane: 256 consecutive output pixels, x fastest.  Neighbouring threads read
// neighbouring input pixels, the ky*kx re-reads of a pixel hit L1.
__global__ void __launch_bounds__(256) dwconv2d_kernel(const DwArgs a, int blocks_per_plane) {
    __shared__ float taps[kMaxTaps];
    const int plane = blockIdx.x / blocks_per_plane, tile = blockIdx.x - plane * blocks_per_plane;
    const int c = plane % a.C;
    const int ntaps = a.ky * a.kx, Q = (a.C + 15) >> 4;
    if (threadIdx.x < ntaps) taps[threadIdx.x] = tap_value(a.W, Q, threadIdx.x, c);
    __syncthreads();
    const int o = tile * 256 + threadIdx.x;
    if (o >= a.OH * a.OW) return;
    const int oy = o / a.OW, ox = o - oy * a.OW;
    const float *x = a.X + (size_t)plane * a.H * a.Wd;
    float acc = 0.0f;
    for (int i = 0; i < a.ky; i++) {
        const int iy = oy * a.sy - a.py + i * a.dy;
        const bool y_ok = iy >= 0 && iy < a.H;
        for (int j = 0; j < a.kx; j++) {
            const int ix = ox * a.sx - a.px + j * a.dx;
            const float v = (y_ok && ix >= 0 && ix < a.Wd) ? __ldg(x + (size_t)iy * a.Wd + ix) : 0.0f;
            acc = __fmaf_rn(v, taps[i * a.kx + j], acc);
        }
    }
    a.Y[(size_t)plane * a.OH * a.OW + o] = finish(acc, a.scale, a.bias, c);
}

// Transposed depthwise convolution in gather form: output pixel (oy, ox) sums the taps (i, j) whose source position
// (oy + py - i*dy) / sy, (ox + px - j*dx) / sx is integral and inside the input.
__global__ void __launch_bounds__(256) dwconvtrans2d_kernel(const DwArgs a, int blocks_per_plane) {
    __shared__ float taps[kMaxTaps];
    const int plane = blockIdx.x / blocks_per_plane, tile = blockIdx.x - plane * blocks_per_plane;
    const int c = plane % a.C;
    const int ntaps = a.ky * a.kx, Q = (a.C + 15) >> 4;
    if (threadIdx.x < ntaps) taps[threadIdx.x] = tap_value(a.W, Q, threadIdx.x, c);
    __syncthreads();
    const int o = tile * 256 + threadIdx.x;
    if (o >= a.OH * a.OW) return;
    const int oy = o / a.OW, ox = o - oy * a.OW;
    const float *x = a.X + (size_t)plane * a.H * a.Wd;
    float acc = 0.0f;
    for (int i = 0; i < a.ky; i++) {
        const int ty = oy + a.py - i * a.dy;
        const int iy = ty / a.sy;
        const bool y_ok = ty >= 0 && iy * a.sy == ty && iy < a.H;
        for (int j = 0; j < a.kx; j++) {
            const int tx = ox + a.px - j * a.dx;
            const int ix = tx / a.sx;
            const bool ok = y_ok && tx >= 0 && ix * a.sx == tx && ix < a.Wd;
            const float v = ok ? __ldg(x + (size_t)iy * a.Wd + ix) : 0.0f;
            acc = __fmaf_rn(v, taps[i * a.kx + j], acc);
        }
    }
    a.Y[(size_t)plane * a.OH * a.OW + o] = finish(acc, a.scale, a.bias, c);
}

// Operator-level forward form: X [rows][ntaps][C] (what F.unfold + permute produces), Y [rows][C].
__global__ void __launch_bounds__(256) dwconv_patches_kernel(const float *__restrict__ X, const uint32_t *__restrict__ W,
                                                              float *__restrict__ Y, long long rows, int C, int ntaps) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * C) return;
    const long long r = idx / C;
    const int c = (int)(idx - r * C);
    const int Q = (C + 15) >> 4;
    const float *x = X + r * (long long)ntaps * C + c;
    float acc = 0.0f;
    for (int t = 0; t < ntaps; t++) acc = __fmaf_rn(__ldg(x + (long long)t * C), tap_value(W, Q, t, c), acc);
    Y[idx] = acc;
}

// Operator-level transposed form: X [B][P][C] -> Y [B][C*ntaps][P], Y[b][c*ntaps + t][p] = X[b][p][c] * T[t][c].
// A 32 x 32 (pixel x channel) tile goes through shared memory so that both the reads (channel fastest) and the
// writes (pixel fastest) are coalesced.
__global__ void __launch_bounds__(256) dwconvtrans_patches_kernel(const float *__restrict__ X,
                                                                   const uint32_t *__restrict__ W, float *__restrict__ Y,
                                                                   int P, int C, int ntaps) {
    __shared__ float tile[32][33];
    const int b = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = X + (size_t)b * P * C;
    for (int i = warp; i < 32; i += 8) {
        const int p = p0 + i, c = c0 + lane;
        tile[i][lane] = (p < P && c < C) ? x[(size_t)p * C + c] : 0.0f;
    }
    __syncthreads();
    const int Q = (C + 15) >> 4;
    float *y = Y + (size_t)b * C * ntaps * P;
    const int p = p0 + lane;
    for (int i = warp; i < 32; i += 8) {        // channel c0 + i: all taps, 32 pixels per store
        const int c = c0 + i;
        if (c >= C || p >= P) continue;
        const float v = tile[lane][i];
        for (int t = 0; t < ntaps; t++) y[((size_t)c * ntaps + t) * P + p] = __fmul_rn(v, tap_value(W, Q, t, c));
    }
}

static int check_dw(const DwArgs &a) {
    if (!a.X || !a.W || !a.Y) return TMQ_ERR_ARG;
    if (a.B <= 0 || a.C <= 0 || a.H <= 0 || a.Wd <= 0 || a.ky <= 0 || a.kx <= 0 || a.sy <= 0 || a.sx <= 0 || a.dy <= 0 ||
        a.dx <= 0 || a.py < 0 || a.px < 0)
        return TMQ_ERR_ARG;
    if (a.ky * a.kx > kMaxTaps) return TMQ_ERR_UNSUPPORTED;
    return TMQ_OK;
}

template <typename Kernel>
static int launch_planes(Kernel kernel, const DwArgs &a, cudaStream_t st) {
    if (a.OH <= 0 || a.OW <= 0) return TMQ_ERR_ARG;
    const long long bpp = ((long long)a.OH * a.OW + 255) / 256;
    const long long blocks = bpp * a.B * a.C;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    kernel<<<(unsigned)blocks, 256, 0, st>>>(a, (int)bpp);
    return launch_status();
}

}  // namespace tmq

using namespace tmq;

extern "C" int tmq_ternary_dwconv2d_f32(const float *X, const uint32_t *W, const float *scale, const float *bias, float *Y,
                                        int B, int C, int H, int Wd, int ky, int kx, int sy, int sx, int py, int px,
                                        int dy, int dx, void *stream) {
    DwArgs a = {X, W, scale, bias, Y, B, C, H, Wd, 0, 0, ky, kx, sy, sx, py, px, dy, dx};
    int rc = check_dw(a);
    if (rc != TMQ_OK) return rc;
    a.OH = (H + 2 * py - dy * (ky - 1) - 1) / sy + 1;
    a.OW = (Wd + 2 * px - dx * (kx - 1) - 1) / sx + 1;
    if (H + 2 * py - dy * (ky - 1) - 1 < 0 || Wd + 2 * px - dx * (kx - 1) - 1 < 0) return TMQ_ERR_ARG;
    return launch_planes(dwconv2d_kernel, a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_dwconvtrans2d_f32(const float *X, const uint32_t *W, const float *scale, const float *bias,
                                             float *Y, int B, int C, int H, int Wd, int ky, int kx, int sy, int sx, int py,
                                             int px, int dy, int dx, int opy, int opx, void *stream) {
    DwArgs a = {X, W, scale, bias, Y, B, C, H, Wd, 0, 0, ky, kx, sy, sx, py, px, dy, dx};
    int rc = check_dw(a);
    if (rc != TMQ_OK) return rc;
    if (opy < 0 || opx < 0) return TMQ_ERR_ARG;
    a.OH = (H - 1) * sy - 2 * py + dy * (ky - 1) + 1 + opy;
    a.OW = (Wd - 1) * sx - 2 * px + dx * (kx - 1) + 1 + opx;
    return launch_planes(dwconvtrans2d_kernel, a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_dwconv_patches_f32(const float *X, const uint32_t *W, float *Y, int64_t rows, int C, int ntaps,
                                              void *stream) {
    if (!X || !W || !Y || rows <= 0 || C <= 0 || ntaps <= 0) return TMQ_ERR_ARG;
    const long long blocks = (rows * C + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    dwconv_patches_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(X, W, Y, rows, C, ntaps);
    return launch_status();
}

extern "C" int tmq_ternary_dwconvtrans_patches_f32(const float *X, const uint32_t *W, float *Y, int B, int P, int C,
                                                   int ntaps, void *stream) {
    if (!X || !W || !Y || B <= 0 || P <= 0 || C <= 0 || ntaps <= 0) return TMQ_ERR_ARG;
    if (B > 65535 || (C + 31) / 32 > 65535) return TMQ_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((P + 31) / 32), (unsigned)((C + 31) / 32), (unsigned)B);
    dwconvtrans_patches_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(X, W, Y, P, C, ntaps);
    return launch_status();
}
