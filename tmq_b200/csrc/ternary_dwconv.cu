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

// Tiled form for unit stride and dilation (the common depthwise layer): a block stages the 16 x 64 output tile's input
// window (halo included, zero outside the image) in shared memory once, then every thread produces four horizontally
// adjacent outputs from a KY x (KX + 3) register window: about 1.5 shared-memory reads and KY*KX multiply-adds per
// output instead of KY*KX bounds-checked global reads.  TRANS selects the transposed convolution, which for unit stride
// is the same window walked backwards; the taps are still accumulated in (ky, kx) order.
template <int KY, int KX, bool TRANS, int ST>
__global__ void __launch_bounds__(256) dw_tile_kernel(const DwArgs a, int tiles_x, int tiles_y) {
    // ST: stride (both directions) of the forward convolution, 1 or 2; the transposed form is tiled for stride 1 only
    static_assert(!TRANS || ST == 1, "transposed tiles are unit-stride");
    constexpr int TH = 16, TW = 64, SH = (TH - 1) * ST + KY, SW = (TW - 1) * ST + KX, S = (SW + 3) / 4 * 4;
    __shared__ __align__(16) float tile[SH * S];
    __shared__ float taps[KY * KX];
    int b = blockIdx.x;
    const int tx = b % tiles_x;
    b /= tiles_x;
    const int ty = b % tiles_y, plane = b / tiles_y;
    const int c = plane % a.C, Q = (a.C + 15) >> 4;
    if (threadIdx.x < KY * KX) taps[threadIdx.x] = tap_value(a.W, Q, threadIdx.x, c);
    const int oy0 = ty * TH, ox0 = tx * TW;
    const int iy0 = TRANS ? oy0 + a.py - (KY - 1) : oy0 * ST - a.py, ix0 = TRANS ? ox0 + a.px - (KX - 1) : ox0 * ST - a.px;
    const float *x = a.X + (size_t)plane * a.H * a.Wd;
    for (int i = threadIdx.x; i < SH * SW; i += 256) {
        const int r = i / SW, col = i - r * SW;
        const int iy = iy0 + r, ix = ix0 + col;
        tile[r * S + col] = (iy >= 0 && iy < a.H && ix >= 0 && ix < a.Wd) ? __ldg(x + (size_t)iy * a.Wd + ix) : 0.0f;
    }
    __syncthreads();
    const int r = threadIdx.x >> 4, cg = threadIdx.x & 15;
    const int oy = oy0 + r, ox = ox0 + 4 * cg;
    if (oy >= a.OH || ox >= a.OW) return;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < KY; i++) {
        const float *row = tile + (r * ST + (TRANS ? KY - 1 - i : i)) * S + 4 * cg * ST;
        float win[KX + 3 * ST];
        const float4 v = *reinterpret_cast<const float4 *>(row);
        win[0] = v.x; win[1] = v.y; win[2] = v.z; win[3] = v.w;
#pragma unroll
        for (int j = 4; j < KX + 3 * ST; j++) win[j] = row[j];
#pragma unroll
        for (int j = 0; j < KX; j++) {
            const float t = taps[i * KX + j];
            const int col = TRANS ? KX - 1 - j : j;
#pragma unroll
            for (int q = 0; q < 4; q++) acc[q] = __fmaf_rn(win[q * ST + col], t, acc[q]);
        }
    }
    float *y = a.Y + ((size_t)plane * a.OH + oy) * a.OW + ox;
    float out[4];
#pragma unroll
    for (int q = 0; q < 4; q++) out[q] = finish(acc[q], a.scale, a.bias, c);
    if (ox + 3 < a.OW && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
        *reinterpret_cast<float4 *>(y) = make_float4(out[0], out[1], out[2], out[3]);
    } else {
#pragma unroll
        for (int q = 0; q < 4; q++)
            if (ox + q < a.OW) y[q] = out[q];
    }
}

// Marching form for unit stride and dilation, image width a multiple of 4 and padding that does not widen the image:
// no shared memory at all.  A thread owns one 16-byte column chunk of one plane and walks down the rows; per input row
// it issues one aligned 128-bit load (the next row is requested before the current one is consumed), gets the few halo
// elements from its lane neighbours with shuffles (lanes at a warp edge load them), keeps the KY most recent rows as a
// register window and emits four outputs per row with KY*KX multiply-adds each: about 12 instructions per output.
// EPX is the distance between the first window column and the first output column: px for the forward convolution,
// KX-1-px for the transposed one, which for unit stride is the same walk with the taps taken backwards (still
// accumulated in (ky, kx) order).
template <int KY, int KX, int EPX, bool TRANS>
__global__ void __launch_bounds__(256) dw_march_kernel(const DwArgs a, int epy, long long items, int rows_per_strip) {
    constexpr int L = EPX, R = KX - 1 - EPX, WN = KX + 3;      // halo left / right, window width
    static_assert(L >= 0 && L <= 4 && R >= 0 && R <= 4, "halo must fit the neighbouring chunk");
    const long long item_raw = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = item_raw < items;
    const long long item = live ? item_raw : items - 1;
    const int nchunks = a.Wd >> 2, lane = threadIdx.x & 31;
    const int plane = (int)(item / nchunks), chunk = (int)(item - (long long)plane * nchunks);
    const int c = plane % a.C, Q = (a.C + 15) >> 4;
    float taps[KY * KX];
#pragma unroll
    for (int t = 0; t < KY * KX; t++) taps[t] = tap_value(a.W, Q, t, c);
    const float *xf = a.X + (size_t)plane * a.H * a.Wd + 4 * chunk;
    // neighbours that a shuffle cannot deliver: the other plane row's end, or another warp
    const bool has_left = chunk > 0, has_right = chunk < nchunks - 1;
    const bool load_left = L > 0 && has_left && (lane == 0), load_right = R > 0 && has_right && (lane == 31);
    struct Row {
        float4 own;
        float lh[L > 0 ? L : 1], rh[R > 0 ? R : 1];   // halo elements, only filled in lanes at a warp edge
    };
    auto fetch = [&](int iy, Row &r) {
        r.own = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < (L > 0 ? L : 1); j++) r.lh[j] = 0.0f;
#pragma unroll
        for (int j = 0; j < (R > 0 ? R : 1); j++) r.rh[j] = 0.0f;
        if (iy >= 0 && iy < a.H) {
            const float *p = xf + (size_t)iy * a.Wd;
            r.own = __ldg(reinterpret_cast<const float4 *>(p));
            if (load_left) {
#pragma unroll
                for (int j = 0; j < L; j++) r.lh[j] = __ldg(p - L + j);
            }
            if (load_right) {
#pragma unroll
                for (int j = 0; j < R; j++) r.rh[j] = __ldg(p + 4 + j);
            }
        }
    };
    float win[KY][WN];
#pragma unroll
    for (int i = 0; i < KY; i++)
#pragma unroll
        for (int j = 0; j < WN; j++) win[i][j] = 0.0f;
    auto push = [&](const Row &r) {
#pragma unroll
        for (int i = 0; i + 1 < KY; i++)
#pragma unroll
            for (int j = 0; j < WN; j++) win[i][j] = win[i + 1][j];
        const float lo[4] = {r.own.x, r.own.y, r.own.z, r.own.w};
#pragma unroll
        for (int j = 0; j < 4; j++) win[KY - 1][L + j] = lo[j];
#pragma unroll
        for (int j = 0; j < L; j++) {           // the last L elements of the chunk to the left
            float v = __shfl_up_sync(0xFFFFFFFFu, lo[4 - L + j], 1);
            if (lane == 0) v = r.lh[j];
            win[KY - 1][j] = has_left ? v : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < R; j++) {           // the first R elements of the chunk to the right
            float v = __shfl_down_sync(0xFFFFFFFFu, lo[j], 1);
            if (lane == 31) v = r.rh[j];
            win[KY - 1][L + 4 + j] = has_right ? v : 0.0f;
        }
    };
    // blockIdx.y selects a strip of output rows (more, shorter walks: fills the last wave of blocks better)
    const int oy_begin = blockIdx.y * rows_per_strip;
    const int oy_end = min(a.OH, oy_begin + rows_per_strip);
    // window rows before the strip's first output row: input rows oy_begin - epy .. + KY - 2
    {
        Row r;
#pragma unroll
        for (int i = 0; i < KY - 1; i++) {
            fetch(oy_begin + i - epy, r);
            push(r);
        }
    }
    // D rows are in flight ahead of the one being consumed.  More than one costs registers (the unrolled window) and
    // with them occupancy; measured 3.65 TB/s at D = 3 against 3.9 TB/s at D = 1 for 3 x 3 kernels.
    constexpr int D = 1;
    Row pre[D];
#pragma unroll
    for (int u = 0; u < D; u++) fetch(oy_begin + u + KY - 1 - epy, pre[u]);
    const float sc = a.scale ? a.scale[c] : 1.0f, bi = a.bias ? a.bias[c] : 0.0f;
    const bool vec = (a.OW & 3) == 0;
    for (int oy0 = oy_begin; oy0 < oy_end; oy0 += D) {
#pragma unroll
        for (int u = 0; u < D; u++) {
            const int oy = oy0 + u;
            if (oy >= oy_end) break;              // uniform over the block
            push(pre[u]);
            fetch(oy + D + KY - 1 - epy, pre[u]);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < KY; i++)
#pragma unroll
                for (int j = 0; j < KX; j++) {
                    const float t = taps[i * KX + j];
                    const int row = TRANS ? KY - 1 - i : i, col = TRANS ? KX - 1 - j : j;
#pragma unroll
                    for (int q = 0; q < 4; q++) acc[q] = __fmaf_rn(win[row][q + col], t, acc[q]);
                }
            if (!live) continue;
            float out[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                out[q] = acc[q];
                if (a.scale) out[q] = __fmul_rn(out[q], sc);
                if (a.bias) out[q] = __fadd_rn(out[q], bi);
            }
            float *y = a.Y + ((size_t)plane * a.OH + oy) * a.OW + 4 * chunk;
            if (vec && 4 * chunk + 3 < a.OW) {
                *reinterpret_cast<float4 *>(y) = make_float4(out[0], out[1], out[2], out[3]);
            } else {
#pragma unroll
                for (int q = 0; q < 4; q++)
                    if (4 * chunk + q < a.OW) y[q] = out[q];
            }
        }
    }
}

template <int KY, int KX, int EPX, bool TRANS>
static int launch_march_one(const DwArgs &a, int epy, cudaStream_t st) {
    const long long items = (long long)a.B * a.C * (a.Wd >> 2);
    const long long blocks = (items + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    // strips of at least 8 output rows, enough of them for about eight full waves of resident threads
    const long long resident = (long long)kNumSMs * 1024;
    long long strips = (8 * resident + items - 1) / items;
    if (strips > a.OH / 8) strips = a.OH / 8;
    if (strips < 1) strips = 1;
    const int rows_per_strip = (int)((a.OH + strips - 1) / strips);
    strips = (a.OH + rows_per_strip - 1) / rows_per_strip;
    dw_march_kernel<KY, KX, EPX, TRANS><<<dim3((unsigned)blocks, (unsigned)strips), 256, 0, st>>>(a, epy, items,
                                                                                                   rows_per_strip);
    return launch_status();
}

// Square 3 / 5 / 7 kernels with "same" or no padding; everything else goes to the tiled or the generic kernel.
template <bool TRANS>
static int launch_march(const DwArgs &a, cudaStream_t st, bool &taken) {
    taken = false;
    if (a.sy != 1 || a.sx != 1 || a.dy != 1 || a.dx != 1 || a.ky != a.kx || (a.Wd & 3) != 0) return TMQ_OK;
    if (!aligned(a.X, 16) || !aligned(a.Y, 16)) return TMQ_OK;
    const int k = a.ky;
    const int epy = TRANS ? k - 1 - a.py : a.py, epx = TRANS ? k - 1 - a.px : a.px;
    if (epy < 0 || epx < 0 || a.OW > a.Wd) return TMQ_OK;
    taken = true;
    if (k == 3 && epx == 1) return launch_march_one<3, 3, 1, TRANS>(a, epy, st);
    if (k == 3 && epx == 0) return launch_march_one<3, 3, 0, TRANS>(a, epy, st);
    if (k == 5 && epx == 2) return launch_march_one<5, 5, 2, TRANS>(a, epy, st);
    if (k == 5 && epx == 0) return launch_march_one<5, 5, 0, TRANS>(a, epy, st);
    if (k == 7 && epx == 3) return launch_march_one<7, 7, 3, TRANS>(a, epy, st);
    taken = false;
    return TMQ_OK;
}

template <bool TRANS>
static int launch_tiles(const DwArgs &a, cudaStream_t st, bool &taken) {
    taken = false;
    if (a.dy != 1 || a.dx != 1 || a.ky != a.kx || (a.ky != 3 && a.ky != 5 && a.ky != 7)) return TMQ_OK;
    const bool unit = a.sy == 1 && a.sx == 1, two = !TRANS && a.sy == 2 && a.sx == 2 && a.ky <= 5;
    if (!unit && !two) return TMQ_OK;
    const long long tiles_x = (a.OW + 63) / 64, tiles_y = (a.OH + 15) / 16;
    const long long blocks = tiles_x * tiles_y * a.B * a.C;
    if (blocks > 0x7FFFFFFF) return TMQ_OK;
    taken = true;
    const unsigned grid = (unsigned)blocks;
    const int tx = (int)tiles_x, ty = (int)tiles_y;
    if (unit) {
        if (a.ky == 3) dw_tile_kernel<3, 3, TRANS, 1><<<grid, 256, 0, st>>>(a, tx, ty);
        else if (a.ky == 5) dw_tile_kernel<5, 5, TRANS, 1><<<grid, 256, 0, st>>>(a, tx, ty);
        else dw_tile_kernel<7, 7, TRANS, 1><<<grid, 256, 0, st>>>(a, tx, ty);
    } else {
        if (a.ky == 3) dw_tile_kernel<3, 3, false, 2><<<grid, 256, 0, st>>>(a, tx, ty);
        else dw_tile_kernel<5, 5, false, 2><<<grid, 256, 0, st>>>(a, tx, ty);
    }
    return launch_status();
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
    bool taken;
    rc = launch_march<false>(a, (cudaStream_t)stream, taken);
    if (taken) return rc;
    rc = launch_tiles<false>(a, (cudaStream_t)stream, taken);
    if (taken) return rc;
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
    if (a.OH <= 0 || a.OW <= 0) return TMQ_ERR_ARG;
    bool taken;
    rc = launch_march<true>(a, (cudaStream_t)stream, taken);
    if (taken) return rc;
    rc = launch_tiles<true>(a, (cudaStream_t)stream, taken);
    if (taken) return rc;
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
