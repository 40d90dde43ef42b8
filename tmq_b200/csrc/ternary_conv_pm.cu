// Stride-1 ternary Conv2d for layers with ONE 64-channel input slice and at most 64 output channels (ResNet's first
// stage): the "pixel-major" form of the shifted-window implicit GEMM.
//
// With 64 output channels the channel-major kernel (ternary_conv_sw.cu: weights as the 128-row A operand) multiplies 64
// rows of zeros, only half of its epilogue warps own real channels, and its single MMA-issuing thread waits on a decode
// barrier per filter tap.  Here the roles are swapped:
//   * the WHOLE decoded weight matrix (ky * kx taps x 64 channels x 64 k = at most 72 KB of bf16) is written to shared
//     memory once per CTA, in the 128-byte-swizzled K-major layout, and stays: it is the B operand (N = 64) of every MMA;
//   * the activations are the A operand (M = 128 output positions), read from the TMA-loaded input tile through a
//     descriptor shifted by the tap's offset, exactly as in the channel-major kernel;
//   * the accumulator holds [128 positions (lanes)] x [64 channels (columns)]: an epilogue thread owns one output pixel,
//     applies scale / bias / residual / ReLU to its 64 channels and writes 128 contiguous bytes - no transposition
//     through shared memory, and all four epilogue warps of a stream have work;
//   * one CTA per SM runs TWO independent streams of tiles (an MMA-issuing warp, four epilogue warps, a two-stage ring of
//     input tiles and two 64-column accumulators each), because one issuing thread cannot feed the tensor core with
//     MMAs this small; a tile's ky * kx * 4 MMAs are issued back to back, with no barrier in between.
// Same operands, geometry arguments and results as tmq_ternary_conv2d_s1_bf16 (which dispatches here).
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "decode.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace tmq {

constexpr int kPmThreads = 352;   // warp 0: TMA, warps 1-2: MMA issuers, warps 3-6 / 7-10: epilogue of stream 0 / 1
constexpr int kPmMaxTaps = 9;

struct PmArgs {
    const uint32_t *Wt;                   // prepacked weights [N][KS words], K order (tap, channel)
    const float *scale, *bias;
    const __nv_bfloat16 *residual;
    __nv_bfloat16 *Y;
    int B, H, W, OH, OW, N;
    int ky, kx, py, px, dy, dx;
    int R, Wt_cols, Wp, Rin;              // tile rows / columns, shared-memory row pitch (positions), input rows per tile
    int col_pieces, row_tiles;
    long long tiles;                      // B * row_tiles * col_pieces
    int region_bytes;                     // multiple of 1024
    int KS;                               // row stride of Wt in words
    int relu;
    int *status;
};

struct PmSmem {
    int w_off, in_off, lut_off, sc_off, bar_off, total;
};

__host__ __device__ inline PmSmem pm_smem(int ntaps, int region_bytes) {
    PmSmem s;
    s.w_off = 0;                                        // ntaps x 8 KB
    s.in_off = ntaps * 8192;                            // [stream][stage] regions
    s.lut_off = s.in_off + 4 * region_bytes;            // [stream][128] ints
    s.sc_off = s.lut_off + 1024;                        // scale[64], bias[64], tap shifts
    s.bar_off = s.sc_off + 1024;
    s.total = s.bar_off + 256 + 1024;
    return s;
}

__device__ __forceinline__ void pm_tma_load_4d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c, int w, int h, int b) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(ptx::smem_u32(bar)), "r"(c), "r"(w), "r"(h),
          "r"(b)
        : "memory");
}

__device__ __forceinline__ void pm_tile(const PmArgs &a, long long tile, int &b, int &oy0, int &ox0) {
    const int per_img = a.row_tiles * a.col_pieces;
    b = (int)(tile / per_img);
    const int rem = (int)(tile - (long long)b * per_img);
    oy0 = (rem / a.col_pieces) * a.R;
    ox0 = (rem % a.col_pieces) * a.Wt_cols;
}

__global__ void __launch_bounds__(kPmThreads, 1)
ternary_conv_pm_kernel(const __grid_constant__ CUtensorMap tmap_x, const PmArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int ntaps = args.ky * args.kx;
    const PmSmem L = pm_smem(ntaps, args.region_bytes);
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem + L.bar_off);       // [stream][stage]
    uint64_t *empty_in = full_in + 4;                                          // [stream][stage]
    uint64_t *acc_full = empty_in + 4;                                         // [stream][buffer]
    uint64_t *acc_empty = acc_full + 4;                                        // [stream][buffer]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 4);
    float *sc_s = reinterpret_cast<float *>(smem + L.sc_off), *bi_s = sc_s + 64;
    int *shtab = reinterpret_cast<int *>(bi_s + 64);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 256;                                        // 2 streams x 2 buffers x 64 columns

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; i++) {
            ptx::mbar_init(full_in + i, 1);
            ptx::mbar_init(empty_in + i, 1);
            ptx::mbar_init(acc_full + i, 1);
            ptx::mbar_init(acc_empty + i, 4);
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
    }
    if (threadIdx.x < ntaps) shtab[threadIdx.x] = (threadIdx.x / args.kx) * args.dy * args.Wp + (threadIdx.x % args.kx) * args.dx;
    if (threadIdx.x < 64) {
        const int n = threadIdx.x;
        sc_s[n] = 0.5f * ((n < args.N && args.scale) ? args.scale[n] : 1.0f);  // operands carried +-2.0
        bi_s[n] = (n < args.N && args.bias) ? args.bias[n] : 0.0f;
    }
    // every thread helps to decode the weights into the resident B tiles: one packed word (16 k of one channel) at a time
    for (int i = threadIdx.x; i < 64 * ntaps * 4; i += kPmThreads) {
        const int n = i / (ntaps * 4), rem = i - n * (ntaps * 4), tap = rem >> 2, w = rem & 3;
        uint32_t r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (n < args.N) decode_word_bf16(__ldg(args.Wt + (size_t)n * args.KS + rem), r);
        uint8_t *row = smem + L.w_off + tap * 8192 + n * 128;
        *reinterpret_cast<uint4 *>(row + (((2 * w) ^ (n & 7)) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<uint4 *>(row + (((2 * w + 1) ^ (n & 7)) << 4)) = make_uint4(r[4], r[5], r[6], r[7]);
    }
    ptx::fence_proxy_async_smem();
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const bool healthy = (*reinterpret_cast<volatile int *>(args.status) == 0);
    const uint32_t in_bytes = (uint32_t)(args.Rin * args.Wp * 128);

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA: one input tile per tile of either stream
        if (lane == 0 && healthy) {
            bool ok = true;
            int k = 0;
            for (long long tile = blockIdx.x; tile < args.tiles && ok; tile += gridDim.x, k++) {
                const int s = k & 1, stage = (k >> 1) & 1, slot = s * 2 + stage;
                ok = ptx::mbar_wait(empty_in + slot, (((uint32_t)(k >> 2)) & 1u) ^ 1u, args.status);
                if (!ok) break;
                int b, oy0, ox0;
                pm_tile(args, tile, b, oy0, ox0);
                ptx::mbar_arrive_expect_tx(full_in + slot, in_bytes);
                pm_tma_load_4d(smem + L.in_off + slot * args.region_bytes, &tmap_x, full_in + slot, 0, ox0 - args.px,
                               oy0 - args.py, b);
            }
        }
    } else if (warp <= 2) {
        // ---------------------------------------------------------------- MMA issuer of stream (warp - 1)
        // the whole warp walks the loop (uniform waits and descriptor arithmetic), one elected lane issues
        if (healthy) {
            const int s = warp - 1;
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t w_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L.w_off));
            bool ok = true;
            int j = 0;
            for (long long tile = blockIdx.x + (long long)s * gridDim.x; tile < args.tiles && ok; tile += 2LL * gridDim.x, j++) {
                const int buf = j & 1, slot = s * 2 + buf;                     // accumulator buffer and input stage alternate together
                const uint32_t ph = ((uint32_t)(j >> 1)) & 1u;
                ok = ptx::mbar_wait_warp(acc_empty + slot, ph ^ 1u, args.status);
                if (ok) ok = ptx::mbar_wait_warp(full_in + slot, ph, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint64_t in_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L.in_off + slot * args.region_bytes));
                const uint32_t d_tmem = tmem_base + (uint32_t)slot * 64u;
                if (ptx::elect_one()) {
#pragma unroll 1
                    for (int tap = 0; tap < ntaps; tap++) {
                        const uint64_t a_desc = in_desc + (uint32_t)(shtab[tap] * 8);   // the tap's row shift, in 16-byte units
                        const uint64_t b_desc = w_desc + (uint32_t)(tap * 512);          // 8 KB per tap
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++)
                            ptx::umma_f16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (tap | k4) ? 1u : 0u);
                    }
                    ptx::umma_commit(empty_in + slot);
                    ptx::umma_commit(acc_full + slot);
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: warps 3-6 stream 0, warps 7-10 stream 1
        const int s = (warp - 3) >> 2;
        const int quarter = warp & 3;
        const int p = quarter * 32 + lane;                                     // this thread's output position of the tile
        // a chunk of 16 channels is one 32-byte sector of the pixel's row: one 256-bit access when rows and bases allow
        const bool vec_ok = ((args.N & 15) == 0) && ((reinterpret_cast<uintptr_t>(args.Y) & 31) == 0) &&
                            ((reinterpret_cast<uintptr_t>(args.residual) & 31) == 0);
        bool ok = healthy;
        int j = 0;
        for (long long tile = blockIdx.x + (long long)s * gridDim.x; tile < args.tiles && ok; tile += 2LL * gridDim.x, j++) {
            const int buf = j & 1, slot = s * 2 + buf;
            int b, oy0, ox0;
            pm_tile(args, tile, b, oy0, ox0);
            const int r = p / args.Wp, jj = p - r * args.Wp;
            const int oy = oy0 + r, ox = ox0 + jj;
            const bool valid = r < args.R && jj < args.Wt_cols && oy < args.OH && ox < args.OW;
            const long long pix = valid ? ((long long)(b * args.OH + oy) * args.OW + ox) : -1;
            // this pixel's residual row is requested before the accumulator is waited for: its latency hides under the
            // multiplications still in flight
            ptx::u32x8 rv[4];
            const bool pre = args.residual != nullptr && vec_ok && pix >= 0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
#pragma unroll
                for (int e = 0; e < 8; e++) rv[q].v[e] = 0u;
                if (pre && 16 * q < args.N) rv[q] = ptx::ldg_v8(args.residual + pix * args.N + 16 * q);
            }
            ok = ptx::mbar_wait(acc_full + slot, ((uint32_t)(j >> 1)) & 1u, args.status);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)slot * 64u;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c0, v);
                ptx::tmem_ld_wait();
                if (c0 == 48) {                                                // drained: the issuer may reuse the buffer
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_empty + slot);
                }
                if (pix >= 0 && c0 < args.N) {
                    float f[16];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float4 sc4 = *reinterpret_cast<const float4 *>(sc_s + c0 + 4 * q);
                        const float4 bi4 = *reinterpret_cast<const float4 *>(bi_s + c0 + 4 * q);
                        f[4 * q + 0] = fmaf(__uint_as_float(v[4 * q + 0]), sc4.x, bi4.x);
                        f[4 * q + 1] = fmaf(__uint_as_float(v[4 * q + 1]), sc4.y, bi4.y);
                        f[4 * q + 2] = fmaf(__uint_as_float(v[4 * q + 2]), sc4.z, bi4.z);
                        f[4 * q + 3] = fmaf(__uint_as_float(v[4 * q + 3]), sc4.w, bi4.w);
                    }
                    const long long off = pix * args.N + c0;
                    if (vec_ok && c0 + 16 <= args.N) {
                        if (args.residual) {
                            const __nv_bfloat16 *rb = reinterpret_cast<const __nv_bfloat16 *>(&rv[c0 / 16]);
#pragma unroll
                            for (int e = 0; e < 16; e++) f[e] += __bfloat162float(rb[e]);
                        }
                        ptx::u32x8 o;
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(args.relu ? fmaxf(f[2 * e], 0.0f) : f[2 * e],
                                                                           args.relu ? fmaxf(f[2 * e + 1], 0.0f) : f[2 * e + 1]);
                            o.v[e] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        ptx::stg_v8(args.Y + off, o);
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; e++) {                         // unrolled: f stays in registers
                            if (c0 + e < args.N) {
                                float x = f[e];
                                if (args.residual) x += __bfloat162float(args.residual[off + e]);
                                args.Y[off + e] = __float2bfloat16_rn(args.relu ? fmaxf(x, 0.0f) : x);
                            }
                        }
                    }
                }
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

static bool pm_make_map_nhwc(CUtensorMap *map, const void *base, int B, int H, int W, int C, int box_w, int box_h) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_w, (cuuint32_t)box_h, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Pixel-major launch; arguments already validated by tmq_ternary_conv2d_s1_bf16.  TMQ_ERR_UNSUPPORTED when the layer is
// not of this kernel's class (the caller then runs the channel-major kernel).
int launch_conv_pixel_major(const void *X, const uint32_t *Wt, const float *scale, const float *bias, const void *residual,
                            void *Y, int B, int H, int W, int C, int N, int ky, int kx, int py, int px, int dy, int dx,
                            int relu, int *status, cudaStream_t st) {
    if (C != 64 || N > 64 || ky * kx > kPmMaxTaps) return TMQ_ERR_UNSUPPORTED;
    const int OH = H + 2 * py - dy * (ky - 1), OW = W + 2 * px - dx * (kx - 1);
    const int halo_x = dx * (kx - 1), halo_y = dy * (ky - 1);
    if (halo_x + 16 > 128) return TMQ_ERR_UNSUPPORTED;
    PmArgs a = {};
    a.Wt = Wt; a.scale = scale; a.bias = bias;
    a.residual = reinterpret_cast<const __nv_bfloat16 *>(residual);
    a.Y = reinterpret_cast<__nv_bfloat16 *>(Y);
    a.B = B; a.H = H; a.W = W; a.OH = OH; a.OW = OW; a.N = N;
    a.ky = ky; a.kx = kx; a.py = py; a.px = px; a.dy = dy; a.dx = dx;
    a.relu = relu; a.status = status;
    a.col_pieces = (OW + halo_x + 127) / 128;
    if (a.col_pieces > 1) a.col_pieces = (OW + (128 - halo_x) - 1) / (128 - halo_x);
    a.Wt_cols = (OW + a.col_pieces - 1) / a.col_pieces;
    a.Wp = a.Wt_cols + halo_x;
    const int rmax = 128 / a.Wp;
    if (rmax < 1) return TMQ_ERR_UNSUPPORTED;
    a.row_tiles = (OH + rmax - 1) / rmax;
    a.R = (OH + a.row_tiles - 1) / a.row_tiles;
    a.Rin = a.R + halo_y;
    if (a.Rin > 256 || a.Wp > 256) return TMQ_ERR_UNSUPPORTED;
    a.tiles = (long long)B * a.row_tiles * a.col_pieces;
    if (a.tiles < 2LL * kNumSMs) return TMQ_ERR_UNSUPPORTED;                    // too few tiles to fill two streams per SM
    const int reach = 128 + halo_y * a.Wp + halo_x;                            // rows the widest shifted read can touch
    int rows = a.Rin * a.Wp > reach ? a.Rin * a.Wp : reach;
    a.region_bytes = (rows * 128 + 1023) / 1024 * 1024;
    const long long K = (long long)ky * kx * 64;
    a.KS = (int)prepack_row_words(K, 0);
    const PmSmem L = pm_smem(ky * kx, a.region_bytes);
    if (L.total > 220 * 1024) return TMQ_ERR_UNSUPPORTED;
    CUtensorMap mx;
    if (!pm_make_map_nhwc(&mx, X, B, H, W, C, a.Wp, a.Rin)) return TMQ_ERR_LAUNCH;
    const int attr_rc = ensure_dynamic_smem(ternary_conv_pm_kernel, 220 * 1024, true);
    if (attr_rc != TMQ_OK) return attr_rc;
    ternary_conv_pm_kernel<<<kNumSMs, kPmThreads, (size_t)L.total, st>>>(mx, a);
    return launch_status();
}

}  // namespace tmq
