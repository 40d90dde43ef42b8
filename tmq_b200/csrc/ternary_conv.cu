// Ternary Conv2d from 2-bit packed weights as an IMPLICIT GEMM on tcgen05: no im2col buffer is ever written.
//   Y[b][oy][ox][n] = act( scale[n] * sum_{ky,kx,c} X[b][oy*s+ky*d-p][ox*s+kx*d-p][c] * T[n][(ky,kx,c)] + bias[n] )
//
// Replaces the reference's convolution path (tmq/tmq.py:822-871): F.unfold materialises every patch in fp32
// (K/C times the input), a CUDA-core GEMM multiplies it (tmq/tmq_cuda.cu:289-427) and F.fold reshapes the result.
// Here activations are bf16 NHWC, K runs as (ky, kx, c) so that 64 consecutive k of one filter tap are 128
// contiguous bytes of the input, and the patch rows of a tile are gathered straight into the swizzled operand layout:
//   * same CTA organisation as the tiled GEMM (ternary_gemm.cu): weights are the 128-row A operand, decoded from a
//     TMA-loaded raw tile into TENSOR memory (tcgen05.st, MMA with A from TMEM: no shared-memory traffic for it), output
//     pixels are the N side (BN = 128 or 256), accumulator in TMEM next to the ring of decoded weight tiles;
//   * 4 gather warps replace the activation TMA: per k-block each thread issues 16-byte cp.async copies (zero-filled
//     outside the image = padding) for its rows, then publishes a stage two k-blocks later, once the copies have landed
//     and a proxy fence has made them visible to the tensor core;
//   * the epilogue applies the folded-BatchNorm scale / bias and ReLU and writes NHWC, which is exactly the row-major
//     [pixels][channels] GEMM output.
// Needs C % 64 == 0 (every ResNet layer but the 3-channel stem).  All mbarrier waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "decode.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace tmq {

constexpr int kConvThreads = 320;  // warp 0: weight TMA, warp 1: MMA, warps 2-5: decode + epilogue, warps 6-9: gather
constexpr int kConvLag = 2;        // a gathered stage is published this many k-blocks after it was issued

struct ConvArgs {
    const void *X;                  // bf16 or int8 NHWC
    const float *scale, *bias;
    const __nv_bfloat16 *residual;  // optional [M][N], added before the ReLU (ResNet skip connection)
    void *Y;                        // bf16 / fp32 (out_f32) / int32 NHWC
    int B, H, W, C, OH, OW, N;
    int ky, kx, sy, sx, py, px, dy, dx;
    long long M;  // B * OH * OW
    int relu;
    int *status;
};

enum { CONV_BF16 = 0, CONV_I8 = 1 };

template <int BN>
struct ConvSmem {
    // a stage = gathered activation tile + raw packed words (the decoded weights sit in tensor memory).  256-pixel tiles:
    // six stages, one CTA per SM; 128-pixel tiles: four stages = 81 KB and 256 TMEM columns, so TWO CTAs share an SM and
    // one CTA's set-up, pipeline fill and epilogue run under the other's main loop.
    static constexpr int kStages = BN > 128 ? 6 : 4;
    static constexpr int STAGE_BYTES = 4 * 2048;     // transpose areas of the four epilogue warps
    static constexpr int B_BYTES = BN * 128;
    static constexpr int RAW_BYTES = 128 * 32;       // 16 bytes per row and k-block for bf16, 32 for int8 activations
    static constexpr int STAGE_OFF = 0;
    static constexpr int B_OFF = STAGE_OFF + STAGE_BYTES;
    static constexpr int RAW_OFF = B_OFF + kStages * B_BYTES;
    static constexpr int BAR_OFF = RAW_OFF + kStages * RAW_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void *gsrc, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// KIND: CONV_BF16 (bf16 activations, 64 k per k-block, fp32 accumulation) or CONV_I8 (int8 activations, 128 k per
// k-block, exact int32 accumulation and int32 output).  A k-block is always 128 bytes of one pixel's K run.
template <int KIND, bool F32OUT, int BN>
__global__ void __launch_bounds__(kConvThreads, BN > 128 ? 1 : 2)
ternary_conv_kernel(const __grid_constant__ CUtensorMap tmap_w, const ConvArgs args) {
    using L = ConvSmem<BN>;
    constexpr int ESZ = KIND == CONV_BF16 ? 2 : 1;        // bytes per activation
    constexpr int RAW_ROW = KIND == CONV_BF16 ? 16 : 32;  // packed bytes per weight row and k-block
    constexpr int kConvStages = L::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_raw = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *full_a = full_raw + kConvStages;
    uint64_t *full_b = full_a + kConvStages;
    uint64_t *empty = full_b + kConvStages;
    uint64_t *acc_full = empty + kConvStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n0 = (long long)blockIdx.x * 128;
    const long long m0 = (long long)blockIdx.y * BN;
    const int ntaps = args.ky * args.kx;
    const int cpb = args.C / 64;                           // bf16: k-blocks per filter tap
    const int nkb = (ntaps * args.C * ESZ + 127) / 128;   // C % 64 == 0: only int8 can end on half a k-block
    constexpr uint32_t A_COLS = 32;                                   // one k-block of a weight row: 64 bf16
    constexpr uint32_t TMEM_NEED = BN + kConvStages * A_COLS;         // accumulator, then the ring of decoded weight tiles
    constexpr uint32_t TMEM_COLS = TMEM_NEED <= 256 ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "tensor memory exceeded");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kConvStages; s++) {
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(full_a + s, 4);   // one arrival per decode warp
            ptx::mbar_init(full_b + s, 4);   // one arrival per gather warp
            ptx::mbar_init(empty + s, 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const bool healthy = (*reinterpret_cast<volatile int *>(args.status) == 0);

    if (warp == 0) {
        // ---------------------------------------------------------------- raw packed weights by TMA
        if (lane == 0 && healthy) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % kConvStages;
                const uint32_t ph = (uint32_t)(kb / kConvStages) & 1u;
                if (!ptx::mbar_wait(empty + s, ph ^ 1u, args.status)) break;
                ptx::mbar_arrive_expect_tx(full_raw + s, (uint32_t)(128 * RAW_ROW));
                ptx::tma_load_2d(smem + L::RAW_OFF + s * L::RAW_BYTES, &tmap_w, full_raw + s, kb * (RAW_ROW / 4), (int)n0);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // the whole warp walks the loop (uniform waits and descriptor arithmetic), one elected lane issues
        if (healthy) {
            constexpr uint32_t idesc = ((KIND == CONV_BF16 ? 1u : 2u) << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % kConvStages;
                const uint32_t ph = (uint32_t)(kb / kConvStages) & 1u;
                ok = ptx::mbar_wait_warp(full_a + s, ph, args.status);
                if (ok) ok = ptx::mbar_wait_warp(full_b + s, ph, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t a_tmem = tmem_base + BN + (uint32_t)s * A_COLS;
                const uint64_t b_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::B_OFF + s * L::B_BYTES));
                if (ptx::elect_one()) {
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {     // 32 bytes of K per instruction
                        if (KIND == CONV_BF16)
                            ptx::umma_f16_ts(tmem_base, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                        else
                            ptx::umma_i8_ts(tmem_base, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                    }
                    ptx::umma_commit(empty + s);
                }
                __syncwarp();
            }
            if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- decode warps, then epilogue
        // the decoded weight tile goes to tensor memory (row m of the tile in lane m); a warp may only touch the lane
        // quarter (warp index % 4), so rows are dealt accordingly
        const int row = (warp & 3) * 32 + lane;
        bool ok = healthy;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % kConvStages;
            const uint32_t ph = (uint32_t)(kb / kConvStages) & 1u;
            ok = ptx::mbar_wait(full_raw + s, ph, args.status);
            if (!ok) break;
            const uint8_t *raw = smem + L::RAW_OFF + s * L::RAW_BYTES + row * RAW_ROW;
            uint32_t cols[32];                        // the row's 128 operand bytes of this k-block, K ascending
            if (KIND == CONV_BF16) {
                const uint4 p = *reinterpret_cast<const uint4 *>(raw);
                const uint32_t words[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
                for (int wi = 0; wi < 4; wi++) {
                    uint32_t r[8];
                    decode_word_bf16(words[wi], r);
#pragma unroll
                    for (int j = 0; j < 8; j++) cols[8 * wi + j] = r[j];
                }
            } else {
                const uint4 p0 = *reinterpret_cast<const uint4 *>(raw);
                const uint4 p1 = *reinterpret_cast<const uint4 *>(raw + 16);
                const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int wi = 0; wi < 8; wi++) {
                    uint32_t r[4];
                    decode_word_i8(words[wi], r);
#pragma unroll
                    for (int j = 0; j < 4; j++) cols[4 * wi + j] = r[j];
                }
            }
            ptx::tmem_st_x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + BN + (uint32_t)s * A_COLS, cols);
            ptx::tmem_st_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(full_a + s);
        }
        if (ok) ok = ptx::mbar_wait(acc_full, 0u, args.status);
        ptx::tc_fence_after_sync();
        const int quarter = warp & 3;
        const long long n = n0 + quarter * 32 + lane;
        const bool n_ok = n < args.N;
        float sc = KIND == CONV_BF16 ? 0.5f : 1.0f, bi = 0.0f;   // bf16 operands are carried as +-2.0
        if (ok && n_ok) {
            if (args.scale) sc *= args.scale[n];
            if (args.bias) bi = args.bias[n];
        }
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float *stage = reinterpret_cast<float *>(smem + L::STAGE_OFF) + (warp - 2) * 512;   // this warp's transpose area
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c, v);
                ptx::tmem_ld_wait();
                if (KIND == CONV_BF16 && !F32OUT) {
                    epilogue_chunk_bf16(v, sc, bi, stage, reinterpret_cast<__nv_bfloat16 *>(args.Y), args.residual, m0 + c,
                                        args.M, args.N, n0 + quarter * 32, args.N, args.relu, lane);
                } else if (n_ok) {
                    // 4-byte outputs: lane = channel, so a store instruction covers 32 consecutive channels of one pixel
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const long long m = m0 + c + j;
                        if (m < args.M) {
                            if (KIND == CONV_I8) {
                                reinterpret_cast<int *>(args.Y)[m * args.N + n] = (int)v[j];
                            } else {
                                float f = fmaf(__uint_as_float(v[j]), sc, bi);
                                if (args.residual) f += __bfloat162float(args.residual[m * args.N + n]);
                                reinterpret_cast<float *>(args.Y)[m * args.N + n] = args.relu ? fmaxf(f, 0.0f) : f;
                            }
                        }
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- gather warps: patches -> swizzled B tile
        // Eight consecutive lanes fetch the eight 16-byte chunks of ONE pixel's 128 bytes, so a warp instruction reads
        // four full 128-byte lines.  (One thread per pixel row made every 16-byte copy its own request: 2048 requests
        // per k-block through the load/store unit, 1.25 us where the MMAs need 0.43.)  A thread serves the pixel rows
        // rg, rg + 16, ... of the tile and keeps their geometry in registers.
        const int g = threadIdx.x - 192;              // 0..127
        const int chunk = g & 7, rg = g >> 3;
        constexpr int RPT = BN / 16;                  // pixel rows per thread
        int roff[RPT];                                // element offset of the pixel at filter tap (0, 0); -1: row past the end
        int ryx[RPT];                                 // (iy0 + 32768) << 16 | (ix0 + 32768)
        {
            // first row by division, the others by stepping 16 pixels at a time (16 divisions per thread took 3.5 us)
            const long long m_first = m0 + rg;
            const long long mm = m_first < args.M ? m_first : 0;
            int b = (int)(mm / ((long long)args.OH * args.OW));
            const int rem = (int)(mm % ((long long)args.OH * args.OW));
            int oy = rem / args.OW, ox = rem % args.OW;
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                const bool valid = m_first + 16 * i < args.M;
                const int iy0 = oy * args.sy - args.py, ix0 = ox * args.sx - args.px;
                roff[i] = valid ? ((b * args.H + iy0) * args.W + ix0) * args.C : -1;
                ryx[i] = ((iy0 + 32768) << 16) | (ix0 + 32768);
                ox += 16;
                while (ox >= args.OW) {
                    ox -= args.OW;
                    if (++oy == args.OH) {
                        oy = 0;
                        b++;
                    }
                }
            }
        }
        bool ok = healthy;
        int published = 0;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % kConvStages;
            const uint32_t ph = (uint32_t)(kb / kConvStages) & 1u;
            ok = ptx::mbar_wait(empty + s, ph ^ 1u, args.status);
            if (!ok) break;
            // this thread's 16-byte chunk of the k-block: which filter tap and which channels (with 64-channel int8
            // layers a k-block spans two taps, so the tap is a per-chunk matter; past the last tap: zeros)
            int tap, c0;
            if (KIND == CONV_BF16) {          // 64 channels per k-block: one tap for the whole k-block
                tap = kb / cpb;
                c0 = (kb - tap * cpb) * 64 + chunk * 8;
            } else {
                const int e0 = kb * 128 + chunk * 16;
                tap = e0 / args.C;
                c0 = e0 - tap * args.C;
            }
            const bool tap_ok = KIND == CONV_BF16 || tap < ntaps;
            const int fy = (tap / args.kx) * args.dy, fx = (tap % args.kx) * args.dx;
            const uint32_t bbase = ptx::smem_u32(smem + L::B_OFF + s * L::B_BYTES);
            const int delta = (fy * args.W + fx) * args.C + c0;   // the chunk's distance from tap (0, 0), channel 0
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                const int r = rg + 16 * i;
                const int iy = (int)((unsigned)ryx[i] >> 16) - 32768 + fy, ix = (ryx[i] & 0xFFFF) - 32768 + fx;
                const bool inb = tap_ok && roff[i] != -1 && (unsigned)iy < (unsigned)args.H && (unsigned)ix < (unsigned)args.W;
                const char *src = reinterpret_cast<const char *>(args.X) + (inb ? (long long)(roff[i] + delta) * ESZ : 0ll);
                // 0 source bytes = zero fill (padding, rows past the end)
                cp_async_16(bbase + r * 128 + ((chunk ^ (r & 7)) << 4), src, inb ? 16u : 0u);
            }
            cp_async_commit();
            if (kb >= kConvLag) {
                cp_async_wait<kConvLag>();            // the stage issued kConvLag k-blocks ago has landed
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(full_b + (published % kConvStages));
                published++;
            }
        }
        if (ok) {
            // drain: publish what is still in flight, oldest first
            if (published < nkb - 1) {
                cp_async_wait<1>();
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(full_b + (published % kConvStages));
                published++;
            }
            cp_async_wait<0>();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            while (published < nkb) {
                if (lane == 0) ptx::mbar_arrive(full_b + (published % kConvStages));
                published++;
            }
        } else {
            cp_async_wait<0>();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int KIND, bool F32OUT, int BN>
static int launch_conv(const uint32_t *Wt, const ConvArgs &a, long long K, cudaStream_t st) {
    using L = ConvSmem<BN>;
    const long long KW = prepack_valid_words(K), KS = prepack_row_words(K, KIND);
    CUtensorMap mw;
    // box: one k-block of 128 rows; words beyond KW (an int8 k-block that ends past K) are filled with zeros
    if (!make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, Wt, (uint64_t)KW, (uint64_t)a.N, (uint64_t)KS * 4,
                     KIND == CONV_BF16 ? 4 : 8, 128, CU_TENSOR_MAP_SWIZZLE_NONE))
        return TMQ_ERR_LAUNCH;
    const int attr_rc = ensure_dynamic_smem(ternary_conv_kernel<KIND, F32OUT, BN>, L::TOTAL);
    if (attr_rc != TMQ_OK) return attr_rc;
    const long long gy = (a.M + BN - 1) / BN;
    if (gy > 65535) return TMQ_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((a.N + 127) / 128), (unsigned)gy);
    ternary_conv_kernel<KIND, F32OUT, BN><<<grid, kConvThreads, L::TOTAL, st>>>(mw, a);
    return launch_status();
}

}  // namespace tmq

using namespace tmq;

// Patch matrix for convolutions whose channel count is too small for the implicit path (the 3-channel stem):
// X fp32 NCHW [B][C][H][W] -> A bf16 [B*OH*OW][Kp], K = ky*kx*C in (ky, kx, c) order, zero padded to Kp (multiple of 8).
__global__ void __launch_bounds__(256) stem_patches_kernel(const float *__restrict__ X, __nv_bfloat16 *__restrict__ A, int B,
                                                            int C, int H, int W, int OH, int OW, int ky, int kx, int sy,
                                                            int sx, int py, int px, int dy, int dx, int Kp) {
    const int chunks = Kp / 8;
    const long long total = (long long)B * OH * OW * chunks;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int ch = (int)(idx % chunks);
    const long long m = idx / chunks;
    const int ox = (int)(m % OW), oy = (int)((m / OW) % OH), b = (int)(m / ((long long)OW * OH));
    const int K = ky * kx * C;
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const int k = ch * 8 + e;
        float f = 0.0f;
        if (k < K) {
            const int tap = k / C, c = k % C;
            const int iy = oy * sy + (tap / kx) * dy - py, ix = ox * sx + (tap % kx) * dx - px;
            if (iy >= 0 && iy < H && ix >= 0 && ix < W) f = __ldg(X + (((long long)b * C + c) * H + iy) * W + ix);
        }
        v[e] = __float2bfloat16_rn(f);
    }
    *reinterpret_cast<uint4 *>(A + m * Kp + ch * 8) = *reinterpret_cast<const uint4 *>(v);
}

// Row-staged form of the same patch matrix for unit dilation: one block per (image, output row).  The C*ky input rows
// the output row touches are converted to bf16 into shared memory once (zero outside the image); a table maps each
// k of the patch to its offset in that tile, so a thread assembles eight consecutive k from shared memory and writes one
// 16-byte vector.  Every input element is then fetched once per output row from L2 instead of once per use, and the
// index arithmetic per element shrinks to one table lookup.
__global__ void __launch_bounds__(256) stem_patches_rows_kernel(const float *__restrict__ X, __nv_bfloat16 *__restrict__ A,
                                                                 int C, int H, int W, int OH, int OW, int ky, int kx, int sy,
                                                                 int sx, int py, int px, int Kp, int RW) {
    extern __shared__ __align__(16) unsigned char dyn[];
    int *lut = reinterpret_cast<int *>(dyn);                                     // [Kp] tile offset of k, -1 = padding
    __nv_bfloat16 *tile = reinterpret_cast<__nv_bfloat16 *>(dyn + (size_t)Kp * 4);  // [C][ky][RW]
    const int oy = blockIdx.x % OH, b = blockIdx.x / OH;
    const int K = ky * kx * C;
    for (int k = threadIdx.x; k < Kp; k += 256) {
        int off = -1;
        if (k < K) {
            const int tap = k / C, c = k - tap * C;
            off = (c * ky + tap / kx) * RW + tap % kx;
        }
        lut[k] = off;
    }
    const int rows = C * ky;
    for (int i = threadIdx.x; i < rows * RW; i += 256) {
        const int r = i / RW, col = i - r * RW;            // tile column col <-> input column col - px
        const int c = r / ky, iy = oy * sy - py + (r - c * ky), ix = col - px;
        float f = 0.0f;
        if (iy >= 0 && iy < H && ix >= 0 && ix < W) f = __ldg(X + (((long long)b * C + c) * H + iy) * W + ix);
        tile[i] = __float2bfloat16_rn(f);
    }
    __syncthreads();
    const int chunks = Kp >> 3;
    __nv_bfloat16 *out = A + ((long long)b * OH + oy) * OW * Kp;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
    for (int i = threadIdx.x; i < OW * chunks; i += 256) {
        const int ox = i / chunks, ch = i - ox * chunks;
        const int base = ox * sx;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int off = lut[ch * 8 + e];
            v[e] = off >= 0 ? tile[off + base] : zero;
        }
        *reinterpret_cast<uint4 *>(out + (long long)i * 8) = *reinterpret_cast<const uint4 *>(v);
    }
}

extern "C" int tmq_conv_patches_bf16(const float *X, void *A, int B, int C, int H, int W, int ky, int kx, int sy, int sx,
                                     int py, int px, int dy, int dx, int Kp, void *stream) {
    if (!X || !A || B <= 0 || C <= 0 || H <= 0 || W <= 0 || ky <= 0 || kx <= 0 || sy <= 0 || sx <= 0 || py < 0 || px < 0 ||
        dy <= 0 || dx <= 0)
        return TMQ_ERR_ARG;
    if (Kp % 8 != 0 || Kp < ky * kx * C) return TMQ_ERR_ARG;
    if (!aligned(A, 16) || !aligned(X, 4)) return TMQ_ERR_ALIGN;
    const int OH = (H + 2 * py - dy * (ky - 1) - 1) / sy + 1, OW = (W + 2 * px - dx * (kx - 1) - 1) / sx + 1;
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    // row-staged form: unit dilation and a tile of C*ky padded input rows that fits 40 KB of shared memory
    const long long RW = (long long)(OW - 1) * sx + kx;   // tile columns an output row can touch
    const long long dyn = (long long)Kp * 4 + (long long)C * ky * RW * 2;
    if (dy == 1 && dx == 1 && dyn <= 40 * 1024 && (long long)B * OH <= 0x7FFFFFFF) {
        stem_patches_rows_kernel<<<(unsigned)(B * OH), 256, (size_t)dyn, (cudaStream_t)stream>>>(
            X, reinterpret_cast<__nv_bfloat16 *>(A), C, H, W, OH, OW, ky, kx, sy, sx, py, px, Kp, (int)RW);
        return launch_status();
    }
    const long long total = (long long)B * OH * OW * (Kp / 8);
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    stem_patches_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(X, reinterpret_cast<__nv_bfloat16 *>(A), B, C, H, W,
                                                                           OH, OW, ky, kx, sy, sx, py, px, dy, dx, Kp);
    return launch_status();
}

// ---- fused stem: few input channels, fp32 NCHW images -------------------------------------------------------------
//
// The implicit kernel above needs 64-channel runs; a 3-channel stem has none.  Writing its patch matrix to memory and
// multiplying it costs about 2 GB of traffic per 256 images (976 MB written, read again, for 154 MB of input).  This
// kernel keeps the patches on chip: one CTA per (image, output row).  The C*ky input rows that row touches are
// converted to bf16 into shared memory once; the gather warps assemble the (up to four) 128-pixel x 64-k operand tiles
// from that window through a k -> offset table, directly in the swizzled layout the MMA reads; weights are decoded into
// tensor memory as in the implicit kernel; the epilogue writes NHWC bf16 with scale / bias / ReLU.  All k-blocks are
// resident at once, so the barriers are single-use.  81 KB of shared memory and 256 TMEM columns: two CTAs per SM.
struct StemArgs {
    const float *X;
    const float *scale, *bias;
    __nv_bfloat16 *Y;
    int B, C, H, W, OH, OW, N, ky, kx, sy, sx, py, px;
    int K, RW;        // K = ky*kx*C (patch length, (ky, kx, c) order); RW = window row width = (OW-1)*sx + kx
    int relu;
    int *status;
};

constexpr int kStemMaxKb = 4;                  // K up to 256
constexpr int kStemWindowBytes = 16 * 1024;

struct StemSmem {
    static constexpr int STAGE_OFF = 0;                                   // 4 x 2 KB transpose areas
    static constexpr int B_OFF = STAGE_OFF + 4 * 2048;                    // kStemMaxKb operand tiles of 128 x 128 B
    static constexpr int RAW_OFF = B_OFF + kStemMaxKb * 128 * 128;
    static constexpr int WIN_OFF = RAW_OFF + kStemMaxKb * 128 * 16;
    static constexpr int LUT_OFF = WIN_OFF + kStemWindowBytes;
    static constexpr int BAR_OFF = LUT_OFF + kStemMaxKb * 64 * 4;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(kConvThreads, 2)
ternary_stem_kernel(const __grid_constant__ CUtensorMap tmap_w, const StemArgs args) {
    using L = StemSmem;
    constexpr int BN = 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_raw = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *full_a = full_raw + kStemMaxKb;
    uint64_t *full_b = full_a + kStemMaxKb;
    uint64_t *acc_full = full_b + kStemMaxKb;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (args.K + 63) / 64;
    const int oy = blockIdx.x % args.OH, b = blockIdx.x / args.OH;
    const long long n0 = (long long)blockIdx.y * 128;
    constexpr uint32_t A_COLS = 32, TMEM_COLS = 256;                     // 128 accumulator columns + 4 x 32

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStemMaxKb; s++) {
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(full_a + s, 4);
            ptx::mbar_init(full_b + s, 8);   // warps 2-9 all build operand tiles
        }
        ptx::mbar_init(acc_full, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const bool healthy = (*reinterpret_cast<volatile int *>(args.status) == 0);

    if (warp >= 2) {
        // ---------------------------------------------------------------- warps 2-9: window, then the operand tiles
        const int g = threadIdx.x - 64;               // 0..255
        int *lut = reinterpret_cast<int *>(smem + L::LUT_OFF);
        __nv_bfloat16 *win = reinterpret_cast<__nv_bfloat16 *>(smem + L::WIN_OFF);
        for (int k = g; k < nkb * 64; k += 256) {
            int off = -1;
            if (k < args.K) {
                const int tap = k / args.C, c = k - tap * args.C;
                off = (c * args.ky + tap / args.kx) * args.RW + tap % args.kx;
            }
            lut[k] = off;
        }
        // one warp per window row at a time: no division per element, loads of a row are consecutive
        const int rows = args.C * args.ky;
        for (int r = warp - 2; r < rows; r += 8) {
            const int c = r / args.ky, iy = oy * args.sy - args.py + (r - c * args.ky);
            const bool y_ok = iy >= 0 && iy < args.H;
            const float *src = args.X + (((long long)b * args.C + c) * args.H + (y_ok ? iy : 0)) * args.W - args.px;
            __nv_bfloat16 *dst = win + r * args.RW;
            for (int col0 = lane; col0 < args.RW; col0 += 256) {   // eight loads in flight per lane, then the stores
                float f[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int col = col0 + 32 * u, ix = col - args.px;
                    f[u] = (y_ok && col < args.RW && ix >= 0 && ix < args.W) ? __ldg(src + col) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int col = col0 + 32 * u;
                    if (col < args.RW) dst[col] = __float2bfloat16_rn(f[u]);
                }
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");   // warps 2-9 only
        const int chunk = g & 7, rg = g >> 3;            // eight lanes write the eight 16-byte chunks of one pixel row
        const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
        for (int kb = 0; kb < nkb; kb++) {
            int loff[8];
#pragma unroll
            for (int e = 0; e < 8; e++) loff[e] = lut[kb * 64 + chunk * 8 + e];
            uint8_t *tile = smem + L::B_OFF + kb * 128 * 128;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = rg + 32 * i;               // pixel ox = r of this output row
                __align__(16) __nv_bfloat16 v[8];
                const int base = r * args.sx;
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = (r < args.OW && loff[e] >= 0) ? win[loff[e] + base] : zero;
                *reinterpret_cast<uint4 *>(tile + r * 128 + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<const uint4 *>(v);
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(full_b + kb);
        }
    }

    if (warp == 0) {
        if (lane == 0 && healthy) {
            for (int kb = 0; kb < nkb; kb++) {
                ptx::mbar_arrive_expect_tx(full_raw + kb, 128 * 16);
                ptx::tma_load_2d(smem + L::RAW_OFF + kb * 128 * 16, &tmap_w, full_raw + kb, kb * 4, (int)n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && healthy) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                ok = ptx::mbar_wait(full_a + kb, 0u, args.status);
                if (ok) ok = ptx::mbar_wait(full_b + kb, 0u, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t a_tmem = tmem_base + BN + (uint32_t)kb * A_COLS;
                const uint64_t b_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::B_OFF + kb * 128 * 128));
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++)
                    ptx::umma_f16_ts(tmem_base, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
            }
            if (ok) ptx::umma_commit(acc_full);
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- weights -> tensor memory, then the epilogue
        const int row = (warp & 3) * 32 + lane;
        bool ok = healthy;
        for (int kb = 0; kb < nkb && ok; kb++) {
            ok = ptx::mbar_wait(full_raw + kb, 0u, args.status);
            if (!ok) break;
            const uint4 p = *reinterpret_cast<const uint4 *>(smem + L::RAW_OFF + kb * 128 * 16 + row * 16);
            const uint32_t words[4] = {p.x, p.y, p.z, p.w};
            uint32_t cols[32];
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                uint32_t r[8];
                decode_word_bf16(words[wi], r);
#pragma unroll
                for (int j = 0; j < 8; j++) cols[8 * wi + j] = r[j];
            }
            ptx::tmem_st_x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + BN + (uint32_t)kb * A_COLS, cols);
            ptx::tmem_st_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(full_a + kb);
        }
        if (ok) ok = ptx::mbar_wait(acc_full, 0u, args.status);
        ptx::tc_fence_after_sync();
        const int quarter = warp & 3;
        const long long n = n0 + quarter * 32 + lane;
        float sc = 0.5f, bi = 0.0f;                   // operands carried +-2.0
        if (ok && n < args.N) {
            if (args.scale) sc *= args.scale[n];
            if (args.bias) bi = args.bias[n];
        }
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float *stage = reinterpret_cast<float *>(smem + L::STAGE_OFF) + (warp - 2) * 512;
        const long long m_base = ((long long)b * args.OH + oy) * args.OW;    // first pixel of this output row
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN && c < args.OW; c += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c, v);
                ptx::tmem_ld_wait();
                epilogue_chunk_bf16(v, sc, bi, stage, args.Y, nullptr, m_base + c, m_base + args.OW, args.N,
                                    n0 + quarter * 32, args.N, args.relu, lane);
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

extern "C" int tmq_ternary_conv2d_stem_bf16(const float *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                            int B, int C, int H, int W, int N, int ky, int kx, int sy, int sx, int py, int px,
                                            int k_rows, int relu, int *status, void *stream) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || N <= 0 || ky <= 0 || kx <= 0 || sy <= 0 || sx <= 0 || py < 0 || px < 0)
        return TMQ_ERR_ARG;
    const int K = ky * kx * C;
    if (k_rows < K) return TMQ_ERR_ARG;
    const int OH = (H + 2 * py - ky) / sy + 1, OW = (W + 2 * px - kx) / sx + 1;
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    const long long RW = (long long)(OW - 1) * sx + kx;
    if (K > kStemMaxKb * 64 || OW > 128 || (long long)C * ky * RW * 2 > kStemWindowBytes || (N & 7) != 0)
        return TMQ_ERR_UNSUPPORTED;
    if ((long long)B * OH > 0x7FFFFFFF || (N + 127) / 128 > 65535) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 4) || !aligned(Wt, 16) || !aligned(Y, 16) || !aligned(status, 4)) return TMQ_ERR_ALIGN;
    StemArgs a = {X, scale, bias, reinterpret_cast<__nv_bfloat16 *>(Y), B, C, H, W, OH, OW, N, ky, kx, sy, sx, py, px, K, (int)RW,
                  relu, status};
    const long long KW = prepack_valid_words(k_rows), KS = prepack_row_words(k_rows, 0);
    CUtensorMap mw;
    if (!make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, Wt, (uint64_t)KW, (uint64_t)N, (uint64_t)KS * 4, 4, 128,
                     CU_TENSOR_MAP_SWIZZLE_NONE))
        return TMQ_ERR_LAUNCH;
    const int attr_rc = ensure_dynamic_smem(ternary_stem_kernel, StemSmem::TOTAL);
    if (attr_rc != TMQ_OK) return attr_rc;
    dim3 grid((unsigned)(B * OH), (unsigned)((N + 127) / 128));
    ternary_stem_kernel<<<grid, kConvThreads, StemSmem::TOTAL, (cudaStream_t)stream>>>(mw, a);
    return launch_status();
}

// Max pooling on bf16 NHWC activations (the layer between the stem and the first residual stage): one thread per
// 8 channels of an output pixel, 16-byte loads, window positions outside the image ignored (torch semantics).
__global__ void __launch_bounds__(256) maxpool_nhwc_kernel(const uint4 *__restrict__ X, uint4 *__restrict__ Y, int B, int H,
                                                            int W, int C8, int OH, int OW, int k, int s, int p, int relu) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)B * OH * OW * C8;
    if (idx >= total) return;
    const int c8 = (int)(idx % C8);
    long long m = idx / C8;
    const int ox = (int)(m % OW);
    m /= OW;
    const int oy = (int)(m % OH), b = (int)(m / OH);
    // relu: max(0, max(window)) equals the pooled ReLU (both are monotone), so the activation costs nothing extra
    const __nv_bfloat162 lowest = __float2bfloat162_rn(relu ? 0.0f : -INFINITY);
    __nv_bfloat162 best[4] = {lowest, lowest, lowest, lowest};
    for (int i = 0; i < k; i++) {
        const int iy = oy * s - p + i;
        if (iy < 0 || iy >= H) continue;
        for (int j = 0; j < k; j++) {
            const int ix = ox * s - p + j;
            if (ix < 0 || ix >= W) continue;
            const uint4 v = __ldg(X + (((long long)b * H + iy) * W + ix) * C8 + c8);
            const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
            for (int q = 0; q < 4; q++) best[q] = __hmax2_nan(best[q], h[q]);
        }
    }
    Y[idx] = *reinterpret_cast<const uint4 *>(best);
}

extern "C" int tmq_maxpool2d_nhwc_bf16(const void *X, void *Y, int B, int H, int W, int C, int k, int s, int p, int relu,
                                       void *stream) {
    if (!X || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || k <= 0 || s <= 0 || p < 0 || 2 * p > k) return TMQ_ERR_ARG;
    if (C % 8 != 0) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 16) || !aligned(Y, 16)) return TMQ_ERR_ALIGN;
    const int OH = (H + 2 * p - k) / s + 1, OW = (W + 2 * p - k) / s + 1;
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    const long long total = (long long)B * OH * OW * (C / 8);
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    maxpool_nhwc_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint4 *>(X), reinterpret_cast<uint4 *>(Y), B, H, W, C / 8, OH, OW, k, s, p, relu);
    return launch_status();
}

static int conv_common(const void *X, const uint32_t *Wt, const float *scale, const float *bias, const void *residual,
                       void *Y, int B, int H, int W, int C, int N, int ky, int kx, int sy, int sx, int py, int px, int dy,
                       int dx, int relu, int out_f32, int *status, int kind, cudaStream_t st) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || N <= 0 || ky <= 0 || kx <= 0 || sy <= 0 || sx <= 0 || py < 0 || px < 0 ||
        dy <= 0 || dx <= 0)
        return TMQ_ERR_ARG;
    if (C % 64 != 0) return TMQ_ERR_UNSUPPORTED;
    // the gather keeps 32-bit element offsets and 16-bit pixel coordinates
    if ((long long)B * H * W * C > 0x7FFFFFFFll || H > 30000 || W > 30000 || py > 2000 || px > 2000) return TMQ_ERR_UNSUPPORTED;
    const int OH = (H + 2 * py - dy * (ky - 1) - 1) / sy + 1, OW = (W + 2 * px - dx * (kx - 1) - 1) / sx + 1;
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    const size_t out_align = (kind == CONV_I8 || out_f32) ? 4 : 2;
    if (!aligned(X, 16) || !aligned(Wt, 16) || !aligned(Y, out_align) || !aligned(residual, 2) || !aligned(status, 4))
        return TMQ_ERR_ALIGN;
    ConvArgs a;
    a.X = X;
    a.scale = scale; a.bias = bias;
    a.residual = reinterpret_cast<const __nv_bfloat16 *>(residual);
    a.Y = Y;
    a.B = B; a.H = H; a.W = W; a.C = C; a.OH = OH; a.OW = OW; a.N = N;
    a.ky = ky; a.kx = kx; a.sy = sy; a.sx = sx; a.py = py; a.px = px; a.dy = dy; a.dx = dx;
    a.M = (long long)B * OH * OW;
    a.relu = relu;
    a.status = status;
    const long long K = (long long)ky * kx * C;
    // 128-pixel tiles, two CTAs per SM: measured 69 k images/s on packed ResNet-18 against 55 k with one 256-pixel CTA per
    // SM wherever that filled the GPU (the second CTA hides set-up, pipeline fill and epilogue of the first)
    if (kind == CONV_I8) return launch_conv<CONV_I8, false, 128>(Wt, a, K, st);
    if (out_f32) return launch_conv<CONV_BF16, true, 128>(Wt, a, K, st);
    return launch_conv<CONV_BF16, false, 128>(Wt, a, K, st);
}

extern "C" int tmq_ternary_conv2d_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias,
                                       const void *residual, void *Y, int B, int H, int W, int C, int N, int ky, int kx,
                                       int sy, int sx, int py, int px, int dy, int dx, int relu, int *status, void *stream) {
    return conv_common(X, Wt, scale, bias, residual, Y, B, H, W, C, N, ky, kx, sy, sx, py, px, dy, dx, relu, 0, status,
                       CONV_BF16, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_conv2d_bf16_f32out(const void *X, const uint32_t *Wt, const float *scale, const float *bias,
                                              const void *residual, float *Y, int B, int H, int W, int C, int N, int ky,
                                              int kx, int sy, int sx, int py, int px, int dy, int dx, int relu, int *status,
                                              void *stream) {
    return conv_common(X, Wt, scale, bias, residual, Y, B, H, W, C, N, ky, kx, sy, sx, py, px, dy, dx, relu, 1, status,
                       CONV_BF16, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_conv2d_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int B, int H, int W, int C, int N,
                                     int ky, int kx, int sy, int sx, int py, int px, int dy, int dx, int *status,
                                     void *stream) {
    return conv_common(X, Wt, nullptr, nullptr, nullptr, Y, B, H, W, C, N, ky, kx, sy, sx, py, px, dy, dx, 0, 0, status,
                       CONV_I8, (cudaStream_t)stream);
}
