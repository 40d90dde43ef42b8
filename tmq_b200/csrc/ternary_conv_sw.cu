// Stride-1 ternary Conv2d from 2-bit packed weights as a SHIFTED-WINDOW implicit GEMM on tcgen05, and the few-channel
// stem whose patches are read by descriptor.
//
// The gather-based implicit GEMM (ternary_conv.cu) fetches every input pixel once per filter tap.  For unit stride the
// patch rows of neighbouring output pixels are neighbouring input pixels, so the input never has to be rearranged at all:
//
//   * a tile is R output rows x Wt output columns of one image.  ONE 4-D TMA copy brings the (R + halo) x (Wt + halo)
//     input pixels of a 64-channel slice into shared memory as consecutive 128-byte rows (128-byte swizzle), with the
//     convolution's zero padding produced by the copy's out-of-bounds fill;
//   * output position n = r * Wp + j of the tile (Wp = Wt + halo: the positions j >= Wt of each row are computed and
//     thrown away) reads, for filter tap (fy, fx), the shared-memory row n + fy * Wp + fx.  The B operand of the MMAs of
//     that tap is therefore the SAME shared-memory tile with its descriptor's start address moved by fy * Wp + fx rows
//     (the swizzle is a function of the address, so a start in the middle of a 1024-byte swizzle atom reads correctly,
//     and measured no slower than an aligned one): ky * kx taps reuse one copy, and the load/store units never touch the
//     activations;
//   * weights are the 128-row A operand, decoded from TMA-loaded packed words into TENSOR memory exactly as in the tiled
//     GEMM (ternary_gemm.cu); their K order is (64-channel slice, ky, kx, channel) so that the words of all taps of a slice
//     are one contiguous run per output channel = one TMA copy per slice;
//   * persistent CTAs, two per SM (see the note above the kernel), each with one 128-column accumulator and a four-stage
//     ring of decoded weight k-blocks in its 256 tensor-memory columns; the epilogue (folded BatchNorm scale / bias,
//     residual, ReLU, NHWC bf16 stores) of one CTA runs under the multiplications of the other;
//   * small images (Wp * R well below 128 positions) put several sub-tiles - different images - side by side in the 128
//     accumulator columns, each with its own input copy; the decoded weights serve all of them.
//
// Limits: unit stride, C % 64 == 0, ky * kx <= 9, (Wt + halo) <= 128 positions per row piece (wider rows are cut into
// column pieces).  Everything else (strides, int8, fp32 output) stays with ternary_conv.cu.  All mbarrier waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "decode.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace tmq {

constexpr int kSwThreads = 320;   // warp 0: TMA, warp 1: MMA, warps 2-5: decode, warps 6-9: epilogue
constexpr int kSwBN = 128;        // accumulator columns (output positions) per tile
constexpr int kSwAStages = 4;     // decoded weight k-blocks in tensor memory (32 columns each)
constexpr int kSwMaxTaps = 9;     // ky * kx
constexpr int kSwMaxSub = 4;      // sub-tiles per tile

#ifdef TMQ_SW_TRACE
// development build only: time stamps (ns) of CTA 0's pipeline events, row = k-block / slice / tile counter
__device__ unsigned long long g_sw_trace[512][8];
__device__ __forceinline__ unsigned long long sw_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define SW_TRACE(row, col) do { if (blockIdx.x == 0 && (row) < 512) g_sw_trace[(row)][(col)] = sw_now(); } while (0)
#else
#define SW_TRACE(row, col) do { } while (0)
#endif

struct SwArgs {
    const float *scale, *bias;
    const __nv_bfloat16 *residual;
    __nv_bfloat16 *Y;
    int B, H, W, C, OH, OW, N;            // N = output channels
    int ky, kx, py, px, dy, dx;
    int R, Wt, Wp, Rin;                    // tile rows / columns, shared-memory row pitch (positions), input rows per tile
    int nsub;                              // sub-tiles per tile (1, 2 or 4), each with kSwBN / nsub accumulator columns
    int col_pieces, row_tiles;             // pieces per output row, tiles per image column piece
    long long subtiles;                    // B * row_tiles * col_pieces
    long long tiles_p;                     // ceil(subtiles / nsub)
    int tiles_n;                           // ceil(N / 128)
    int region_rows;                       // 128-byte rows reserved per sub-tile region in a stage
    int in_stages, raw_stages;
    int relu;
    int *status;
};

// dynamic shared memory: [epilogue staging 4 x 2 KB][position -> pixel table 128 ints + tap shifts][regions][raw words][barriers]
struct SwSmem {
    int stage_off, lut_off, in_off, raw_off, bar_off, total;
    int in_stage_bytes, raw_stage_bytes;
};

__host__ __device__ inline SwSmem sw_smem(int region_rows, int nsub, int in_stages, int ntaps, int raw_stages) {
    SwSmem s;
    s.stage_off = 0;
    s.lut_off = 4 * 2048;
    s.in_off = s.lut_off + 1024;                                  // 1024-aligned as long as the base is
    s.in_stage_bytes = ((region_rows * nsub * 128) + 1023) / 1024 * 1024;
    s.raw_off = s.in_off + in_stages * s.in_stage_bytes;
    s.raw_stage_bytes = ntaps * 128 * 16;                          // 16 packed bytes per row and k-block
    s.bar_off = s.raw_off + raw_stages * s.raw_stage_bytes;
    s.total = s.bar_off + 256 + 1024;
    return s;
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c, int w, int h, int b) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(ptx::smem_u32(bar)), "r"(c), "r"(w), "r"(h),
          "r"(b)
        : "memory");
}

// decomposition of a sub-tile index into (image, first output row, first output column)
__device__ __forceinline__ void sw_subtile(const SwArgs &a, long long st, int &b, int &oy0, int &ox0) {
    const int per_img = a.row_tiles * a.col_pieces;
    b = (int)(st / per_img);
    const int rem = (int)(st - (long long)b * per_img);
    oy0 = (rem / a.col_pieces) * a.R;
    ox0 = (rem % a.col_pieces) * a.Wt;
}

// Two CTAs share an SM (256 tensor-memory columns and at most ~110 KB of shared memory each).  A single thread per CTA
// issues the MMAs and needs several hundred cycles of its own instructions per k-block - more than the tensor core needs
// for the k-block's four 128 x 128 x 16 MMAs - so one CTA alone cannot keep the tensor core busy; the second CTA's issue
// thread fills the gaps, and one CTA's epilogue runs under the other's multiplications.  The issue loop is kept small on
// purpose: unrolled over the filter taps it measured TWICE as slow (the lone issuing warp then misses the instruction
// cache on every pass).
__global__ void __launch_bounds__(kSwThreads, 2)
ternary_conv_sw_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const SwArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int ntaps = args.ky * args.kx;
    const SwSmem L = sw_smem(args.region_rows, args.nsub, args.in_stages, ntaps, args.raw_stages);
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem + L.bar_off);       // [in_stages]  input regions landed
    uint64_t *empty_in = full_in + 4;                                          // [in_stages]  MMAs done reading them
    uint64_t *full_raw = empty_in + 4;                                         // [raw_stages] packed words landed
    uint64_t *empty_raw = full_raw + 4;                                        // [raw_stages] 4 decode warps done with them
    uint64_t *full_a = empty_raw + 4;                                          // [kSwAStages] decoded k-block in tensor memory
    uint64_t *empty_a = full_a + kSwAStages;                                   // [kSwAStages] MMAs done reading it
    uint64_t *acc_full = empty_a + kSwAStages;
    uint64_t *acc_empty = acc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    int *lut = reinterpret_cast<int *>(smem + L.lut_off);                      // [128] output pixel of a position, -1 = none
    int *shtab = lut + 128;                                                    // [ntaps] row shift of a filter tap

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nslices = args.C / 64;
    const long long ntiles = args.tiles_p * args.tiles_n;
    const int nsubcols = kSwBN / args.nsub;
    constexpr uint32_t TMEM_COLS = 256;                                        // 128 accumulator + 4 x 32 weight ring
    constexpr uint32_t A_BASE = kSwBN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 4; s++) {
            ptx::mbar_init(full_in + s, 1);
            ptx::mbar_init(empty_in + s, 1);
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(empty_raw + s, 4);
        }
        for (int s = 0; s < kSwAStages; s++) {
            ptx::mbar_init(full_a + s, 4);     // one arrival per decode warp
            ptx::mbar_init(empty_a + s, 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, 4);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (threadIdx.x < ntaps) shtab[threadIdx.x] = (threadIdx.x / args.kx) * args.dy * args.Wp + (threadIdx.x % args.kx) * args.dx;
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
        // ---------------------------------------------------------------- TMA: input regions and packed words per slice
        if (lane == 0 && healthy) {
            int si = 0, sr = 0;
            uint32_t in_phase = 1, raw_phase = 1;                              // producer side: first pass over a stage is free
            bool ok = true;
            const uint32_t in_bytes = (uint32_t)(args.Rin * args.Wp * 128);
            for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int n0 = (int)(tile % args.tiles_n) * 128;
                const long long st0 = (tile / args.tiles_n) * args.nsub;
                int bb[kSwMaxSub], oy[kSwMaxSub], ox[kSwMaxSub];
                for (int g = 0; g < args.nsub; g++) sw_subtile(args, st0 + g, bb[g], oy[g], ox[g]);   // past the end: zeros
                for (int sl = 0; sl < nslices; sl++) {
                    ok = ptx::mbar_wait(empty_in + si, in_phase, args.status);
                    if (!ok) break;
                    SW_TRACE(sl, 0);
                    ptx::mbar_arrive_expect_tx(full_in + si, in_bytes * (uint32_t)args.nsub);
                    for (int g = 0; g < args.nsub; g++)
                        tma_load_4d(smem + L.in_off + si * L.in_stage_bytes + g * args.region_rows * 128, &tmap_x, full_in + si,
                                    sl * 64, ox[g] - args.px, oy[g] - args.py, bb[g]);
                    ok = ptx::mbar_wait(empty_raw + sr, raw_phase, args.status);
                    if (!ok) break;
                    ptx::mbar_arrive_expect_tx(full_raw + sr, (uint32_t)L.raw_stage_bytes);
                    ptx::tma_load_2d(smem + L.raw_off + sr * L.raw_stage_bytes, &tmap_w, full_raw + sr, sl * ntaps * 4, n0);
                    if (++si == args.in_stages) { si = 0; in_phase ^= 1u; }
                    if (++sr == args.raw_stages) { sr = 0; raw_phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (keep this loop small)
        // The whole warp walks the loop - waits, stage counters and descriptor arithmetic are warp-uniform - and one elected
        // lane issues the MMAs and commits.
        if (healthy) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(nsubcols >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t sub_units = (uint32_t)(args.region_rows * 8);       // next sub-tile's region, in 16-byte units
            int si = 0, sa = 0, ka = 0;
            uint32_t in_phase = 0, a_phase = 0, acc_phase = 1;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                ok = ptx::mbar_wait_warp(acc_empty, acc_phase, args.status);        // the epilogue has drained the accumulator
                if (!ok) break;
                acc_phase ^= 1u;
                ptx::tc_fence_after_sync();
                uint32_t accum = 0u;
                for (int sl = 0; sl < nslices && ok; sl++) {
                    ok = ptx::mbar_wait_warp(full_in + si, in_phase, args.status);
                    if (!ok) break;
                    if (lane == 0) SW_TRACE(sl, 1);
                    const uint64_t in_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L.in_off + si * L.in_stage_bytes));
#pragma unroll 1
                    for (int tap = 0; tap < ntaps; tap++, ka++) {
                        ok = ptx::mbar_wait_warp(full_a + sa, a_phase, args.status);
                        if (!ok) break;
                        if (lane == 0) SW_TRACE(ka, 4);
                        ptx::tc_fence_after_sync();
                        const uint32_t a_tmem = tmem_base + A_BASE + (uint32_t)sa * 32u;
                        uint64_t b_desc = in_desc + (uint32_t)(shtab[tap] * 8);    // the tap's row shift, in 16-byte units
                        uint32_t d_tmem = tmem_base;
                        if (ptx::elect_one()) {
                            for (int g = 0; g < args.nsub; g++, b_desc += sub_units, d_tmem += (uint32_t)nsubcols) {
#pragma unroll
                                for (int k4 = 0; k4 < 4; k4++)
                                    ptx::umma_f16_ts(d_tmem, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, (accum | (uint32_t)k4) ? 1u : 0u);
                            }
                            ptx::umma_commit(empty_a + sa);
                        }
                        __syncwarp();
                        accum = 1u;
                        if (lane == 0) SW_TRACE(ka, 5);
                        sa = (sa + 1) & (kSwAStages - 1);
                        a_phase ^= (sa == 0) ? 1u : 0u;
                    }
                    if (ok && ptx::elect_one()) ptx::umma_commit(empty_in + si);   // every tap of the slice has read the region
                    __syncwarp();
                    if (++si == args.in_stages) { si = 0; in_phase ^= 1u; }
                }
                if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
                __syncwarp();
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- decode warps 2..5: one tensor-memory lane quarter each
        const int row = (warp & 3) * 32 + lane;
        bool ok = healthy;
        int sr = 0, sa = 0;
        uint32_t raw_phase = 0, a_phase = 1;
        int ka = 0;
        for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            for (int sl = 0; sl < nslices && ok; sl++) {
                ok = ptx::mbar_wait(full_raw + sr, raw_phase, args.status);
                if (!ok) break;
                const uint8_t *raw = smem + L.raw_off + sr * L.raw_stage_bytes + row * (ntaps * 16);
#pragma unroll 1
                for (int tap = 0; tap < ntaps; tap++, ka++) {
                    ok = ptx::mbar_wait(empty_a + sa, a_phase, args.status);
                    if (!ok) break;
                    if (warp == 2 && lane == 0) SW_TRACE(ka, 2);
                    const uint4 p = *reinterpret_cast<const uint4 *>(raw + tap * 16);
                    const uint32_t words[4] = {p.x, p.y, p.z, p.w};
                    uint32_t cols[32];
#pragma unroll
                    for (int wi = 0; wi < 4; wi++) {
                        uint32_t r[8];
                        decode_word_bf16(words[wi], r);
#pragma unroll
                        for (int j = 0; j < 8; j++) cols[8 * wi + j] = r[j];
                    }
                    ptx::tmem_st_x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + A_BASE + (uint32_t)sa * 32u, cols);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(full_a + sa);
                    if (warp == 2 && lane == 0) SW_TRACE(ka, 3);
                    sa = (sa + 1) & (kSwAStages - 1);
                    a_phase ^= (sa == 0) ? 1u : 0u;
                }
                __syncwarp();
                if (lane == 0 && ok) ptx::mbar_arrive(empty_raw + sr);         // this warp has read its words of the slice
                if (++sr == args.raw_stages) { sr = 0; raw_phase ^= 1u; }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps 6..9
        // The residual values of the first half of the tile are requested BEFORE the accumulator is waited for, those of
        // the second half while the first is being written, so their latency hides under work already in flight.
        const int quarter = warp & 3;
        float *stage = reinterpret_cast<float *>(smem + L.stage_off) + (warp - 6) * 512;
        const int et = threadIdx.x - 192;                                      // 0..127
        bool ok = healthy;
        uint32_t acc_phase = 0;
        int ti = 0;
        for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ti++) {
            const long long n0 = (tile % args.tiles_n) * 128;
            const long long st0 = (tile / args.tiles_n) * args.nsub;
            {   // position -> output pixel index of this tile (one position per epilogue thread)
                const int g = et / nsubcols, pos = et - g * nsubcols;
                int b, oy0, ox0;
                sw_subtile(args, st0 + g, b, oy0, ox0);
                const int r = pos / args.Wp, j = pos - r * args.Wp;
                const int oy = oy0 + r, ox = ox0 + j;
                const bool valid = (st0 + g) < args.subtiles && r < args.R && j < args.Wt && oy < args.OH && ox < args.OW;
                lut[et] = valid ? ((b * args.OH + oy) * args.OW + ox) : -1;
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");                     // the four epilogue warps: table complete
            const long long n = n0 + quarter * 32 + lane;
            float sc = 0.5f, bi = 0.0f;                                        // operands carried +-2.0
            if (n < args.N) {
                if (args.scale) sc *= args.scale[n];
                if (args.bias) bi = args.bias[n];
            }
            const int cg = (lane & 3) * 8;
            const long long nv = n0 + quarter * 32 + cg;                       // first channel of this lane's 8-channel vector
            const bool vec_ok = ((args.N & 7) == 0) && (nv + 8 <= args.N) && ((reinterpret_cast<uintptr_t>(args.Y) & 15) == 0) &&
                                ((reinterpret_cast<uintptr_t>(args.residual) & 15) == 0);
            const bool pre = args.residual != nullptr && vec_ok;
            uint4 rv[8];                                                       // residual vectors, four chunks ahead
#pragma unroll
            for (int q = 0; q < 8; q++) {
                rv[q] = make_uint4(0, 0, 0, 0);
                if (pre) {
                    const int pix = lut[(q >> 1) * 16 + (q & 1) * 8 + (lane >> 2)];
                    if (pix >= 0) rv[q] = __ldg(reinterpret_cast<const uint4 *>(args.residual + (long long)pix * args.N + nv));
                }
            }
            ok = ptx::mbar_wait(acc_full, acc_phase, args.status);
            if (!ok) break;
            acc_phase ^= 1u;
            if (warp == 6 && lane == 0) SW_TRACE(ti, 6);
            ptx::tc_fence_after_sync();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int cc = 0; cc < 8; cc++) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)(cc * 16), v);
                ptx::tmem_ld_wait();
                if (cc == 7) {                                                 // drained: the MMA thread may start the next tile
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_empty);
                }
#pragma unroll
                for (int j = 0; j < 16; j++) stage[j * 32 + lane] = fmaf(__uint_as_float(v[j]), sc, bi);
                __syncwarp();
#pragma unroll
                for (int itr = 0; itr < 2; itr++) {
                    const int p = itr * 8 + (lane >> 2);
                    const int pix = lut[cc * 16 + p];
                    const uint4 rcur = rv[(cc & 3) * 2 + itr];
                    if (cc < 4 && pre) {                                       // request the residual of chunk cc + 4 into the freed slot
                        const int pix4 = lut[(cc + 4) * 16 + p];
                        rv[(cc & 3) * 2 + itr] = make_uint4(0, 0, 0, 0);
                        if (pix4 >= 0)
                            rv[(cc & 3) * 2 + itr] = __ldg(reinterpret_cast<const uint4 *>(args.residual + (long long)pix4 * args.N + nv));
                    }
                    if (pix >= 0 && nv < args.N) {
                        const float4 lo = *reinterpret_cast<const float4 *>(stage + p * 32 + cg);
                        const float4 hi = *reinterpret_cast<const float4 *>(stage + p * 32 + cg + 4);
                        float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                        const long long off = (long long)pix * args.N + nv;
                        if (vec_ok) {
                            if (args.residual) {
                                const __nv_bfloat16 *rb = reinterpret_cast<const __nv_bfloat16 *>(&rcur);
#pragma unroll
                                for (int e = 0; e < 8; e++) f[e] += __bfloat162float(rb[e]);
                            }
                            __align__(16) __nv_bfloat16 o[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(args.relu ? fmaxf(f[e], 0.0f) : f[e]);
                            *reinterpret_cast<uint4 *>(args.Y + off) = *reinterpret_cast<const uint4 *>(o);
                        } else {
                            for (int e = 0; e < 8 && nv + e < args.N; e++) {
                                float x = f[e];
                                if (args.residual) x += __bfloat162float(args.residual[off + e]);
                                args.Y[off + e] = __float2bfloat16_rn(args.relu ? fmaxf(x, 0.0f) : x);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            if (warp == 6 && lane == 0) SW_TRACE(ti, 7);
            asm volatile("bar.sync 2, 128;" ::: "memory");                     // everyone is done with the table
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn4)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int launch_conv_pixel_major(const void *X, const uint32_t *Wt, const float *scale, const float *bias, const void *residual,
                            void *Y, int B, int H, int W, int C, int N, int ky, int kx, int py, int px, int dy, int dx,
                            int relu, int *status, cudaStream_t st);   // ternary_conv_pm.cu

static bool make_map_nhwc(CUtensorMap *map, const void *base, int B, int H, int W, int C, int box_w, int box_h) {
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


// ---- few-channel layers (an image stem): patches by descriptor, no operand tile -------------------------------------
//
// X fp32 NCHW with C <= CP channels, horizontal stride sx, CP = 8 / sx (sx = 2: up to 4 channels, sx = 1: up to 8), at
// most 64 output channels.  The input rows an output row needs are kept in shared memory as bf16 [row][pixel][CP
// channels]: a pixel is CP * 2 bytes, so the patch rows of neighbouring OUTPUT pixels start sx * CP * 2 = 16 bytes apart -
// exactly the row pitch of the tensor core's unswizzled K-major operand layout (8 rows x 16 bytes per core matrix).  The
// A operand (M = 128 output pixels of one output row) of the MMAs of filter row fy is therefore that shared-memory row
// itself, read through a descriptor whose core matrices overlap (K-neighbour 16 bytes on, next 8 pixels 128 bytes on): no
// patch matrix, no operand tile.  K runs as (filter row, [kx x CP] padded to a multiple of 16) with zero weights in the
// padding; the decoded weights (B operand, N = 64) sit in shared memory for the life of the CTA.
//   * the window is a RING of ky + sy input rows: consecutive tiles of a CTA are consecutive output rows of an image, so a
//     new tile converts only the sy rows it does not share with its predecessor;
//   * accumulator [128 pixels (lanes)] x [64 channels (columns)], double-buffered: an epilogue thread owns one pixel and
//     writes its 64 channels (scale / bias / ReLU, bf16 NHWC) as 128 contiguous bytes while the next row is multiplied;
//   * persistent CTAs, two per SM, each walking a contiguous range of (image, output row) tiles.
struct StemRowsArgs {
    const float *X;
    const uint32_t *Wt;       // prepacked weights [N][KS words], K order (ky, [kx, CP] padded to 16)
    const float *scale, *bias;
    __nv_bfloat16 *Y;
    int B, C, H, W, OH, OW, N;
    int ky, kx, sy, sx, py, px;
    int KR;          // MMAs (16 k each) per filter row
    int KS;          // row stride of Wt in words
    int WB;          // bytes of one window row
    int ring;        // window rows kept: ky + sy
    long long tiles; // B * OH
    long long per_cta;   // tiles per CTA (contiguous)
    int relu;
    int use_tma;     // the sy new rows of a tile arrive by TMA in a staging ring (needs W % 4 == 0)
    int stg_bytes;   // bytes of one staging slot: C planes x sy rows x W floats, rounded up to 128
    int pool;        // fuse a 3x3 / stride 2 / pad 1 max pooling behind the ReLU: Y is [B][OH/2][OW/2][64]
    int pool_off;    // byte offset (from the staging area) of the two pooling row buffers
    int *status;
};

constexpr int kStemRowsThreads = 320;   // warp 0: row copies (TMA), warp 1: MMA, warps 2-5: epilogue, warps 6-9: window
constexpr int kStemStages = 4;          // staging slots of fp32 input rows
constexpr int kStemSmemMax = 112 * 1024;  // two CTAs per SM

__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(ptx::smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ uint64_t desc_k16(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // unswizzled K-major: K-adjacent 16-byte chunk lbo_bytes on (leading byte offset), next 8 rows sbo_bytes on (stride)
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

template <int CP>
__global__ void __launch_bounds__(kStemRowsThreads, 2)
ternary_stem_rows_kernel(const __grid_constant__ CUtensorMap tmap_x, const StemRowsArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int ksteps = args.ky * args.KR;
    uint8_t *wsm = smem;                                                       // [kstep][2 chunks][64 rows x 16 B] = 2 KB each
    uint8_t *win = wsm + ksteps * 2048;                                        // [ring][WB]
    const int win_bytes = (args.ring * args.WB + 127) / 128 * 128;
    float *sc_s = reinterpret_cast<float *>(win + win_bytes), *bi_s = sc_s + 64;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bi_s + 64);
    // every barrier exists twice, for even and odd tiles: a producer can then never complete two phases of one barrier
    // before its consumer has looked at the first (a parity wait cannot tell phase n from phase n + 2)
    uint64_t *win_full = bars, *win_empty = bars + 2, *acc_full = bars + 4, *acc_empty = bars + 6;
    uint64_t *stg_full = bars + 8, *stg_empty = bars + 8 + kStemStages;        // staging ring of fp32 rows
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 8 + 2 * kStemStages);
    uint8_t *stg = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 127) & ~uintptr_t(127));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 128;                                        // two 64-column accumulators

    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(win_full + b, 4);   // the four window warps
            ptx::mbar_init(win_empty + b, 1);
            ptx::mbar_init(acc_full + b, 1);
            ptx::mbar_init(acc_empty + b, 4);
        }
        for (int i = 0; i < kStemStages; i++) {
            ptx::mbar_init(stg_full + i, 1);
            ptx::mbar_init(stg_empty + i, 4);
        }
        ptx::fence_mbar_init();
        if (args.use_tma) ptx::prefetch_tensormap(&tmap_x);
    }
    if (threadIdx.x < 64) {
        const int n = threadIdx.x;
        sc_s[n] = 0.5f * ((n < args.N && args.scale) ? args.scale[n] : 1.0f);  // operands carried +-2.0
        bi_s[n] = (n < args.N && args.bias) ? args.bias[n] : 0.0f;
    }
    // resident weights: word ks of channel n = its 16 k of MMA step ks -> two 16-byte chunks of the unswizzled B tile
    for (int i = threadIdx.x; i < 64 * ksteps; i += kStemRowsThreads) {
        const int n = i / ksteps, ks = i - n * ksteps;
        uint32_t r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (n < args.N) decode_word_bf16(__ldg(args.Wt + (size_t)n * args.KS + ks), r);
        uint8_t *dst = wsm + ks * 2048 + n * 16;
        *reinterpret_cast<uint4 *>(dst) = make_uint4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<uint4 *>(dst + 1024) = make_uint4(r[4], r[5], r[6], r[7]);
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
    long long t_begin = (long long)blockIdx.x * args.per_cta;
    long long t_end = t_begin + args.per_cta;
    if (t_end > args.tiles) t_end = args.tiles;
    // pooling: a chunk starts on an even output row (per_cta and OH are even); when that row is not the top of an image,
    // the odd row above it - the previous CTA's last - is computed here once more, only for its part in the 3-row maximum
    const bool pool_halo = args.pool && (t_begin % args.OH) != 0;
    if (pool_halo) t_begin -= 1;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA: the sy new input rows of every non-refill tile
        if (lane == 0 && healthy && args.use_tma) {
            bool ok = true;
            int ti = 0, n = 0;                                                 // n counts the tiles that arrive by TMA
            for (long long tile = t_begin; tile < t_end && ok; tile++, ti++) {
                const int b = (int)(tile / args.OH), oy = (int)(tile - (long long)b * args.OH);
                if (ti == 0 || oy == 0) continue;                              // refill: the window warps load it themselves
                const int sg = n % kStemStages;
                ok = ptx::mbar_wait(stg_empty + sg, (((uint32_t)(n / kStemStages)) & 1u) ^ 1u, args.status);
                if (!ok) break;
                ptx::mbar_arrive_expect_tx(stg_full + sg, (uint32_t)(args.C * args.sy * args.W * 4));
                tma_load_3d(stg + (size_t)sg * args.stg_bytes, &tmap_x, stg_full + sg, 0, oy * args.sy - args.py + args.ky - args.sy,
                            b * args.C);
                n++;
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (whole warp walks the loop, one lane issues)
        if (healthy) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t win_addr = ptx::smem_u32(win);
            const uint64_t w_desc = desc_k16(ptx::smem_u32(wsm), 1024, 128);
            bool ok = true;
            int ti = 0;
            for (long long tile = t_begin; tile < t_end && ok; tile++, ti++) {
                const int buf = ti & 1;
                ok = ptx::mbar_wait_warp(acc_empty + buf, (((uint32_t)(ti >> 1)) & 1u) ^ 1u, args.status);
                if (ok) ok = ptx::mbar_wait_warp(win_full + buf, ((uint32_t)(ti >> 1)) & 1u, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const int oy = (int)(tile % args.OH);
                int slot = (oy * args.sy) % args.ring;                         // ring slot of the tile's first input row
                uint64_t b_desc = w_desc;
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * 64u;
                if (ptx::elect_one()) {
#pragma unroll 1
                    for (int r = 0; r < args.ky; r++) {
                        const uint64_t a_desc = desc_k16(win_addr + (uint32_t)(slot * args.WB), 16, 128);
                        for (int j = 0; j < args.KR; j++, b_desc += 128)       // 2 KB per step, in 16-byte units
                            ptx::umma_f16(d_tmem, a_desc + 2u * (uint32_t)j, b_desc, idesc, (r | j) != 0 ? 1u : 0u);
                        if (++slot == args.ring) slot = 0;
                    }
                    ptx::umma_commit(win_empty + buf);
                    ptx::umma_commit(acc_full + buf);
                }
                __syncwarp();
            }
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------------------------------------------------------- epilogue: one output pixel per thread
        const int quarter = warp & 3;
        const int p = quarter * 32 + lane;
        // a chunk of 16 channels is one 32-byte sector of the pixel's row: one 256-bit store when rows and base allow
        const bool vec_ok = ((args.N & 15) == 0) && ((reinterpret_cast<uintptr_t>(args.Y) & 31) == 0);
        bool ok = healthy;
        int ti = 0;
        // pooling buffers, one 128-byte row per pixel, 16-byte chunks XOR-swizzled by the pixel index (a thread walks its
        // own row): V = running maximum over the rows of the current 3-row window, Hb = finished 3-row maxima of a pooled row
        uint8_t *Vrow = stg + args.pool_off + p * 128, *Hb = stg + args.pool_off + 128 * 128;
        for (long long tile = t_begin; tile < t_end && ok; tile++, ti++) {
            const int buf = ti & 1;
            ok = ptx::mbar_wait(acc_full + buf, ((uint32_t)(ti >> 1)) & 1u, args.status);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const long long pix = p < args.OW ? tile * args.OW + p : -1;       // tile = b * OH + oy
            const int oy = (int)(tile % args.OH);
            const bool odd = (oy & 1) != 0, emit = odd && !(pool_halo && ti == 0);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * 64u;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c0, v);
                ptx::tmem_ld_wait();
                if (c0 == 48) {
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_empty + buf);
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
                    if (args.pool) {
                        // rows 2p-1, 2p, 2p+1 -> pooled row p.  Even row: V = max(V, row) (top of an image: V = row, the
                        // padding row above cannot win against values >= 0); odd row: Hb = max(V, row), then V = row
#pragma unroll
                        for (int hc = 0; hc < 2; hc++) {
                            __nv_bfloat162 o[4];
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                o[e] = __floats2bfloat162_rn(fmaxf(f[8 * hc + 2 * e], 0.0f), fmaxf(f[8 * hc + 2 * e + 1], 0.0f));
                            const int chunk = ((c0 >> 3) + hc) ^ (p & 7);
                            uint4 *vp = reinterpret_cast<uint4 *>(Vrow + chunk * 16);
                            uint4 cur = *reinterpret_cast<const uint4 *>(o);
                            if (oy != 0 && !(odd && !emit)) {
                                const uint4 old = *vp;
                                const __nv_bfloat162 *a2 = reinterpret_cast<const __nv_bfloat162 *>(&old);
                                __nv_bfloat162 m[4];
#pragma unroll
                                for (int e = 0; e < 4; e++) m[e] = __hmax2_nan(a2[e], o[e]);
                                const uint4 mx = *reinterpret_cast<const uint4 *>(m);
                                if (odd) *reinterpret_cast<uint4 *>(Hb + p * 128 + chunk * 16) = mx;
                                else cur = mx;
                            }
                            *vp = cur;
                        }
                    } else if (vec_ok && c0 + 16 <= args.N) {
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
                        for (int e = 0; e < 16; e++)
                            if (c0 + e < args.N) args.Y[off + e] = __float2bfloat16_rn(args.relu ? fmaxf(f[e], 0.0f) : f[e]);
                    }
                }
            }
            if (args.pool && emit) {
                // the 3-row maxima of the whole row are in Hb: columns 2q-1, 2q, 2q+1 -> pooled pixel q.  Thread = (q, half
                // of the channels): 64 contiguous output bytes
                asm volatile("bar.sync 3, 128;" ::: "memory");
                const int q = p >> 1, half = p & 1;
                if (q < args.OW / 2) {
                    const int b = (int)(tile / args.OH);
                    __nv_bfloat16 *dst = args.Y + (((long long)b * (args.OH / 2) + (oy >> 1)) * (args.OW / 2) + q) * 64 + half * 32;
                    ptx::u32x8 out[2];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint4 m = make_uint4(0, 0, 0, 0);                          // values are >= 0: zero is the padding
#pragma unroll
                        for (int dxp = -1; dxp <= 1; dxp++) {
                            const int px = 2 * q + dxp;
                            if (px >= 0) {
                                const uint4 v4 = *reinterpret_cast<const uint4 *>(Hb + px * 128 + (((half * 4 + c) ^ (px & 7)) << 4));
                                const __nv_bfloat162 *a2 = reinterpret_cast<const __nv_bfloat162 *>(&v4);
                                __nv_bfloat162 *m2 = reinterpret_cast<__nv_bfloat162 *>(&m);
#pragma unroll
                                for (int e = 0; e < 4; e++) m2[e] = __hmax2_nan(m2[e], a2[e]);
                            }
                        }
                        out[c >> 1].v[4 * (c & 1) + 0] = m.x; out[c >> 1].v[4 * (c & 1) + 1] = m.y;
                        out[c >> 1].v[4 * (c & 1) + 2] = m.z; out[c >> 1].v[4 * (c & 1) + 3] = m.w;
                    }
                    ptx::stg_v8(dst, out[0]);
                    ptx::stg_v8(dst + 16, out[1]);
                }
                asm volatile("bar.sync 3, 128;" ::: "memory");                     // Hb may be rewritten by the next odd row
            }
        }
    } else if (warp >= 6) {
        // ---------------------------------------------------------------- window warps 6..9: fp32 NCHW rows -> bf16 ring rows
        const int t = threadIdx.x - 192;                                       // 0..127
        const int slots = args.WB / (CP * 2);                                   // pixel slots per window row
        bool ok = healthy;
        int ti = 0, n_tma = 0;
        for (long long tile = t_begin; tile < t_end && ok; tile++, ti++) {
            const int b = (int)(tile / args.OH), oy = (int)(tile - (long long)b * args.OH);
            const float *img = args.X + (long long)b * args.C * args.H * args.W;
            // first tile of this CTA or of an image: every row of the window; otherwise only the sy rows that are new
            const bool refill = ti == 0 || oy == 0;
            const int r_first = refill ? 0 : args.ky - args.sy;
            // the sy new rows overwrite rows last read by the tile two back; a refill also those of the previous tile
            if (ti >= 2) ok = ptx::mbar_wait(win_empty + (ti & 1), (((uint32_t)(ti >> 1)) & 1u) ^ 1u, args.status);
            if (ok && refill && ti >= 1) ok = ptx::mbar_wait(win_empty + ((ti - 1) & 1), ((uint32_t)((ti - 1) >> 1)) & 1u, args.status);
            if (!ok) break;
            if (args.use_tma && !refill) {
                // the new rows are already in shared memory as fp32 [channel][row][W]: convert them into the ring
                const int sg = n_tma % kStemStages;
                ok = ptx::mbar_wait(stg_full + sg, ((uint32_t)(n_tma / kStemStages)) & 1u, args.status);
                if (!ok) break;
                const float *src = reinterpret_cast<const float *>(stg + (size_t)sg * args.stg_bytes);
                for (int i = t; i < args.sy * slots; i += 128) {
                    const int dr = i / slots, sl = i - dr * slots;
                    const int ix = sl - args.px;
                    __align__(16) __nv_bfloat16 o[CP];
#pragma unroll
                    for (int c = 0; c < CP; c++) {
                        const float v = ((unsigned)ix < (unsigned)args.W && c < args.C) ? src[(c * args.sy + dr) * args.W + ix] : 0.0f;
                        o[c] = __float2bfloat16_rn(v);
                    }
                    const int slot = (oy * args.sy + args.ky - args.sy + dr) % args.ring;
                    uint8_t *dst = win + (size_t)slot * args.WB + (size_t)sl * (CP * 2);
                    if (CP == 4) *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(o);
                    else *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(o);
                }
                n_tma++;
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(stg_empty + sg);
                    ptx::mbar_arrive(win_full + (ti & 1));
                }
                continue;
            }
            const int iy0 = oy * args.sy - args.py;
            // two rows x three slots per thread in one batch: every load of a (non-refill) tile is in flight before the
            // first value is consumed, so a tile costs one memory round trip
            for (int r0 = r_first; r0 < args.ky; r0 += 2) {
                for (int s0 = t; s0 < slots; s0 += 384) {
                    float f[2][3][CP];
#pragma unroll
                    for (int dr = 0; dr < 2; dr++)
#pragma unroll
                        for (int u = 0; u < 3; u++) {
                            const int r = r0 + dr, sl = s0 + 128 * u;
                            const int iy = iy0 + r, ix = sl - args.px;
                            const bool in = r < args.ky && sl < slots && (unsigned)iy < (unsigned)args.H && (unsigned)ix < (unsigned)args.W;
                            const float *p = img + (long long)(in ? iy : 0) * args.W + (in ? ix : 0);
#pragma unroll
                            for (int c = 0; c < CP; c++) f[dr][u][c] = (in && c < args.C) ? __ldg(p + (long long)c * args.H * args.W) : 0.0f;
                        }
#pragma unroll
                    for (int dr = 0; dr < 2; dr++)
#pragma unroll
                        for (int u = 0; u < 3; u++) {
                            const int r = r0 + dr, sl = s0 + 128 * u;
                            if (r < args.ky && sl < slots) {
                                __align__(16) __nv_bfloat16 o[CP];
#pragma unroll
                                for (int c = 0; c < CP; c++) o[c] = __float2bfloat16_rn(f[dr][u][c]);
                                const int slot = (oy * args.sy + r) % args.ring;
                                uint8_t *dst = win + (size_t)slot * args.WB + (size_t)sl * (CP * 2);
                                if (CP == 4) *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(o);
                                else *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(o);
                            }
                        }
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(win_full + (ti & 1));
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace tmq

using namespace tmq;

#ifdef TMQ_SW_TRACE
extern "C" int tmq_sw_trace_read(unsigned long long *host) {
    return cudaMemcpyFromSymbol(host, g_sw_trace, sizeof(g_sw_trace)) == cudaSuccess ? 0 : -3;
}
#endif

extern "C" int tmq_ternary_conv2d_s1_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias,
                                          const void *residual, void *Y, int B, int H, int W, int C, int N, int ky, int kx,
                                          int py, int px, int dy, int dx, int relu, int *status, void *stream) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || N <= 0 || ky <= 0 || kx <= 0 || py < 0 || px < 0 || dy <= 0 || dx <= 0)
        return TMQ_ERR_ARG;
    if (C % 64 != 0 || ky * kx > kSwMaxTaps) return TMQ_ERR_UNSUPPORTED;
    const int OH = H + 2 * py - dy * (ky - 1), OW = W + 2 * px - dx * (kx - 1);
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    if ((long long)B * OH * OW > 0x7FFFFFFFll) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 16) || !aligned(Wt, 16) || !aligned(Y, 2) || !aligned(residual, 2) || !aligned(status, 4))
        return TMQ_ERR_ALIGN;
    const int halo_x = dx * (kx - 1), halo_y = dy * (ky - 1);
    if (halo_x + 16 > kSwBN) return TMQ_ERR_UNSUPPORTED;
    {   // one input slice and at most 64 output channels: the pixel-major kernel, where it covers the layer
        const int rc = launch_conv_pixel_major(X, Wt, scale, bias, residual, Y, B, H, W, C, N, ky, kx, py, px, dy, dx, relu,
                                               status, (cudaStream_t)stream);
        if (rc != TMQ_ERR_UNSUPPORTED) return rc;
    }
    SwArgs a = {};
    a.scale = scale; a.bias = bias;
    a.residual = reinterpret_cast<const __nv_bfloat16 *>(residual);
    a.Y = reinterpret_cast<__nv_bfloat16 *>(Y);
    a.B = B; a.H = H; a.W = W; a.C = C; a.OH = OH; a.OW = OW; a.N = N;
    a.ky = ky; a.kx = kx; a.py = py; a.px = px; a.dy = dy; a.dx = dx;
    a.relu = relu; a.status = status;
    // tile geometry: whole output rows when a padded row fits the 128 accumulator columns, else column pieces
    a.col_pieces = (OW + halo_x + kSwBN - 1) / kSwBN;
    if (a.col_pieces > 1) a.col_pieces = (OW + (kSwBN - halo_x) - 1) / (kSwBN - halo_x);
    a.Wt = (OW + a.col_pieces - 1) / a.col_pieces;
    a.Wp = a.Wt + halo_x;
    // sub-tiles: several images side by side when one image's rows leave most of the columns idle
    a.nsub = 1;
    while (a.nsub < kSwMaxSub && (long long)OH * a.Wp * (a.nsub * 2) <= kSwBN && B >= a.nsub * 2) a.nsub *= 2;
    const int cols = kSwBN / a.nsub;
    int rmax = cols / a.Wp;
    if (rmax < 1) return TMQ_ERR_UNSUPPORTED;
    a.row_tiles = (OH + rmax - 1) / rmax;
    a.R = (OH + a.row_tiles - 1) / a.row_tiles;
    a.Rin = a.R + halo_y;
    if (a.Rin > 256 || a.Wp > 256) return TMQ_ERR_UNSUPPORTED;
    a.subtiles = (long long)B * a.row_tiles * a.col_pieces;
    a.tiles_p = (a.subtiles + a.nsub - 1) / a.nsub;
    a.tiles_n = (N + 127) / 128;
    // a region must hold the copied rows and everything the widest shifted read of `cols` positions can touch
    const int reach = cols + halo_y * a.Wp + halo_x;
    a.region_rows = a.Rin * a.Wp > reach ? a.Rin * a.Wp : reach;
    a.region_rows = (a.region_rows + 7) / 8 * 8;                                // regions start on a swizzle-atom boundary
    const int ntaps = ky * kx;
    // two stages of each suffice (the MMAs of a slice take longer than its copies); what matters is staying under half an
    // SM's shared memory so that two CTAs are resident
    a.raw_stages = 2;
    a.in_stages = 2;
    const SwSmem L = sw_smem(a.region_rows, a.nsub, a.in_stages, ntaps, a.raw_stages);
    if (L.total > 220 * 1024) return TMQ_ERR_UNSUPPORTED;
    CUtensorMap mx, mw;
    if (!make_map_nhwc(&mx, X, B, H, W, C, a.Wp, a.Rin)) return TMQ_ERR_LAUNCH;
    const long long K = (long long)ntaps * C;
    const long long KW = prepack_valid_words(K), KS = prepack_row_words(K, 0);
    if (!make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, Wt, (uint64_t)KW, (uint64_t)N, (uint64_t)KS * 4, (uint32_t)(ntaps * 4),
                     128, CU_TENSOR_MAP_SWIZZLE_NONE))
        return TMQ_ERR_LAUNCH;
    const int attr_rc = ensure_dynamic_smem(ternary_conv_sw_kernel, 220 * 1024, true);
    if (attr_rc != TMQ_OK) return attr_rc;
    const long long ntiles = a.tiles_p * a.tiles_n;
    const long long resident = (L.total <= 112 * 1024 ? 2 : 1) * (long long)kNumSMs;
    const unsigned grid = (unsigned)(ntiles < resident ? ntiles : resident);
    ternary_conv_sw_kernel<<<grid, kSwThreads, (size_t)L.total, (cudaStream_t)stream>>>(mx, mw, a);
    return launch_status();
}

// Few-channel convolution (image stem) with the patches read by descriptor: X fp32 NCHW, C <= 8 / sx channels, sx in {1, 2}.
// Wt = prepack (fmt 0) of the packed weights with rows ordered (ky, [kx, CP channels] zero-padded to a multiple of 16);
// tmq_stem_rows_k gives that row count.
extern "C" int tmq_stem_rows_k(int C, int ky, int kx, int sx) {
    if (C <= 0 || ky <= 0 || kx <= 0 || (sx != 1 && sx != 2)) return 0;
    const int CP = 8 / sx;
    if (C > CP) return 0;
    return ky * ((kx * CP + 15) / 16) * 16;
}

static int stem_rows_launch(const float *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, int B, int C,
                            int H, int W, int N, int ky, int kx, int sy, int sx, int py, int px, int relu, int pool,
                            int *status, void *stream) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || N <= 0 || ky <= 0 || kx <= 0 || sy <= 0 || sx <= 0 || py < 0 || px < 0)
        return TMQ_ERR_ARG;
    const int Kp = tmq_stem_rows_k(C, ky, kx, sx);
    if (Kp == 0) return TMQ_ERR_UNSUPPORTED;
    const int CP = 8 / sx, KR = (kx * CP + 15) / 16;
    const int OH = (H + 2 * py - ky) / sy + 1, OW = (W + 2 * px - kx) / sx + 1;
    if (OH <= 0 || OW <= 0) return TMQ_ERR_ARG;
    // one output row per tile (M = 128 pixels), all channels in one accumulator (N = 64), the ring must reuse rows
    if (OW > 128 || N > 64 || sy >= ky || ky * KR > 24) return TMQ_ERR_UNSUPPORTED;
    if ((long long)B * OH > 0x7FFFFFFFll) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 4) || !aligned(Wt, 16) || !aligned(Y, 2) || !aligned(status, 4)) return TMQ_ERR_ALIGN;
    StemRowsArgs a = {};
    a.X = X; a.Wt = Wt; a.scale = scale; a.bias = bias;
    a.Y = reinterpret_cast<__nv_bfloat16 *>(Y);
    a.B = B; a.C = C; a.H = H; a.W = W; a.OH = OH; a.OW = OW; a.N = N;
    a.ky = ky; a.kx = kx; a.sy = sy; a.sx = sx; a.py = py; a.px = px;
    a.KR = KR;
    a.KS = (int)prepack_row_words(Kp, 0);
    // a window row must hold every byte the MMAs of one filter row read: 128 rows 16 bytes apart, KR * 32 bytes each,
    // and every pixel slot an output row can touch
    const int need_mma = 127 * 16 + KR * 32, need_px = ((OW - 1) * sx + kx) * CP * 2;
    a.WB = ((need_mma > need_px ? need_mma : need_px) + 15) / 16 * 16;
    a.ring = ky + sy;
    a.tiles = (long long)B * OH;
    a.relu = relu; a.status = status;
    a.pool = pool;
    // pooling: zero stands in for the padding, so the values must be >= 0 (ReLU); row and column pairs; the vector path
    if (pool && (!relu || N != 64 || (OH & 1) || (OW & 1) || !aligned(Y, 32))) return TMQ_ERR_UNSUPPORTED;
    const int win_bytes = (a.ring * a.WB + 127) / 128 * 128;
    // the new rows of a tile by TMA: X as a 3-D tensor [B*C planes][H][W] of fp32, box = C planes x sy rows x W
    CUtensorMap mx = {};
    a.use_tma = (W % 4 == 0 && W <= 256 && C <= 256 && sy <= 256 && aligned(X, 16)) ? 1 : 0;
    a.stg_bytes = (C * sy * W * 4 + 127) / 128 * 128;
    if (a.use_tma) {
        EncodeTiledFn fn = encode_tiled();
        cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B * C};
        cuuint64_t strides[2] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4};
        cuuint32_t box[3] = {(cuuint32_t)W, (cuuint32_t)sy, (cuuint32_t)C};
        cuuint32_t estr[3] = {1, 1, 1};
        if (!fn || fn(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(X), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            a.use_tma = 0;
    }
    a.pool_off = a.use_tma ? kStemStages * a.stg_bytes : 0;
    const int smem = ky * KR * 2048 + win_bytes + 512 + 256 + 128 + a.pool_off + (pool ? 2 * 128 * 128 : 0) + 1024;
    if (smem > kStemSmemMax) return TMQ_ERR_UNSUPPORTED;
    const long long want = 2LL * kNumSMs;
    const long long grid = a.tiles < want ? a.tiles : want;
    a.per_cta = (a.tiles + grid - 1) / grid;
    if (pool) a.per_cta += a.per_cta & 1;          // chunks start on even rows
    const unsigned nblocks = (unsigned)((a.tiles + a.per_cta - 1) / a.per_cta);
    int rc;
    if (CP == 4) {
        if ((rc = ensure_dynamic_smem(ternary_stem_rows_kernel<4>, kStemSmemMax)) != TMQ_OK) return rc;   // the limit, not this call's size
        ternary_stem_rows_kernel<4><<<nblocks, kStemRowsThreads, (size_t)smem, (cudaStream_t)stream>>>(mx, a);
    } else {
        if ((rc = ensure_dynamic_smem(ternary_stem_rows_kernel<8>, kStemSmemMax)) != TMQ_OK) return rc;
        ternary_stem_rows_kernel<8><<<nblocks, kStemRowsThreads, (size_t)smem, (cudaStream_t)stream>>>(mx, a);
    }
    return launch_status();
}

extern "C" int tmq_ternary_conv2d_stem_rows_bf16(const float *X, const uint32_t *Wt, const float *scale, const float *bias,
                                                 void *Y, int B, int C, int H, int W, int N, int ky, int kx, int sy, int sx,
                                                 int py, int px, int relu, int *status, void *stream) {
    return stem_rows_launch(X, Wt, scale, bias, Y, B, C, H, W, N, ky, kx, sy, sx, py, px, relu, 0, status, stream);
}

extern "C" int tmq_ternary_conv2d_stem_rows_pool_bf16(const float *X, const uint32_t *Wt, const float *scale,
                                                      const float *bias, void *Y, int B, int C, int H, int W, int N, int ky,
                                                      int kx, int sy, int sx, int py, int px, int *status, void *stream) {
    return stem_rows_launch(X, Wt, scale, bias, Y, B, C, H, W, N, ky, kx, sy, sx, py, px, 1, 1, status, stream);
}
