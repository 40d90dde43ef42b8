// Ternary GEMM from 2-bit packed weights on the 5th-generation tensor cores:  Y[m][n] = scale[n] * sum_k X[m][k] *
// T[n][k] + bias[n],  T in {-1, 0, +1}.
//
// Replaces the reference's CUDA-core kernel (tmq/tmq_cuda.cu:289-427, launcher :478-549), which multiplies fp32
// activations with a constant-memory LUT decode of the packed words.  Here the packed tile is decoded in shared
// memory to EXACT bf16 / int8 values and fed to tcgen05.mma with the accumulator in tensor memory:
//
//   * persistent CTAs (one per SM, 320 threads) walk the output tiles; roles: warp 0 issues TMA loads (activation
//     tile with 128-byte swizzle + the raw packed-weight tile), warps 2-5 decode the packed tile into the swizzled
//     K-major operand layout, one thread of warp 1 issues the MMAs, warps 6-9 drain the accumulator (tcgen05.ld),
//     apply scale/bias and store.  The accumulator is double-buffered in tensor memory, so the epilogue of one
//     tile overlaps the multiplication of the next.
//   * the WEIGHT tile is the 128-row "A" operand and the ACTIVATION tile the N-side "B" operand (BN = 32..256
//     rows), so one decoded weight tile is reused by up to 256 activation rows and skinny problems use a small BN.
//     TMEM lane i therefore holds output column n0+i, TMEM column j holds output row m0+j.
//   * 4-stage mbarrier pipeline: full_raw (TMA bytes landed) -> full_a (decode done) -> MMA -> empty (tcgen05.commit).
//   * exactness: bf16 operands carry the code bits directly as {0, +2.0, -2.0} (sign and top exponent bit), the
//     factor 2 is folded into the epilogue scale; products and int8 dot products are exact, accumulation is
//     fp32 / int32 in TMEM.
//   * every mbarrier wait is bounded and reports TMQ_ERR_TIMEOUT through a status word instead of hanging.
//
// Prepacked weight layout (built once from the reference layout by tmq_prepack): Wt[N][Kp/16] words, Kp = K rounded
// up to 64, word = 16 consecutive k of one output channel, bit order chosen per activation type so that decode is
// a shift+mask (bf16) or a byte-permute table lookup (int8).
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "decode.cuh"
#include "epilogue.cuh"
#include "tma_host.cuh"
#include "ptx.cuh"

namespace tmq {

constexpr int kGemmThreads = 320;  // warp 0: TMA, warp 1: MMA, warps 2-5: decode, warps 6-9: epilogue
constexpr int kTileN = 128;    // weight rows (output channels) per CTA = UMMA M
// Pipeline depth: four stages when the decoded weight tile sits in shared memory (one 256-row CTA with 4 stages
// measured 20 % faster than two 128-row CTAs per SM with 3); with the weight tile in tensor memory a stage is only the
// activation tile plus the raw packed words, and shared memory holds six of the largest.
template <int BN, bool TA>
struct StagesFor {
    static constexpr int value = TA ? (BN > 128 ? 6 : 8) : 4;
};
constexpr int kRowBytes = 128; // bytes of one operand row per k-block (64 bf16 or 128 int8)

enum { KIND_BF16 = 0, KIND_I8 = 1 };

struct GemmArgs {
    const float *scale;  // [N] or null (=1)
    const float *bias;   // [N] or null (=0)
    void *Y;
    long long M, N, K, ldy;
    int out_f32;         // bf16 kind: write fp32 instead of bf16
    int *status;
    PeerList peers;      // bf16 output only: the same block is also stored into these buffers (other GPUs' memory)
    // K split over several CTAs per output tile (skinny problems with fewer tiles than SMs): raw accumulators go to
    // partial[split][M][N] (fp32 or int32) and a second kernel sums them in split order and applies scale / bias
    void *partial;
    int splits;          // >= 1
    int kb_per_split;    // k-blocks of one split
};

// Work unit u = (output tile, K split): the k-blocks [kb0, kb1) of tile u / splits.
struct GemmUnit {
    long long tile;
    int split, kb0, kb1;
};
template <bool EXT>
__device__ __forceinline__ GemmUnit gemm_unit(const GemmArgs &a, long long u, int nkb) {
    GemmUnit q;
    if (!EXT) {                 // the plain kernel: one unit per tile, all of K
        q.tile = u; q.split = 0; q.kb0 = 0; q.kb1 = nkb;
        return q;
    }
    q.tile = u / a.splits;
    q.split = (int)(u - q.tile * a.splits);
    q.kb0 = q.split * a.kb_per_split;
    q.kb1 = q.kb0 + a.kb_per_split < nkb ? q.kb0 + a.kb_per_split : nkb;
    return q;
}

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<KIND_BF16> {
    static constexpr int BK = 64;          // k per block
    static constexpr int RAW_ROW = 16;     // packed bytes per row per k-block
    static constexpr uint32_t C_FMT = 1u;  // f32 accumulator
};
template <>
struct KindTraits<KIND_I8> {
    static constexpr int BK = 128;
    static constexpr int RAW_ROW = 32;
    static constexpr uint32_t C_FMT = 2u;  // s32 accumulator
};

// BC: the all-gather form (tmq_ternary_gemm_bf16_bcast on full tiles).  The epilogue first parks the whole bf16 output tile
// in shared memory (64 KB, paid for with two pipeline stages), hands the accumulator back, and only then writes the tile
// out - to this GPU and to the peers - in whole 256-byte rows while the next tile is already being multiplied.
template <int KIND, int BN, bool TA, bool BC = false>
struct SmemLayout {
    static constexpr int kStages = BC ? 4 : StagesFor<BN, TA>::value;
    static constexpr int A_BYTES = TA ? 0 : kTileN * kRowBytes;              // 16 KB, or none: operand in tensor memory
    static constexpr int B_BYTES = BN * kRowBytes;
    static constexpr int RAW_BYTES = kTileN * KindTraits<KIND>::RAW_ROW;     // 2 KB / 4 KB
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = A_OFF + kStages * A_BYTES;
    static constexpr int RAW_OFF = B_OFF + kStages * B_BYTES;
    static constexpr int STAGE_OFF = RAW_OFF + kStages * RAW_BYTES;          // 4 x 2 KB transpose areas of the epilogue warps
    static constexpr int OUT_OFF = STAGE_OFF + 4 * 2048;                     // BC: [BN rows][128 channels] bf16, 16-byte chunks swizzled
    static constexpr int BAR_OFF = OUT_OFF + (BC ? BN * 256 : 0);
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;                       // + barriers + alignment slack
};

// ---- the kernel -----------------------------------------------------------------------------------------------------
//
// Persistent: min(#tiles, 148) CTAs, CTA c works on tiles c, c + grid, ... (channel-tile index fastest, so the CTAs of
// one sweep share an activation tile through L2).  The TMA / decode / MMA pipeline runs on across tile boundaries and
// the accumulator is double-buffered in TMEM (2 x BN columns): four dedicated epilogue warps drain tile i while tile
// i+1 is being multiplied.

// TA: the decoded weight tile (A operand) lives in tensor memory instead of shared memory.  Per k-block that takes the
// 16 KB decode write and the 16 KB operand read off shared memory, whose bandwidth otherwise bounds the kernel; the
// accumulator is then single-buffered for 256-row activation tiles (512 TMEM columns: 256 + 4 x 32 for the A ring).
// MODE 0: the plain GEMM.  MODE 1 (BC): the all-gather form on full tiles.  MODE 2 (EXT): K split over CTAs (partial sums
// to a workspace) and / or further destinations written from the ordinary epilogue.  The extras are compiled out of
// MODE 0: with the accumulator single-buffered its epilogue is on the critical path, and carrying them cost 3 - 4 %.
template <int KIND, int BN, bool TA, int MODE = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
ternary_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, GemmArgs args) {
    using KT = KindTraits<KIND>;
    constexpr bool BC = MODE == 1, EXT = MODE == 2;
    using L = SmemLayout<KIND, BN, TA, BC>;
    constexpr int kStages = L::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_raw = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *full_a = full_raw + kStages;
    uint64_t *empty = full_a + kStages;
    uint64_t *acc_full = empty + kStages;   // [2]
    uint64_t *acc_empty = acc_full + 2;     // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((args.K + KT::BK - 1) / KT::BK);
    const long long tiles_n = (args.N + kTileN - 1) / kTileN;
    const long long tiles_m = (args.M + BN - 1) / BN;
    const long long ntiles = tiles_n * tiles_m * (EXT ? args.splits : 1);   // work units: (tile, K split)
    constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN;
    constexpr int ACC_BUFS = (TA && BN > 128) ? 1 : 2;
    constexpr uint32_t A_COLS = kRowBytes / 4;                       // one k-block of a row: 32 columns
    constexpr uint32_t A_BASE = ACC_BUFS * ACC_COLS;                 // A ring behind the accumulators
    constexpr uint32_t TMEM_NEED = A_BASE + (TA ? kStages * A_COLS : 0);
    constexpr uint32_t TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128
                                   : TMEM_NEED <= 256 ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "tensor memory exceeded");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(full_a + s, 4);    // one arrival per decode warp
            ptx::mbar_init(empty + s, 1);
        }
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(acc_full + b, 1);
            ptx::mbar_init(acc_empty + b, 4); // one arrival per epilogue warp
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
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
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && healthy) {
            long long it = 0;
            bool ok = true;
            for (long long u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
                const GemmUnit q = gemm_unit<EXT>(args, u, nkb);
                const int n0 = (int)(q.tile % tiles_n) * kTileN, m0 = (int)(q.tile / tiles_n) * BN;
                for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                    ok = ptx::mbar_wait(empty + s, ph ^ 1u, args.status);
                    if (!ok) break;
                    ptx::mbar_arrive_expect_tx(full_raw + s, (uint32_t)(L::RAW_BYTES + L::B_BYTES));
                    ptx::tma_load_2d(smem + L::RAW_OFF + s * L::RAW_BYTES, &tmap_w, full_raw + s, kb * (KT::RAW_ROW / 4), n0);
                    ptx::tma_load_2d(smem + L::B_OFF + s * L::B_BYTES, &tmap_x, full_raw + s, kb * KT::BK, m0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // The whole warp walks the loop - waits, stage arithmetic and descriptors are warp-uniform, which lets them live
        // in uniform registers - and one elected lane issues the MMAs and commits.
        if (healthy) {
            constexpr uint32_t idesc = (KT::C_FMT << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((128u >> 4) << 24);
            long long it = 0;
            int ti = 0;
            bool ok = true;
            for (long long u = blockIdx.x; u < ntiles && ok; u += gridDim.x, ti++) {
                const GemmUnit q = gemm_unit<EXT>(args, u, nkb);
                const int buf = ACC_BUFS == 2 ? (ti & 1) : 0;
                const uint32_t use = (uint32_t)(ACC_BUFS == 2 ? (ti >> 1) : ti);
                // the epilogue must have drained this accumulator (its previous use)
                ok = ptx::mbar_wait_warp(acc_empty + buf, (use & 1u) ^ 1u, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * ACC_COLS;
                for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                    ok = ptx::mbar_wait_warp(full_a + s, ph, args.status);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint64_t a_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::A_OFF + s * L::A_BYTES));
                    const uint64_t b_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::B_OFF + s * L::B_BYTES));
                    const uint32_t a_tmem = tmem_base + A_BASE + (uint32_t)s * A_COLS;
                    if (ptx::elect_one()) {
#pragma unroll
                        for (int k4 = 0; k4 < kRowBytes / 32; k4++) {  // 32 bytes of K per instruction (16 bf16 / 32 int8)
                            const uint32_t accum = (kb > q.kb0 || k4 > 0) ? 1u : 0u;
                            if (TA) {
                                if (KIND == KIND_BF16) ptx::umma_f16_ts(d_tmem, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, accum);
                                else ptx::umma_i8_ts(d_tmem, a_tmem + 8 * k4, b_desc + 2 * k4, idesc, accum);
                            } else {
                                if (KIND == KIND_BF16) ptx::umma_f16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, accum);
                                else ptx::umma_i8(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, accum);
                            }
                        }
                        ptx::umma_commit(empty + s);  // stage reusable once these MMAs have read it
                    }
                    __syncwarp();
                }
                if (ok && ptx::elect_one()) ptx::umma_commit(acc_full + buf);
                __syncwarp();
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- decode warps (2..5)
        // weight row inside the tile, 0..127.  With the operand in tensor memory a warp may only touch the lane quarter
        // (warp index % 4), so rows are dealt accordingly.
        const int row = (warp & 3) * 32 + lane;
        const int sw = row & 7;
        bool ok = healthy;
        long long it = 0;
        for (long long u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
            const GemmUnit q = gemm_unit<EXT>(args, u, nkb);
            for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                const int s = (int)(it % kStages);
                const uint32_t ph = (uint32_t)(it / kStages) & 1u;
                ok = ptx::mbar_wait(full_raw + s, ph, args.status);
                if (!ok) break;
                const uint8_t *raw = smem + L::RAW_OFF + s * L::RAW_BYTES + row * KT::RAW_ROW;
                uint8_t *arow = smem + L::A_OFF + s * L::A_BYTES + row * kRowBytes;
                if (TA) {
                    uint32_t cols[32];               // the row's 128 operand bytes, K ascending
                    if (KIND == KIND_BF16) {
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
                    ptx::tmem_st_x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + A_BASE + (uint32_t)s * A_COLS, cols);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(full_a + s);
                    continue;
                }
                if (KIND == KIND_BF16) {
                    const uint4 p = *reinterpret_cast<const uint4 *>(raw);
                    const uint32_t words[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
                    for (int wi = 0; wi < 4; wi++) {
                        uint32_t r[8];
                        decode_word_bf16(words[wi], r);
                        *reinterpret_cast<uint4 *>(arow + (((2 * wi) ^ sw) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
                        *reinterpret_cast<uint4 *>(arow + (((2 * wi + 1) ^ sw) << 4)) = make_uint4(r[4], r[5], r[6], r[7]);
                    }
                } else {
                    const uint4 p0 = *reinterpret_cast<const uint4 *>(raw);
                    const uint4 p1 = *reinterpret_cast<const uint4 *>(raw + 16);
                    const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                    for (int wi = 0; wi < 8; wi++) {
                        uint32_t r[4];
                        decode_word_i8(words[wi], r);
                        *reinterpret_cast<uint4 *>(arow + ((wi ^ sw) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
                    }
                }
                ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(full_a + s);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps (6..9)
        const int quarter = warp & 3;                    // TMEM lanes this warp may touch: 32*quarter .. +31
        float *stage = reinterpret_cast<float *>(smem + L::STAGE_OFF) + (warp - 6) * 512;
        bool ok = healthy;
        int ti = 0;
        for (long long u = blockIdx.x; u < ntiles && ok; u += gridDim.x, ti++) {
            const GemmUnit q = gemm_unit<EXT>(args, u, nkb);
            const long long n0 = (q.tile % tiles_n) * kTileN, m0 = (q.tile / tiles_n) * BN;
            const int buf = ACC_BUFS == 2 ? (ti & 1) : 0;
            ok = ptx::mbar_wait(acc_full + buf, (uint32_t)(ACC_BUFS == 2 ? (ti >> 1) : ti) & 1u, args.status);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const long long n = n0 + quarter * 32 + lane;
            const bool n_ok = n < args.N;
            float sc = 1.0f, bi = 0.0f;
            if (n_ok) {
                if (args.scale) sc = args.scale[n];
                if (args.bias) bi = args.bias[n];
            }
            if (KIND == KIND_BF16) sc *= 0.5f;           // operands carried +-2.0
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_COLS;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c, v);
                ptx::tmem_ld_wait();
                if (c + 16 >= BN) {                      // last chunk read: hand the accumulator back to the MMA warp
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_empty + buf);
                }
                if (EXT && args.partial) {
                    // split K: raw accumulators of this split; a warp writes 128 contiguous bytes per output row
                    uint32_t *part = reinterpret_cast<uint32_t *>(args.partial) + (long long)q.split * args.M * args.N;
                    if (n_ok) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const long long m = m0 + c + j;
                            if (m < args.M) part[m * args.N + n] = v[j];
                        }
                    }
                } else if (BC) {
                    // scaled chunk -> per-warp transposition area -> 16-byte vectors (8 channels of one row) -> the parked tile
#pragma unroll
                    for (int j = 0; j < 16; j++) stage[j * 32 + lane] = fmaf(__uint_as_float(v[j]), sc, bi);
                    __syncwarp();
                    uint8_t *outb = smem + L::OUT_OFF;
#pragma unroll
                    for (int it = 0; it < 2; it++) {
                        const int p = it * 8 + (lane >> 2), cg = (lane & 3) * 8, row = c + p;
                        const float4 lo = *reinterpret_cast<const float4 *>(stage + p * 32 + cg);
                        const float4 hi = *reinterpret_cast<const float4 *>(stage + p * 32 + cg + 4);
                        __align__(16) __nv_bfloat162 o[4] = {__floats2bfloat162_rn(lo.x, lo.y), __floats2bfloat162_rn(lo.z, lo.w),
                                                             __floats2bfloat162_rn(hi.x, hi.y), __floats2bfloat162_rn(hi.z, hi.w)};
                        const int chunk = (quarter * 4 + (lane & 3)) ^ (row & 7);
                        *reinterpret_cast<uint4 *>(outb + row * 256 + chunk * 16) = *reinterpret_cast<const uint4 *>(o);
                    }
                    __syncwarp();
                } else if (KIND == KIND_BF16 && !args.out_f32) {
                    epilogue_chunk_bf16(v, sc, bi, stage, reinterpret_cast<__nv_bfloat16 *>(args.Y), nullptr, m0 + c, args.M,
                                        args.ldy, n0 + quarter * 32, args.N, 0, lane, EXT ? &args.peers : nullptr);
                } else if (n_ok) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const long long m = m0 + c + j;
                        if (m < args.M) {
                            if (KIND == KIND_I8) reinterpret_cast<int *>(args.Y)[m * args.ldy + n] = (int)v[j];
                            else reinterpret_cast<float *>(args.Y)[m * args.ldy + n] = fmaf(__uint_as_float(v[j]), sc, bi);
                        }
                    }
                }
            }
            if (BC) {
                // the accumulator is back with the MMA warp; write the parked tile out in whole rows (256 bytes of one output
                // row per half warp), once to this GPU and once to every peer.  Host-checked: N % 8 == 0, ldy % 8 == 0 and
                // 16-byte aligned destinations, so a vector never straddles the matrix edge
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const uint8_t *outb = smem + L::OUT_OFF;
                const int col = lane & 15;
                const long long nn = n0 + col * 8;
                __nv_bfloat16 *Yl = reinterpret_cast<__nv_bfloat16 *>(args.Y);
#pragma unroll 4
                for (int r = (warp - 6) * (BN / 4) + (lane >> 4); r < (warp - 5) * (BN / 4); r += 2) {
                    const long long m = m0 + r;
                    if (m < args.M && nn < args.N) {
                        const uint4 val = *reinterpret_cast<const uint4 *>(outb + r * 256 + ((col ^ (r & 7)) << 4));
                        const long long off = m * args.ldy + nn;
                        *reinterpret_cast<uint4 *>(Yl + off) = val;
                        for (int q = 0; q < args.peers.n; q++) *reinterpret_cast<uint4 *>(args.peers.y[q] + off) = val;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");                 // the tile area is free for the next tile
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

// ---- prepack: reference layout P[K][ceil(N/16)] -> Wt[N][Kp/16] ----------------------------------------------------------

__device__ __forceinline__ uint32_t ref_code(const uint32_t *__restrict__ P, long long Q, long long K, long long n,
                                             long long k) {
    if (k >= K) return 0u;
    return (P[k * Q + (n >> 4)] >> (2 * (15 - (int)(n & 15)))) & 3u;
}

// fmt 0 = bf16-ready words, 1 = int8-ready words; row-major Wt[N][KS].  This kernel never executes
// griddepcontrol.launch_dependents: a skinny kernel launched right behind it with programmatic stream serialisation
// (which fetches Wt before its griddepcontrol.wait) therefore cannot start before every block of this grid has exited.
__global__ void __launch_bounds__(256) prepack_kernel(const uint32_t *__restrict__ P, uint32_t *__restrict__ Wt,
                                                       long long N, long long K, long long KW, long long KS,
                                                       long long rows_out, int fmt) {
    // KW: words of a row that carry weights, KS >= KW: row stride of the row-major form (padding words are zeroed)
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows_out * KS) return;
    // consecutive threads take consecutive n for one kw: their reads of P share 32-bit words and rows
    const long long n = idx % rows_out, kw = idx / rows_out;
    const long long Q = (N + 15) / 16;
    const int kind = fmt & 1;
    uint32_t word = 0;
    if (n < N && kw < KW) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const uint32_t c = ref_code(P, Q, K, n, kw * 16 + i);  // 0: zero, 1: +1, 2: -1 (3 never produced -> zero)
            if (kind == KIND_BF16) {
                const uint32_t v = (c == 1u) ? 1u : ((c == 2u) ? 3u : 0u);  // (sign, nonzero)
                const int j = i >> 1;
                const int pos = (i & 1) ? (30 - 2 * j) : (14 - 2 * j);
                word |= v << pos;
            } else {
                const uint32_t v = (c == 3u) ? 0u : c;
                const int pos = ((i >> 3) << 4) + ((i & 3) << 2) + (((i >> 2) & 1) << 1);
                word |= v << pos;
            }
        }
    }
    Wt[n * KS + kw] = word;
}

// Ends tmq_prepack's work in the stream with an ordinary kernel boundary.  The skinny kernels read Wt ahead of their
// griddepcontrol.wait; a plain launch between the writer of Wt and them guarantees the writer has completed and its
// stores are visible before any such early read can be issued.
__global__ void prepack_fence_kernel() {}

// Test helper for the bounded waits: one thread waits on an mbarrier nobody ever completes, with the given budget,
// and the kernel returns normally once the wait has given up (TMQ_ERR_TIMEOUT lands in *status).
__global__ void wait_selftest_kernel(int *status, long long budget, long long *waited_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
        const long long t0 = clock64();
        const bool ok = ptx::mbar_wait(&bar, 0u, status, budget);
        if (waited_cycles) *waited_cycles = ok ? -1 : clock64() - t0;
    }
}

// Split-K epilogue: Y = scale * (sum over the splits, in split order) + bias.  KIND 0: fp32 partial sums of operands
// carried as +-2 (the factor 0.5 is applied here), output bf16 or fp32; KIND 1: exact int32.
template <int KIND>
__global__ void __launch_bounds__(256) gemm_combine_kernel(const void *__restrict__ partial, const float *__restrict__ scale,
                                                           const float *__restrict__ bias, void *__restrict__ Y, long long M,
                                                           long long N, long long ldy, int splits, int out_f32) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * N) return;
    const long long m = i / N, n = i - m * N;
    if (KIND == KIND_I8) {
        const int *p = reinterpret_cast<const int *>(partial);
        int s = p[i];
        for (int q = 1; q < splits; q++) s += p[(long long)q * M * N + i];
        reinterpret_cast<int *>(Y)[m * ldy + n] = s;
    } else {
        const float *p = reinterpret_cast<const float *>(partial);
        float s = p[i];
        for (int q = 1; q < splits; q++) s += p[(long long)q * M * N + i];
        const float f = fmaf(s, 0.5f * (scale ? scale[n] : 1.0f), bias ? bias[n] : 0.0f);
        if (out_f32) reinterpret_cast<float *>(Y)[m * ldy + n] = f;
        else reinterpret_cast<__nv_bfloat16 *>(Y)[m * ldy + n] = __float2bfloat16_rn(f);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------------

template <int KIND, int BN, bool TA, int MODE = 0>
static int launch_gemm(const void *X, const uint32_t *Wt, const GemmArgs &a_in, cudaStream_t st) {
    using KT = KindTraits<KIND>;
    using L = SmemLayout<KIND, BN, TA, MODE == 1>;
    GemmArgs a = a_in;
    const long long KW = prepack_valid_words(a.K), KS = prepack_row_words(a.K, KIND);  // words / stride of a row
    CUtensorMap mx, mw;
    const bool okx = (KIND == KIND_BF16)
        ? make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, X, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.K * 2, KT::BK, BN,
                      CU_TENSOR_MAP_SWIZZLE_128B)
        : make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, X, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.K, KT::BK, BN,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    const bool okw = make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, Wt, (uint64_t)KW, (uint64_t)a.N, (uint64_t)KS * 4,
                                 KT::RAW_ROW / 4, kTileN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!okx || !okw) return TMQ_ERR_LAUNCH;
    const int attr_rc = ensure_dynamic_smem(ternary_gemm_kernel<KIND, BN, TA, MODE>, L::TOTAL);
    if (attr_rc != TMQ_OK) return attr_rc;
    const long long nkb = (a.K + KT::BK - 1) / KT::BK;
    if (a.splits < 1 || !a.partial || MODE != 2) a.splits = 1;
    a.kb_per_split = (int)((nkb + a.splits - 1) / a.splits);
    a.splits = (int)((nkb + a.kb_per_split - 1) / a.kb_per_split);      // no empty split
    if (a.splits == 1) a.partial = nullptr;
    const long long ntiles = ((a.N + kTileN - 1) / kTileN) * ((a.M + BN - 1) / BN) * a.splits;
    const unsigned grid = (unsigned)(ntiles < kNumSMs ? ntiles : kNumSMs);
    ternary_gemm_kernel<KIND, BN, TA, MODE><<<grid, kGemmThreads, L::TOTAL, st>>>(mx, mw, a);
    int rc = launch_status();
    if (rc != TMQ_OK || !a.partial) return rc;
    const long long total = a.M * a.N;
    gemm_combine_kernel<KIND><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.partial, a.scale, a.bias, a.Y, a.M, a.N, a.ldy,
                                                                               a.splits, a.out_f32);
    return launch_status();
}

// K splits for a problem whose output tiles do not fill the machine: as many as keep all units in ONE wave and leave
// every split at least four k-blocks.  More splits than that do not pay: on 11008 x 4096 (86 tiles) three splits in two
// waves measured 18.5 us against 18.7 us unsplit at 16 rows and twice the time at 256 rows (partial sums + combine).
// 1 = do not split.
template <int KIND>
static int gemm_splits(long long M, long long N, long long K) {
    if (M > 256) return 1;
    const long long BN = M > 128 ? 256 : M > 64 ? 128 : M > 32 ? 64 : 32;
    const long long tiles = ((N + kTileN - 1) / kTileN) * ((M + BN - 1) / BN);
    const long long nkb = (K + KindTraits<KIND>::BK - 1) / KindTraits<KIND>::BK;
    long long splits = kNumSMs / tiles;
    if (splits > nkb / 4) splits = nkb / 4;
    if (M > 128 && splits < 6) splits = 1;      // 256-row tiles: the partial sums cost more than four splits save
    return splits < 1 ? 1 : (int)splits;
}

template <int KIND, int MODE>
static int dispatch_gemm_mode(const void *X, const uint32_t *Wt, const GemmArgs &a, cudaStream_t st) {
    // bf16: weight operand in tensor memory (+3 .. +13 % measured); int8: in shared memory (the tensor-memory form
    // measured 20 % slower there)
    constexpr bool TA = (KIND == KIND_BF16);
    // short reductions (a handful of k-blocks per tile) are bound by the epilogue: 128-row tiles keep the accumulator
    // double-buffered in the tensor-memory-operand form, so the drain of one tile hides under the next
    if (a.M > 128 && !(TA && a.K <= 512)) return launch_gemm<KIND, 256, TA, MODE>(X, Wt, a, st);
    if (a.M > 64) return launch_gemm<KIND, 128, TA, MODE>(X, Wt, a, st);
    if (a.M > 32) return launch_gemm<KIND, 64, TA, MODE>(X, Wt, a, st);
    return launch_gemm<KIND, 32, TA, MODE>(X, Wt, a, st);
}

template <int KIND>
static int dispatch_gemm(const void *X, const uint32_t *Wt, const GemmArgs &a, cudaStream_t st) {
    if ((a.partial && a.splits > 1) || a.peers.n > 0) return dispatch_gemm_mode<KIND, 2>(X, Wt, a, st);
    return dispatch_gemm_mode<KIND, 0>(X, Wt, a, st);
}

static int check_gemm_common(const void *X, const uint32_t *Wt, const void *Y, long long M, long long N, long long K,
                             long long ldy, const int *status, int x_elem_bytes) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || ldy < N) return TMQ_ERR_ARG;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    if ((K * x_elem_bytes) % 16 != 0) return TMQ_ERR_UNSUPPORTED;  // TMA row pitch must be a multiple of 16 bytes
    if (!aligned(X, 16) || !aligned(Wt, 16) || !aligned(status, 4)) return TMQ_ERR_ALIGN;
    return TMQ_OK;
}

}  // namespace tmq

using namespace tmq;

extern "C" size_t tmq_prepack_row_words(int64_t K, int fmt) {
    if (K <= 0 || fmt < 0 || fmt > 1) return 0;
    return (size_t)prepack_row_words(K, fmt & 1);
}

extern "C" size_t tmq_prepack_words(int64_t N, int64_t K, int fmt) {
    if (N <= 0) return 0;
    return (size_t)N * tmq_prepack_row_words(K, fmt);
}

extern "C" int tmq_prepack(const uint32_t *P, uint32_t *Wt, int64_t N, int64_t K, int fmt, void *stream) {
    if (!P || !Wt || N <= 0 || K <= 0 || fmt < 0 || fmt > 1) return TMQ_ERR_ARG;
    if (!aligned(Wt, 16)) return TMQ_ERR_ALIGN;
    const long long KW = prepack_valid_words(K);
    const long long KS = prepack_row_words(K, fmt & 1);
    const long long total = N * KS;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    prepack_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(P, Wt, N, K, KW, KS, N, fmt);
    int rc = launch_status();
    if (rc != TMQ_OK) return rc;
    prepack_fence_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    return launch_status();
}

extern "C" int tmq_selftest_wait_timeout(long long budget_cycles, int *status, long long *waited_cycles, void *stream) {
    if (!status || budget_cycles <= 0 || budget_cycles > 4000000000ll) return TMQ_ERR_ARG;
    if (!aligned(status, 4) || !aligned(waited_cycles, 8)) return TMQ_ERR_ALIGN;
    wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, budget_cycles, waited_cycles);
    return launch_status();
}

extern "C" int tmq_ternary_gemm_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                     int64_t M, int64_t N, int64_t K, int64_t ldy, int out_f32, int *status,
                                     void *stream) {
    int rc = check_gemm_common(X, Wt, Y, M, N, K, ldy, status, 2);
    if (rc != TMQ_OK) return rc;
    if (!aligned(Y, out_f32 ? 4 : 2)) return TMQ_ERR_ALIGN;
    GemmArgs a = {scale, bias, Y, M, N, K, ldy, out_f32, status, {}, nullptr, 1, 0};
    return dispatch_gemm<KIND_BF16>(X, Wt, a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemm_bf16_bcast(const void *X, const uint32_t *Wt, const float *scale, const float *bias,
                                           void *const *Ys, int ndst, int64_t M, int64_t N, int64_t K, int64_t ldy,
                                           int *status, void *stream) {
    if (!Ys || ndst < 1 || ndst > 1 + kMaxPeers) return TMQ_ERR_ARG;
    int rc = check_gemm_common(X, Wt, Ys[0], M, N, K, ldy, status, 2);
    if (rc != TMQ_OK) return rc;
    GemmArgs a = {scale, bias, Ys[0], M, N, K, ldy, 0, status, {}, nullptr, 1, 0};
    for (int q = 0; q < ndst; q++) {
        if (!Ys[q]) return TMQ_ERR_ARG;
        if (!aligned(Ys[q], 2)) return TMQ_ERR_ALIGN;
        if (q > 0) a.peers.y[q - 1] = reinterpret_cast<__nv_bfloat16 *>(Ys[q]);
    }
    a.peers.n = ndst - 1;
    // tall problems with vector-friendly geometry: the form that parks the tile and writes whole rows under the next
    // tile's multiplication; anything else: the ordinary epilogue, which stores to every destination as it goes
    bool rows_ok = M > 128 && K > 512 && (N % 8) == 0 && (ldy % 8) == 0;
    for (int q = 0; q < ndst; q++) rows_ok = rows_ok && aligned(Ys[q], 16);
    if (rows_ok) return launch_gemm<KIND_BF16, 256, true, 1>(X, Wt, a, (cudaStream_t)stream);
    return dispatch_gemm<KIND_BF16>(X, Wt, a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemm_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K,
                                   int64_t ldy, int *status, void *stream) {
    int rc = check_gemm_common(X, Wt, Y, M, N, K, ldy, status, 1);
    if (rc != TMQ_OK) return rc;
    if (!aligned(Y, 4)) return TMQ_ERR_ALIGN;
    GemmArgs a = {nullptr, nullptr, Y, M, N, K, ldy, 0, status, {}, nullptr, 1, 0};
    return dispatch_gemm<KIND_I8>(X, Wt, a, (cudaStream_t)stream);
}

extern "C" size_t tmq_ternary_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int int8_activations) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int splits = int8_activations ? gemm_splits<KIND_I8>(M, N, K) : gemm_splits<KIND_BF16>(M, N, K);
    return splits > 1 ? (size_t)splits * (size_t)M * (size_t)N * 4 : 0;
}

extern "C" int tmq_ternary_gemm_bf16_splitk(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                            int64_t M, int64_t N, int64_t K, int64_t ldy, int out_f32, void *workspace,
                                            size_t workspace_bytes, int *status, void *stream) {
    int rc = check_gemm_common(X, Wt, Y, M, N, K, ldy, status, 2);
    if (rc != TMQ_OK) return rc;
    if (!aligned(Y, out_f32 ? 4 : 2) || !aligned(workspace, 16)) return TMQ_ERR_ALIGN;
    GemmArgs a = {scale, bias, Y, M, N, K, ldy, out_f32, status, {}, nullptr, 1, 0};
    const size_t need = tmq_ternary_gemm_workspace_bytes(M, N, K, 0);
    if (need > 0 && workspace && workspace_bytes >= need) {
        a.partial = workspace;
        a.splits = gemm_splits<KIND_BF16>(M, N, K);
    }
    return dispatch_gemm<KIND_BF16>(X, Wt, a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemm_i8_splitk(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K,
                                          int64_t ldy, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    int rc = check_gemm_common(X, Wt, Y, M, N, K, ldy, status, 1);
    if (rc != TMQ_OK) return rc;
    if (!aligned(Y, 4) || !aligned(workspace, 16)) return TMQ_ERR_ALIGN;
    GemmArgs a = {nullptr, nullptr, Y, M, N, K, ldy, 0, status, {}, nullptr, 1, 0};
    const size_t need = tmq_ternary_gemm_workspace_bytes(M, N, K, 1);
    if (need > 0 && workspace && workspace_bytes >= need) {
        a.partial = workspace;
        a.splits = gemm_splits<KIND_I8>(M, N, K);
    }
    return dispatch_gemm<KIND_I8>(X, Wt, a, (cudaStream_t)stream);
}
