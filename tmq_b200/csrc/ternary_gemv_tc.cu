// Skinny ternary GEMM (1..32 activation rows) on tcgen05: the decode-like shapes, made to stream.
//   Y[m][n] = scale[n] * sum_k X[m][k] * T[n][k] + bias[n]
//
// Why a second tensor-core kernel: the tiled GEMM (ternary_gemm.cu) keeps one CTA per 128 output channels and walks K
// through a 4-stage pipeline, which for M <= 32 leaves most SMs idle and every CTA latency-bound; the warp-level MMA
// kernel (ternary_gemv.cu) is limited by the legacy mma.sync rate.  Here the same decode-in-shared-memory scheme is
// rearranged as a persistent stream-K kernel:
//   * the work is the list of (128-channel tile, k-block) units in tile-major order; each of the 2 x 148 resident CTAs
//     takes one contiguous, equally long range of it, so every SM streams the same number of weight bytes and the TMA
//     pipeline never drains between tiles;
//   * raw packed tiles (2-4 KB) and the matching activation tiles ride an 8-deep TMA ring, decoded operand tiles a
//     3-deep ring; 8 decode warps, one MMA thread (weights are the 128-row A operand, N = 16 or 32 activation rows),
//     two TMEM accumulators so that 4 epilogue warps drain one tile segment while the next one accumulates;
//   * a tile whose k range is split over several CTAs gets its partials written to workspace slots ordered by CTA;
//     the last contributor (ticket counter) adds them in slot order and applies scale / bias: deterministic, no second
//     kernel, counters re-armed for the next call.
// Every mbarrier wait is bounded (TMQ_ERR_TIMEOUT through the status word).
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "decode.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace tmq {

constexpr int kTcThreads = 448;  // warp 0: TMA, warp 1: MMA + TMEM, warps 2-9: decode, warps 10-13: epilogue
constexpr int kTcRing = 8;       // raw-weights + activation tiles in flight
constexpr int kTcARing = 3;     // decoded operand tiles
constexpr int kTcTile = 128;
constexpr size_t kTcCounterBytes = 4096 * 4;  // ticket counters for up to 4096 channel tiles

struct TcArgs {
    const float *scale, *bias;
    void *Y;
    long long M, N, K, ldy;
    int out_f32;
    int nkb;             // k-blocks per tile
    long long units;     // tiles * nkb
    int max_contrib;     // workspace slots per tile
    unsigned *counters;  // [tiles]
    float *partials;     // [tiles][max_contrib][BN][128]
    int *status;
};

template <int KIND, int BN>
struct TcSmem {
    static constexpr int BK = KIND == 0 ? 64 : 128;
    static constexpr int RAW_ROW = KIND == 0 ? 16 : 32;
    static constexpr int A_BYTES = kTcTile * 128;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int RAW_BYTES = kTcTile * RAW_ROW;
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = A_OFF + kTcARing * A_BYTES;
    static constexpr int RAW_OFF = B_OFF + kTcRing * B_BYTES;
    static constexpr int BAR_OFF = RAW_OFF + kTcRing * RAW_BYTES;
    static constexpr int TOTAL = BAR_OFF + 512 + 1024;
};

// first unit of CTA c when `units` units are dealt to `g` CTAs in contiguous, near-equal ranges
__device__ __forceinline__ long long tc_range_start(long long c, long long units, long long g) { return c * units / g; }
// CTA that owns unit u under that split
__device__ __forceinline__ long long tc_owner(long long u, long long units, long long g) {
    return ((u + 1) * g + units - 1) / units - 1;
}

template <int KIND, int BN>
__global__ void __launch_bounds__(kTcThreads, 2)
ternary_gemv_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint32_t *__restrict__ wt_tiled, TcArgs args) {
    using L = TcSmem<KIND, BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_raw = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *empty_raw = full_raw + kTcRing;
    uint64_t *a_full = empty_raw + kTcRing;
    uint64_t *a_empty = a_full + kTcARing;
    uint64_t *acc_full = a_empty + kTcARing;   // [2]
    uint64_t *acc_empty = acc_full + 2;        // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    int *is_last = reinterpret_cast<int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long G = gridDim.x;
    const long long u0 = tc_range_start(blockIdx.x, args.units, G), u1 = tc_range_start(blockIdx.x + 1, args.units, G);
    const int nkb = args.nkb;
    constexpr uint32_t TMEM_COLS = 64;  // two accumulators of BN <= 32 columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcRing; s++) {
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(empty_raw + s, 1);
        }
        for (int s = 0; s < kTcARing; s++) {
            ptx::mbar_init(a_full + s, 8);     // one arrival per decode warp
            ptx::mbar_init(a_empty + s, 1);
        }
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(acc_full + s, 1);
            ptx::mbar_init(acc_empty + s, 4);  // one arrival per epilogue warp
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
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
            for (long long u = u0; u < u1; u++, it++) {
                const int s = (int)(it % kTcRing);
                const uint32_t ph = (uint32_t)(it / kTcRing) & 1u;
                const int tile = (int)(u / nkb), kb = (int)(u % nkb);
                if (!ptx::mbar_wait(empty_raw + s, ph ^ 1u, args.status)) break;
                ptx::mbar_arrive_expect_tx(full_raw + s, (uint32_t)(L::RAW_BYTES + L::B_BYTES));
                // tile-contiguous weights: the raw tile of this unit is one contiguous run -> one bulk copy
                ptx::bulk_load(smem + L::RAW_OFF + s * L::RAW_BYTES,
                               wt_tiled + ((size_t)tile * nkb + kb) * (L::RAW_BYTES / 4), L::RAW_BYTES, full_raw + s);
                ptx::tma_load_2d(smem + L::B_OFF + s * L::B_BYTES, &tmap_x, full_raw + s, kb * L::BK, 0);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && healthy) {
            constexpr uint32_t idesc = ((KIND == 0 ? 1u : 2u) << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((128u >> 4) << 24);
            long long it = 0;
            int seg = 0;
            bool good = true;
            for (long long u = u0; u < u1 && good; u++, it++) {
                const int s = (int)(it % kTcRing), a = (int)(it % kTcARing);
                const uint32_t aph = (uint32_t)(it / kTcARing) & 1u;
                const int kb = (int)(u % nkb);
                const bool seg_first = (u == u0) || kb == 0;
                const bool seg_last = (u + 1 == u1) || kb == nkb - 1;
                const int buf = seg & 1;
                if (seg_first) {  // the epilogue must have drained this accumulator (two segments ago)
                    good = ptx::mbar_wait(acc_empty + buf, ((uint32_t)(seg >> 1) & 1u) ^ 1u, args.status);
                    if (!good) break;
                    ptx::tc_fence_after_sync();
                }
                good = ptx::mbar_wait(a_full + a, aph, args.status);
                if (!good) break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 32);
                const uint64_t a_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::A_OFF + a * L::A_BYTES));
                const uint64_t b_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::B_OFF + s * L::B_BYTES));
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++) {
                    const uint32_t accum = (!seg_first || k4 > 0) ? 1u : 0u;
                    if (KIND == 0) ptx::umma_f16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, accum);
                    else ptx::umma_i8(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, accum);
                }
                ptx::umma_commit(a_empty + a);
                ptx::umma_commit(empty_raw + s);
                if (seg_last) {
                    ptx::umma_commit(acc_full + buf);
                    seg++;
                }
            }
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------------- decode: 256 threads, half a row each
        const int t = threadIdx.x - 64;
        const int row = t & 127, half = t >> 7;
        const int sw = row & 7;
        bool ok = healthy;
        long long it = 0;
        for (long long u = u0; u < u1 && ok; u++, it++) {
            const int s = (int)(it % kTcRing), a = (int)(it % kTcARing);
            const uint32_t ph = (uint32_t)(it / kTcRing) & 1u, aph = (uint32_t)(it / kTcARing) & 1u;
            ok = ptx::mbar_wait(full_raw + s, ph, args.status);
            if (ok) ok = ptx::mbar_wait(a_empty + a, aph ^ 1u, args.status);
            if (!ok) break;
            const uint8_t *raw = smem + L::RAW_OFF + s * L::RAW_BYTES + row * L::RAW_ROW;
            uint8_t *arow = smem + L::A_OFF + a * L::A_BYTES + row * 128;
            if (KIND == 0) {
                const uint2 p = *reinterpret_cast<const uint2 *>(raw + 8 * half);  // words 2h, 2h+1
                const uint32_t words[2] = {p.x, p.y};
#pragma unroll
                for (int wi = 0; wi < 2; wi++) {
                    uint32_t r[8];
                    decode_word_bf16(words[wi], r);
                    const int c = 4 * half + 2 * wi;
                    *reinterpret_cast<uint4 *>(arow + ((c ^ sw) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
                    *reinterpret_cast<uint4 *>(arow + (((c + 1) ^ sw) << 4)) = make_uint4(r[4], r[5], r[6], r[7]);
                }
            } else {
                const uint4 p = *reinterpret_cast<const uint4 *>(raw + 16 * half);  // words 4h .. 4h+3
                const uint32_t words[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
                for (int wi = 0; wi < 4; wi++) {
                    uint32_t r[4];
                    decode_word_i8(words[wi], r);
                    const int c = 4 * half + wi;
                    *reinterpret_cast<uint4 *>(arow + ((c ^ sw) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(a_full + a);  // 8 arrivals instead of 256 on one barrier word
        }
    } else {
        // ---------------------------------------------------------------- epilogue: 4 warps, one tile segment at a time
        const int quarter = warp & 3;                 // TMEM lanes this warp may touch
        const int erow = quarter * 32 + lane;
        const int et = threadIdx.x - 320;             // 0..127
        bool ok = healthy;
        int seg = 0;
        long long u = u0;
        while (u < u1 && ok) {
            const int tile = (int)(u / nkb), kb_begin = (int)(u % nkb);
            const long long tile_end = (long long)(tile + 1) * nkb;
            const long long seg_end = tile_end < u1 ? tile_end : u1;
            const bool whole = (kb_begin == 0) && (seg_end == tile_end);
            const int buf = seg & 1;
            ok = ptx::mbar_wait(acc_full + buf, (uint32_t)(seg >> 1) & 1u, args.status);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            uint32_t v[BN];
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 32);
#pragma unroll
            for (int c = 0; c < BN; c += 16) {
                uint32_t part[16];
                ptx::tmem_ld_x16(lane_addr + (uint32_t)c, part);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++) v[c + j] = part[j];
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty + buf);  // accumulator free for the segment after next
            bool finalize = true;
            if (!whole) {
                // contributors of this tile are consecutive CTAs; this CTA's slot is its rank among them
                const long long c_first = tc_owner((long long)tile * nkb, args.units, G);
                const long long c_last = tc_owner(tile_end - 1, args.units, G);
                const int slot = (int)(blockIdx.x - c_first), ncontrib = (int)(c_last - c_first + 1);
                float *dst = args.partials + ((size_t)tile * args.max_contrib + slot) * (BN * 128) + erow;
#pragma unroll
                for (int j = 0; j < BN; j++)
                    if (j < args.M) dst[j * 128] = __uint_as_float(v[j]);
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) {
                    const unsigned ticket = atomicAdd(args.counters + tile, 1u);
                    const int last = (ticket == (unsigned)ncontrib - 1u);
                    if (last) args.counters[tile] = 0u;  // re-armed for the next call
                    *is_last = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finalize = (*is_last != 0);
                if (finalize) {
                    __threadfence();
                    const float *src = args.partials + (size_t)tile * args.max_contrib * (BN * 128) + erow;
#pragma unroll
                    for (int j = 0; j < BN; j++) {
                        if (j < args.M) {
                            if (KIND == 0) {
                                float sum = 0.f;
                                for (int c = 0; c < ncontrib; c++) sum += __ldcg(src + ((size_t)c * BN + j) * 128);
                                v[j] = __float_as_uint(sum);
                            } else {
                                int sum = 0;
                                for (int c = 0; c < ncontrib; c++) sum += __float_as_int(__ldcg(src + ((size_t)c * BN + j) * 128));
                                v[j] = (uint32_t)sum;
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");  // is_last is reused by the next segment
            }
            const long long n = (long long)tile * kTcTile + erow;
            if (finalize && n < args.N) {
                float sc = 1.0f, bi = 0.0f;
                if (KIND == 0) {
                    if (args.scale) sc = args.scale[n];
                    if (args.bias) bi = args.bias[n];
                    sc *= 0.5f;  // operands carried +-2.0
                }
#pragma unroll
                for (int j = 0; j < BN; j++) {
                    if (j < args.M) {
                        if (KIND == 1) {
                            reinterpret_cast<int *>(args.Y)[(long long)j * args.ldy + n] = (int)v[j];
                        } else {
                            const float f = fmaf(__uint_as_float(v[j]), sc, bi);
                            if (args.out_f32) reinterpret_cast<float *>(args.Y)[(long long)j * args.ldy + n] = f;
                            else reinterpret_cast<__nv_bfloat16 *>(args.Y)[(long long)j * args.ldy + n] = __float2bfloat16_rn(f);
                        }
                    }
                }
            }
            u = seg_end;
            seg++;
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host ---------------------------------------------------------------------------------------------------------------

struct TcPlan {
    int bn, bk, nkb, max_contrib;
    long long tiles, units, grid;
};

static TcPlan tc_plan(long long M, long long N, long long K, int kind) {
    TcPlan p;
    p.bn = M <= 16 ? 16 : 32;
    p.bk = kind == 0 ? 64 : 128;
    p.nkb = (int)((K + p.bk - 1) / p.bk);
    p.tiles = (N + kTcTile - 1) / kTcTile;
    p.units = p.tiles * p.nkb;
    p.grid = 2LL * kNumSMs;                    // two resident CTAs per SM
    if (p.grid > p.units) p.grid = p.units;
    const long long per_cta = p.units / p.grid;  // every CTA gets per_cta or per_cta + 1 units
    p.max_contrib = (int)((p.nkb + per_cta - 1) / per_cta) + 1;
    return p;
}

template <int KIND, int BN>
static int launch_tc(const void *X, const uint32_t *Wt, TcArgs a, const TcPlan &p, cudaStream_t st) {
    using L = TcSmem<KIND, BN>;
    CUtensorMap mx;
    const bool okx = (KIND == 0)
        ? make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, X, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.K * 2, L::BK, BN,
                      CU_TENSOR_MAP_SWIZZLE_128B)
        : make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, X, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.K, L::BK, BN,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (!okx) return TMQ_ERR_LAUNCH;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ternary_gemv_tc_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    if (attr_err != cudaSuccess) return cuda_status(attr_err);
    ternary_gemv_tc_kernel<KIND, BN><<<(unsigned)p.grid, kTcThreads, L::TOTAL, st>>>(mx, Wt, a);
    return launch_status();
}

template <int KIND>
static int run_tc(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, long long M, long long N,
                  long long K, long long ldy, int out_f32, void *workspace, size_t workspace_bytes, int *status,
                  cudaStream_t st) {
    if (!X || !Wt || !Y || !status || !workspace) return TMQ_ERR_ARG;
    if (M <= 0 || M > 32 || N <= 0 || K <= 0 || ldy < N) return TMQ_ERR_ARG;
    if (N > 0x7FFFFFFF || K > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    if ((K * (KIND == 0 ? 2 : 1)) % 16 != 0) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 16) || !aligned(Wt, 16) || !aligned(workspace, 256) || !aligned(status, 4)) return TMQ_ERR_ALIGN;
    const TcPlan p = tc_plan(M, N, K, KIND);
    if (p.tiles > 4096) return TMQ_ERR_UNSUPPORTED;
    const size_t need = kTcCounterBytes + (size_t)p.tiles * p.max_contrib * p.bn * 128 * sizeof(float);
    if (workspace_bytes < need) return TMQ_ERR_SCRATCH;
    TcArgs a = {scale, bias, Y, M, N, K, ldy, out_f32, p.nkb, p.units, p.max_contrib,
                reinterpret_cast<unsigned *>(workspace),
                reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + kTcCounterBytes), status};
    return p.bn == 16 ? launch_tc<KIND, 16>(X, Wt, a, p, st) : launch_tc<KIND, 32>(X, Wt, a, p, st);
}

}  // namespace tmq

using namespace tmq;

extern "C" size_t tmq_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const TcPlan a = tc_plan(M, N, K, 0), b = tc_plan(M, N, K, 1);
    const size_t pa = (size_t)a.tiles * a.max_contrib * a.bn * 128 * sizeof(float);
    const size_t pb = (size_t)b.tiles * b.max_contrib * b.bn * 128 * sizeof(float);
    return kTcCounterBytes + (pa > pb ? pa : pb);
}

extern "C" int tmq_ternary_gemv_tc_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                        int64_t M, int64_t N, int64_t K, int64_t ldy, int out_f32, void *workspace,
                                        size_t workspace_bytes, int *status, void *stream) {
    return run_tc<0>(X, Wt, scale, bias, Y, M, N, K, ldy, out_f32, workspace, workspace_bytes, status, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemv_tc_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K,
                                      int64_t ldy, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    return run_tc<1>(X, Wt, nullptr, nullptr, Y, M, N, K, ldy, 0, workspace, workspace_bytes, status, (cudaStream_t)stream);
}
