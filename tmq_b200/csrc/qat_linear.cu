// Forward of a quantisation-aware-training Linear layer with the soft staircase fused into the weight-operand load:
//   Y[m][n] = sum_k X[m][k] * S(W[n][k]) + bias[n]
// X bf16 [M][K], W the latent fp32 weights [N][K], S the transfer function of the current hardness, Y fp32.
//
// Replaces, for bf16 activations, the two passes of the reference's training forward (tmq/tmq.py:637-659:
// SoftStep.apply over the whole weight tensor, then F.linear on the result): the staircase values never exist in
// global memory.  Built like the ternary tensor-core GEMM (ternary_gemm.cu) with the operand producer swapped:
//
//   * warp 0 streams, per 64-wide k-block, the fp32 weight tile (128 rows, two 128-byte-swizzled boxes of 32 floats)
//     and the bf16 activation tile (BN rows, 128-byte swizzle) into a 3-stage ring with TMA;
//   * sixteen producer warps evaluate S (bit-identical to the elementwise kernel, softstep_math.cuh, two weights per packed fp32 instruction) on the weight
//     tile, split each value into two bf16 terms hi = bf16(S), lo = bf16(S - hi) (S is then carried to ~2^-17
//     relative) and store both terms as A operands in tensor memory (tcgen05.st);
//   * one elected lane of warp 1 issues, per 16 k, MMA(A_hi, B) and MMA(A_lo, B) into the same fp32 accumulator
//     (tcgen05.mma kind::f16, A from tensor memory, B from shared memory);
//   * four epilogue warps drain the accumulator, add the bias and store fp32 rows.
//
// The kernel is bound by the producers (about 30 fp32 instructions per weight, every 128 x 64 weight tile evaluated
// once per BN activation rows): it pays when M is at most a few hundred rows, where it saves writing and re-reading
// S(W); for tall activations evaluating S once with the elementwise kernel and running a dense GEMM is cheaper.
// Every mbarrier wait is bounded and reports through the status word, as in the ternary GEMM.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "softstep_math.cuh"
#include "tma_host.cuh"

namespace tmq {

namespace {

constexpr int kQatProducers = 16;      // producer warps: four per tensor-memory lane quarter, 16 floats of the k-block each
constexpr int kQatThreads = (2 + kQatProducers + 4) * 32;   // warp 0: TMA, warp 1: MMA, then producers, then 4 epilogue warps
constexpr int kQatStages = 3;
constexpr int kQatRows = 128;          // weight rows (output channels) per tile = UMMA M
constexpr int kQatBK = 64;             // k per block
constexpr int kQatWBytes = kQatRows * kQatBK * 4;   // 32 KB: two boxes of 128 rows x 128 bytes

struct QatArgs {
    const float *bias;   // [N] or null
    float *Y;
    long long M, N, K, ldy;
    Hardness s;
    int *status;
    float *partial;      // [splits][M][N] partial sums when K is split over several CTAs, else null
    int splits;          // CTAs sharing one output tile, each with a contiguous range of k-blocks
    int kb_per_split;
    float one, nzero;    // 1.0f and -0.0f, passed in so the packed FMAs keep operands the assembler cannot fold
};

// Work unit u = (output tile, K split): the k-blocks [kb0, kb1) of tile u / splits.
struct QatUnit {
    long long tile;
    int split, kb0, kb1;
};
__device__ __forceinline__ QatUnit qat_unit(const QatArgs &a, long long u, int nkb) {
    QatUnit q;
    q.tile = u / a.splits;
    q.split = (int)(u - q.tile * a.splits);
    q.kb0 = q.split * a.kb_per_split;
    q.kb1 = q.kb0 + a.kb_per_split < nkb ? q.kb0 + a.kb_per_split : nkb;
    return q;
}

template <int BN>
struct QatSmem {
    static constexpr int X_BYTES = BN * 128;
    static constexpr int W_OFF = 0;
    static constexpr int X_OFF = W_OFF + kQatStages * kQatWBytes;
    static constexpr int BAR_OFF = X_OFF + kQatStages * X_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;   // + barriers + alignment slack
};

// 32 lanes x 8 consecutive 32-bit columns: thread i of the warp writes lane (base_lane + i)
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kQatThreads, 1)
qat_linear_fwd_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, QatArgs args) {
    using L = QatSmem<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_raw = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *full_a = full_raw + kQatStages;
    uint64_t *empty = full_a + kQatStages;
    uint64_t *acc_full = empty + kQatStages;   // [2]
    uint64_t *acc_empty = acc_full + 2;        // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((args.K + kQatBK - 1) / kQatBK);
    const long long tiles_n = (args.N + kQatRows - 1) / kQatRows;
    const long long tiles_m = (args.M + BN - 1) / BN;
    const long long nunits = tiles_n * tiles_m * args.splits;
    constexpr int ACC_BUFS = BN > 128 ? 1 : 2;
    constexpr uint32_t A_COLS = 64;                              // per stage: 32 columns of hi terms, 32 of lo terms
    constexpr uint32_t A_BASE = ACC_BUFS * BN;
    constexpr uint32_t TMEM_NEED = A_BASE + kQatStages * A_COLS;
    constexpr uint32_t TMEM_COLS = TMEM_NEED <= 256 ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "tensor memory exceeded");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kQatStages; s++) {
            ptx::mbar_init(full_raw + s, 1);
            ptx::mbar_init(full_a + s, kQatProducers);    // one arrival per producer warp
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
            for (long long u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
                const QatUnit q = qat_unit(args, u, nkb);
                const int n0 = (int)(q.tile % tiles_n) * kQatRows, m0 = (int)(q.tile / tiles_n) * BN;
                for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                    const int s = (int)(it % kQatStages);
                    const uint32_t ph = (uint32_t)(it / kQatStages) & 1u;
                    ok = ptx::mbar_wait(empty + s, ph ^ 1u, args.status);
                    if (!ok) break;
                    ptx::mbar_arrive_expect_tx(full_raw + s, (uint32_t)(kQatWBytes + L::X_BYTES));
                    uint8_t *w = smem + L::W_OFF + s * kQatWBytes;
                    ptx::tma_load_2d(w, &tmap_w, full_raw + s, kb * kQatBK, n0);                       // k 0..31 of the block
                    ptx::tma_load_2d(w + kQatWBytes / 2, &tmap_w, full_raw + s, kb * kQatBK + 32, n0);  // k 32..63
                    ptx::tma_load_2d(smem + L::X_OFF + s * L::X_BYTES, &tmap_x, full_raw + s, kb * kQatBK, m0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (whole warp walks, one lane issues)
        if (healthy) {
            // f32 accumulator, bf16 x bf16, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((128u >> 4) << 24);
            long long it = 0;
            int ti = 0;
            bool ok = true;
            for (long long u = blockIdx.x; u < nunits && ok; u += gridDim.x, ti++) {
                const QatUnit q = qat_unit(args, u, nkb);
                const int buf = ACC_BUFS == 2 ? (ti & 1) : 0;
                const uint32_t use = (uint32_t)(ACC_BUFS == 2 ? (ti >> 1) : ti);
                ok = ptx::mbar_wait_warp(acc_empty + buf, (use & 1u) ^ 1u, args.status);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                    const int s = (int)(it % kQatStages);
                    const uint32_t ph = (uint32_t)(it / kQatStages) & 1u;
                    ok = ptx::mbar_wait_warp(full_a + s, ph, args.status);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint64_t b_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem + L::X_OFF + s * L::X_BYTES));
                    const uint32_t a_hi = tmem_base + A_BASE + (uint32_t)s * A_COLS, a_lo = a_hi + 32;
                    if (ptx::elect_one()) {
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {           // 16 k per instruction
                            ptx::umma_f16_ts(d_tmem, a_lo + 8 * k4, b_desc + 2 * k4, idesc, (kb > q.kb0 || k4 > 0) ? 1u : 0u);
                            ptx::umma_f16_ts(d_tmem, a_hi + 8 * k4, b_desc + 2 * k4, idesc, 1u);
                        }
                        ptx::umma_commit(empty + s);
                    }
                    __syncwarp();
                }
                if (ok && ptx::elect_one()) ptx::umma_commit(acc_full + buf);
                __syncwarp();
            }
        }
    } else if (warp < 2 + kQatProducers) {
        // ---------------------------------------------------------------- producers: S(W) -> bf16 hi / lo -> TMEM
        // A warp may only touch the tensor-memory lane quarter (warp index % 4); the four warps of a quarter take 16
        // floats of the k-block each (many warps: the staircase is a long dependent chain per element, and the SM hides
        // its latency with warps, not with registers).
        const int quarter = warp & 3, part = (warp - 2) >> 2;        // part 0..3: floats 16 part .. 16 part + 15
        const int row = quarter * 32 + lane;
        const int sw = row & 7;
        const Hardness hs = args.s;
        bool ok = healthy;
        long long it = 0;
        for (long long u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
            const QatUnit q = qat_unit(args, u, nkb);
            for (int kb = q.kb0; kb < q.kb1; kb++, it++) {
                const int s = (int)(it % kQatStages);
                const uint32_t ph = (uint32_t)(it / kQatStages) & 1u;
                ok = ptx::mbar_wait(full_raw + s, ph, args.status);
                if (!ok) break;
                const uint8_t *wrow = smem + L::W_OFF + s * kQatWBytes + (part >> 1) * (kQatWBytes / 2) + row * 128;
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int c = 0; c < 4; c++) {        // 16-byte chunk cc of the 128-byte row sits at position cc ^ (row % 8)
                    const int cc = (part & 1) * 4 + c;
                    const float4 v = *reinterpret_cast<const float4 *>(wrow + ((cc ^ sw) << 4));
                    const float2 f[2] = {softstep_forward2<true>(make_float2(v.x, v.y), hs, args.one, args.nzero),
                                         softstep_forward2<true>(make_float2(v.z, v.w), hs, args.one, args.nzero)};
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[e].x, f[e].y);
                        const __nv_bfloat162 l2 = __floats2bfloat162_rn(f[e].x - __low2float(h2), f[e].y - __high2float(h2));
                        hi[2 * c + e] = *reinterpret_cast<const uint32_t *>(&h2);
                        lo[2 * c + e] = *reinterpret_cast<const uint32_t *>(&l2);
                    }
                }
                const uint32_t a_hi = tmem_base + ((uint32_t)(quarter * 32) << 16) + A_BASE + (uint32_t)s * A_COLS + 8 * part;
                tmem_st_x8(a_hi, hi);
                tmem_st_x8(a_hi + 32, lo);
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(full_a + s);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps (the last four)
        const int quarter = warp & 3;                    // TMEM lanes this warp may touch: 32*quarter .. +31
        bool ok = healthy;
        int ti = 0;
        for (long long u = blockIdx.x; u < nunits && ok; u += gridDim.x, ti++) {
            const QatUnit q = qat_unit(args, u, nkb);
            const long long n0 = (q.tile % tiles_n) * kQatRows, m0 = (q.tile / tiles_n) * BN;
            const int buf = ACC_BUFS == 2 ? (ti & 1) : 0;
            ok = ptx::mbar_wait(acc_full + buf, (uint32_t)(ACC_BUFS == 2 ? (ti >> 1) : ti) & 1u, args.status);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const long long n = n0 + quarter * 32 + lane;
            const bool n_ok = n < args.N;
            const float bi = (n_ok && args.bias && !args.partial) ? args.bias[n] : 0.0f;   // split sums get it when combined
            float *out = args.partial ? args.partial + (long long)q.split * args.M * args.N : args.Y;
            const long long ld = args.partial ? args.N : args.ldy;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * BN;
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
                if (n_ok) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const long long m = m0 + c + j;
                        if (m < args.M) out[m * ld + n] = __uint_as_float(v[j]) + bi;   // a warp writes 128 contiguous bytes
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

// Y = bias + sum over the K splits, in split order: deterministic
__global__ void __launch_bounds__(256) qat_combine_kernel(const float *__restrict__ partial, const float *__restrict__ bias,
                                                          float *__restrict__ Y, long long M, long long N, long long ldy,
                                                          int splits) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * N) return;
    const long long m = i / N, n = i - m * N;
    float s = partial[i];
    for (int q = 1; q < splits; q++) s += partial[(long long)q * M * N + i];
    Y[m * ldy + n] = s + (bias ? bias[n] : 0.0f);
}

// K is split over several CTAs when there are fewer output tiles than SMs (the producers, not the tensor cores, bound
// the kernel, so idle SMs are the first thing to avoid): as many splits as keep every unit in one wave and leave each
// at least four k-blocks.
int qat_splits(long long M, long long N, long long K) {
    const long long BN = M > 128 ? 256 : 128;
    const long long tiles = ((N + kQatRows - 1) / kQatRows) * ((M + BN - 1) / BN);
    const long long nkb = (K + kQatBK - 1) / kQatBK;
    long long splits = kNumSMs / tiles;
    if (splits > nkb / 4) splits = nkb / 4;
    return splits < 1 ? 1 : (int)splits;
}

template <int BN>
int launch_qat(const void *X, const float *W, QatArgs a, cudaStream_t st) {
    using L = QatSmem<BN>;
    CUtensorMap mx, mw;
    const bool okx = make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, X, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.K * 2,
                                 kQatBK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    const bool okw = make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, W, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K * 4,
                                 32, kQatRows, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!okx || !okw) return TMQ_ERR_LAUNCH;
    const int rc = ensure_dynamic_smem(qat_linear_fwd_kernel<BN>, L::TOTAL);
    if (rc != TMQ_OK) return rc;
    const long long nkb = (a.K + kQatBK - 1) / kQatBK;
    a.kb_per_split = (int)((nkb + a.splits - 1) / a.splits);
    a.splits = (int)((nkb + a.kb_per_split - 1) / a.kb_per_split);       // no empty split
    if (a.splits == 1) a.partial = nullptr;
    const long long nunits = ((a.N + kQatRows - 1) / kQatRows) * ((a.M + BN - 1) / BN) * a.splits;
    const unsigned grid = (unsigned)(nunits < kNumSMs ? nunits : kNumSMs);
    qat_linear_fwd_kernel<BN><<<grid, kQatThreads, L::TOTAL, st>>>(mx, mw, a);
    int lrc = cuda_status(cudaGetLastError());
    if (lrc != TMQ_OK || !a.partial) return lrc;
    const long long total = a.M * a.N;
    qat_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.partial, a.bias, a.Y, a.M, a.N, a.ldy, a.splits);
    return cuda_status(cudaGetLastError());
}

}  // namespace

}  // namespace tmq

using namespace tmq;

extern "C" size_t tmq_qat_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int splits = qat_splits(M, N, K);
    return splits > 1 ? (size_t)splits * (size_t)M * (size_t)N * sizeof(float) : 0;
}

extern "C" int tmq_qat_linear_fwd_bf16(const void *X, const float *W, const float *bias, float *Y, int64_t M, int64_t N,
                                       int64_t K, int64_t ldy, double hardness, void *workspace, size_t workspace_bytes,
                                       int *status, void *stream) {
    if (!X || !W || !Y || !status) return TMQ_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || ldy < N) return TMQ_ERR_ARG;
    if (!(hardness >= 1e-3 && hardness <= 1e3)) return TMQ_ERR_ARG;       // also rejects NaN
    if (K % 8 != 0) return TMQ_ERR_UNSUPPORTED;                           // 16-byte row pitch of both operands
    if (!aligned(X, 16) || !aligned(W, 16) || !aligned(Y, 4) || !aligned(status, 4) || !aligned(workspace, 16))
        return TMQ_ERR_ALIGN;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    QatArgs a = {bias, Y, M, N, K, ldy, make_hardness(hardness), status, nullptr, 1, 0, 1.0f, -0.0f};
    const size_t need = tmq_qat_linear_workspace_bytes(M, N, K);
    if (need > 0 && workspace && workspace_bytes >= need) {               // without a workspace: one CTA per output tile
        a.partial = reinterpret_cast<float *>(workspace);
        a.splits = qat_splits(M, N, K);
    }
    // The quotient by the constant D uses the reciprocal sequence, as the elementwise forward does for every admissible
    // hardness (its operand is 0 or of magnitude >= 2^-60: no underflow).
    cudaStream_t st = (cudaStream_t)stream;
    return M > 128 ? launch_qat<256>(X, W, a, st) : launch_qat<128>(X, W, a, st);
}
