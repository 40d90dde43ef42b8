// Skinny ternary GEMV / GEMM (M <= 8 activation rows per pass) from 2-bit packed weights: the decode-like path.
//   Y[m][n] = scale[n] * sum_k X[m][k] * T[n][k] + bias[n]
//
// Replaces the reference's batch-1 kernel (tmq/tmq_cuda.cu:242-286, launcher :563-603), which reads the packed words
// with a stride of N/16 words between threads, multiplies by a constant-memory LUT and finishes with shared atomics.
// Here the packed weights are read exactly once and HBM is the resource that should matter.  Two forms:
//
//   * resident (default whenever one SM's share of the rows fits half its shared memory; see "resident variant"
//     below): a CTA bulk-copies its rows into shared memory before it waits for its predecessor in the stream;
//   * streaming (fallback): one small CTA (4 warps) per group of 16 output channels or a 16-warp CTA per 5 groups,
//     weights loaded with 128-bit loads straight into registers, again before griddepcontrol.wait.
//
// Common to both:
//   * consecutive launches are chained with programmatic dependent launch: weights depend on nothing, so they are
//     requested while the previous launch is still computing; activations and outputs are only touched after
//     griddepcontrol.wait, i.e. after the previous kernel in the stream has completed.
//   * arithmetic: a 2-bit code costs about one integer instruction to decode, which already fills half the issue
//     slots at HBM speed; an fp32 add/sub per weight on top (the CUDA-core formulation) cannot keep up.  The decoded
//     codes are fed, exact, to warp-level mma (m16n8k16 bf16 / m16n8k32 s8) with the <= 8 activation rows as the 8
//     MMA columns and fp32 / int32 accumulation: products with {-1,0,+1} are exact either way.
//   * the per-warp partial sums are combined through shared memory in a fixed order: deterministic.
//
// Weights use the same prepacked layout as the tensor-core GEMM (tmq_prepack, fmt 0 / 1).
#include <cuda_bf16.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace tmq {

#ifndef TMQ_GEMV_MINB
#define TMQ_GEMV_MINB 1      // min resident CTAs per SM handed to __launch_bounds__ (capping registers at 64 to fit 8 measured slower)
#endif

constexpr int kGemvWarps = 4;        // warps per CTA
constexpr int kGemvBatch = 4;        // K slices a warp has in flight at once

struct GemvArgs {
    const void *X;          // [M][K] bf16 or int8
    const uint32_t *Wt;     // [N][KW]
    const float *scale, *bias;
    void *Y;
    long long M, N, K, KW, KS, ldy;   // KW: words of a row that carry weights, KS: row stride in words
    int out_f32;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint32_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// KIND 0: bf16 activations (fmt-0 words), KIND 1: int8 activations (fmt-1 words)
template <int KIND>
__global__ void __launch_bounds__(kGemvWarps * 32, TMQ_GEMV_MINB) ternary_gemv_kernel(const GemvArgs a) {
    using Acc = typename std::conditional<KIND == 0, float, int>::type;
    __shared__ Acc red[kGemvWarps][16][8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next launch may start its own prologue
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long r0 = (long long)blockIdx.x * 16 + g, r1 = r0 + 8;  // the two output channels of this lane
    const uint32_t *w0 = a.Wt + r0 * a.KS, *w1 = a.Wt + r1 * a.KS;
    const bool ok0 = r0 < a.N, ok1 = r1 < a.N;
    const int nslices = (int)((a.K + 255) / 256);
    bool waited = false;

    Acc acc[4] = {0, 0, 0, 0};
    for (int s0 = warp; s0 < nslices; s0 += kGemvWarps * kGemvBatch) {
        // ---- weights of up to kGemvBatch slices: every load issued before anything consumes them
        uint4 wlo[kGemvBatch], whi[kGemvBatch];
#pragma unroll
        for (int b = 0; b < kGemvBatch; b++) {
            const int slice = s0 + b * kGemvWarps;
            const long long word = ((long long)slice * 256 + 64 * t) >> 4;  // KW is a multiple of 4 words
            wlo[b] = make_uint4(0, 0, 0, 0);
            whi[b] = make_uint4(0, 0, 0, 0);
            if (slice < nslices && word < a.KW) {
                if (ok0) wlo[b] = ldg_stream(w0 + word);
                if (ok1) whi[b] = ldg_stream(w1 + word);
            }
        }
        if (!waited) {  // everything above read only the weights, which no kernel of the chain writes
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
#pragma unroll
        for (int b = 0; b < kGemvBatch; b++) {
            const int slice = s0 + b * kGemvWarps;
            if (slice >= nslices) break;
            const long long k_lane = (long long)slice * 256 + 64 * t;
            // ---- activations of row g for these 64 k (zero beyond M or K); K % 8 == 0 (bf16) / K % 16 == 0 (int8)
            constexpr int XR = (KIND == 0) ? 32 : 16;
            uint32_t xr[XR];
#pragma unroll
            for (int q = 0; q < XR / 4; q++) {
                uint4 v = make_uint4(0, 0, 0, 0);
                const long long k = k_lane + (long long)q * (KIND == 0 ? 8 : 16);
                if (g < a.M && k < a.K) {
                    const char *p = reinterpret_cast<const char *>(a.X) + ((long long)g * a.K + k) * (KIND == 0 ? 2 : 1);
                    v = __ldg(reinterpret_cast<const uint4 *>(p));
                }
                xr[4 * q + 0] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
            }
            const uint32_t lo[4] = {wlo[b].x, wlo[b].y, wlo[b].z, wlo[b].w};
            const uint32_t hi[4] = {whi[b].x, whi[b].y, whi[b].z, whi[b].w};
#pragma unroll
            for (int w = 0; w < 4; w++) {  // word w = k offsets 16w .. 16w+15 of the lane's 64
                if (KIND == 0) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {  // k offsets 16w+4j .. +3: pairs 2j and 2j+1 of the word
                        const uint32_t a0 = (lo[w] << (4 * j)) & 0xC000C000u, a2 = (lo[w] << (4 * j + 2)) & 0xC000C000u;
                        const uint32_t a1 = (hi[w] << (4 * j)) & 0xC000C000u, a3 = (hi[w] << (4 * j + 2)) & 0xC000C000u;
                        mma_bf16(reinterpret_cast<float(&)[4]>(acc), a0, a1, a2, a3, xr[8 * w + 2 * j], xr[8 * w + 2 * j + 1]);
                    }
                } else {
                    const uint32_t table = 0x00FF0100u;
                    const uint32_t l0 = lo[w] & 0x33333333u, l1 = (lo[w] >> 2) & 0x33333333u;
                    const uint32_t h0 = hi[w] & 0x33333333u, h1 = (hi[w] >> 2) & 0x33333333u;
                    // k 0-3 / 4-7 of the word, then k 8-11 / 12-15
                    mma_s8(reinterpret_cast<int(&)[4]>(acc), __byte_perm(table, 0u, l0), __byte_perm(table, 0u, h0),
                           __byte_perm(table, 0u, l1), __byte_perm(table, 0u, h1), xr[4 * w + 0], xr[4 * w + 1]);
                    mma_s8(reinterpret_cast<int(&)[4]>(acc), __byte_perm(table, 0u, l0 >> 16), __byte_perm(table, 0u, h0 >> 16),
                           __byte_perm(table, 0u, l1 >> 16), __byte_perm(table, 0u, h1 >> 16), xr[4 * w + 2], xr[4 * w + 3]);
                }
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- combine the warps' K slices in a fixed order
    red[warp][g][2 * t] = acc[0];
    red[warp][g][2 * t + 1] = acc[1];
    red[warp][g + 8][2 * t] = acc[2];
    red[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();
    {
        const int row = threadIdx.x & 15, col = threadIdx.x >> 4;  // 128 threads = 16 channels x 8 activation rows
        const long long n = (long long)blockIdx.x * 16 + row;
        if (n < a.N && col < a.M) {
            Acc sum = 0;
#pragma unroll
            for (int w = 0; w < kGemvWarps; w++) sum += red[w][row][col];
            if (KIND == 1) {
                reinterpret_cast<int *>(a.Y)[(long long)col * a.ldy + n] = (int)sum;
            } else {
                const float sc = (a.scale ? a.scale[n] : 1.0f) * 0.5f;  // operands carried +-2.0
                const float f = fmaf((float)sum, sc, a.bias ? a.bias[n] : 0.0f);
                if (a.out_f32) reinterpret_cast<float *>(a.Y)[(long long)col * a.ldy + n] = f;
                else reinterpret_cast<__nv_bfloat16 *>(a.Y)[(long long)col * a.ldy + n] = __float2bfloat16_rn(f);
            }
        }
    }
}

template <int KIND>
static int launch_gemv(GemvArgs a, cudaStream_t st) {
    const long long grid = (a.N + 15) / 16;
    if (grid > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, ternary_gemv_kernel<KIND>, a));
}

constexpr int kWideGroups = 5;   // 16-channel groups per CTA of the wide variant
constexpr int kWideWarps = 16;   // K slices handled concurrently

struct WideArgs {
    const void *X;
    const uint32_t *Wt;
    const float *scale, *bias;
    void *Y;
    long long M, N, K, KW, KS, ldy;
    int groups_per_cta, nwarps, out_f32;
};

// Wide variant: a CTA of 16 warps owns up to 5 channel groups and all of K; each warp keeps the activations of its
// 256-wide K slice in registers and reuses them for every group, which cuts the activation reads five-fold.  Measured
// faster than the small-CTA kernel for bf16 activations (whose 64 activations per lane take 32 registers to fetch).
template <int KIND>
__global__ void __launch_bounds__(kWideWarps * 32, 1) ternary_gemv_wide_kernel(const WideArgs a) {
    using Acc = typename std::conditional<KIND == 0, float, int>::type;
    __shared__ Acc red[kWideWarps][kWideGroups][16][8];  // 40 KB
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next launch may start its own prologue
    bool waited = false;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = a.groups_per_cta;
    const long long group0 = (long long)blockIdx.x * G;
    const long long ngroups = (a.N + 15) / 16;

    Acc acc[kWideGroups][4];
#pragma unroll
    for (int i = 0; i < kWideGroups; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0;

    const long long nslices = (a.K + 255) / 256;
    for (long long slice = warp; slice < nslices; slice += a.nwarps) {
        const long long k_lane = slice * 256 + 64 * t;  // first k of this lane
        // ---- weights: issue every load of this slice before anything consumes them
        uint4 wlo[kWideGroups], whi[kWideGroups];
        const bool k_ok = (k_lane >> 4) < a.KW;  // KW is a multiple of 4 words: a lane's 4 words are all in or all out
#pragma unroll
        for (int i = 0; i < kWideGroups; i++) {
            wlo[i] = make_uint4(0, 0, 0, 0);
            whi[i] = make_uint4(0, 0, 0, 0);
            if (i < G && group0 + i < ngroups && k_ok) {
                const long long r0 = (group0 + i) * 16 + g, r1 = r0 + 8;
                if (r0 < a.N) wlo[i] = ldg_stream(a.Wt + r0 * a.KS + (k_lane >> 4));
                if (r1 < a.N) whi[i] = ldg_stream(a.Wt + r1 * a.KS + (k_lane >> 4));
            }
        }
        if (!waited) {  // everything before this point read only the weights, which no kernel writes
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
        // ---- activations of row g for these 64 k (zero beyond M or K); K % 8 == 0 (bf16) / K % 16 == 0 (int8)
        constexpr int XR = (KIND == 0) ? 32 : 16;  // 32-bit registers holding the lane's 64 activations
        uint32_t xr[XR];
#pragma unroll
        for (int q = 0; q < XR / 4; q++) {
            uint4 v = make_uint4(0, 0, 0, 0);
            const long long k = k_lane + (long long)q * (KIND == 0 ? 8 : 16);
            if (g < a.M && k < a.K) {
                const char *p = reinterpret_cast<const char *>(a.X) + ((long long)g * a.K + k) * (KIND == 0 ? 2 : 1);
                v = __ldg(reinterpret_cast<const uint4 *>(p));
            }
            xr[4 * q + 0] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
        }
        // ---- decode + MMA
#pragma unroll
        for (int i = 0; i < kWideGroups; i++) {
            if (i < G) {
                const uint32_t lo[4] = {wlo[i].x, wlo[i].y, wlo[i].z, wlo[i].w};
                const uint32_t hi[4] = {whi[i].x, whi[i].y, whi[i].z, whi[i].w};
#pragma unroll
                for (int w = 0; w < 4; w++) {  // word w = k offsets 16w .. 16w+15 of the lane's 64
                    if (KIND == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {  // k offsets 16w+4j .. +3: pairs 2j and 2j+1 of the word
                            const uint32_t a0 = (lo[w] << (4 * j)) & 0xC000C000u, a2 = (lo[w] << (4 * j + 2)) & 0xC000C000u;
                            const uint32_t a1 = (hi[w] << (4 * j)) & 0xC000C000u, a3 = (hi[w] << (4 * j + 2)) & 0xC000C000u;
                            mma_bf16(reinterpret_cast<float(&)[4]>(acc[i]), a0, a1, a2, a3, xr[8 * w + 2 * j],
                                     xr[8 * w + 2 * j + 1]);
                        }
                    } else {
                        const uint32_t table = 0x00FF0100u;
                        const uint32_t l0 = lo[w] & 0x33333333u, l1 = (lo[w] >> 2) & 0x33333333u;
                        const uint32_t h0 = hi[w] & 0x33333333u, h1 = (hi[w] >> 2) & 0x33333333u;
                        // k 0-3 / 4-7 of the word, then k 8-11 / 12-15
                        mma_s8(reinterpret_cast<int(&)[4]>(acc[i]), __byte_perm(table, 0u, l0), __byte_perm(table, 0u, h0),
                               __byte_perm(table, 0u, l1), __byte_perm(table, 0u, h1), xr[4 * w + 0], xr[4 * w + 1]);
                        mma_s8(reinterpret_cast<int(&)[4]>(acc[i]), __byte_perm(table, 0u, l0 >> 16),
                               __byte_perm(table, 0u, h0 >> 16), __byte_perm(table, 0u, l1 >> 16),
                               __byte_perm(table, 0u, h1 >> 16), xr[4 * w + 2], xr[4 * w + 3]);
                    }
                }
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- combine the K slices: fixed order over warps
#pragma unroll
    for (int i = 0; i < kWideGroups; i++) {
        if (i < G) {
            red[warp][i][g][2 * t] = acc[i][0];
            red[warp][i][g][2 * t + 1] = acc[i][1];
            red[warp][i][g + 8][2 * t] = acc[i][2];
            red[warp][i][g + 8][2 * t + 1] = acc[i][3];
        }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < G * 128; o += blockDim.x) {
        const int row = o & 15, col = (o >> 4) & 7, grp = o >> 7;
        const long long n = (group0 + grp) * 16 + row;
        if (n < a.N && col < a.M) {
            Acc s = 0;
            for (int w = 0; w < a.nwarps; w++) s += red[w][grp][row][col];
            if (KIND == 1) {
                reinterpret_cast<int *>(a.Y)[(long long)col * a.ldy + n] = (int)s;
            } else {
                const float sc = (a.scale ? a.scale[n] : 1.0f) * 0.5f;  // operands carried +-2.0
                const float f = fmaf((float)s, sc, a.bias ? a.bias[n] : 0.0f);
                if (a.out_f32) reinterpret_cast<float *>(a.Y)[(long long)col * a.ldy + n] = f;
                else reinterpret_cast<__nv_bfloat16 *>(a.Y)[(long long)col * a.ldy + n] = __float2bfloat16_rn(f);
            }
        }
    }
}

template <int KIND>
static int launch_gemv_wide(WideArgs a, cudaStream_t st) {
    const long long ngroups = (a.N + 15) / 16;
    long long G = (ngroups + kNumSMs - 1) / kNumSMs;
    if (G > kWideGroups) G = kWideGroups;
    if (G < 1) G = 1;
    const long long grid = (ngroups + G - 1) / G;
    if (grid > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    long long nslices = (a.K + 255) / 256;
    a.groups_per_cta = (int)G;
    a.nwarps = (int)(nslices < kWideWarps ? nslices : kWideWarps);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)(a.nwarps * 32));
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, ternary_gemv_wide_kernel<KIND>, a));
}

// ---- resident variant ---------------------------------------------------------------------------------------------
//
// One CTA per SM owns a contiguous range of channel groups and copies ALL of its packed rows (N*K/4/148 bytes: 76 KB
// for 11008 x 4096) into shared memory BEFORE it waits for the previous kernel of the stream.  Registers are capped
// at 64 so that two CTAs fit one SM: the CTA of launch i+1 becomes resident the moment the CTA of launch i-1
// retires, and its rows stream from HBM while launch i decodes and multiplies.  In a chain of launches (what decoding
// is) the weight traffic is therefore hidden entirely and the chain runs at the speed of the work that follows the
// wait: activation fetch, decode + multiply, reduction, plus the hand-over latency between two kernels.
//
// The rows travel as ONE bulk copy: the TMA unit spends about 40 ns per bulk copy whatever its size (measured: 80
// row-sized copies took 4.4 us to issue, 16 four-times larger ones 1 us), so the prepacked format itself carries the
// row padding that keeps the fragment reads (8 rows x 8 / 16 bytes per warp) free of bank conflicts.
//
// Warp-level mma costs the same for 1..8 activation rows; for int8 activations with M <= 2 the four-way byte dot
// product (dp4a) on the CUDA cores is faster than the legacy mma path on this part and is used instead.  Either way
// the integer decode (about 0.6 - 0.8 instructions per weight) bounds the arithmetic phase.

// Warps per CTA: 16 warps of <= 64 registers or 8 warps of <= 128, two CTAs per SM either way.  Sixteen give a lone
// launch the shorter critical path after griddepcontrol.wait (one K slice per warp); eight leave the compiler the
// registers to keep the decode free of spills and moves, which is what counts when launches run back to back inside
// one kernel (the batched form) or carry more than one activation row of int8 (measured per case in the launchers).
constexpr int kResWarpsMany = 16, kResWarpsFew = 8;
constexpr int kResGroups = 5;                 // channel groups per CTA at most
template <int WARPS>
struct ResOut {
    static constexpr int passes = (kResGroups * 128 + WARPS * 32 - 1) / (WARPS * 32);   // outputs per thread
};
constexpr int kResSmemMax = 110 * 1024;       // two CTAs per SM
constexpr int kResSlack = 64;                 // bytes kept readable behind the last packed row

struct ResArgs {
    const void *X;
    const uint32_t *Wt;
    const float *scale, *bias;
    void *Y;
    long long M, N, K, KW, KS, ldy;           // KS: row stride in words, in global and in shared memory
    int ngroups, out_f32;
    int bar_offset;                           // byte offset of the mbarrier inside dynamic shared memory
    int *status;
};


// Prologue shared by both resident kernels, executed by warp 0 only and kept as short as possible: a CTA that has
// just become resident competes for issue slots with the CTA of the previous launch, which is in the middle of its
// arithmetic.  The other warps learn of the barrier at the __syncthreads that follows griddepcontrol.wait.
__device__ __forceinline__ void resident_groups(const ResArgs &a, int &group0, int &G) {
    // balanced contiguous split of the channel groups (at most 5 * 148 of them) over the CTAs
    group0 = (int)((blockIdx.x * (unsigned)a.ngroups) / gridDim.x);
    G = (int)(((blockIdx.x + 1) * (unsigned)a.ngroups) / gridDim.x) - group0;
}
__device__ __forceinline__ void resident_prologue(const ResArgs &a, uint32_t *wsm, uint64_t *bar, int group0, int G) {
    if (threadIdx.x == 0) {
        long long valid = a.N - (long long)group0 * 16;                // rows of this CTA that exist
        if (valid > G * 16) valid = G * 16;
        const uint32_t bytes = (uint32_t)(valid * a.KS * 4);            // one contiguous run: rows keep their stride
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
        ptx::mbar_arrive_expect_tx(bar, bytes);
        ptx::bulk_load(wsm, a.Wt + (long long)group0 * 16 * a.KS, bytes, bar);
    }
}

__device__ __forceinline__ void lds_v2(uint32_t addr, uint32_t &a, uint32_t &b) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}
__device__ __forceinline__ void lds_v4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}

// One fmt-1 word (16 codes) -> four registers of four int8 weights: nine instructions, spelled out so that the
// compiler keeps exactly these (its own lowering of the C expression measured 60 % more integer instructions).
__device__ __forceinline__ void decode_word_dp4a(uint32_t w, uint32_t &w0, uint32_t &w1, uint32_t &w2, uint32_t &w3) {
    asm("{\n\t"
        ".reg .b32 l0, l1, s, h0, h1;\n\t"
        "and.b32 l0, %4, 0x33333333;\n\t"
        "shr.b32 s, %4, 2;\n\t"
        "and.b32 l1, s, 0x33333333;\n\t"
        "shr.b32 h0, l0, 16;\n\t"
        "shr.b32 h1, l1, 16;\n\t"
        "prmt.b32 %0, %5, 0, l0;\n\t"
        "prmt.b32 %1, %5, 0, l1;\n\t"
        "prmt.b32 %2, %5, 0, h0;\n\t"
        "prmt.b32 %3, %5, 0, h1;\n\t"
        "}"
        : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
        : "r"(w), "r"(0x00FF0100u));
}

// acc += four-way signed byte dot product, in place (spelled out for the same reason)
__device__ __forceinline__ void dp4a_acc(int &acc, uint32_t a, uint32_t b) {
    asm("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}

// Pieces of the resident kernels that the one-matrix and the batched forms share.  Lane (g, t) of a warp owns rows g
// and g + 8 of every 16-channel group and the k range [slice * 4 LK + LK t, + LK) of K slice `slice`; warps take the
// slices round-robin.
template <int KIND, int WARPS>
struct ResMma {
    using Acc = typename std::conditional<KIND == 0, float, int>::type;
    static constexpr int LK = (KIND == 0) ? 32 : 64;     // k per lane and slice: 2 / 4 packed words per channel
    static constexpr int LW = LK / 16;
    static constexpr int XR = 16;                        // 32 bf16 or 64 int8 activations of row g

    // activations of row g for one slice; zero beyond M or K; K % 8 == 0 (bf16) / K % 16 == 0 (int8)
    static __device__ __forceinline__ void load_x(const void *X, long long M, long long K, int slice, int g, int t,
                                                  uint32_t (&xr)[XR]) {
        const long long k_lane = (long long)slice * (4 * LK) + LK * t;
#pragma unroll
        for (int q = 0; q < XR / 4; q++) {
            uint4 v = make_uint4(0, 0, 0, 0);
            const long long k = k_lane + (long long)q * (KIND == 0 ? 8 : 16);
            if (g < M && k < K) {
                const char *p = reinterpret_cast<const char *>(X) + ((long long)g * K + k) * (KIND == 0 ? 2 : 1);
                v = __ldg(reinterpret_cast<const uint4 *>(p));
            }
            xr[4 * q + 0] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
        }
    }

    // all slices of this warp; `xr` holds the activations of slice `warp` on entry.  No K tail handling is needed:
    // the activations are zero beyond K, every decoded code is finite (0, +-2), and the words a lane reads past the
    // valid part of its row (at most 12: the row padding, the next row, or the slack the launcher leaves behind the
    // last row) therefore contribute exact zeros.
    // FULL: every CTA's shared-memory area holds kResGroups groups (the launcher's per-CTA maximum), so the group loop
    // runs without its predicate; a CTA that owns fewer groups multiplies rows nobody loaded - any bits decode to finite
    // values - and never stores those sums.  The slowest CTA owns kResGroups groups anyway.
    template <bool FULL>
    static __device__ __forceinline__ void slices(const uint32_t *wsm, const void *X, long long M, long long K,
                                                  long long KS, int G, int warp, int g, int t, uint32_t (&xr)[XR],
                                                  Acc (&acc)[kResGroups][4]) {
        const int nslices = (int)((K + 4 * LK - 1) / (4 * LK));
        const uint32_t hi_off = (uint32_t)KS * 32u;           // 8 rows further, in bytes
        uint32_t addr = ptx::smem_u32(wsm) + (uint32_t)g * ((uint32_t)KS * 4u) + (uint32_t)(LK / 4) * t +
                        (uint32_t)warp * (uint32_t)LK;     // slice s starts 4 LK / 16 words = LK bytes after slice s - 1
        for (int slice = warp; slice < nslices; slice += WARPS, addr += WARPS * LK) {
            if (slice != warp) load_x(X, M, K, slice, g, t, xr);
#pragma unroll
            for (int i = 0; i < kResGroups; i++) {
                if (FULL || i < G) {                            // warp-uniform: every lane takes part in the mma below
                    const uint32_t p0 = addr + (uint32_t)i * (2u * hi_off), p1 = p0 + hi_off;
                    uint32_t lo[LW], hi[LW];
                    if (KIND == 0) {
                        lds_v2(p0, lo[0], lo[1]);
                        lds_v2(p1, hi[0], hi[1]);
                    } else {
                        lds_v4(p0, lo[0], lo[1], lo[LW - 2], lo[LW - 1]);
                        lds_v4(p1, hi[0], hi[1], hi[LW - 2], hi[LW - 1]);
                    }
#pragma unroll
                    for (int w = 0; w < LW; w++) {
                        if (KIND == 0) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const uint32_t a0 = (lo[w] << (4 * j)) & 0xC000C000u, a2 = (lo[w] << (4 * j + 2)) & 0xC000C000u;
                                const uint32_t a1 = (hi[w] << (4 * j)) & 0xC000C000u, a3 = (hi[w] << (4 * j + 2)) & 0xC000C000u;
                                mma_bf16(reinterpret_cast<float(&)[4]>(acc[i]), a0, a1, a2, a3, xr[8 * w + 2 * j],
                                         xr[8 * w + 2 * j + 1]);
                            }
                        } else {
                            const uint32_t table = 0x00FF0100u;
                            const uint32_t l0 = lo[w] & 0x33333333u, l1 = (lo[w] >> 2) & 0x33333333u;
                            const uint32_t h0 = hi[w] & 0x33333333u, h1 = (hi[w] >> 2) & 0x33333333u;
                            mma_s8(reinterpret_cast<int(&)[4]>(acc[i]), __byte_perm(table, 0u, l0), __byte_perm(table, 0u, h0),
                                   __byte_perm(table, 0u, l1), __byte_perm(table, 0u, h1), xr[4 * w + 0], xr[4 * w + 1]);
                            mma_s8(reinterpret_cast<int(&)[4]>(acc[i]), __byte_perm(table, 0u, l0 >> 16),
                                   __byte_perm(table, 0u, h0 >> 16), __byte_perm(table, 0u, l1 >> 16),
                                   __byte_perm(table, 0u, h1 >> 16), xr[4 * w + 2], xr[4 * w + 3]);
                        }
                    }
                }
            }
        }
    }

    // this warp's partial sums into red[warp][group][16 channels][mc rows]; mc: even, >= M, <= 8
    static __device__ __forceinline__ void partials(Acc *red, int G, int warp, int g, int t, const Acc (&acc)[kResGroups][4],
                                                    int mc = 8) {
        if (2 * t >= mc) return;
#pragma unroll
        for (int i = 0; i < kResGroups; i++) {
            if (i < G) {
                Acc *r = red + ((size_t)(warp * kResGroups + i) * 16) * mc;
                r[g * mc + 2 * t] = acc[i][0];
                r[g * mc + 2 * t + 1] = acc[i][1];
                r[(g + 8) * mc + 2 * t] = acc[i][2];
                r[(g + 8) * mc + 2 * t + 1] = acc[i][3];
            }
        }
    }

    // sum over the warps of output o (< G * 128: channel o & 15 of group o >> 7, row (o >> 4) & 7), fixed order
    static __device__ __forceinline__ Acc total(const Acc *red, int o, int mc = 8) {
        const int row = o & 15, col = (o >> 4) & 7, grp = o >> 7;
        Acc s = 0;
#pragma unroll
        for (int w = 0; w < WARPS; w++) s += red[((size_t)(w * kResGroups + grp) * 16 + row) * mc + col];
        return s;
    }
};

template <int KIND, int WARPS, bool FULL>
__global__ void __launch_bounds__(WARPS * 32, 2) ternary_gemv_resident_kernel(const ResArgs a) {
    using R = ResMma<KIND, WARPS>;
    using Acc = typename R::Acc;
    extern __shared__ __align__(16) uint32_t wsm[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(wsm) + a.bar_offset);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    int group0, G;
    resident_groups(a, group0, G);
    resident_prologue(a, wsm, bar, group0, G);
    // per-channel scale / bias of the outputs this thread will write (they belong to the weights, not to the chain):
    // fetched here so that their latency is not paid after the arithmetic
    float psc[ResOut<WARPS>::passes], pbi[ResOut<WARPS>::passes];
    if (KIND == 0) {
#pragma unroll
        for (int q = 0; q < ResOut<WARPS>::passes; q++) {
            psc[q] = 0.5f;                                    // operands carried +-2.0
            pbi[q] = 0.0f;
            const int o = threadIdx.x + q * (WARPS * 32);
            const long long n = ((long long)group0 + (o >> 7)) * 16 + (o & 15);
            if (o < G * 128 && n < a.N) {
                if (a.scale) psc[q] *= a.scale[n];
                if (a.bias) pbi[q] = a.bias[n];
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");   // activations and outputs belong to the chain
    __syncthreads();                                     // the barrier warp 0 initialised is visible to every warp

    Acc acc[kResGroups][4];
#pragma unroll
    for (int i = 0; i < kResGroups; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0;
    uint32_t xr[R::XR];
    R::load_x(a.X, a.M, a.K, warp, g, t, xr);      // in flight while the last packed rows land
    const bool ok = __syncthreads_and(ptx::mbar_wait(bar, 0, a.status));
    if (ok) R::template slices<FULL>(wsm, a.X, a.M, a.K, a.KS, G, warp, g, t, xr, acc);
    __syncthreads();   // every warp is done reading the packed rows: the area becomes the reduction buffer
    if (!ok) return;   // uniform: the copies never completed and the status word says so
    Acc *red = reinterpret_cast<Acc *>(wsm);  // [warp][group][16][8]
    R::partials(red, G, warp, g, t, acc);
    __syncthreads();
#pragma unroll
    for (int q = 0; q < ResOut<WARPS>::passes; q++) {            // G * 128 <= 640 outputs
        const int o = threadIdx.x + q * (WARPS * 32);
        if (o >= G * 128) break;
        const int row = o & 15, col = (o >> 4) & 7, grp = o >> 7;
        const long long n = ((long long)group0 + grp) * 16 + row;
        if (n < a.N && col < a.M) {
            const Acc s = R::total(red, o);
            if (KIND == 1) {
                reinterpret_cast<int *>(a.Y)[(long long)col * a.ldy + n] = (int)s;
            } else {
                const float f = fmaf((float)s, psc[q], pbi[q]);
                if (a.out_f32) reinterpret_cast<float *>(a.Y)[(long long)col * a.ldy + n] = f;
                else reinterpret_cast<__nv_bfloat16 *>(a.Y)[(long long)col * a.ldy + n] = __float2bfloat16_rn(f);
            }
        }
    }
}

// int8 activations, MR = 1 or 2 rows: lane (g, t) of warp w owns the 64 k  [256 w + 64 t, +64)  of the channels
// g, g+8, g+16, ... of the CTA and accumulates them with dp4a; the four t lanes and the 16 warps are then summed.
template <int MR, int WARPS>
struct ResDp4a {
    static constexpr int RL = 2 * kResGroups;             // channels per lane at most

    static __device__ __forceinline__ void load_x(const void *X, long long M, long long K, int slice, int t,
                                                  uint32_t (&xr)[MR][16]) {
        const long long k_lane = (long long)slice * 256 + 64 * t;
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint4 v = make_uint4(0, 0, 0, 0);
                const long long k = k_lane + 16 * q;
                if (m < M && k < K)
                    v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(X) + (long long)m * K + k));
                xr[m][4 * q + 0] = v.x; xr[m][4 * q + 1] = v.y; xr[m][4 * q + 2] = v.z; xr[m][4 * q + 3] = v.w;
            }
    }

    // all slices of this warp (`xr` holds slice `warp` on entry), then the sum over the four t lanes of a channel;
    // no K tail handling, for the reasons given at ResMma::slices
    template <bool FULL>
    static __device__ __forceinline__ void slices(const uint32_t *wsm, const void *X, long long M, long long K,
                                                  long long KS, int G, int warp, int g, int t, uint32_t (&xr)[MR][16],
                                                  int (&acc)[RL][MR]) {
        const int nslices = (int)((K + 255) / 256);
        const uint32_t row8 = (uint32_t)KS * 32u;             // 8 rows further, in bytes
        uint32_t addr = ptx::smem_u32(wsm) + (uint32_t)g * ((uint32_t)KS * 4u) + 16u * t + 64u * warp;
        for (int slice = warp; slice < nslices; slice += WARPS, addr += WARPS * 64) {
            if (slice != warp) load_x(X, M, K, slice, t, xr);
#pragma unroll
            for (int i = 0; i < RL; i++) {
                if (FULL || i < 2 * G) {
                    uint32_t words[4];
                    lds_v4(addr + (uint32_t)i * row8, words[0], words[1], words[2], words[3]);
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        // word w = k 16w .. 16w+15 of the lane's 64, in the order the activations sit in memory
                        uint32_t w0, w1, w2, w3;
                        decode_word_dp4a(words[w], w0, w1, w2, w3);
#pragma unroll
                        for (int m = 0; m < MR; m++) {
                            dp4a_acc(acc[i][m], w0, xr[m][4 * w + 0]);
                            dp4a_acc(acc[i][m], w1, xr[m][4 * w + 1]);
                            dp4a_acc(acc[i][m], w2, xr[m][4 * w + 2]);
                            dp4a_acc(acc[i][m], w3, xr[m][4 * w + 3]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < RL; i++)
#pragma unroll
            for (int m = 0; m < MR; m++) {
                acc[i][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[i][m], 1);
                acc[i][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[i][m], 2);
            }
    }

    // red[warp][channel of the CTA][MR]
    static __device__ __forceinline__ void partials(int *red, int G, int warp, int g, int t, const int (&acc)[RL][MR]) {
        if (t == 0) {
#pragma unroll
            for (int i = 0; i < RL; i++)
                if (i < 2 * G)
#pragma unroll
                    for (int m = 0; m < MR; m++) red[(warp * (RL * 8) + i * 8 + g) * MR + m] = acc[i][m];
        }
    }
    static __device__ __forceinline__ int total(const int *red, int row, int m) {
        int s = 0;
#pragma unroll
        for (int w = 0; w < WARPS; w++) s += red[(w * (RL * 8) + row) * MR + m];
        return s;
    }
};

template <int MR, int WARPS, bool FULL>
__global__ void __launch_bounds__(WARPS * 32, 2) ternary_gemv_resident_dp4a_kernel(const ResArgs a) {
    using R = ResDp4a<MR, WARPS>;
    extern __shared__ __align__(16) uint32_t wsm[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(wsm) + a.bar_offset);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    int group0, G;
    resident_groups(a, group0, G);
    resident_prologue(a, wsm, bar, group0, G);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();                                     // the barrier warp 0 initialised is visible to every warp

    int acc[R::RL][MR];
#pragma unroll
    for (int i = 0; i < R::RL; i++)
#pragma unroll
        for (int m = 0; m < MR; m++) acc[i][m] = 0;
    uint32_t xr[MR][16];
    R::load_x(a.X, a.M, a.K, warp, t, xr);
    const bool ok = __syncthreads_and(ptx::mbar_wait(bar, 0, a.status));
    if (ok) R::template slices<FULL>(wsm, a.X, a.M, a.K, a.KS, G, warp, g, t, xr, acc);
    __syncthreads();   // every warp is done reading the packed rows: the area becomes the reduction buffer
    if (!ok) return;
    int *red = reinterpret_cast<int *>(wsm);
    R::partials(red, G, warp, g, t, acc);
    __syncthreads();
    for (int o = threadIdx.x; o < G * 16 * MR; o += blockDim.x) {
        const int m = o % MR, row = o / MR;
        const long long n = (long long)group0 * 16 + row;
        if (n < a.N && m < a.M) reinterpret_cast<int *>(a.Y)[(long long)m * a.ldy + n] = R::total(red, row, m);
    }
}

// 9 .. 16 activation rows in ONE pass: the decoded weight fragment of a k16 step is fed to NB = 2 MMAs (two 8-row
// activation tiles), so the integer decode - the cost that bounds the one-tile kernel - is paid once for both.  Eight
// warps and up to 128 registers per thread (two accumulator sets and two activation fragments per lane), two CTAs per
// SM as above, so the next launch's rows still stream in under this launch's arithmetic.
constexpr int kRowsWarps = 8;

template <int KIND, int NB>
__global__ void __launch_bounds__(kRowsWarps * 32, 2) ternary_gemv_resident_rows_kernel(const ResArgs a) {
    using Acc = typename std::conditional<KIND == 0, float, int>::type;
    constexpr int LK = (KIND == 0) ? 32 : 64;     // k per lane and slice: 2 / 4 packed words per channel
    constexpr int LW = LK / 16;
    extern __shared__ __align__(16) uint32_t wsm[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(wsm) + a.bar_offset);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    int group0, G;
    resident_groups(a, group0, G);
    resident_prologue(a, wsm, bar, group0, G);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // activations and outputs belong to the chain
    __syncthreads();                                     // the barrier warp 0 initialised is visible to every warp

    Acc acc[kResGroups][NB][4];
#pragma unroll
    for (int i = 0; i < kResGroups; i++)
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][b][j] = 0;

    const int nslices = (int)((a.K + 4 * LK - 1) / (4 * LK));
    constexpr int XR = 16;                         // 32 bf16 or 64 int8 activations of one row
    uint32_t xr[NB][XR];
    auto load_x = [&](int slice) {                 // rows g, g + 8, ...; zero beyond M or K
        const long long k_lane = (long long)slice * (4 * LK) + LK * t;
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int q = 0; q < XR / 4; q++) {
                uint4 v = make_uint4(0, 0, 0, 0);
                const long long k = k_lane + (long long)q * (KIND == 0 ? 8 : 16);
                const int m = 8 * b + g;
                if (m < a.M && k < a.K) {
                    const char *p = reinterpret_cast<const char *>(a.X) + ((long long)m * a.K + k) * (KIND == 0 ? 2 : 1);
                    v = __ldg(reinterpret_cast<const uint4 *>(p));
                }
                xr[b][4 * q + 0] = v.x; xr[b][4 * q + 1] = v.y; xr[b][4 * q + 2] = v.z; xr[b][4 * q + 3] = v.w;
            }
    };
    load_x(warp);
    const bool ok = __syncthreads_and(ptx::mbar_wait(bar, 0, a.status));
    for (int slice = warp; ok && slice < nslices; slice += kRowsWarps) {
        if (slice != warp) load_x(slice);
        const long long k_lane = (long long)slice * (4 * LK) + LK * t;
        const bool k_ok = (k_lane >> 4) < a.KW;
#pragma unroll
        for (int i = 0; i < kResGroups; i++) {
            if (i < G) {                            // warp-uniform: every lane takes part in the mma below
                const uint32_t *p0 = wsm + (size_t)(i * 16 + g) * a.KS + (k_lane >> 4);
                const uint32_t *p1 = p0 + (size_t)8 * a.KS;
                uint32_t lo[LW], hi[LW];
#pragma unroll
                for (int w = 0; w < LW; w++) lo[w] = hi[w] = 0;
                if (k_ok) {
                    if (KIND == 0) {
                        const uint2 u0 = *reinterpret_cast<const uint2 *>(p0), u1 = *reinterpret_cast<const uint2 *>(p1);
                        lo[0] = u0.x; lo[1] = u0.y; hi[0] = u1.x; hi[1] = u1.y;
                    } else {
                        const uint4 u0 = *reinterpret_cast<const uint4 *>(p0), u1 = *reinterpret_cast<const uint4 *>(p1);
                        lo[0] = u0.x; lo[1] = u0.y; lo[LW - 2] = u0.z; lo[LW - 1] = u0.w;
                        hi[0] = u1.x; hi[1] = u1.y; hi[LW - 2] = u1.z; hi[LW - 1] = u1.w;
                    }
                }
#pragma unroll
                for (int w = 0; w < LW; w++) {
                    if (KIND == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint32_t a0 = (lo[w] << (4 * j)) & 0xC000C000u, a2 = (lo[w] << (4 * j + 2)) & 0xC000C000u;
                            const uint32_t a1 = (hi[w] << (4 * j)) & 0xC000C000u, a3 = (hi[w] << (4 * j + 2)) & 0xC000C000u;
#pragma unroll
                            for (int b = 0; b < NB; b++)
                                mma_bf16(reinterpret_cast<float(&)[4]>(acc[i][b]), a0, a1, a2, a3, xr[b][8 * w + 2 * j],
                                         xr[b][8 * w + 2 * j + 1]);
                        }
                    } else {
                        const uint32_t table = 0x00FF0100u;
                        const uint32_t l0 = lo[w] & 0x33333333u, l1 = (lo[w] >> 2) & 0x33333333u;
                        const uint32_t h0 = hi[w] & 0x33333333u, h1 = (hi[w] >> 2) & 0x33333333u;
                        const uint32_t e0 = __byte_perm(table, 0u, l0), e1 = __byte_perm(table, 0u, h0);
                        const uint32_t e2 = __byte_perm(table, 0u, l1), e3 = __byte_perm(table, 0u, h1);
                        const uint32_t f0 = __byte_perm(table, 0u, l0 >> 16), f1 = __byte_perm(table, 0u, h0 >> 16);
                        const uint32_t f2 = __byte_perm(table, 0u, l1 >> 16), f3 = __byte_perm(table, 0u, h1 >> 16);
#pragma unroll
                        for (int b = 0; b < NB; b++) {
                            mma_s8(reinterpret_cast<int(&)[4]>(acc[i][b]), e0, e1, e2, e3, xr[b][4 * w + 0], xr[b][4 * w + 1]);
                            mma_s8(reinterpret_cast<int(&)[4]>(acc[i][b]), f0, f1, f2, f3, xr[b][4 * w + 2], xr[b][4 * w + 3]);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();   // every warp is done reading the packed rows: the area becomes the reduction buffer
    if (!ok) return;   // uniform: the copies never completed and the status word says so
    constexpr int MC = 8 * NB;                      // activation rows (columns of the reduction tile)
    Acc *red = reinterpret_cast<Acc *>(wsm);        // [warp][group][16][MC]
#pragma unroll
    for (int i = 0; i < kResGroups; i++) {
        if (i < G) {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                Acc *r = red + ((size_t)(warp * kResGroups + i) * 16) * MC + 8 * b;
                r[g * MC + 2 * t] = acc[i][b][0];
                r[g * MC + 2 * t + 1] = acc[i][b][1];
                r[(g + 8) * MC + 2 * t] = acc[i][b][2];
                r[(g + 8) * MC + 2 * t + 1] = acc[i][b][3];
            }
        }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < G * 16 * MC; o += kRowsWarps * 32) {
        const int row = o & 15, col = (o >> 4) % MC, grp = o / (16 * MC);
        const long long n = ((long long)group0 + grp) * 16 + row;
        if (n < a.N && col < a.M) {
            Acc s = 0;
#pragma unroll
            for (int w = 0; w < kRowsWarps; w++) s += red[((size_t)(w * kResGroups + grp) * 16 + row) * MC + col];
            if (KIND == 1) {
                reinterpret_cast<int *>(a.Y)[(long long)col * a.ldy + n] = (int)s;
            } else {
                const float sc = (a.scale ? a.scale[n] : 1.0f) * 0.5f;   // operands carried +-2.0
                const float f = fmaf((float)s, sc, a.bias ? a.bias[n] : 0.0f);
                if (a.out_f32) reinterpret_cast<float *>(a.Y)[(long long)col * a.ldy + n] = f;
                else reinterpret_cast<__nv_bfloat16 *>(a.Y)[(long long)col * a.ldy + n] = __float2bfloat16_rn(f);
            }
        }
    }
}

// ---- batched form: several matrices of one shape in ONE launch -----------------------------------------------------
//
// Q/K/V or gate/up projections share an activation vector, experts or independent layers bring their own; either way
// nothing orders the matrices of such a group, so one launch can take them all and the hand-over between two kernels
// (completion -> dependent released, activation fetch, barrier: about 1.5 us) is paid once per group instead of once
// per matrix.  Two CTAs per SM as in the one-matrix kernels; the CTAs of an SM take the even and the odd matrices, each
// with one resident buffer: while one multiplies matrix j the other's rows of matrix j + 1 stream in, and the reduction
// and store of one overlap the arithmetic of the other.  Per matrix the launch then costs max(row traffic, arithmetic).
constexpr int kBatchMax = TMQ_GEMV_BATCH_MAX;

struct BatchArgs {
    const void *X;
    long long x_stride;                        // bytes between the activation blocks of consecutive matrices, 0: shared
    const uint32_t *Wt[kBatchMax];
    const float *scale[kBatchMax], *bias[kBatchMax];
    void *Y[kBatchMax];
    long long M, N, K, KW, KS, ldy;
    int nmat, ngroups, nslots, out_f32;
    int bar_offset, red_offset, red_alias;     // red_alias: the reduction area overlays the rows (they did not both fit)
    int red_cols;                              // activation rows the reduction area keeps per channel: even, >= M
    int *status;
};

struct BatchCta {
    int group0, G, first, step;
    uint32_t bytes;
};
__device__ __forceinline__ BatchCta batch_cta(const BatchArgs &a) {
    BatchCta c;
    const int slot = (int)(blockIdx.x % (unsigned)a.nslots);
    c.first = (int)(blockIdx.x / (unsigned)a.nslots);
    c.step = (int)(gridDim.x / (unsigned)a.nslots);
    c.group0 = (int)((slot * (unsigned)a.ngroups) / (unsigned)a.nslots);
    c.G = (int)(((slot + 1) * (unsigned)a.ngroups) / (unsigned)a.nslots) - c.group0;
    long long valid = a.N - (long long)c.group0 * 16;
    if (valid > c.G * 16) valid = c.G * 16;
    c.bytes = (uint32_t)(valid * a.KS * 4);
    return c;
}
__device__ __forceinline__ void batch_fetch(const BatchArgs &a, const BatchCta &c, uint32_t *wsm, uint64_t *bar, int j) {
    ptx::mbar_arrive_expect_tx(bar, c.bytes);
    ptx::bulk_load(wsm, a.Wt[j] + (long long)c.group0 * 16 * a.KS, c.bytes, bar);
}

template <int KIND, int WARPS, bool FULL>
__global__ void __launch_bounds__(WARPS * 32, 2) ternary_gemv_batched_kernel(const __grid_constant__ BatchArgs a) {
    using R = ResMma<KIND, WARPS>;
    using Acc = typename R::Acc;
    extern __shared__ __align__(16) uint32_t wsm[];
    unsigned char *base = reinterpret_cast<unsigned char *>(wsm);
    uint64_t *bar = reinterpret_cast<uint64_t *>(base + a.bar_offset);
    Acc *red = reinterpret_cast<Acc *>(base + a.red_offset);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const BatchCta c = batch_cta(a);
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
        if (c.first < a.nmat) batch_fetch(a, c, wsm, bar, c.first);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    uint32_t phase = 0;
    for (int j = c.first; j < a.nmat; j += c.step, phase ^= 1) {
        float psc[ResOut<WARPS>::passes], pbi[ResOut<WARPS>::passes];
        if (KIND == 0) {
            const float *scale = a.scale[j], *bias = a.bias[j];
#pragma unroll
            for (int q = 0; q < ResOut<WARPS>::passes; q++) {
                psc[q] = 0.5f;                                // operands carried +-2.0
                pbi[q] = 0.0f;
                const int o = threadIdx.x + q * (WARPS * 32);
                const long long n = ((long long)c.group0 + (o >> 7)) * 16 + (o & 15);
                if (o < c.G * 128 && n < a.N) {
                    if (scale) psc[q] *= scale[n];
                    if (bias) pbi[q] = bias[n];
                }
            }
        }
        Acc acc[kResGroups][4];
#pragma unroll
        for (int i = 0; i < kResGroups; i++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[i][q] = 0;
        const void *X = reinterpret_cast<const char *>(a.X) + (long long)j * a.x_stride;
        uint32_t xr[R::XR];
        R::load_x(X, a.M, a.K, warp, g, t, xr);
        if (!__syncthreads_and(ptx::mbar_wait(bar, phase, a.status))) return;   // uniform; the status word says why
        R::template slices<FULL>(wsm, X, a.M, a.K, a.KS, c.G, warp, g, t, xr, acc);
        __syncthreads();                                   // every warp is done with the rows of matrix j
        const bool more = j + c.step < a.nmat;
        if (!a.red_alias && more && threadIdx.x == 0) batch_fetch(a, c, wsm, bar, j + c.step);
        R::partials(red, c.G, warp, g, t, acc, a.red_cols);
        __syncthreads();
        void *Y = a.Y[j];
#pragma unroll
        for (int q = 0; q < ResOut<WARPS>::passes; q++) {
            const int o = threadIdx.x + q * (WARPS * 32);
            if (o >= c.G * 128) break;
            const int row = o & 15, col = (o >> 4) & 7, grp = o >> 7;
            const long long n = ((long long)c.group0 + grp) * 16 + row;
            if (n < a.N && col < a.M) {
                const Acc s = R::total(red, o, a.red_cols);
                if (KIND == 1) {
                    reinterpret_cast<int *>(Y)[(long long)col * a.ldy + n] = (int)s;
                } else {
                    const float f = fmaf((float)s, psc[q], pbi[q]);
                    if (a.out_f32) reinterpret_cast<float *>(Y)[(long long)col * a.ldy + n] = f;
                    else reinterpret_cast<__nv_bfloat16 *>(Y)[(long long)col * a.ldy + n] = __float2bfloat16_rn(f);
                }
            }
        }
        // a separate reduction area is next written after two more barriers; an overlaid one must be read out first
        if (a.red_alias) {
            __syncthreads();
            if (more && threadIdx.x == 0) batch_fetch(a, c, wsm, bar, j + c.step);
        }
    }
}

template <int MR, int WARPS, bool FULL>
__global__ void __launch_bounds__(WARPS * 32, 2) ternary_gemv_batched_dp4a_kernel(const __grid_constant__ BatchArgs a) {
    using R = ResDp4a<MR, WARPS>;
    extern __shared__ __align__(16) uint32_t wsm[];
    unsigned char *base = reinterpret_cast<unsigned char *>(wsm);
    uint64_t *bar = reinterpret_cast<uint64_t *>(base + a.bar_offset);
    int *red = reinterpret_cast<int *>(base + a.red_offset);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const BatchCta c = batch_cta(a);
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
        if (c.first < a.nmat) batch_fetch(a, c, wsm, bar, c.first);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    uint32_t phase = 0;
    for (int j = c.first; j < a.nmat; j += c.step, phase ^= 1) {
        int acc[R::RL][MR];
#pragma unroll
        for (int i = 0; i < R::RL; i++)
#pragma unroll
            for (int m = 0; m < MR; m++) acc[i][m] = 0;
        const void *X = reinterpret_cast<const char *>(a.X) + (long long)j * a.x_stride;
        uint32_t xr[MR][16];
        R::load_x(X, a.M, a.K, warp, t, xr);
        if (!__syncthreads_and(ptx::mbar_wait(bar, phase, a.status))) return;
        R::template slices<FULL>(wsm, X, a.M, a.K, a.KS, c.G, warp, g, t, xr, acc);
        __syncthreads();
        const bool more = j + c.step < a.nmat;
        if (!a.red_alias && more && threadIdx.x == 0) batch_fetch(a, c, wsm, bar, j + c.step);
        R::partials(red, c.G, warp, g, t, acc);
        __syncthreads();
        int *Y = reinterpret_cast<int *>(a.Y[j]);
        for (int o = threadIdx.x; o < c.G * 16 * MR; o += blockDim.x) {
            const int m = o % MR, row = o / MR;
            const long long n = (long long)c.group0 * 16 + row;
            if (n < a.N && m < a.M) Y[(long long)m * a.ldy + n] = R::total(red, row, m);
        }
        if (a.red_alias) {
            __syncthreads();
            if (more && threadIdx.x == 0) batch_fetch(a, c, wsm, bar, j + c.step);
        }
    }
}

template <typename Args>
static int launch_resident_form(void (*kernel)(const Args), const Args &a, unsigned grid, int warps, long long smem,
                                cudaStream_t st) {
    int rc = ensure_dynamic_smem(kernel, kResSmemMax, true);
    if (rc != TMQ_OK) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, a));
}

template <int KIND>
static int launch_gemv_batched(BatchArgs a, cudaStream_t st) {
    constexpr int W = kResWarpsFew;               // measured faster than 16 warps for every batched case
    const long long ngroups = (a.N + 15) / 16;
    const long long nslots = ngroups < kNumSMs ? ngroups : kNumSMs;
    const long long G = (ngroups + nslots - 1) / nslots;
    if (G > kResGroups || ngroups > 0x7FFFFFFF) return TMQ_ERR_UNSUPPORTED;
    const bool dp4a = KIND == 1 && a.M <= 2;
    const long long rows = G * 16 * a.KS * 4 + kResSlack;   // a lane may read up to 48 bytes past the last row
    a.red_cols = (int)((a.M + 1) / 2 * 2);
    const long long red = dp4a ? (long long)W * 2 * kResGroups * 8 * a.M * 4
                               : (long long)W * kResGroups * 16 * a.red_cols * 4;
    long long smem = rows + red;
    a.red_offset = (int)rows;
    a.red_alias = 0;
    if (smem + 16 > kResSmemMax) {                 // overlay: the next fetch then waits for the reduction
        smem = rows > red ? rows : red;
        a.red_offset = 0;
        a.red_alias = 1;
    }
    a.bar_offset = (int)smem;
    smem += 16;
    if (smem > kResSmemMax) return TMQ_ERR_UNSUPPORTED;
    a.ngroups = (int)ngroups;
    a.nslots = (int)nslots;
    const unsigned grid = (unsigned)(nslots * (a.nmat > 1 ? 2 : 1));
    if (G == kResGroups) {         // every CTA's area holds the full five groups: the unpredicated group loop
        if (dp4a && a.M == 1) return launch_resident_form(ternary_gemv_batched_dp4a_kernel<1, W, true>, a, grid, W, smem, st);
        if (dp4a) return launch_resident_form(ternary_gemv_batched_dp4a_kernel<2, W, true>, a, grid, W, smem, st);
        return launch_resident_form(ternary_gemv_batched_kernel<KIND, W, true>, a, grid, W, smem, st);
    }
    if (dp4a && a.M == 1) return launch_resident_form(ternary_gemv_batched_dp4a_kernel<1, W, false>, a, grid, W, smem, st);
    if (dp4a) return launch_resident_form(ternary_gemv_batched_dp4a_kernel<2, W, false>, a, grid, W, smem, st);
    return launch_resident_form(ternary_gemv_batched_kernel<KIND, W, false>, a, grid, W, smem, st);
}

// Returns TMQ_ERR_UNSUPPORTED when the CTA's rows do not fit the shared-memory budget (the caller then streams).
template <int KIND>
static int launch_gemv_resident(ResArgs a, cudaStream_t st) {
    const long long ngroups = (a.N + 15) / 16;
    const long long grid = ngroups < kNumSMs ? ngroups : kNumSMs;
    const long long G = (ngroups + grid - 1) / grid;
    if (G > kResGroups || ngroups > 0x7FFFFFFF || !a.status) return TMQ_ERR_UNSUPPORTED;
    long long smem = G * 16 * a.KS * 4;            // the row stride already carries the bank padding
    const bool rows16 = a.M > 8;                   // 9 .. 16 rows: the two-tile kernel (8 warps, 16 reduction columns)
    // int8 with more than one row: 8 warps (measured: M = 2 6.7 -> 5.3 us, M = 8 5.9 -> 5.4 us per matrix); bf16 and
    // the one-row int8 case keep 16 (bf16 M = 1 5.6 us against 6.3 with 8 warps)
    const int warps = rows16 ? kRowsWarps : (KIND == 1 && a.M >= 2) ? kResWarpsFew : kResWarpsMany;
    const long long red_bytes = (long long)warps * kResGroups * 16 * (rows16 ? 16 : 8) * 4;   // covers the dp4a layout too
    if (smem < red_bytes) smem = red_bytes;
    smem += kResSlack;                             // a lane may read up to 48 bytes past the last row (zero activations)
    a.bar_offset = (int)smem;                      // multiple of 16
    smem += 16;
    if (smem > kResSmemMax) return TMQ_ERR_UNSUPPORTED;
    a.ngroups = (int)ngroups;
    const unsigned g = (unsigned)grid;
    if (rows16) return launch_resident_form(ternary_gemv_resident_rows_kernel<KIND, 2>, a, g, warps, smem, st);
    if (G == kResGroups) {         // every CTA's area holds the full five groups: the unpredicated group loop
        if (KIND == 1 && a.M == 1)
            return launch_resident_form(ternary_gemv_resident_dp4a_kernel<1, kResWarpsMany, true>, a, g, warps, smem, st);
        if (KIND == 1 && a.M == 2)
            return launch_resident_form(ternary_gemv_resident_dp4a_kernel<2, kResWarpsFew, true>, a, g, warps, smem, st);
        if (KIND == 1) return launch_resident_form(ternary_gemv_resident_kernel<1, kResWarpsFew, true>, a, g, warps, smem, st);
        return launch_resident_form(ternary_gemv_resident_kernel<0, kResWarpsMany, true>, a, g, warps, smem, st);
    }
    if (KIND == 1 && a.M == 1)
        return launch_resident_form(ternary_gemv_resident_dp4a_kernel<1, kResWarpsMany, false>, a, g, warps, smem, st);
    if (KIND == 1 && a.M == 2)
        return launch_resident_form(ternary_gemv_resident_dp4a_kernel<2, kResWarpsFew, false>, a, g, warps, smem, st);
    if (KIND == 1) return launch_resident_form(ternary_gemv_resident_kernel<1, kResWarpsFew, false>, a, g, warps, smem, st);
    return launch_resident_form(ternary_gemv_resident_kernel<0, kResWarpsMany, false>, a, g, warps, smem, st);
}

static int check_gemv(const void *X, const uint32_t *Wt, const void *Y, long long M, long long N, long long K,
                      long long ldy, int elem) {
    if (!X || !Wt || !Y) return TMQ_ERR_ARG;
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || ldy < N) return TMQ_ERR_ARG;
    if ((K * elem) % 16 != 0) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 16) || !aligned(Wt, 16)) return TMQ_ERR_ALIGN;
    return TMQ_OK;
}

}  // namespace tmq

using namespace tmq;

extern "C" int tmq_ternary_gemv_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                     int64_t M, int64_t N, int64_t K, int64_t ldy, int out_f32, int *status, void *stream) {
    int rc = check_gemv(X, Wt, Y, M, N, K, ldy, 2);
    if (rc != TMQ_OK) return rc;
    if (status) {   // resident form; falls through when one SM's share of the rows exceeds the shared-memory budget
        ResArgs r = {X, Wt, scale, bias, Y, M, N, K, prepack_valid_words(K), prepack_row_words(K, 0), ldy, 0, out_f32, 0, status};
        rc = launch_gemv_resident<0>(r, (cudaStream_t)stream);
        if (rc != TMQ_ERR_UNSUPPORTED) return rc;
    }
    if (M > 8) return TMQ_ERR_UNSUPPORTED;   // the streaming fallback takes 8 rows per pass: the caller splits
    WideArgs a = {X, Wt, scale, bias, Y, M, N, K, prepack_valid_words(K), prepack_row_words(K, 0), ldy, 0, 0, out_f32};
    return launch_gemv_wide<0>(a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemv_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K,
                                   int64_t ldy, int *status, void *stream) {
    int rc = check_gemv(X, Wt, Y, M, N, K, ldy, 1);
    if (rc != TMQ_OK) return rc;
    if (status) {
        ResArgs r = {X, Wt, nullptr, nullptr, Y, M, N, K, prepack_valid_words(K), prepack_row_words(K, 1), ldy, 0, 0, 0, status};
        rc = launch_gemv_resident<1>(r, (cudaStream_t)stream);
        if (rc != TMQ_ERR_UNSUPPORTED) return rc;
    }
    if (M > 8) return TMQ_ERR_UNSUPPORTED;
    GemvArgs a = {X, Wt, nullptr, nullptr, Y, M, N, K, prepack_valid_words(K), prepack_row_words(K, 1), ldy, 0};
    return launch_gemv<1>(a, (cudaStream_t)stream);
}

static int check_gemv_batched(const void *X, const void *const *Wt, void *const *Y, int nmat, long long M, long long N,
                              long long K, long long ldy, long long x_stride, int elem, const int *status) {
    if (!X || !Wt || !Y || !status) return TMQ_ERR_ARG;
    if (nmat <= 0 || nmat > kBatchMax || M <= 0 || M > 8 || N <= 0 || K <= 0 || ldy < N || x_stride < 0) return TMQ_ERR_ARG;
    if ((K * elem) % 16 != 0 || (x_stride * elem) % 16 != 0) return TMQ_ERR_UNSUPPORTED;
    if (!aligned(X, 16)) return TMQ_ERR_ALIGN;
    for (int j = 0; j < nmat; j++) {
        if (!Wt[j] || !Y[j]) return TMQ_ERR_ARG;
        if (!aligned(Wt[j], 16)) return TMQ_ERR_ALIGN;
    }
    return TMQ_OK;
}

extern "C" int tmq_ternary_gemv_batched_bf16(const void *X, int64_t x_stride, const uint32_t *const *Wt,
                                             const float *const *scale, const float *const *bias, void *const *Y, int nmat,
                                             int64_t M, int64_t N, int64_t K, int64_t ldy, int out_f32, int *status,
                                             void *stream) {
    int rc = check_gemv_batched(X, reinterpret_cast<const void *const *>(Wt), Y, nmat, M, N, K, ldy, x_stride, 2, status);
    if (rc != TMQ_OK) return rc;
    BatchArgs a = {};
    a.X = X; a.x_stride = x_stride * 2;
    for (int j = 0; j < nmat; j++) {
        a.Wt[j] = Wt[j]; a.scale[j] = scale ? scale[j] : nullptr; a.bias[j] = bias ? bias[j] : nullptr; a.Y[j] = Y[j];
    }
    a.M = M; a.N = N; a.K = K; a.KW = prepack_valid_words(K); a.KS = prepack_row_words(K, 0); a.ldy = ldy;
    a.nmat = nmat; a.out_f32 = out_f32; a.status = status;
    return launch_gemv_batched<0>(a, (cudaStream_t)stream);
}

extern "C" int tmq_ternary_gemv_batched_i8(const int8_t *X, int64_t x_stride, const uint32_t *const *Wt, int32_t *const *Y,
                                           int nmat, int64_t M, int64_t N, int64_t K, int64_t ldy, int *status, void *stream) {
    int rc = check_gemv_batched(X, reinterpret_cast<const void *const *>(Wt), reinterpret_cast<void *const *>(Y), nmat, M, N,
                                K, ldy, x_stride, 1, status);
    if (rc != TMQ_OK) return rc;
    BatchArgs a = {};
    a.X = X; a.x_stride = x_stride;
    for (int j = 0; j < nmat; j++) { a.Wt[j] = Wt[j]; a.Y[j] = Y[j]; }
    a.M = M; a.N = N; a.K = K; a.KW = prepack_valid_words(K); a.KS = prepack_row_words(K, 1); a.ldy = ldy;
    a.nmat = nmat; a.status = status;
    return launch_gemv_batched<1>(a, (cudaStream_t)stream);
}
