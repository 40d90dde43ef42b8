// Soft-staircase transfer function for ternary QAT: forward, backward, loss integrand (+ fused reduction),
// its backward, clamp, and the one-pass fusion of all of them.  fp32, HBM-bound streaming kernels.
//
// Arithmetic contract: every operation below is one IEEE round-to-nearest fp32 operation in exactly the order
// PyTorch CPU eager evaluates the reference's formulas (tmq/tmq.py:353-381 sigmoid/dsigmoid/d2sigmoid,
// :417-419 forward, :434-438 backward, :469-473 derivative forward, :488-493 derivative backward).  The
// explicit __f*_rn intrinsics keep the compiler from contracting a multiply and an add into one FMA, which
// would change results by up to 2 ulp of 1.0 and far more relative to outputs near zero.
//
// Layout: flat contiguous fp32.  Each thread keeps U independent 128-bit loads in flight per input stream; one
// block per tile of 256*4*U elements, in address order, streaming cache hints on both sides because no byte is
// touched twice.
#include <math.h>

#include "common.cuh"
#include "softstep_math.cuh"


namespace tmq {

thread_local int g_last_cuda_error = 0;

// ---------------------------------------------------------------------------------------------------- constants

static bool hardness_ok(double d) { return isfinite(d) && d >= 1e-3 && d <= 1e3; }

// A scalar factor is safe for the constant-divisor sequence when products with it stay far from the
// subnormal and overflow ranges (the integrands it multiplies lie in [0, 16]).
static bool factor_ok(float f) {
    float a = fabsf(f);
    return (f == 0.0f && !signbit(f)) || (a >= 1e-15f && a <= 1e15f);
}

struct Args {
    const float *w;
    const float *g;
    float *y;     // forward output
    float *gw;    // gradient output
    float *o;     // materialised loss integrand
    float *wc;    // clamped weights
    size_t n;
    Hardness s;   // hardness of the transfer function (digamma)
    Hardness q;   // hardness of the loss integrand (sharpness)
    float scale;  // gradient scale of the transfer function
    float sd;     // fp32(strength * sharpness)
    float sdd;    // fp32(strength * sharpness * sharpness)
    float gq;     // upstream gradient of the loss term when it is a broadcast scalar
    float lo, hi;
    float one, nzero;  // 1.0f and -0.0f, passed in so the packed FMAs keep operands the assembler cannot fold
    void *scratch;
    double *loss_out;
};

enum : unsigned {
    F_FWD = 1u,       // y
    F_BWD = 2u,       // gw  = scale*g*S'(w)
    F_DFWD = 4u,      // o   = sd*S'_q(w)/D        (materialised)
    F_DBWD = 8u,      // gw  = g*sdd*S''_q(w)/D    (tensor upstream gradient)
    F_QSUM = 16u,     // loss_out = sum o
    F_QGRAD = 32u,    // gw += gq*sdd*S''_q(w)/D   (scalar upstream gradient)
    F_CLAMP = 64u,    // wc
};

// ---------------------------------------------------------------------------------------------------- element math

struct Out {
    float y, gw, o, wc, term;
};

template <unsigned F, bool FAST>
__device__ __forceinline__ Out element(float w, float g, const Args &a) {
    Out r;
    const float fw = floorf(w);
    const float fr = __fsub_rn(w, fw);
    if (F & (F_FWD | F_BWD)) {
        const float t = __fmul_rn(a.s.d, fr);
        const float x = clamp_nan(__fsub_rn(t, a.s.h), -3.0f, 3.0f);
        const float x2 = __fmul_rn(x, x);
        if (F & F_FWD) r.y = softstep_value<FAST>(x, x2, fw, a.s);
        if (F & F_BWD) {
            const float e = __fsub_rn(x2, 9.0f);
            const float n = __fmul_rn(e, e);
            const float b = __fadd_rn(3.0f, x2);
            const float m = __fmul_rn(__fmul_rn(9.0f, b), b);
            const float ds = __fdiv_rn(n, m);
            const float G = div_const<FAST>(__fmul_rn(a.s.d, ds), a.s.D, a.s.rD);
            r.gw = __fmul_rn(__fmul_rn(a.scale, g), G);  // scale is 1.0 in every reference call site; 1*g is exact
        }
    }
    if (F & (F_DFWD | F_DBWD | F_QSUM | F_QGRAD)) {
        const float t = __fmul_rn(a.q.d, fr);
        const float x = clamp_nan(__fsub_rn(t, a.q.h), -3.0f, 3.0f);
        const float x2 = __fmul_rn(x, x);
        if (F & (F_DFWD | F_QSUM)) {
            const float e = __fsub_rn(x2, 9.0f);
            const float n = __fmul_rn(e, e);
            const float b = __fadd_rn(3.0f, x2);
            const float m = __fmul_rn(__fmul_rn(9.0f, b), b);
            const float ds = __fdiv_rn(n, m);
            r.o = div_const<FAST>(__fmul_rn(a.sd, ds), a.q.D, a.q.rD);
            r.term = r.o;
        }
        if (F & (F_DBWD | F_QGRAD)) {
            const float A = __fadd_rn(x2, 3.0f);
            const float i = __fmul_rn(16.0f, x);
            const float j = __fsub_rn(x2, 9.0f);
            const float N2 = __fmul_rn(i, j);
            const float Dd = __fmul_rn(__fmul_rn(__fmul_rn(3.0f, A), A), A);
            const float d2 = __fdiv_rn(N2, Dd);
            const float num = __fmul_rn(a.sdd, d2);
            // num is -0 when the argument sits on the lower clamp; IEEE division keeps that sign
            const float gr = FAST ? copysignf(div_const<true>(num, a.q.D, a.q.rD), num) : __fdiv_rn(num, a.q.D);
            const float up = (F & F_QGRAD) ? a.gq : g;
            const float g2 = __fmul_rn(up, gr);
            r.gw = (F & F_BWD) ? __fadd_rn(r.gw, g2) : g2;
        }
    }
    if (F & F_CLAMP) r.wc = clamp_nan(w, a.lo, a.hi);
    return r;
}

// Two elements at a time on Blackwell's packed fp32 pipe: add/mul/fma.rn.f32x2 round each lane exactly like the
// scalar instruction, so results are unchanged while the issue slots spent on plain arithmetic halve.  Divisions,
// floor, the NaN-propagating min/max and copysign have no packed form and stay per lane.
struct Out2 {
    float2 y, gw, o, wc, term;
};

template <unsigned F, bool FAST>
__device__ __forceinline__ Out2 element2(float2 w, float2 g, const Args &a) {
    Out2 r;
    const float2 ONE = f2(a.one), NZ = f2(a.nzero);
    const float2 fw = make_float2(floorf(w.x), floorf(w.y));
    const float2 fr = __ffma2_rn(fw, f2(-a.one), w);  // w - fw in one rounding
    if (F & (F_FWD | F_BWD)) {
        const float2 t = mul2(f2(a.s.d), fr);
        const float2 x = clamp2(add2(t, f2(-a.s.h)), -3.0f, 3.0f);
        const float2 x2 = mul2(x, x);
        if (F & F_FWD) r.y = softstep_value2<FAST>(x, x2, fw, a.s, ONE, NZ);
        if (F & F_BWD) {
            const float2 e = add2(x2, f2(-9.0f));
            const float2 n = mul2(e, e);
            const float2 b = add2(f2(3.0f), x2);
            const float2 m = mul2(mul2(f2(9.0f), b), b);
            const float2 ds = TMQ_SS_FASTDIV ? div_ranged2(n, m, ONE, NZ) : div2(n, m);
            const float2 G = div_const2<FAST>(mul2(f2(a.s.d), ds), a.s.D, a.s.rD, ONE, NZ);
            r.gw = mul2(mul2(f2(a.scale), g), G);
        }
    }
    if (F & (F_DFWD | F_DBWD | F_QSUM | F_QGRAD)) {
        const float2 t = mul2(f2(a.q.d), fr);
        const float2 x = clamp2(add2(t, f2(-a.q.h)), -3.0f, 3.0f);
        const float2 x2 = mul2(x, x);
        const float2 e = add2(x2, f2(-9.0f));   // x2 - 9
        const float2 b = add2(f2(3.0f), x2);    // 3 + x2 == x2 + 3
        if (F & (F_DFWD | F_QSUM)) {
            const float2 n = mul2(e, e);
            const float2 m = mul2(mul2(f2(9.0f), b), b);
            const float2 ds = TMQ_SS_FASTDIV ? div_ranged2(n, m, ONE, NZ) : div2(n, m);
            r.o = div_const2<FAST>(mul2(f2(a.sd), ds), a.q.D, a.q.rD, ONE, NZ);
            r.term = r.o;
        }
        if (F & (F_DBWD | F_QGRAD)) {
            const float2 i = mul2(f2(16.0f), x);
            const float2 N2 = mul2(i, e);
            const float2 Dd = mul2(mul2(mul2(f2(3.0f), b), b), b);
            float2 d2;
            if (TMQ_SS_FASTDIV) {
                d2 = div_ranged2(N2, Dd, ONE, NZ);
                d2 = make_float2(copysignf(d2.x, N2.x), copysignf(d2.y, N2.y));  // -0 numerators (argument on the lower clamp)
            } else {
                d2 = div2(N2, Dd);
            }
            const float2 num = mul2(f2(a.sdd), d2);
            float2 gr;
            if (FAST) {
                gr = div_const2<true>(num, a.q.D, a.q.rD, ONE, NZ);
                gr = make_float2(copysignf(gr.x, num.x), copysignf(gr.y, num.y));  // keep the sign of a -0 numerator
            } else {
                gr = make_float2(__fdiv_rn(num.x, a.q.D), __fdiv_rn(num.y, a.q.D));
            }
            const float2 up = (F & F_QGRAD) ? f2(a.gq) : g;
            const float2 g2 = mul2(up, gr);
            r.gw = (F & F_BWD) ? add2(r.gw, g2) : g2;
        }
    }
    if (F & F_CLAMP) r.wc = clamp2(w, a.lo, a.hi);
    return r;
}

// ---------------------------------------------------------------------------------------------------- flat kernel

template <int VEC>
struct Pack;
template <>
struct Pack<4> {
    float v[4];
    __device__ __forceinline__ static Pack load(const float *p, size_t i) {
        float4 t = __ldcs(reinterpret_cast<const float4 *>(p) + i);
        Pack r;
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
        return r;
    }
    __device__ __forceinline__ void store(float *p, size_t i) const {
        __stcs(reinterpret_cast<float4 *>(p) + i, make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <>
struct Pack<1> {
    float v[1];
    __device__ __forceinline__ static Pack load(const float *p, size_t i) {
        Pack r;
        r.v[0] = __ldcs(p + i);
        return r;
    }
    __device__ __forceinline__ void store(float *p, size_t i) const { __stcs(p + i, v[0]); }
};

constexpr int kThreads = 256;

#ifndef TMQ_SS_U
#define TMQ_SS_U 4          // 128-bit loads in flight per thread and input stream in the fused kernel
#endif
#ifndef TMQ_SS_TPB
#define TMQ_SS_TPB 2        // consecutive tiles per block
#endif
#ifndef TMQ_SS_PACKED
#define TMQ_SS_PACKED 1     // arithmetic on the packed f32x2 pipe, two elements per instruction
#endif
#ifndef TMQ_SS_FASTDIV
#define TMQ_SS_FASTDIV 1    // range-specialised division for the data-dependent quotients of the packed path
#endif
#ifndef TMQ_SS_MINB
#define TMQ_SS_MINB 4       // min resident blocks per SM handed to __launch_bounds__
#endif

template <unsigned F, int VEC, int U>
struct Tile {
    static constexpr bool NEED_G = (F & (F_BWD | F_DBWD)) != 0;
    Pack<VEC> w[U], g[U];
    __device__ __forceinline__ void load(const Args &a, size_t tile, size_t nv) {
        const size_t base = tile * ((size_t)kThreads * U) + threadIdx.x;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const size_t i = base + (size_t)u * kThreads;
            if (i < nv) {
                w[u] = Pack<VEC>::load(a.w, i);
                if (NEED_G) g[u] = Pack<VEC>::load(a.g, i);
            }
        }
    }
    template <bool FAST>
    __device__ __forceinline__ void process(const Args &a, size_t tile, size_t nv, double &acc) const {
        constexpr bool SUM = (F & F_QSUM) != 0;
        const size_t base = tile * ((size_t)kThreads * U) + threadIdx.x;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const size_t i = base + (size_t)u * kThreads;
            if (i < nv) {
                Pack<VEC> y, gw, o, wc;
                float part = 0.0f;
                if (VEC == 4 && TMQ_SS_PACKED) {
#pragma unroll
                    for (int k = 0; k < VEC; k += 2) {
                        const float2 gg = NEED_G ? make_float2(g[u].v[k], g[u].v[k + 1 < VEC ? k + 1 : k]) : f2(0.0f);
                        Out2 r = element2<F, FAST>(make_float2(w[u].v[k], w[u].v[k + 1 < VEC ? k + 1 : k]), gg, a);
                        const int k1 = k + 1 < VEC ? k + 1 : k;
                        if (F & F_FWD) { y.v[k] = r.y.x; y.v[k1] = r.y.y; }
                        if (F & (F_BWD | F_DBWD | F_QGRAD)) { gw.v[k] = r.gw.x; gw.v[k1] = r.gw.y; }
                        if (F & F_DFWD) { o.v[k] = r.o.x; o.v[k1] = r.o.y; }
                        if (F & F_CLAMP) { wc.v[k] = r.wc.x; wc.v[k1] = r.wc.y; }
                        if (SUM) {  // same association as the scalar path: ((t0+t1)+t2)+t3
                            part = (k == 0) ? __fadd_rn(r.term.x, r.term.y) : __fadd_rn(__fadd_rn(part, r.term.x), r.term.y);
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; k++) {
                        Out r = element<F, FAST>(w[u].v[k], NEED_G ? g[u].v[k] : 0.0f, a);
                        if (F & F_FWD) y.v[k] = r.y;
                        if (F & (F_BWD | F_DBWD | F_QGRAD)) gw.v[k] = r.gw;
                        if (F & F_DFWD) o.v[k] = r.o;
                        if (F & F_CLAMP) wc.v[k] = r.wc;
                        if (SUM) part = (k == 0) ? r.term : __fadd_rn(part, r.term);
                    }
                }
                if (F & F_FWD) y.store(a.y, i);
                if (F & (F_BWD | F_DBWD | F_QGRAD)) gw.store(a.gw, i);
                if (F & F_DFWD) o.store(a.o, i);
                if (F & F_CLAMP) wc.store(a.wc, i);
                if (SUM) acc += (double)part;
            }
        }
    }
};

template <unsigned F, int VEC, int U, bool FAST>
__global__ void __launch_bounds__(kThreads, TMQ_SS_MINB) softstep_kernel(const Args a) {
    constexpr bool NEED_G = (F & (F_BWD | F_DBWD)) != 0;
    constexpr bool SUM = (F & F_QSUM) != 0;
    const size_t nv = a.n / VEC;  // whole vectors
    const size_t ntiles = (nv + (size_t)kThreads * U - 1) / ((size_t)kThreads * U);
    double acc = 0.0;

    // Blocks take TMQ_SS_TPB consecutive tiles each, in address order (more only beyond kMaxPartials blocks).
    const size_t per_block = (ntiles + gridDim.x - 1) / gridDim.x;
    size_t tile = (size_t)blockIdx.x * per_block;
    const size_t tile_end = (tile + per_block < ntiles) ? tile + per_block : ntiles;
    for (; tile < tile_end; tile++) {
        Tile<F, VEC, U> A;
        A.load(a, tile, nv);
        A.template process<FAST>(a, tile, nv, acc);
    }
    // ragged tail (n not a multiple of VEC): the first few threads of block 0, scalar
    if (VEC > 1 && blockIdx.x == 0) {
        const size_t i = nv * VEC + threadIdx.x;
        if (i < a.n) {
            Out r = element<F, FAST>(a.w[i], NEED_G ? a.g[i] : 0.0f, a);
            if (F & F_FWD) a.y[i] = r.y;
            if (F & (F_BWD | F_DBWD | F_QGRAD)) a.gw[i] = r.gw;
            if (F & F_DFWD) a.o[i] = r.o;
            if (F & F_CLAMP) a.wc[i] = r.wc;
            if (SUM) acc += (double)r.term;
        }
    }
    if (SUM) {
        __shared__ double red[8];
        double total = block_sum_256(acc, red);
        grid_sum_finish(total, a.scratch, a.loss_out, red);
    }
}

template <unsigned F, int VEC, int U, bool FAST>
static int launch_flat(const Args &a, cudaStream_t st) {
    const size_t nv = a.n / VEC;
    size_t ntiles = (nv + (size_t)kThreads * U - 1) / ((size_t)kThreads * U);
    if (ntiles == 0) ntiles = 1;
    const size_t cap = (F & F_QSUM) ? (size_t)kMaxPartials : (size_t)0x7FFFFFFF;
    size_t blocks = (ntiles + TMQ_SS_TPB - 1) / TMQ_SS_TPB;
    const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
    softstep_kernel<F, VEC, U, FAST><<<grid, kThreads, 0, st>>>(a);
    return launch_status();
}

template <unsigned F, int U>
static int dispatch(const Args &a, bool vec_ok, bool fast_ok, cudaStream_t st) {
    if (vec_ok) return fast_ok ? launch_flat<F, 4, U, true>(a, st) : launch_flat<F, 4, U, false>(a, st);
    return fast_ok ? launch_flat<F, 1, 4, true>(a, st) : launch_flat<F, 1, 4, false>(a, st);
}

// ---------------------------------------------------------------------------------------------------- multi-tensor

constexpr int kChunk = 4096;  // elements per chunk: 256 threads x 4 x float4

struct MtTensor {
    const float *w;
    float *out;
    unsigned long long n;
    unsigned long long out_offset;
};
struct MtChunk {
    unsigned tensor;
    unsigned index;  // chunk number inside the tensor
};

template <unsigned F, bool FAST>
__global__ void __launch_bounds__(kThreads) softstep_mt_kernel(const MtTensor *__restrict__ tensors,
                                                                const MtChunk *__restrict__ chunks, int nchunks,
                                                                Args a, const float *__restrict__ upstream,
                                                                float *__restrict__ out_base) {
    constexpr bool SUM = (F & F_QSUM) != 0;
    double acc = 0.0;
    const float up = (F & F_QGRAD) ? (upstream ? *upstream : 1.0f) : 0.0f;
    for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const MtChunk ch = chunks[c];
        const MtTensor t = tensors[ch.tensor];
        const size_t begin = (size_t)ch.index * kChunk;
        const size_t count = (t.n - begin) < (size_t)kChunk ? (size_t)(t.n - begin) : (size_t)kChunk;
        const float *w = t.w + begin;
        float *out = (F & F_CLAMP) ? const_cast<float *>(t.w) + begin
                                   : (out_base ? out_base + t.out_offset : t.out) + begin;
        if (F & F_QGRAD) a.gq = __fdiv_rn(up, (float)t.n);  // what autograd's mean backward hands down
        double csum = 0.0;
        const size_t nv = count / 4;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const size_t i = threadIdx.x + (size_t)u * kThreads;
            if (i < nv) {
                float4 wv = __ldg(reinterpret_cast<const float4 *>(w) + i);
                float in[4] = {wv.x, wv.y, wv.z, wv.w}, res[4];
                float part = 0.0f;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    Out r = element<F, FAST>(in[k], 0.0f, a);
                    res[k] = (F & F_CLAMP) ? r.wc : r.gw;
                    if (SUM) part = (k == 0) ? r.term : __fadd_rn(part, r.term);
                }
                if (F & (F_CLAMP | F_QGRAD))
                    reinterpret_cast<float4 *>(out)[i] = make_float4(res[0], res[1], res[2], res[3]);
                if (SUM) csum += (double)part;
            }
        }
        const size_t i = nv * 4 + threadIdx.x;
        if (i < count) {
            Out r = element<F, FAST>(w[i], 0.0f, a);
            if (F & (F_CLAMP | F_QGRAD)) out[i] = (F & F_CLAMP) ? r.wc : r.gw;
            if (SUM) csum += (double)r.term;
        }
        if (SUM) acc += csum / (double)t.n;  // contribution to this tensor's mean
    }
    if (SUM) {
        __shared__ double red[8];
        double total = block_sum_256(acc, red);
        grid_sum_finish(total, a.scratch, a.loss_out, red);
    }
}

// ---------------------------------------------------------------------------------------------------- fused optimizer

// Adam update of every tensor of a plan in one launch, optionally followed by the clamp of the QAT step, so that the
// weights are read and written once for both: per element 16 bytes read (w, g, m, v) and 12 written (w, m, v).
// The plan's `out` field of a tensor carries its GRADIENT, `out_offset` its slice of the flat moment buffers.
// Arithmetic: torch.optim.Adam's single-tensor sequence (torch/optim/adam.py, _single_tensor_adam) in fp32, one rounding
// per operation:   m += (g - m) * (1 - b1);  v = v * b2 + ((1 - b2) * g) * g;
//                  w += -(lr / (1 - b1^t)) * (m / (sqrt(v) / sqrt(1 - b2^t) + eps));   w = clamp(w, lo, hi)
struct AdamArgs {
    float w1, b2, w2, bc2_sqrt, eps, neg_step, lo, hi;
    int clamp;
};

__global__ void __launch_bounds__(kThreads) adam_clamp_mt_kernel(const MtTensor *__restrict__ tensors,
                                                                  const MtChunk *__restrict__ chunks, int nchunks,
                                                                  float *__restrict__ m_base, float *__restrict__ v_base,
                                                                  const AdamArgs a) {
    auto update = [&](float &w, float g, float &m, float &v) {
        m = __fadd_rn(m, __fmul_rn(__fsub_rn(g, m), a.w1));
        v = __fadd_rn(__fmul_rn(v, a.b2), __fmul_rn(__fmul_rn(a.w2, g), g));
        const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), a.bc2_sqrt), a.eps);
        w = __fadd_rn(w, __fmul_rn(a.neg_step, __fdiv_rn(m, denom)));
        if (a.clamp) w = clamp_nan(w, a.lo, a.hi);
    };
    for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const MtChunk ch = chunks[c];
        const MtTensor t = tensors[ch.tensor];
        const size_t begin = (size_t)ch.index * kChunk;
        const size_t count = (t.n - begin) < (size_t)kChunk ? (size_t)(t.n - begin) : (size_t)kChunk;
        float *w = const_cast<float *>(t.w) + begin;
        const float *g = t.out + begin;
        float *m = m_base + t.out_offset + begin, *v = v_base + t.out_offset + begin;
        const size_t nv = count / 4;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const size_t i = threadIdx.x + (size_t)u * kThreads;
            if (i < nv) {
                float4 wv = reinterpret_cast<float4 *>(w)[i], gv = __ldg(reinterpret_cast<const float4 *>(g) + i);
                float4 mv = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
                update(wv.x, gv.x, mv.x, vv.x);
                update(wv.y, gv.y, mv.y, vv.y);
                update(wv.z, gv.z, mv.z, vv.z);
                update(wv.w, gv.w, mv.w, vv.w);
                reinterpret_cast<float4 *>(w)[i] = wv;
                reinterpret_cast<float4 *>(m)[i] = mv;
                reinterpret_cast<float4 *>(v)[i] = vv;
            }
        }
        const size_t i = nv * 4 + threadIdx.x;
        if (i < count) update(w[i], g[i], m[i], v[i]);
    }
}

extern "C" int tmq_mt_adam_clamp(const void *d_plan, int ntensors, int nchunks, float *m_base, float *v_base, double lr,
                                 double beta1, double beta2, double eps, long long step, int clamp, float lo, float hi,
                                 void *stream) {
    if (!d_plan || ntensors <= 0 || nchunks <= 0 || !m_base || !v_base || step < 1) return TMQ_ERR_ARG;
    if (!(lr >= 0.0) || !(beta1 >= 0.0 && beta1 < 1.0) || !(beta2 >= 0.0 && beta2 < 1.0) || !(eps >= 0.0)) return TMQ_ERR_ARG;
    if (clamp && !(lo <= hi)) return TMQ_ERR_ARG;
    if (!aligned(d_plan, 8) || !aligned(m_base, 16) || !aligned(v_base, 16)) return TMQ_ERR_ALIGN;
    // scalars as torch forms them: Python doubles, cast to the tensors' fp32 inside the kernel
    const double bc1 = 1.0 - pow(beta1, (double)step), bc2 = 1.0 - pow(beta2, (double)step);
    AdamArgs a;
    a.w1 = (float)(1.0 - beta1);
    a.b2 = (float)beta2;
    a.w2 = (float)(1.0 - beta2);
    a.bc2_sqrt = (float)sqrt(bc2);
    a.eps = (float)eps;
    a.neg_step = (float)(-(lr / bc1));
    a.lo = lo; a.hi = hi; a.clamp = clamp;
    const MtTensor *T = reinterpret_cast<const MtTensor *>(d_plan);
    const MtChunk *C = reinterpret_cast<const MtChunk *>(T + ntensors);
    const unsigned grid = (unsigned)(nchunks < kMaxPartials ? nchunks : kMaxPartials);
    adam_clamp_mt_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(T, C, nchunks, m_base, v_base, a);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------------- self-test

__global__ void const_div_selftest_kernel(float D, float rD, unsigned long long *mismatches) {
    // exponents 2^-60 .. 2^60 (biased 67..187), both signs, every mantissa
    const unsigned long long total = 121ull << 24;  // 121 exponents x 2 signs x 2^23 mantissas
    unsigned long long bad = 0;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < total;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned mant = (unsigned)(i & 0x7FFFFFu);
        const unsigned sign = (unsigned)((i >> 23) & 1u);
        const unsigned expo = 67u + (unsigned)(i >> 24);
        const float a = __uint_as_float((sign << 31) | (expo << 23) | mant);
        const float fast = div_const<true>(a, D, rD);
        const float exact = __fdiv_rn(a, D);
        bad += (__float_as_uint(fast) != __float_as_uint(exact));
    }
    bad = (unsigned long long)__reduce_add_sync(0xffffffffu, (unsigned)bad);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(mismatches, bad);
}

// Compares div_ranged with IEEE division: every denominator bit pattern of the binades [2^lo_exp, 2^hi_exp), each with
// `per_b` numerators (mantissas from a counter-based hash, or - when per_b == 2^23 - every mantissa), numerator exponent
// fixed at 2^0 and both signs alternating (the sequence is scale-invariant in the numerator barring under/overflow).
__global__ void div_selftest_kernel(int lo_exp, int hi_exp, unsigned per_b, unsigned long long b_begin,
                                    unsigned long long b_count, unsigned long long *mismatches) {
    unsigned long long bad = 0;
    const unsigned long long total = b_count * per_b;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < total;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long bi = b_begin + i / per_b;
        const unsigned ai = (unsigned)(i % per_b);
        const unsigned bexp = (unsigned)(127 + lo_exp) + (unsigned)(bi >> 23);
        const float b = __uint_as_float((bexp << 23) | (unsigned)(bi & 0x7FFFFFu));
        unsigned mant;
        if (per_b == (1u << 23)) {
            mant = ai;
        } else {
            unsigned h = ai * 0x9E3779B1u ^ (unsigned)(bi * 0x85EBCA77ull);
            h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12;
            mant = h & 0x7FFFFFu;
        }
        const float a = __uint_as_float(((ai & 1u) << 31) | (127u << 23) | mant);
        bad += (__float_as_uint(div_ranged(a, b)) != __float_as_uint(__fdiv_rn(a, b)));
    }
    (void)hi_exp;
    bad = (unsigned long long)__reduce_add_sync(0xffffffffu, (unsigned)bad);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(mismatches, bad);
}

}  // namespace tmq

// ---------------------------------------------------------------------------------------------------- C ABI

using namespace tmq;

static bool vec_ok(std::initializer_list<const void *> ptrs) {
    for (const void *p : ptrs)
        if (p && !aligned(p, 16)) return false;
    return true;
}
static bool ptr_ok(std::initializer_list<const void *> ptrs) {
    for (const void *p : ptrs)
        if (!p || !aligned(p, 4)) return false;
    return true;
}

extern "C" int tmq_softstep_fwd(const float *w, float *y, size_t n, double digamma, void *stream) {
    if (n == 0) return TMQ_OK;
    if (!hardness_ok(digamma)) return TMQ_ERR_ARG;
    if (!w || !y) return TMQ_ERR_ARG;
    if (!ptr_ok({w, y})) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.y = y; a.n = n; a.s = make_hardness(digamma);
    return dispatch<F_FWD, 4>(a, vec_ok({w, y}), true, (cudaStream_t)stream);
}

extern "C" int tmq_softstep_bwd(const float *w, const float *g, float *gw, size_t n, double digamma, double scale,
                                void *stream) {
    if (n == 0) return TMQ_OK;
    if (!hardness_ok(digamma) || !isfinite(scale)) return TMQ_ERR_ARG;
    if (!w || !g || !gw) return TMQ_ERR_ARG;
    if (!ptr_ok({w, g, gw})) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.g = g; a.gw = gw; a.n = n; a.s = make_hardness(digamma); a.scale = (float)scale;
    return dispatch<F_BWD, 4>(a, vec_ok({w, g, gw}), true, (cudaStream_t)stream);
}

extern "C" int tmq_softstep_deriv_fwd(const float *w, float *o, size_t n, double digamma, double strength,
                                      void *stream) {
    if (n == 0) return TMQ_OK;
    if (!hardness_ok(digamma) || !isfinite(strength)) return TMQ_ERR_ARG;
    if (!w || !o) return TMQ_ERR_ARG;
    if (!ptr_ok({w, o})) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.o = o; a.n = n; a.q = make_hardness(digamma); a.sd = (float)(strength * digamma);
    return dispatch<F_DFWD, 4>(a, vec_ok({w, o}), factor_ok(a.sd), (cudaStream_t)stream);
}

extern "C" int tmq_softstep_deriv_bwd(const float *w, const float *g, float *gw, size_t n, double digamma,
                                      double strength, void *stream) {
    if (n == 0) return TMQ_OK;
    if (!hardness_ok(digamma) || !isfinite(strength)) return TMQ_ERR_ARG;
    if (!w || !g || !gw) return TMQ_ERR_ARG;
    if (!ptr_ok({w, g, gw})) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.g = g; a.gw = gw; a.n = n; a.q = make_hardness(digamma);
    a.sdd = (float)(strength * digamma * digamma);
    return dispatch<F_DBWD, 4>(a, vec_ok({w, g, gw}), factor_ok(a.sdd), (cudaStream_t)stream);
}

extern "C" int tmq_clamp(const float *w, float *out, size_t n, float lo, float hi, void *stream) {
    if (n == 0) return TMQ_OK;
    if (!w || !out || !(lo <= hi)) return TMQ_ERR_ARG;
    if (!ptr_ok({w, out})) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.wc = out; a.n = n; a.lo = lo; a.hi = hi;
    return dispatch<F_CLAMP, 4>(a, vec_ok({w, out}), true, (cudaStream_t)stream);
}

extern "C" size_t tmq_reduce_scratch_bytes(void) { return kScratchBytes; }

extern "C" int tmq_qloss_sum(const float *w, size_t n, double sharpness, double strength, double *sum_out,
                             void *scratch, size_t scratch_bytes, void *stream) {
    if (!hardness_ok(sharpness) || !isfinite(strength)) return TMQ_ERR_ARG;
    if (!w || !sum_out || !scratch) return TMQ_ERR_ARG;
    if (scratch_bytes < kScratchBytes) return TMQ_ERR_SCRATCH;
    if (!ptr_ok({w}) || !aligned(sum_out, 8) || !aligned(scratch, 256)) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.n = n; a.q = make_hardness(sharpness); a.sd = (float)(strength * sharpness);
    a.scratch = scratch; a.loss_out = sum_out;
    return dispatch<F_QSUM, 4>(a, vec_ok({w}), factor_ok(a.sd), (cudaStream_t)stream);
}

extern "C" int tmq_softstep_fused_step(const float *w, const float *g, float *y, float *gw, float *wc,
                                       double *loss_sum, size_t n, double digamma, double scale, double sharpness,
                                       double strength, float gq, float lo, float hi, void *scratch,
                                       size_t scratch_bytes, void *stream) {
    if (!hardness_ok(digamma) || !hardness_ok(sharpness) || !isfinite(strength) || !isfinite(scale) || !(lo <= hi))
        return TMQ_ERR_ARG;
    if (!w || !g || !y || !gw || !wc || !loss_sum || !scratch) return TMQ_ERR_ARG;
    if (scratch_bytes < kScratchBytes) return TMQ_ERR_SCRATCH;
    if (!ptr_ok({w, g, y, gw, wc}) || !aligned(loss_sum, 8) || !aligned(scratch, 256)) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.w = w; a.g = g; a.y = y; a.gw = gw; a.wc = wc; a.n = n;
    a.s = make_hardness(digamma); a.q = make_hardness(sharpness);
    a.scale = (float)scale; a.sd = (float)(strength * sharpness); a.sdd = (float)(strength * sharpness * sharpness);
    a.gq = gq; a.lo = lo; a.hi = hi; a.scratch = scratch; a.loss_out = loss_sum;
    constexpr unsigned F = F_FWD | F_BWD | F_QSUM | F_QGRAD | F_CLAMP;
    return dispatch<F, TMQ_SS_U>(a, vec_ok({w, g, y, gw, wc}), factor_ok(a.sd) && factor_ok(a.sdd), (cudaStream_t)stream);
}

// ---- multi-tensor plan: [MtTensor x ntensors][MtChunk x nchunks]

static size_t mt_chunks(const tmq_mt_tensor *t, int n) {
    size_t c = 0;
    for (int i = 0; i < n; i++) c += (size_t)((t[i].n + kChunk - 1) / kChunk);
    return c;
}

extern "C" size_t tmq_mt_plan_bytes(const tmq_mt_tensor *tensors, int ntensors) {
    if (!tensors || ntensors <= 0) return 0;
    return sizeof(MtTensor) * (size_t)ntensors + sizeof(MtChunk) * mt_chunks(tensors, ntensors);
}

extern "C" int tmq_mt_plan_build(const tmq_mt_tensor *tensors, int ntensors, void *host_plan, size_t plan_bytes,
                                 int *nchunks) {
    if (!tensors || ntensors <= 0 || !host_plan || !nchunks) return TMQ_ERR_ARG;
    const size_t nc = mt_chunks(tensors, ntensors);
    if (nc > 0x7FFFFFFFull) return TMQ_ERR_UNSUPPORTED;
    if (plan_bytes < sizeof(MtTensor) * (size_t)ntensors + sizeof(MtChunk) * nc) return TMQ_ERR_SCRATCH;
    MtTensor *T = reinterpret_cast<MtTensor *>(host_plan);
    MtChunk *C = reinterpret_cast<MtChunk *>(T + ntensors);
    size_t k = 0;
    for (int i = 0; i < ntensors; i++) {
        if (!tensors[i].w || tensors[i].n == 0) return TMQ_ERR_ARG;
        if (!aligned(tensors[i].w, 16) || (tensors[i].out && !aligned(tensors[i].out, 16))) return TMQ_ERR_ALIGN;
        if (tensors[i].out_offset % 4 != 0) return TMQ_ERR_ALIGN;
        T[i].w = tensors[i].w; T[i].out = tensors[i].out; T[i].n = tensors[i].n; T[i].out_offset = tensors[i].out_offset;
        const unsigned cnt = (unsigned)((tensors[i].n + kChunk - 1) / kChunk);
        for (unsigned c = 0; c < cnt; c++) { C[k].tensor = (unsigned)i; C[k].index = c; k++; }
    }
    *nchunks = (int)nc;
    return TMQ_OK;
}

template <unsigned F>
static int launch_mt(const void *d_plan, int ntensors, int nchunks, Args a, const float *up, float *out_base, bool fast,
                     cudaStream_t st) {
    if (!d_plan || ntensors <= 0 || nchunks <= 0) return TMQ_ERR_ARG;
    if (!aligned(d_plan, 8)) return TMQ_ERR_ALIGN;
    const MtTensor *T = reinterpret_cast<const MtTensor *>(d_plan);
    const MtChunk *C = reinterpret_cast<const MtChunk *>(T + ntensors);
    const unsigned grid = (unsigned)(nchunks < kMaxPartials ? nchunks : kMaxPartials);
    if (fast) softstep_mt_kernel<F, true><<<grid, kThreads, 0, st>>>(T, C, nchunks, a, up, out_base);
    else softstep_mt_kernel<F, false><<<grid, kThreads, 0, st>>>(T, C, nchunks, a, up, out_base);
    return launch_status();
}

extern "C" int tmq_mt_qloss(const void *d_plan, int ntensors, int nchunks, double sharpness, double strength,
                            double *loss_out, void *scratch, size_t scratch_bytes, void *stream) {
    if (!hardness_ok(sharpness) || !isfinite(strength) || !loss_out || !scratch) return TMQ_ERR_ARG;
    if (scratch_bytes < kScratchBytes) return TMQ_ERR_SCRATCH;
    if (!aligned(loss_out, 8) || !aligned(scratch, 256)) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.q = make_hardness(sharpness); a.sd = (float)(strength * sharpness); a.scratch = scratch; a.loss_out = loss_out;
    return launch_mt<F_QSUM>(d_plan, ntensors, nchunks, a, nullptr, nullptr, factor_ok(a.sd), (cudaStream_t)stream);
}

extern "C" int tmq_mt_qloss_bwd(const void *d_plan, int ntensors, int nchunks, double sharpness, double strength,
                                const float *d_upstream, float *out_base, void *stream) {
    if (!hardness_ok(sharpness) || !isfinite(strength)) return TMQ_ERR_ARG;
    if (out_base && !aligned(out_base, 16)) return TMQ_ERR_ALIGN;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.q = make_hardness(sharpness); a.sdd = (float)(strength * sharpness * sharpness);
    return launch_mt<F_QGRAD>(d_plan, ntensors, nchunks, a, d_upstream, out_base, factor_ok(a.sdd), (cudaStream_t)stream);
}

extern "C" int tmq_mt_clamp(const void *d_plan, int ntensors, int nchunks, float lo, float hi, void *stream) {
    if (!(lo <= hi)) return TMQ_ERR_ARG;
    Args a = {};
    a.one = 1.0f; a.nzero = -0.0f;
    a.lo = lo; a.hi = hi;
    return launch_mt<F_CLAMP>(d_plan, ntensors, nchunks, a, nullptr, nullptr, true, (cudaStream_t)stream);
}

extern "C" int tmq_selftest_div(unsigned per_b, unsigned long long b_begin, unsigned long long b_count,
                                unsigned long long *mismatches, void *stream) {
    // denominators of the soft-step quotients live in [27, 5184]: binades 2^4 .. 2^13
    const unsigned long long all_b = 9ull << 23;
    if (!mismatches || per_b == 0 || per_b > (1u << 23) || b_begin >= all_b || b_count == 0 || b_begin + b_count > all_b)
        return TMQ_ERR_ARG;
    div_selftest_kernel<<<kNumSMs * 16, 256, 0, (cudaStream_t)stream>>>(4, 13, per_b, b_begin, b_count, mismatches);
    return launch_status();
}

extern "C" int tmq_selftest_const_div(double digamma, unsigned long long *mismatches, void *stream) {
    if (!hardness_ok(digamma) || !mismatches) return TMQ_ERR_ARG;
    Hardness h = make_hardness(digamma);
    const_div_selftest_kernel<<<kNumSMs * 8, 256, 0, (cudaStream_t)stream>>>(h.D, h.rD, mismatches);
    return launch_status();
}
