/* tmq_b200 -- C ABI of the B200 (sm_100a) kernels behind TMQ's two data-parallel hot paths.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, a cudaStream_t),
 * returns an int status (0 = TMQ_OK, negative = error), never allocates device memory, never synchronises
 * and never throws.  Work is enqueued on the given stream; outputs are valid once that stream reaches them.
 *
 * "replaces:" names the reference interface an entry point stands in for, as file:line of the reference
 * project (mtnwrw/tmq).
 */
#ifndef TMQ_B200_H
#define TMQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TMQ_OK 0
#define TMQ_ERR_ARG (-1)         /* null pointer, bad size, unsupported combination              */
#define TMQ_ERR_ALIGN (-2)       /* a pointer misses the alignment the entry point documents      */
#define TMQ_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch (see tmq_last_cuda_error) */
#define TMQ_ERR_TIMEOUT (-4)     /* a bounded device-side wait ran out                            */
#define TMQ_ERR_SCRATCH (-5)     /* scratch buffer too small                                      */
#define TMQ_ERR_UNSUPPORTED (-6) /* shape outside what the kernel family covers                   */

const char *tmq_status_string(int status);
int tmq_last_cuda_error(void);  /* cudaError_t of the most recent failed runtime call on this thread, 0 if none */
int tmq_abi_version(void);

/* ------------------------------------------------------------------------------------------------
 * Hot path 1: soft-staircase transfer function, fp32, flat contiguous tensors of n elements.
 * Arithmetic follows the reference's PyTorch-CPU-eager formulas operation by operation (one IEEE
 * rounding each, no FMA contraction); the host scalars d, d/2 and 2*sigma(d/2) are derived from the
 * double `digamma` exactly as Python derives them.  Pointers need 4-byte alignment; 16-byte aligned
 * pointers take the 128-bit vector path.
 * ------------------------------------------------------------------------------------------------ */

/* y = softstep(w; digamma).  replaces: fwd_softstep, tmq/tmq_cuda.cu:740-764 (kernel :80-92), tmq/tmq.py:404-419 */
int tmq_softstep_fwd(const float *w, float *y, size_t n, double digamma, void *stream);

/* gw = scale * g * softstep'(w).  replaces: bwd_softstep, tmq/tmq_cuda.cu:768-794 (kernel :95-110), tmq/tmq.py:422-438 */
int tmq_softstep_bwd(const float *w, const float *g, float *gw, size_t n, double digamma, double scale, void *stream);

/* o = strength * softstep'(w; digamma)  (the quantization-loss integrand).
 * replaces: fwd_softstep_derivative, tmq/tmq_cuda.cu:690-709 (kernel :45-59), tmq/tmq.py:456-473 */
int tmq_softstep_deriv_fwd(const float *w, float *o, size_t n, double digamma, double strength, void *stream);

/* gw = g * strength * softstep''(w; digamma).
 * replaces: bwd_softstep_derivative, tmq/tmq_cuda.cu:713-735 (kernel :63-77), tmq/tmq.py:475-493 */
int tmq_softstep_deriv_bwd(const float *w, const float *g, float *gw, size_t n, double digamma, double strength,
                           void *stream);

/* out = min(max(w, lo), hi); out may alias w.  replaces: torch.clamp in Linear.clamp / Conv2d.clamp, tmq/tmq.py:691-696, :874-879 */
int tmq_clamp(const float *w, float *out, size_t n, float lo, float hi, void *stream);

/* Scratch for the deterministic two-stage reductions below: tmq_reduce_scratch_bytes() bytes of device memory,
 * 256-byte aligned, zero-filled ONCE before first use (the kernels leave it zeroed again).  Calls that share
 * one scratch buffer must be ordered on one stream. */
size_t tmq_reduce_scratch_bytes(void);

/* *sum_out (device, fp64) = sum_i strength * softstep'(w_i; sharpness), without materialising the integrand.
 * replaces: torch.mean(SoftStepDerivative.apply(...)) numerator, tmq/tmq.py:698-699, :889-891 */
int tmq_qloss_sum(const float *w, size_t n, double sharpness, double strength, double *sum_out, void *scratch,
                  size_t scratch_bytes, void *stream);

/* Same result as tmq_qloss_sum for callers that cannot hand over a scratch buffer because they cannot allocate
 * device memory at all (hosts whose device memory was partitioned once at start-up, plug-ins inside a framework
 * that owns the whole pool, paths where cudaMalloc is off limits because it may stall the device).  The scratch is
 * a fixed 33 KB array inside the library image, resident on every GPU that loads the library.  No counterpart in
 * the reference.  Limits: n <= TMQ_QLOSS_NOALLOC_MAX_ELEMS, else TMQ_ERR_SCRATCH and nothing runs.  All calls on a
 * GPU share that one array (each call re-zeroes what must start at zero), so calls whose kernels could overlap on
 * the GPU race with each other: keep them ordered.  The first call on each device also resolves the array's device
 * address; issue that first call before any stream capture begins. */
#define TMQ_QLOSS_NOALLOC_MAX_ELEMS 33554432ull
int tmq_qloss_sum_noalloc(const float *w, size_t n, double sharpness, double strength, double *sum_out, void *stream);

/* One pass over a weight tensor doing everything the QAT step does to it elementwise:
 *   y   = softstep(w; digamma)                                         (forward,            tmq/tmq.py:417-419)
 *   gw  = scale*g*softstep'(w; digamma) + gq*strength*softstep''(w; sharpness)
 *                                                                      (both backward terms, tmq/tmq.py:434-438, :488-493)
 *   *loss_sum = sum_i strength*softstep'(w_i; sharpness)               (loss numerator,     tmq/tmq.py:469-473, :698-699)
 *   wc  = clamp(w, lo, hi)                                             (tmq/tmq.py:696)
 * gq is the upstream gradient of the mean (1/n for a plain sum of layer losses).  Reads 8 and writes 12 bytes per element. */
int tmq_softstep_fused_step(const float *w, const float *g, float *y, float *gw, float *wc, double *loss_sum, size_t n,
                            double digamma, double scale, double sharpness, double strength, float gq, float lo,
                            float hi, void *scratch, size_t scratch_bytes, void *stream);

/* Multi-tensor forms: one launch over every registered layer (tmq/tmq.py:263-272, :298-310 loop over layers).
 * A plan is a host-built table the caller uploads once to device memory (8-byte aligned) and reuses. */
typedef struct {
    const float *w;      /* weights (device)                                                        */
    float *out;          /* per-tensor output (gradient for qloss_bwd), used when out_base is NULL   */
    uint64_t n;          /* elements                                                                */
    uint64_t out_offset; /* element offset of this tensor's output inside out_base (multiple of 4)  */
} tmq_mt_tensor;

size_t tmq_mt_plan_bytes(const tmq_mt_tensor *tensors, int ntensors);
/* Fills host_plan (tmq_mt_plan_bytes bytes); *nchunks receives the launch extent to pass back below. */
int tmq_mt_plan_build(const tmq_mt_tensor *tensors, int ntensors, void *host_plan, size_t plan_bytes, int *nchunks);
/* *loss_out (device fp64) = sum_l mean_i(strength*softstep'(w_li; sharpness)) */
int tmq_mt_qloss(const void *d_plan, int ntensors, int nchunks, double sharpness, double strength, double *loss_out,
                 void *scratch, size_t scratch_bytes, void *stream);
/* out_l = (upstream / n_l) * strength * softstep''(w_l; sharpness); d_upstream: device fp32 scalar or NULL (= 1).
 * Outputs go to out_base + out_offset_l when out_base is given (a fresh flat buffer per call, 16-byte aligned),
 * else to the per-tensor pointers stored in the plan. */
int tmq_mt_qloss_bwd(const void *d_plan, int ntensors, int nchunks, double sharpness, double strength,
                     const float *d_upstream, float *out_base, void *stream);
/* Fused optimizer of the QAT step: torch.optim.Adam's update (single-tensor sequence, fp32, one rounding per operation)
 * of every tensor of a plan in one launch, followed by clamp(w, lo, hi) when `clamp` is set - the optimizer step and
 * QuantizationControl.clamp (tmq/tmq.py:263-272) read and write the weights once between them.  In THIS plan a tensor's
 * `out` field is its gradient and `out_offset` its slice of the flat moment buffers m_base / v_base (exp_avg,
 * exp_avg_sq); `step` is the 1-based step count of the bias corrections. */
int tmq_mt_adam_clamp(const void *d_plan, int ntensors, int nchunks, float *m_base, float *v_base, double lr, double beta1,
                      double beta2, double eps, long long step, int clamp, float lo, float hi, void *stream);
/* w_l = clamp(w_l, lo, hi) in place */
int tmq_mt_clamp(const void *d_plan, int ntensors, int nchunks, float lo, float hi, void *stream);

/* Device self-check of the constant-divisor fast path used inside the kernels above: counts, over every finite
 * fp32 numerator with |a| in [2^-60, 2^60], results that differ from IEEE division by 2*sigma(digamma/2).
 * *mismatches is a device uint64 the caller zeroes first. */
int tmq_selftest_const_div(double digamma, unsigned long long *mismatches, void *stream);

/* Device self-check of the range-specialised division used for the data-dependent quotients (denominators in
 * [16, 8192)): compares it with IEEE division for the denominators number b_begin .. b_begin + b_count - 1 of those nine
 * binades (9 * 2^23 in all), each against per_b numerators (per_b = 2^23: every mantissa).  *mismatches: device
 * uint64, zeroed by the caller. */
int tmq_selftest_div(unsigned per_b, unsigned long long b_begin, unsigned long long b_count,
                     unsigned long long *mismatches, void *stream);

/* Self-check of the bounded device-side waits every tensor-core kernel uses: one thread waits, with a budget of
 * budget_cycles SM clocks (<= 4e9), on a barrier that nothing completes.  The kernel returns normally; afterwards
 * *status (device int, zero before the call) holds TMQ_ERR_TIMEOUT and *waited_cycles (device int64, may be NULL)
 * the clocks spent waiting.  Nothing faults or hangs: this is how the time-out path is tested. */
int tmq_selftest_wait_timeout(long long budget_cycles, int *status, long long *waited_cycles, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Hot path 2a: bit-exact 2-bit packing.  W is [N][K] row-major (Linear [out][in]; a conv kernel
 * [O][I][ky][kx] is the same thing with K = I*ky*kx).  P is [K][ceil(N/16)] 32-bit words, element i of a
 * word in bits [31-2i : 30-2i], codes 0 -> 00, +1 -> 01, -1 -> 10, tail elements zero.
 * ------------------------------------------------------------------------------------------------ */

/* replaces: compactify_ternary, tmq/tmq_native.cpp:418-425 (matrix :303-319/:152-171, conv kernel :279-294/:185-208) */
int tmq_pack2b_f32(const float *W, uint32_t *P, int64_t N, int64_t K, void *stream);
int tmq_pack2b_i32(const int32_t *W, uint32_t *P, int64_t N, int64_t K, void *stream);
int tmq_pack2b_i8(const int8_t *W, uint32_t *P, int64_t N, int64_t K, void *stream);
/* replaces: expand_ternary, tmq/tmq_native.cpp:516-544 (:249-266; the 2-D routine :220-234 drops the transpose,
 * this is the true inverse for both ranks) */
int tmq_unpack2b_f32(const uint32_t *P, float *W, int64_t N, int64_t K, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Hot path 2b: ternary GEMM / GEMV from packed weights, tensor-core path (tcgen05 + TMEM + TMA).
 *   Y[m][n] = scale[n] * sum_k X[m][k] * T[n][k] + bias[n],   T[n][k] in {-1, 0, +1}
 * replaces: ternary_mmm_cuda / ternary_mvm_cuda, tmq/tmq_cuda.cu:478-549 (kernel :289-427), :563-603 (kernel
 * :242-286); callers tmq/tmq.py:662-688 (Linear.compact_forward), :822-871 (Conv2d.compact_forward, after im2col).
 * The reference multiplies fp32 activations on CUDA cores and applies post_scale / bias in Python; here scale and
 * bias are per output channel and fused (pass NULL for none).
 *
 * Weights are consumed in a PREPACKED layout derived once from the reference layout P[K][ceil(N/16)]:
 * Wt[N][row stride] words, Kp = K rounded up to 64, 16 consecutive k of one output channel per word, bit order per
 * activation type (fmt 0: bf16 activations, fmt 1: int8 activations).  tmq_prepack_words gives the word count.
 *
 * Status word: `status` is a device int the caller zeroes once.  A kernel whose bounded device-side wait runs out
 * stores TMQ_ERR_TIMEOUT there and returns; the word is STICKY: while it is non-zero every later GEMM / GEMV /
 * convolution launch that is given the same word returns at once without touching its output, and the C call still
 * returns TMQ_OK (it only enqueues).  Callers must read the word at a point where they synchronise anyway (at least
 * before they trust a batch of results), treat non-zero as a failed batch, and re-zero it before they continue.
 * ------------------------------------------------------------------------------------------------ */
size_t tmq_prepack_row_words(int64_t K, int fmt); /* row stride in 32-bit words (valid words + bank padding) */
size_t tmq_prepack_words(int64_t N, int64_t K, int fmt); /* N * row stride */
/* Enqueues the conversion followed by an empty kernel, so that Wt is complete and visible before ANY later launch on
 * the stream starts - including the skinny kernels below, which read Wt ahead of their wait on the stream's previous
 * kernel (see tmq_ternary_gemv_bf16). */
int tmq_prepack(const uint32_t *P, uint32_t *Wt, int64_t N, int64_t K, int fmt, void *stream);

/* X: bf16 [M][K] row-major, K % 8 == 0, 16-byte aligned.  Y: bf16 (out_f32 = 0) or fp32 (out_f32 = 1) [M][ldy],
 * element-aligned; ldy >= N lets Y be a column block of a wider matrix (Y = base + n0).  bf16 rows are written as
 * 16-byte vectors when Y is 16-byte aligned and ldy % 8 == 0, element by element otherwise.  fp32 accumulation.
 * *status: see "Status word" above. */
int tmq_ternary_gemm_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, int64_t M,
                          int64_t N, int64_t K, int64_t ldy, int out_f32, int *status, void *stream);
/* X: int8 [M][K], K % 16 == 0.  Y: int32 [M][ldy], exact. */
int tmq_ternary_gemm_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K, int64_t ldy,
                        int *status, void *stream);

/* Split-K forms for skinny problems (M <= 256 with fewer 128-channel output tiles than SMs, e.g. a decode batch of 32 - 256
 * rows against an 11008 x 4096 matrix: 86 - 172 tiles on 148 SMs): K is split over up to floor(148 / tiles) CTAs per tile
 * (at least four k-blocks each), the raw accumulators go to `workspace` and a second small kernel adds them in split
 * order and applies scale / bias: deterministic, int32 results exact.  workspace: tmq_ternary_gemm_workspace_bytes(M, N, K,
 * int8_activations) bytes of device scratch, 16-byte aligned; 0 bytes = the problem is not split; NULL / too small =
 * the plain kernel runs.  Everything else as tmq_ternary_gemm_bf16 / _i8. */
size_t tmq_ternary_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int int8_activations);
int tmq_ternary_gemm_bf16_splitk(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, int64_t M,
                                 int64_t N, int64_t K, int64_t ldy, int out_f32, void *workspace, size_t workspace_bytes,
                                 int *status, void *stream);
int tmq_ternary_gemm_i8_splitk(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K, int64_t ldy,
                               void *workspace, size_t workspace_bytes, int *status, void *stream);

/* GEMM + all-gather in one kernel: tmq_ternary_gemm_bf16 (bf16 output) whose epilogue stores every output vector into
 * ndst (1 .. 8) buffers: Ys[0] in this GPU's memory and Ys[1 ..] in OTHER GPUs' memory (peer mappings of buffers of the
 * same shape, e.g. CUDA IPC or symmetric memory), all with row stride ldy.  A rank of a column-sharded linear passes
 * every rank's full-width output buffer offset to its own column block: when the kernel has completed on every rank
 * (the caller orders that with a barrier on the stream, and must not let a rank overwrite a buffer a peer still reads),
 * each buffer holds the whole row-major result and no separate all-gather has run; the transfers over NVLink overlap
 * the multiplication tile by tile.  Ys: HOST array of device pointers.  Plain stores only, no multicast.
 * extends: ternary_mmm_cuda, tmq/tmq_cuda.cu:478-549 (the reference is single-GPU). */
int tmq_ternary_gemm_bf16_bcast(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *const *Ys,
                                int ndst, int64_t M, int64_t N, int64_t K, int64_t ldy, int *status, void *stream);

/* Skinny form for M <= 16 activation rows (decode-like GEMV): reads the packed weights once, exactly decoded operands
 * (warp-level MMA, the decoded fragment shared by both 8-row tiles when M > 8; byte dot products for int8 with M <= 2),
 * deterministic.  M > 8 needs the resident form (a status word, and one SM's share of the rows within the shared-memory
 * budget): TMQ_ERR_UNSUPPORTED otherwise, and the caller makes two calls of up to 8 rows.  Same operand conventions as the GEMM
 * entry points above.  When one SM's share of the packed rows fits half its shared memory the rows are made
 * resident with bulk copies issued BEFORE the kernel waits for its predecessor in the stream (programmatic dependent
 * launch), so consecutive launches overlap their weight traffic with the predecessor's arithmetic; `status` (device
 * int, zero before the first call, may be NULL: then the non-resident streaming kernel is used) receives
 * TMQ_ERR_TIMEOUT if those copies never complete.
 * CONTRACT that follows from the early fetch: Wt, scale and bias must be complete in memory before the kernel that
 * PRECEDES this call in the stream starts, i.e. they must not be written by the immediately preceding launch
 * (tmq_prepack ends with an empty kernel for exactly this reason; weights written by a caller's own kernel need one
 * launch or an event between them and this call).  X and Y carry no such restriction.
 * replaces: ternary_mvm_cuda, tmq/tmq_cuda.cu:563-603 (kernel :242-286). */
int tmq_ternary_gemv_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, int64_t M,
                          int64_t N, int64_t K, int64_t ldy, int out_f32, int *status, void *stream);
int tmq_ternary_gemv_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int64_t M, int64_t N, int64_t K, int64_t ldy,
                        int *status, void *stream);

/* Batched skinny form: nmat (1 .. TMQ_GEMV_BATCH_MAX) weight matrices of ONE shape [N][K] in one launch, M <= 8
 * activation rows each.  Projections that share their input (query / key / value, gate / up) and independent experts
 * are not ordered among themselves, so one launch can take them all: the hand-over between two dependent kernels is
 * paid once per group instead of once per matrix, and inside the launch the rows of matrix j + 1 stream into shared
 * memory while matrix j is multiplied.  Same exact products as nmat calls of tmq_ternary_gemv_*: int32 results are
 * identical, fp32 sums differ only by summation order (the K slices are spread over a different number of warps).
 * Wt / scale / bias / Y: HOST arrays of nmat device pointers (scale, bias: NULL arrays or NULL entries allowed; Wt as
 * for tmq_ternary_gemv_*, same early-fetch CONTRACT).  X: activations of matrix j start x_stride ELEMENTS after those
 * of matrix j - 1 (0: all matrices share one block; otherwise a multiple of 16 bytes).  status: required.
 * TMQ_ERR_UNSUPPORTED when one SM's share of a matrix exceeds the shared-memory budget (call the one-matrix form).
 * extends: ternary_mvm_cuda, tmq/tmq_cuda.cu:563-603 (the reference launches one matrix per call). */
#define TMQ_GEMV_BATCH_MAX 16
int tmq_ternary_gemv_batched_bf16(const void *X, int64_t x_stride, const uint32_t *const *Wt, const float *const *scale,
                                  const float *const *bias, void *const *Y, int nmat, int64_t M, int64_t N, int64_t K,
                                  int64_t ldy, int out_f32, int *status, void *stream);
int tmq_ternary_gemv_batched_i8(const int8_t *X, int64_t x_stride, const uint32_t *const *Wt, int32_t *const *Y, int nmat,
                                int64_t M, int64_t N, int64_t K, int64_t ldy, int *status, void *stream);

/* Training forward of a quantisation-aware Linear layer with the soft staircase fused into the weight-operand load:
 *   Y[m][n] = sum_k X[m][k] * S(W[n][k]; hardness) + bias[n]
 * X bf16 [M][K] (K % 8 == 0, 16-byte aligned), W the latent fp32 weights [N][K] (16-byte aligned), bias fp32 [N] or
 * NULL, Y fp32 [M][ldy].  S is evaluated bit-identically to tmq_softstep_fwd inside the GEMM's producer warps and fed to
 * the tensor cores as two bf16 terms (hi + lo, ~2^-17 relative), fp32 accumulation: the staircase values are never
 * written to memory.  Producer-bound (every weight tile is evaluated once per 128 / 256 activation rows): meant for
 * M up to a few hundred rows; for tall activations run tmq_softstep_fwd once and a dense GEMM.
 * hardness in [1e-3, 1e3]; status: see "Status word" above (required).
 * workspace: device scratch of tmq_qat_linear_workspace_bytes(M, N, K) bytes (16-byte aligned; 0 bytes when the problem
 * has at least as many output tiles as SMs).  With it, K is split over several CTAs per output tile and the partial sums
 * are combined in a fixed order by a second small kernel (deterministic); without it (NULL / too small) every output
 * tile is one CTA's work, which leaves SMs idle on small layers.
 * replaces: SoftStep.apply + F.linear in Linear.forward, tmq/tmq.py:637-659 (:404-433 for S). */
size_t tmq_qat_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
int tmq_qat_linear_fwd_bf16(const void *X, const float *W, const float *bias, float *Y, int64_t M, int64_t N, int64_t K,
                            int64_t ldy, double hardness, void *workspace, size_t workspace_bytes, int *status,
                            void *stream);

/* Ternary Conv2d as an implicit GEMM (no im2col buffer): X bf16 NHWC [B][H][W][C], C % 64 == 0; Wt = fmt-0 prepack of
 * the packed weight with its K rows reordered to (ky, kx, c); Y bf16 NHWC [B][OH][OW][N] with the output geometry of
 * F.conv2d; scale / bias per output channel (folded BatchNorm, NULL for none), optional residual (bf16, shape of Y,
 * added before the activation), optional ReLU.  X 16-byte aligned; Y and residual element-aligned (16-byte aligned
 * pointers with N % 8 == 0 take the vector stores).
 * replaces: Conv2d.compact_forward, tmq/tmq.py:822-871 (F.unfold + ternary_mmm_cuda + F.fold). */
int tmq_ternary_conv2d_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, const void *residual,
                            void *Y, int B, int H, int W, int C, int N, int ky, int kx, int sy, int sx, int py, int px,
                            int dy, int dx, int relu, int *status, void *stream);
/* Unit-stride form with the input tile resident in shared memory for all filter taps ("shifted window"): one 4-D TMA
 * copy per 64-channel slice brings a tile's input pixels (zero padding = the copy's out-of-bounds fill) and every
 * tap's MMAs read that one copy through a descriptor shifted by the tap's offset; persistent CTAs, double-buffered
 * accumulator.  Same operands and results as tmq_ternary_conv2d_bf16 with sy = sx = 1, except the K order of Wt:
 * (64-channel slice, ky, kx, channel within the slice).  ky * kx <= 9; TMQ_ERR_UNSUPPORTED outside its limits.
 * replaces: Conv2d.compact_forward for stride-1 layers, tmq/tmq.py:822-871. */
int tmq_ternary_conv2d_s1_bf16(const void *X, const uint32_t *Wt, const float *scale, const float *bias, const void *residual,
                               void *Y, int B, int H, int W, int C, int N, int ky, int kx, int py, int px, int dy, int dx,
                               int relu, int *status, void *stream);

/* The same convolution with fp32 NHWC output (no output rounding; residual stays bf16), and with int8 activations:
 * X int8 NHWC, Wt = fmt-1 prepack of the (ky, kx, c)-ordered packed weight, Y int32 NHWC, exact.  The fp32-output form
 * is also how fp32 activations are convolved exactly: split them into three bf16 terms along the channels
 * (tmq_nchw_f32_to_nhwc_bf16 / tmq_split_f32_bf16 with terms = 3) and stack three copies of the weights per tap.
 * replaces: Conv2d.compact_forward, tmq/tmq.py:822-871. */
int tmq_ternary_conv2d_bf16_f32out(const void *X, const uint32_t *Wt, const float *scale, const float *bias,
                                   const void *residual, float *Y, int B, int H, int W, int C, int N, int ky, int kx, int sy,
                                   int sx, int py, int px, int dy, int dx, int relu, int *status, void *stream);
int tmq_ternary_conv2d_i8(const int8_t *X, const uint32_t *Wt, int32_t *Y, int B, int H, int W, int C, int N, int ky, int kx,
                          int sy, int sx, int py, int px, int dy, int dx, int *status, void *stream);

/* Activation layout helpers of the packed inference path (replace the eager tensor glue between compact layers,
 * tmq/tmq.py:857-863): fp32 rows [M][K] -> bf16 [M][terms*Kp] (terms = 1: rounded; terms = 3: the exact split
 * x = lo + mid + hi, smallest term first, term t at column t*Kp + k; columns K..Kp-1 zero); fp32 NCHW -> bf16 NHWC [B][H][W][terms*C];
 * global average pooling of bf16 NHWC [B][P][C] -> bf16 [B][C] (fp32 sum, C even). */
int tmq_split_f32_bf16(const float *X, void *out, int64_t M, int64_t K, int64_t Kp, int terms, void *stream);
int tmq_nchw_f32_to_nhwc_bf16(const float *X, void *Y, int B, int C, int H, int W, int terms, void *stream);
int tmq_avgpool_nhwc_bf16(const void *X, void *Y, int B, int P, int C, void *stream);

/* Patch matrix for layers the implicit path cannot take (channel count not a multiple of 64, e.g. a 3-channel stem):
 * X fp32 NCHW -> A bf16 [B*OH*OW][Kp], K = ky*kx*C in (ky, kx, c) order zero-padded to Kp (% 8 == 0); feed A to
 * tmq_ternary_gemm_bf16.  replaces: F.unfold in Conv2d.compact_forward, tmq/tmq.py:857-858. */
int tmq_conv_patches_bf16(const float *X, void *A, int B, int C, int H, int W, int ky, int kx, int sy, int sx, int py, int px,
                          int dy, int dx, int Kp, void *stream);

/* Convolution for layers with few input channels (the image stem), patches kept on chip: X fp32 NCHW [B][C][H][W],
 * Wt = tmq_prepack(fmt 0) of the packed weights with rows in (ky, kx, c) order (k_rows of them, zero rows beyond
 * ky*kx*C allowed), Y bf16 NHWC [B][OH][OW][N] = act(scale[n] * conv + bias[n]), unit dilation.  One CTA per (image,
 * output row): limits ky*kx*C <= 256, OW <= 128, C*ky*((OW-1)*sx+kx)*2 <= 16 KB, N % 8 == 0; TMQ_ERR_UNSUPPORTED beyond
 * them (then: tmq_conv_patches_bf16 + tmq_ternary_gemm_bf16).
 * replaces: Conv2d.compact_forward for such layers, tmq/tmq.py:822-871. */
int tmq_ternary_conv2d_stem_bf16(const float *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y, int B,
                                 int C, int H, int W, int N, int ky, int kx, int sy, int sx, int py, int px, int k_rows,
                                 int relu, int *status, void *stream);

/* The same layer class with the patches read by descriptor instead of being assembled: the input rows an output row
 * touches are kept in shared memory as bf16 [row][pixel][CP channels], CP = 8 / sx channel slots per pixel (sx = 2: up to
 * 4 channels, sx = 1: up to 8), which puts the patch rows of neighbouring output pixels 16 bytes apart - the row pitch of
 * the tensor core's unswizzled operand layout - so every MMA reads its operand straight from that window.  Wt = fmt-0
 * prepack of the packed weights with K ordered (ky, [kx, CP] zero-padded to a multiple of 16): tmq_stem_rows_k rows
 * (0 = layer not covered).  The output pixels of a row are the MMA's M side and the (at most 64) output channels its N
 * side, so an epilogue thread writes one pixel's channels contiguously; the window is a ring of ky + sy rows and a tile
 * converts only the rows its predecessor did not have.  Limits: OW <= 128, N <= 64, sy < ky, ky * ceil(kx * CP / 16) <= 24;
 * TMQ_ERR_UNSUPPORTED beyond (then: tmq_ternary_conv2d_stem_bf16).  replaces: Conv2d.compact_forward for such layers, tmq/tmq.py:822-871. */
int tmq_stem_rows_k(int C, int ky, int kx, int sx);
int tmq_ternary_conv2d_stem_rows_bf16(const float *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                      int B, int C, int H, int W, int N, int ky, int kx, int sy, int sx, int py, int px,
                                      int relu, int *status, void *stream);
/* The same convolution followed by ReLU and a 3 x 3 / stride 2 / padding 1 max pooling, all in the epilogue (the ResNet
 * stem): Y bf16 NHWC [B][OH/2][OW/2][64], 32-byte aligned; N == 64, OH and OW even.  The convolution's own output row is
 * kept in shared memory (running maximum over the three rows of a pooling window, then over the three columns) and
 * never written: a quarter of the output traffic and no pooling launch.  Bit-identical to the unfused sequence.
 * TMQ_ERR_UNSUPPORTED outside those limits.
 * replaces: conv1 + bn1 + relu + maxpool of the reference's ResNet pipelines (samples/resnet_train.py model definition). */
int tmq_ternary_conv2d_stem_rows_pool_bf16(const float *X, const uint32_t *Wt, const float *scale, const float *bias, void *Y,
                                           int B, int C, int H, int W, int N, int ky, int kx, int sy, int sx, int py, int px,
                                           int *status, void *stream);

/* Max pooling between packed layers: X bf16 NHWC [B][H][W][C] (C % 8 == 0) -> Y [B][OH][OW][C], square window k, stride s,
 * padding p (positions outside the image are ignored), OH = (H + 2p - k) / s + 1; relu != 0 applies max(0, .) as well
 * (ReLU and max pooling commute, so a preceding ReLU can be folded in).  Keeps the packed inference pipeline in NHWC bf16
 * (the reference pipeline runs torch's NCHW fp32 pooling between its compact layers). */
int tmq_maxpool2d_nhwc_bf16(const void *X, void *Y, int B, int H, int W, int C, int k, int s, int p, int relu,
                            void *stream);

/* Max pooling for training on fp32 NHWC activations [B][H][W][C], C % 4 == 0, square window k <= 11, stride s, padding p
 * (2p <= k), torch's max_pool2d output geometry and winner rule (first maximum in scan order; a NaN wins).  The forward
 * pass also writes the winning window position of every output element (idx, one signed byte each, shape of Y); the
 * backward pass gathers: every input element sums the gradients of the windows it won - deterministic, no atomics, no
 * zero-fill pass.  16-byte aligned X / Y / gX / gY.
 * replaces: the max_pool2d forward / backward pair between the stem and layer1 of the QAT ResNet step
 * (samples/resnet_train.py:102-160 runs torch's own). */
int tmq_maxpool2d_nhwc_f32_fwd(const float *X, float *Y, signed char *idx, int B, int H, int W, int C, int k, int s, int p,
                               void *stream);
int tmq_maxpool2d_nhwc_f32_bwd(const float *gY, const signed char *idx, float *gX, int B, int H, int W, int C, int k, int s,
                               int p, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Depthwise ternary convolutions (groups == channels), fp32, forward and transposed.  W is the reference's packed form
 * of a [C][1][ky][kx] kernel tensor: int32 [ky*kx][ceil(C/16)].  Arithmetic: taps accumulated in (ky, kx) order from +0
 * with one fused multiply-add each (x = 0 outside the image), then acc * scale[c] + bias[c] with two roundings
 * (NULL = skip).
 *
 * Direct NCHW forms: X [B][C][H][W] -> Y [B][C][OH][OW], no unfold / fold.
 *   forward:    OH = (H + 2*py - dy*(ky-1) - 1) / sy + 1                                   (torch conv2d)
 *   transposed: OH = (H - 1)*sy - 2*py + dy*(ky-1) + 1 + opy                               (torch conv_transpose2d)
 * replaces: Conv2d.compact_forward groups != 1 branch, tmq/tmq.py:849-854, and ConvTranspose2d.compact_forward
 * groups != 1 branch, tmq/tmq.py:1025-1029 (F.unfold / F.fold around the operators below).
 *
 * Operator-level forms on the reference operators' own layouts:
 *   tmq_ternary_dwconv_patches_f32:      X [rows][ntaps][C] -> Y [rows][C]          (rows = batch * pixels)
 *     replaces: ternary_dwconv_cuda, tmq/tmq_cuda.cu:607-644 (kernel :163-238; the reference reads batch element 0 only)
 *   tmq_ternary_dwconvtrans_patches_f32: X [B][P][C] -> Y [B][C*ntaps][P], Y[b][c*ntaps+t][p] = X[b][p][c] * T[t][c]
 *     replaces: ternary_dwconvtrans_cuda, tmq/tmq_cuda.cu:647-686 (kernel :118-159)
 * ------------------------------------------------------------------------------------------------ */
int tmq_ternary_dwconv2d_f32(const float *X, const uint32_t *W, const float *scale, const float *bias, float *Y, int B,
                             int C, int H, int Wd, int ky, int kx, int sy, int sx, int py, int px, int dy, int dx,
                             void *stream);
int tmq_ternary_dwconvtrans2d_f32(const float *X, const uint32_t *W, const float *scale, const float *bias, float *Y,
                                  int B, int C, int H, int Wd, int ky, int kx, int sy, int sx, int py, int px, int dy,
                                  int dx, int opy, int opx, void *stream);
int tmq_ternary_dwconv_patches_f32(const float *X, const uint32_t *W, float *Y, int64_t rows, int C, int ntaps,
                                   void *stream);
int tmq_ternary_dwconvtrans_patches_f32(const float *X, const uint32_t *W, float *Y, int B, int P, int C, int ntaps,
                                        void *stream);

/* ------------------------------------------------------------------------------------------------
 * Entropy-coded storage of packed weights (HOST pointers; sequential range coder, no GPU work).  Streams are
 * byte-identical to the reference's: 26-byte big-endian header + range-coder payload.  P is the packed matrix
 * [rows][ceil(cols/16)] with rows = K and cols = N of the weight (the coder walks the packed, transposed matrix).
 * replaces: compress_ternary / decompress_ternary, tmq/tmq_native.cpp:439-503 (:50-140), tmq/rangecoder.h:41-193.
 * ------------------------------------------------------------------------------------------------ */
size_t tmq_rc_encode_bound(int64_t rows, int64_t cols);
int tmq_rc_encode(const uint32_t *P, int64_t rows, int64_t cols, uint8_t *out, size_t out_cap, size_t *out_len);
int tmq_rc_decode(const uint8_t *in, size_t in_len, uint32_t *P, int64_t rows, int64_t cols);

#ifdef __cplusplus
}
#endif
#endif /* TMQ_B200_H */
