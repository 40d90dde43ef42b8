// Quantization-loss sum for hosts that must not allocate device memory.
//
// Who needs this: a program that links the C ABI from a place where it has no device allocator to call - a
// plain-C inference or training host whose device memory was carved up once at start-up and handed out in full,
// a plug-in running inside a framework that owns every byte of the memory pool, or code on a path where
// cudaMalloc is forbidden because it can stall the whole device.  The regular entry point (tmq_qloss_sum) asks
// such a caller for a scratch buffer it has no way to provide.  Here the scratch lives inside the library image
// instead: one fixed array in device global memory, present on every GPU that loads the library, for as long as
// the process lives.
//
// Consequences the caller has to know:
//   * the array is small, so the tensor size is capped (TMQ_QLOSS_NOALLOC_MAX_ELEMS); larger tensors are refused
//     with TMQ_ERR_SCRATCH and nothing is launched;
//   * all calls on one GPU share the one array, and it still holds whatever the previous call left there, so
//     every call clears the part that has to start at zero; two calls whose kernels can overlap on the GPU
//     (different streams, no ordering between them) would corrupt each other's partial sums;
//   * the first call on each device looks up the array's device address (a host-side query, no allocation).
//     Make that first call ahead of any stream capture.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kPartials = 4096;                    // one fp64 partial per block
constexpr int kBlockThreads = 256;
constexpr size_t kElemsPerBlock = 8192;            // 256 threads x 8 iterations x 4 floats
constexpr size_t kMaxElems = (size_t)kPartials * kElemsPerBlock;
static_assert(kMaxElems == TMQ_QLOSS_NOALLOC_MAX_ELEMS, "header and kernel disagree on the size cap");
constexpr size_t kArrayBytes = tmq::kScratchHeader + sizeof(double) * kPartials;  // 33,024 bytes per GPU

// Device global memory owned by the library image.  In HOST code this name is only a handle for
// cudaGetSymbolAddress, never an address a kernel could use; the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_scratch[kArrayBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void *g_scratch_addr[kMaxDevices] = {};

struct Consts {
    float d, h, D, sd;
};

// strength * S'(w; d), one IEEE operation per line in the order of tmq/tmq.py:469-472 and :368-370
__device__ __forceinline__ float integrand(float w, const Consts c) {
    const float fw = floorf(w);
    const float fr = __fsub_rn(w, fw);
    const float a = __fsub_rn(__fmul_rn(c.d, fr), c.h);
    float x = fminf(fmaxf(a, -3.0f), 3.0f);
    x = (a != a) ? a : x;
    const float x2 = __fmul_rn(x, x);
    const float e = __fsub_rn(x2, 9.0f);
    const float n = __fmul_rn(e, e);
    const float b = __fadd_rn(3.0f, x2);
    const float m = __fmul_rn(__fmul_rn(9.0f, b), b);
    const float ds = __fdiv_rn(n, m);
    return __fdiv_rn(__fmul_rn(c.sd, ds), c.D);
}

__global__ void __launch_bounds__(kBlockThreads) qloss_noalloc_kernel(const float *__restrict__ w, size_t n,
                                                                      Consts c, void *scratch, double *out,
                                                                      bool vec) {
    const size_t begin = (size_t)blockIdx.x * kElemsPerBlock;
    const size_t end = begin + kElemsPerBlock < n ? begin + kElemsPerBlock : n;
    double acc = 0.0;
    if (vec) {
        const size_t v0 = begin / 4, v1 = end / 4;  // begin is a multiple of 4
        for (size_t i = v0 + threadIdx.x; i < v1; i += kBlockThreads) {
            const float4 t = __ldg(reinterpret_cast<const float4 *>(w) + i);
            float p = __fadd_rn(integrand(t.x, c), integrand(t.y, c));
            p = __fadd_rn(p, integrand(t.z, c));
            p = __fadd_rn(p, integrand(t.w, c));
            acc += (double)p;
        }
        for (size_t i = v1 * 4 + threadIdx.x; i < end; i += kBlockThreads) acc += (double)integrand(w[i], c);
    } else {
        for (size_t i = begin + threadIdx.x; i < end; i += kBlockThreads) acc += (double)integrand(w[i], c);
    }
    __shared__ double red[8];
    const double total = tmq::block_sum_256(acc, red);
    tmq::grid_sum_finish(total, scratch, out, red);
}

double scalar_sigmoid(double v) {
    const double x = v > 3.0 ? 3.0 : (v < -3.0 ? -3.0 : v);
    const double x2 = x * x;
    return x * (x2 + 27.0) / (27.0 + x2 * 9.0);
}

}  // namespace

extern "C" int tmq_qloss_sum_noalloc(const float *w, size_t n, double sharpness, double strength, double *sum_out,
                                     void *stream) {
    if (!(sharpness >= 1e-3 && sharpness <= 1e3) || !(strength == strength) || strength > 3e38 || strength < -3e38)
        return TMQ_ERR_ARG;
    if (!sum_out || (!w && n)) return TMQ_ERR_ARG;
    if (n > kMaxElems) return TMQ_ERR_SCRATCH;  // the built-in array has one partial per 8192 elements, 4096 of them
    if (!tmq::aligned(w, 4) || !tmq::aligned(sum_out, 8)) return TMQ_ERR_ALIGN;

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return tmq::cuda_status(e);
    if (dev < 0 || dev >= kMaxDevices) return TMQ_ERR_UNSUPPORTED;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_addr[dev]) {
            // set-up, once per device, with that device current: translate the symbol into its device address
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_scratch);
            if (e != cudaSuccess || !p) return tmq::cuda_status(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
            g_scratch_addr[dev] = p;
        }
        scratch = g_scratch_addr[dev];
    }
    cudaStream_t st = (cudaStream_t)stream;
    // the arrival counter must be zero when the kernel starts, whatever an earlier call left behind
    e = cudaMemsetAsync(scratch, 0, tmq::kScratchHeader, st);
    if (e != cudaSuccess) return tmq::cuda_status(e);

    Consts c;
    c.d = (float)sharpness;
    c.h = (float)(sharpness / 2.0);
    c.D = (float)(2.0 * scalar_sigmoid(sharpness / 2.0));
    c.sd = (float)(strength * sharpness);
    size_t blocks = (n + kElemsPerBlock - 1) / kElemsPerBlock;
    if (blocks == 0) blocks = 1;
    qloss_noalloc_kernel<<<(unsigned)blocks, kBlockThreads, 0, st>>>(w, n, c, scratch, sum_out, tmq::aligned(w, 16));
    return tmq::launch_status();
}
