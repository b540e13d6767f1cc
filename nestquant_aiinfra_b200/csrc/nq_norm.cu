// RMS normalisation of activation rows in one launch (Llama's LlamaRMSNorm as Hugging Face
// writes it: float32 mean of squares, x * rsqrt(mean + eps) rounded to the tensor dtype, then the
// product with the weight rounded again).  Sits in front of every rotate-then-encode launch of
// a decoder layer, where the stock module costs six small tensor kernels.  The sum of squares
// uses a fixed order (per-thread strided partial sums, butterfly over the warp, warps in
// order), so results are deterministic; they are not bit-identical to the tensor-op version,
// whose reduction order differs.
#include <math.h>

#include "nq_common.cuh"
#include "nq_rotate_core.cuh"

namespace {

constexpr int kNormThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
nq_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ weight, int64_t rows, int n, float eps,
                  T* __restrict__ out) {
    __shared__ float s_part[kNormThreads / 32];
    const int64_t row = blockIdx.x;
    const T* src = x + row * n;
    T* dst = out + row * n;
    const int groups = n >> 3;
    float acc = 0.0f;
    for (int g = threadIdx.x; g < groups; g += kNormThreads) {
        float v[8];
        nq_load8<T>(src + g * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(v[j], v[j], acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += s_part[w];
    const float r = rsqrtf(total / (float)n + eps);
    for (int g = threadIdx.x; g < groups; g += kNormThreads) {
        float v[8], w[8], o[8];
        nq_load8<T>(src + g * 8, v);
        nq_load8<T>(weight + g * 8, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = nq_mul(w[j], nq_round_to<T>(nq_mul(v[j], r)));
        nq_store8<T>(dst + g * 8, o);
    }
}

template <typename T>
int launch_rmsnorm(const void* x, const void* weight, int64_t rows, int64_t n, float eps, void* out, cudaStream_t s) {
    nq_rmsnorm_kernel<T><<<(unsigned)rows, kNormThreads, 0, s>>>(reinterpret_cast<const T*>(x),
                                                               reinterpret_cast<const T*>(weight), rows, (int)n, eps,
                                                               reinterpret_cast<T*>(out));
    NQ_CHECK_LAUNCH("nq_rmsnorm");
    return NQ_OK;
}

}  // namespace

extern "C" int nq_rmsnorm(const void* x, const void* weight, int dtype, int64_t rows, int64_t n, float eps, void* out,
                          nq_stream_t stream) {
    NQ_RANGE("nq_rmsnorm");
    NQ_REQUIRE(x && weight && out, NQ_ERR_ARG, "nq_rmsnorm: null pointer");
    NQ_REQUIRE(rows >= 1 && rows <= 0x7fffffff && n >= 8 && n % 8 == 0 && n <= (1 << 20), NQ_ERR_ARG,
               "nq_rmsnorm: rows=%lld n=%lld (n must be a multiple of 8)", (long long)rows, (long long)n);
    NQ_REQUIRE(nq_aligned16(x) && nq_aligned16(weight) && nq_aligned16(out), NQ_ERR_ALIGN,
               "nq_rmsnorm: 16-byte alignment required");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_rmsnorm<float>(x, weight, rows, n, eps, out, s);
        case NQ_BF16: return launch_rmsnorm<__nv_bfloat16>(x, weight, rows, n, eps, out, s);
        case NQ_F16: return launch_rmsnorm<__half>(x, weight, rows, n, eps, out, s);
        default: nq_set_error("nq_rmsnorm: unknown dtype %d", dtype); return NQ_ERR_ARG;
    }
}
