// Normalised Sylvester Hadamard (fast Walsh-Hadamard transform) along the last
// axis, one launch instead of ~2*log2(n) tensor ops.  Replaces hadamard()
// (core/rotation.py:12-27) at its three hot call sites (Linear inputs in their
// own dtype, models/fused_linear.py:287-290; Q and K in float32,
// runtime/nqkv_batched_hf_backend.py:381,549).
//
// Bit-exact with the reference: every butterfly stage is one float32 add/sub
// whose result is rounded to the tensor dtype (what each torch op does on a
// BF16/FP16 tensor), and the final division is an IEEE division by
// float32(sqrt(n)).
#include <math.h>

#include "nq_common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return nq_bf16_round(v); }
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <typename T> __device__ __forceinline__ float load_as_float(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_as_float<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float load_as_float<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }

template <typename T> __device__ __forceinline__ void store_from_float(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void store_from_float<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_from_float<__half>(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
nq_hadamard_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int n, int rows_per_cta,
                   float root, float inv_root) {
    extern __shared__ float buf[];
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    const int nrows = (int)min((int64_t)rows_per_cta, rows - row0);
    const int total = nrows * n;
    for (int i = threadIdx.x; i < total; i += 256) buf[i] = load_as_float<T>(x, row0 * n + i);
    __syncthreads();
    const int pairs = total >> 1, half_n = n >> 1;
    for (int w = 1; w < n; w <<= 1) {
        for (int p = threadIdx.x; p < pairs; p += 256) {
            const int r = p / half_n, q = p - r * half_n;
            const int g = q / w, i = q - g * w;
            const int a = r * n + g * 2 * w + i, b = a + w;
            const float l = buf[a], rr = buf[b];
            buf[a] = round_to<T>(nq_add(l, rr));
            buf[b] = round_to<T>(nq_sub(l, rr));
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < total; i += 256)
        store_from_float<T>(out, row0 * n + i, nq_div_by(buf[i], root, inv_root));
}

template <typename T>
int launch_hadamard(const void* x, void* out, int64_t rows, int64_t n, cudaStream_t stream) {
    int rpc = (int)(n >= 2048 ? 1 : 2048 / n);
    const size_t smem = (size_t)rpc * n * sizeof(float);
    auto kernel = nq_hadamard_kernel<T>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            nq_set_error("nq_hadamard: shared memory: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    const float root = (float)sqrt((double)n);
    const int64_t grid = (rows + rpc - 1) / rpc;
    kernel<<<(unsigned)grid, 256, smem, stream>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(out), rows,
                                                  (int)n, rpc, root, 1.0f / root);
    NQ_CHECK_LAUNCH("nq_hadamard");
    return NQ_OK;
}

}  // namespace

extern "C" int nq_hadamard(const void* x, void* out, int dtype, int64_t rows, int64_t n, nq_stream_t stream) {
    NQ_REQUIRE(x && out, NQ_ERR_ARG, "nq_hadamard: null pointer");
    NQ_REQUIRE(rows >= 1 && n >= 2 && n <= 32768 && (n & (n - 1)) == 0, NQ_ERR_ARG,
               "nq_hadamard: n=%lld must be a power of two in [2, 32768]", (long long)n);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_hadamard<float>(x, out, rows, n, s);
        case NQ_BF16: return launch_hadamard<__nv_bfloat16>(x, out, rows, n, s);
        case NQ_F16: return launch_hadamard<__half>(x, out, rows, n, s);
        default: nq_set_error("nq_hadamard: unknown dtype %d", dtype); return NQ_ERR_ARG;
    }
}
