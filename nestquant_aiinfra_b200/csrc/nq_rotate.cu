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
#include "nq_rotate_core.cuh"

namespace {

// The butterfly passes live in nq_rotate_core.cuh; the last pass here applies the 1/sqrt(n)
// division and stores to global memory in the tensor dtype.
template <typename T>
__global__ void __launch_bounds__(1024)
nq_hadamard_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int n, int rows_per_cta,
                   float root, float inv_root) {
    extern __shared__ __align__(16) float buf[];
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    const int nrows = (int)min((int64_t)rows_per_cta, rows - row0);
    const int total = nrows * n;           // elements of this CTA (rows are independent, n >= 8)
    nq_fwht_rows_to_smem<T>(x + row0 * n, buf, total, n);
    for (int g = threadIdx.x; g < (total >> 3); g += blockDim.x) {
        const float4 lo = reinterpret_cast<const float4*>(buf + g * 8)[0];
        const float4 hi = reinterpret_cast<const float4*>(buf + g * 8)[1];
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = nq_div_by(v[j], root, inv_root);
        nq_store8<T>(out + row0 * n + (int64_t)g * 8, v);
    }
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
    // one group of 8 elements per thread and pass for long rows (a row of 8192 is a chain of five passes:
    // with 256 threads each pass took four rounds)
    const int64_t groups = (int64_t)rpc * n / 8;
    const unsigned threads = groups >= 1024 ? 1024u : (groups >= 512 ? 512u : 256u);
    kernel<<<(unsigned)grid, threads, smem, stream>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(out), rows,
                                                  (int)n, rpc, root, 1.0f / root);
    NQ_CHECK_LAUNCH("nq_hadamard");
    return NQ_OK;
}

}  // namespace

extern "C" int nq_hadamard(const void* x, void* out, int dtype, int64_t rows, int64_t n, nq_stream_t stream) {
    NQ_RANGE("nq_hadamard");
    NQ_REQUIRE(x && out, NQ_ERR_ARG, "nq_hadamard: null pointer");
    NQ_REQUIRE(rows >= 1 && n >= 8 && n <= 32768 && (n & (n - 1)) == 0, NQ_ERR_ARG,
               "nq_hadamard: n=%lld must be a power of two in [8, 32768]", (long long)n);
    NQ_REQUIRE(nq_aligned16(x) && nq_aligned16(out), NQ_ERR_ALIGN, "nq_hadamard: 16-byte alignment required");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_hadamard<float>(x, out, rows, n, s);
        case NQ_BF16: return launch_hadamard<__nv_bfloat16>(x, out, rows, n, s);
        case NQ_F16: return launch_hadamard<__half>(x, out, rows, n, s);
        default: nq_set_error("nq_hadamard: unknown dtype %d", dtype); return NQ_ERR_ARG;
    }
}
