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

// store 8 consecutive results (16-byte aligned) in the tensor dtype
template <typename T> __device__ __forceinline__ void store8(T* p, const float v[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float v[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float v[8]) {
    *reinterpret_cast<uint4*>(p) = nq_pack_bf16x8(v);
}
template <> __device__ __forceinline__ void store8<__half>(__half* p, const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}


// Radix-8 passes: a thread takes 8 elements spaced `w` apart, runs three butterfly stages
// (widths w, 2w, 4w -- exactly the reference's stage order, every result rounded to the
// tensor dtype) in registers and writes them back, so a row needs log2(n)/3 shared-memory
// round trips instead of log2(n).  The first pass reads its 8 consecutive elements straight
// from global memory, the last pass applies the 1/sqrt(n) division and stores to global.
template <typename T, int STAGES>
__device__ __forceinline__ void butterflies(float v[8]) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        const int h = 1 << s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if ((j & h) == 0) {
                const float l = v[j], r = v[j | h];
                v[j] = round_to<T>(nq_add(l, r));
                v[j | h] = round_to<T>(nq_sub(l, r));
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
nq_hadamard_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int n, int rows_per_cta,
                   float root, float inv_root) {
    extern __shared__ __align__(16) float buf[];
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    const int nrows = (int)min((int64_t)rows_per_cta, rows - row0);
    const int total = nrows * n;           // elements of this CTA (rows are independent, n >= 8)
    const int groups = total >> 3;
    int log_n = 0;
    while ((1 << log_n) < n) ++log_n;

    // pass 0: widths 1, 2, 4 on 8 consecutive elements loaded from global memory
    for (int g = threadIdx.x; g < groups; g += 256) {
        float v[8];
        nq_load8<T>(x + row0 * n + (int64_t)g * 8, v);
        butterflies<T, 3>(v);
        float4* dst = reinterpret_cast<float4*>(buf + g * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    int done = 3;
    while (done < log_n) {
        const int stages = min(3, log_n - done);
        const int w = 1 << done;               // spacing of the elements a thread combines
        const int span = w << stages;          // elements covered by one group family
        const int per = 1 << stages;           // elements per thread in this pass
        const int work = total >> stages;
        for (int t = threadIdx.x; t < work; t += 256) {
            const int base = (t / w) * span + (t % w);
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = j < per ? buf[base + j * w] : 0.0f;
            if (stages == 3) butterflies<T, 3>(v);
            else if (stages == 2) butterflies<T, 2>(v);
            else butterflies<T, 1>(v);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j < per) buf[base + j * w] = v[j];
        }
        __syncthreads();
        done += stages;
    }
    for (int g = threadIdx.x; g < groups; g += 256) {
        const float4 lo = reinterpret_cast<const float4*>(buf + g * 8)[0];
        const float4 hi = reinterpret_cast<const float4*>(buf + g * 8)[1];
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = nq_div_by(v[j], root, inv_root);
        store8<T>(out + row0 * n + (int64_t)g * 8, v);
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
    kernel<<<(unsigned)grid, 256, smem, stream>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(out), rows,
                                                  (int)n, rpc, root, 1.0f / root);
    NQ_CHECK_LAUNCH("nq_hadamard");
    return NQ_OK;
}

}  // namespace

extern "C" int nq_hadamard(const void* x, void* out, int dtype, int64_t rows, int64_t n, nq_stream_t stream) {
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
