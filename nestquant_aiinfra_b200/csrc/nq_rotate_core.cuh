// Fast Walsh-Hadamard transform of rows held by one CTA, shared by the stand-alone rotation
// kernel and the rotate-then-encode kernel.
//
// Bit-exact with the reference's hadamard() (core/rotation.py:12-27): every butterfly stage is one
// float32 add/sub whose result is rounded to the tensor dtype T (what each torch op does on a
// BF16/FP16 tensor), in the reference's stage order (widths 1, 2, 4, ...); the final division
// is an IEEE division by float32(sqrt(n)).
//
// Radix-8 passes: a thread takes 8 elements spaced `w` apart, runs three butterfly stages
// (widths w, 2w, 4w) in registers and writes them back, so a row needs log2(n)/3 shared-memory
// round trips instead of log2(n).  The first pass reads its 8 consecutive elements straight
// from global memory.
#pragma once

#include "nq_common.cuh"

template <typename T> __device__ __forceinline__ float nq_round_to(float v);
template <> __device__ __forceinline__ float nq_round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float nq_round_to<__nv_bfloat16>(float v) { return nq_bf16_round(v); }
template <> __device__ __forceinline__ float nq_round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }

// store 8 consecutive results (16-byte aligned) in the tensor dtype
template <typename T> __device__ __forceinline__ void nq_store8(T* p, const float v[8]);
template <> __device__ __forceinline__ void nq_store8<float>(float* p, const float v[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void nq_store8<__nv_bfloat16>(__nv_bfloat16* p, const float v[8]) {
    *reinterpret_cast<uint4*>(p) = nq_pack_bf16x8(v);
}
template <> __device__ __forceinline__ void nq_store8<__half>(__half* p, const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T, int STAGES>
__device__ __forceinline__ void nq_butterflies(float v[8]) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        const int h = 1 << s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if ((j & h) == 0) {
                const float l = v[j], r = v[j | h];
                v[j] = nq_round_to<T>(nq_add(l, r));
                v[j | h] = nq_round_to<T>(nq_sub(l, r));
            }
        }
    }
}

// All butterfly stages of `total / n` independent rows of n elements (n a power of two >= 8),
// result in buf[0, total) as float32 values of dtype T, NOT yet divided by sqrt(n).
// load(g, v) supplies the 8 consecutive elements of group g (elements 8g .. 8g+7 of the CTA's
// rows) as float32 values of dtype T.  Called by every thread of the CTA; ends with a barrier.
template <typename T, class Load>
__device__ __forceinline__ void nq_fwht_groups_to_smem(Load&& load, float* buf, int total, int n) {
    const int nthreads = blockDim.x;
    const int groups = total >> 3;
    int log_n = 0;
    while ((1 << log_n) < n) ++log_n;

    // pass 0: widths 1, 2, 4 on 8 consecutive elements
    for (int g = threadIdx.x; g < groups; g += nthreads) {
        float v[8];
        load(g, v);
        nq_butterflies<T, 3>(v);
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
        for (int t = threadIdx.x; t < work; t += nthreads) {
            const int base = (t / w) * span + (t % w);
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = j < per ? buf[base + j * w] : 0.0f;
            if (stages == 3) nq_butterflies<T, 3>(v);
            else if (stages == 2) nq_butterflies<T, 2>(v);
            else nq_butterflies<T, 1>(v);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j < per) buf[base + j * w] = v[j];
        }
        __syncthreads();
        done += stages;
    }
}

// Same with the rows read from global memory (contiguous in `x`).
template <typename T>
__device__ __forceinline__ void nq_fwht_rows_to_smem(const T* __restrict__ x, float* buf, int total, int n) {
    nq_fwht_groups_to_smem<T>([&](int g, float v[8]) { nq_load8<T>(x + (int64_t)g * 8, v); }, buf, total, n);
}
