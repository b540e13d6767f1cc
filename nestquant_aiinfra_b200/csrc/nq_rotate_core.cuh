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

// ---- 16-bit tensor dtypes: two values per register ------------------------------------------
//
// A float32 add of two BF16 (FP16) values followed by rounding to BF16 (FP16) equals ONE correctly
// rounded BF16 (FP16) add: the float32 sum is exact unless the exponents differ by more than 16 (13),
// and then the small operand is so far below half an ulp of the result that no rounding boundary is
// near.  So a butterfly of the reference is add.rn / sub.rn on the packed pair type, two butterflies
// per instruction, and the row lives in shared memory in its own dtype (half the bytes).
//
// A thread always works on TWO radix-8 groups at once, value j of both groups in one register, so
// that all three stages of a pass combine different registers: in pass 0 the two groups are
// neighbours (16 consecutive elements), in the later passes neighbouring columns, whose values are
// already adjacent in memory (one 32-bit word).  Every 32 words are followed by 4 words of padding
// (word w lives at w + (w >> 5) * 4): the pass with eight-element spacing is then free of bank
// conflicts as well, and since the spacing of every pass is 4 words or a multiple of 32 words the
// addresses of a thread's values stay an arithmetic sequence (one add per access).
template <typename T> struct NqPacked;
template <> struct NqPacked<__nv_bfloat16> {
    using pair = __nv_bfloat162;
    static __device__ __forceinline__ void to_floats(uint32_t w, float& lo, float& hi) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xffff0000u);
    }
};
template <> struct NqPacked<__half> {
    using pair = __half2;
    static __device__ __forceinline__ void to_floats(uint32_t w, float& lo, float& hi) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w);
        lo = __low2float(h);
        hi = __high2float(h);
    }
};

template <typename T>
__device__ __forceinline__ void nq_butterfly_packed(uint32_t& l, uint32_t& r) {
    using P = typename NqPacked<T>::pair;
    const P a = *reinterpret_cast<const P*>(&l), b = *reinterpret_cast<const P*>(&r);
    const P sum = __hadd2(a, b), diff = __hsub2(a, b);
    l = *reinterpret_cast<const uint32_t*>(&sum);
    r = *reinterpret_cast<const uint32_t*>(&diff);
}

template <typename T, int STAGES>
__device__ __forceinline__ void nq_butterflies_packed(uint32_t v[8]) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        const int h = 1 << s;
#pragma unroll
        for (int j = 0; j < (1 << STAGES); ++j)
            if ((j & h) == 0) nq_butterfly_packed<T>(v[j], v[j | h]);
    }
}

__device__ __forceinline__ int nq_fwht_pad(int word) { return word + ((word >> 5) << 2); }
// words a padded buffer of `total` elements takes
__host__ __device__ __forceinline__ int nq_fwht_padded_words(int total) { return (total >> 1) + (total >> 4) + 4; }

// All butterfly stages of total / n rows of n elements (n a power of two >= 16, total a multiple of 16)
// read from x; the result stays in `words` (nq_fwht_padded_words(total) words, element 2i in the
// low half of word i at its padded address), NOT yet divided by sqrt(n).  Ends with a barrier.
// load(g) supplies the 8 consecutive elements of group g as four packed words.
template <typename T, class Load>
__device__ __forceinline__ void nq_fwht_groups_packed(Load&& load, uint32_t* words, int total, int n) {
    static_assert(sizeof(T) == 2, "packed path of the 16-bit dtypes");
    const int nthreads = blockDim.x;
    int log_n = 0;
    while ((1 << log_n) < n) ++log_n;

    // pass 0: widths 1, 2, 4 inside two neighbouring groups of 8 consecutive elements
    for (int pg = threadIdx.x; pg < (total >> 4); pg += nthreads) {
        const uint4 a = load(2 * pg);
        const uint4 b = load(2 * pg + 1);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __byte_perm(aw[i], bw[i], 0x5410);      // (a[2i], b[2i])
            v[2 * i + 1] = __byte_perm(aw[i], bw[i], 0x7632);  // (a[2i+1], b[2i+1])
        }
        nq_butterflies_packed<T, 3>(v);
        uint4 oa, ob;
        oa.x = __byte_perm(v[0], v[1], 0x5410); ob.x = __byte_perm(v[0], v[1], 0x7632);
        oa.y = __byte_perm(v[2], v[3], 0x5410); ob.y = __byte_perm(v[2], v[3], 0x7632);
        oa.z = __byte_perm(v[4], v[5], 0x5410); ob.z = __byte_perm(v[4], v[5], 0x7632);
        oa.w = __byte_perm(v[6], v[7], 0x5410); ob.w = __byte_perm(v[6], v[7], 0x7632);
        uint4* dst = reinterpret_cast<uint4*>(words + nq_fwht_pad(8 * pg));  // 8 words of one 32-word segment
        dst[0] = oa;
        dst[1] = ob;
    }
    __syncthreads();
    int done = 3;
    while (done < log_n) {
        const int stages = min(3, log_n - done);
        const int wp = 1 << (done - 1);        // words between the values a thread combines (w / 2): 4, 32, 256, ...
        const int spanw = wp << stages;        // words covered by one family of column pairs
        const int work = (total >> 1) >> stages;
        // padded distance of wp words: a thread's 4-word steps stay inside one 32-word segment (its first word has
        // bits 2..4 clear), larger steps are whole segments
        const int step = wp >= 32 ? wp + (wp >> 3) : wp;
        for (int t = threadIdx.x; t < work; t += nthreads) {
            uint32_t* mine = words + nq_fwht_pad((t / wp) * spanw + (t % wp));
            uint32_t v[8];
            if (stages == 3) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = mine[j * step];
                nq_butterflies_packed<T, 3>(v);
#pragma unroll
                for (int j = 0; j < 8; ++j) mine[j * step] = v[j];
            } else if (stages == 2) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = mine[j * step];
                nq_butterflies_packed<T, 2>(v);
#pragma unroll
                for (int j = 0; j < 4; ++j) mine[j * step] = v[j];
            } else {
                v[0] = mine[0];
                v[1] = mine[step];
                nq_butterflies_packed<T, 1>(v);
                mine[0] = v[0];
                mine[step] = v[1];
            }
        }
        __syncthreads();
        done += stages;
    }
}

// Same with the rows read from global memory (contiguous in `x`).
template <typename T>
__device__ __forceinline__ void nq_fwht_rows_packed(const T* __restrict__ x, uint32_t* words, int total, int n) {
    nq_fwht_groups_packed<T>([&](int g) { return __ldg(reinterpret_cast<const uint4*>(x) + g); }, words, total, n);
}

// 8 float32 values of dtype T (already rounded to it) as four packed words.
template <typename T> __device__ __forceinline__ uint4 nq_pack_exact8(const float v[8]);
template <> __device__ __forceinline__ uint4 nq_pack_exact8<__nv_bfloat16>(const float v[8]) {
    return make_uint4(__byte_perm(__float_as_uint(v[0]), __float_as_uint(v[1]), 0x7632),
                      __byte_perm(__float_as_uint(v[2]), __float_as_uint(v[3]), 0x7632),
                      __byte_perm(__float_as_uint(v[4]), __float_as_uint(v[5]), 0x7632),
                      __byte_perm(__float_as_uint(v[6]), __float_as_uint(v[7]), 0x7632));
}
template <> __device__ __forceinline__ uint4 nq_pack_exact8<__half>(const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// SiLU(gate) * up on tensors of dtype T as the tensor ops compute it: x / (1 + exp(-x)) in float32 rounded to
// T, then the product rounded to T.
template <typename T>
__device__ __forceinline__ void nq_silu_mul8(float gate[8], const float up[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float s = nq_round_to<T>(nq_div(gate[j], nq_add(1.0f, expf(-gate[j]))));
        gate[j] = nq_round_to<T>(nq_mul(s, up[j]));
    }
}

// The 8 consecutive elements of group g (elements 8g .. 8g+7) of a packed row buffer, as float32.
template <typename T>
__device__ __forceinline__ void nq_fwht_packed_group(const uint32_t* words, int g, float v[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(words + nq_fwht_pad(4 * g));
    NqPacked<T>::to_floats(w.x, v[0], v[1]);
    NqPacked<T>::to_floats(w.y, v[2], v[3]);
    NqPacked<T>::to_floats(w.z, v[4], v[5]);
    NqPacked<T>::to_floats(w.w, v[6], v[7]);
}

// In-place hand-over of a packed transform to a consumer that reads float32: `floats` is a region of `total`
// floats whose END holds the padded packed words of nq_fwht_groups_packed (nq_fwht_words_in_place).  Every
// value is divided by `root` (IEEE), rounded to T and written as float32 at its element index.  Chunks of 8
// groups per thread (C elements) go front to back; inside a chunk all words are read before the first float is
// written (one barrier), and the floats of a chunk never reach words of a later chunk: chunk c ends at byte
// 4 (c+1) C of the region, the words not yet read start at byte ~1.75 total + 2.25 (c+1) C, which is larger
// while elements remain ((c+1) C <= total - C, against at most 28 bytes of rounding of the start).
// Called by all `nthreads` threads of the CTA; ends with a barrier.
__device__ __forceinline__ uint32_t* nq_fwht_words_in_place(float* floats, int total) {
    const int start = (total - nq_fwht_padded_words(total)) & ~3;  // 16-byte aligned, never negative for total >= 16
    return reinterpret_cast<uint32_t*>(floats + (start > 0 ? start : 0));
}

template <typename T>
__device__ __forceinline__ void nq_fwht_packed_to_floats(float* floats, int total, float root, float inv_root) {
    const uint32_t* words = nq_fwht_words_in_place(floats, total);
    const int groups = total >> 3;
    const int nthreads = blockDim.x;
    for (int g0 = 0; g0 < groups; g0 += nthreads * 8) {
        uint4 w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int g = g0 + i * nthreads + threadIdx.x;
            w[i] = g < groups ? *reinterpret_cast<const uint4*>(words + nq_fwht_pad(4 * g)) : make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int g = g0 + i * nthreads + threadIdx.x;
            if (g < groups) {
                float v[8];
                NqPacked<T>::to_floats(w[i].x, v[0], v[1]);
                NqPacked<T>::to_floats(w[i].y, v[2], v[3]);
                NqPacked<T>::to_floats(w[i].z, v[4], v[5]);
                NqPacked<T>::to_floats(w[i].w, v[6], v[7]);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = nq_round_to<T>(nq_div_by(v[j], root, inv_root));
                float4* dst = reinterpret_cast<float4*>(floats + g * 8);
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
    }
    __syncthreads();
}
