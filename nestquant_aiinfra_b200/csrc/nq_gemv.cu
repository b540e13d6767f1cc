// Packed W4A4 projection for small token counts (M <= 16): a split-K GEMV on
// the CUDA cores.  Each lane decodes one packed weight block per step (32-bit
// codeword load, dither regenerated from the block counter, two E8
// projections), rounds the 8 weights to BF16 and multiplies them with the M
// BF16 activation rows held in shared memory; FP32 accumulation.
//
// Work split: grid = (N/8, ksplit).  A CTA owns 8 output channels (one per
// warp) and one K slice; lanes stride over the slice's blocks.  With
// ksplit > 1 the per-slice sums go to a workspace and the LAST CTA to arrive
// for a channel group adds them in slice order, so the result does not depend
// on scheduling (no floating-point atomics).
//
// Replaces nqrt4_w4a4_gemv_m1_packed_word_probe_kernel / split-K partial +
// reduce / small-M and M16 mma.sync kernels of the reference
// (runtime/nqrt4_w4a4_mma.cu:901-1061, 229-409, 124-171).
#include <math.h>

#include "nq_common.cuh"

namespace {

constexpr int kRowsPerCta = 8;
constexpr int kThreads = 256;

struct SmallMParams {
    const __nv_bfloat16* a_dec;  // [m, k] bf16
    const uint32_t* w_codes;
    const uint8_t* w_beta_ids;
    const float* w_norms;
    const float* w_betas;
    int m, n, k;
    int slice_blocks;  // blocks per K slice (multiple of 32)
    int ksplit;
    NqDitherSegments seg;   // dither counters: base (8 * w_block_offset + seed) mod 2^32 per stacked tensor
    float sqrt_k;
    float* partial;      // [ksplit, m, n] when ksplit > 1
    unsigned* counters;  // [n / 8], zero on entry, zero on exit
    void* out;           // [m, n]
    int out_bf16;
};

template <int MT>
__global__ void __launch_bounds__(kThreads) nq_w4a4_small_m_kernel(const SmallMParams p) {
    extern __shared__ uint4 a_smem[];  // [MT][slice_blocks] blocks of 8 bf16
    __shared__ unsigned s_ticket;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bpr = p.k >> 3;
    const int ks = blockIdx.y;
    const int slice0 = ks * p.slice_blocks;
    const int slice_n = min(p.slice_blocks, bpr - slice0);

    // stage the activation slice (rows >= m are zero)
    for (int i = tid; i < MT * p.slice_blocks; i += kThreads) {
        const int mrow = i / p.slice_blocks, b = i - mrow * p.slice_blocks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (mrow < p.m && b < slice_n)
            v = __ldg(reinterpret_cast<const uint4*>(p.a_dec) + (int64_t)mrow * bpr + slice0 + b);
        a_smem[i] = v;
    }
    __syncthreads();

    const int row = blockIdx.x * kRowsPerCta + warp;
    const float ds = nq_div(__ldg(p.w_norms + row), p.sqrt_k);
    const uint32_t counter_base = nq_segment_base(p.seg, row);

    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;

    for (int b = lane; b < slice_n; b += 32) {
        const int64_t g = (int64_t)row * bpr + slice0 + b;
        float w[8];
        nq_decode_weight_block(__ldg(p.w_codes + g), counter_base + (uint32_t)g * 8u, w);
        const float bt = __ldg(p.w_betas + nq_beta_id(p.w_beta_ids, g));
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = nq_bf16_round(nq_mul(nq_mul(w[j], bt), ds));
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            float a[8];
            nq_unpack_bf16x8(a_smem[i * p.slice_blocks + b], a);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i] = fmaf(a[j], w[j], acc[i]);
        }
    }

#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }

    if (p.ksplit == 1) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                if (i < p.m) {
                    const int64_t o = (int64_t)i * p.n + row;
                    if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(acc[i]);
                    else reinterpret_cast<float*>(p.out)[o] = acc[i];
                }
            }
        }
        return;
    }

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < MT; ++i)
            if (i < p.m) p.partial[((int64_t)ks * p.m + i) * p.n + row] = acc[i];
        __threadfence();
    }
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(p.counters + blockIdx.x, 1u);
    __syncthreads();
    if (s_ticket != (unsigned)(p.ksplit - 1)) return;

    // last CTA of this channel group: fixed-order sum over slices
    __threadfence();
    for (int i = tid; i < p.m * kRowsPerCta; i += kThreads) {
        const int mrow = i / kRowsPerCta, r = blockIdx.x * kRowsPerCta + (i - mrow * kRowsPerCta);
        float total = 0.0f;
        for (int s = 0; s < p.ksplit; ++s) total += __ldcg(p.partial + ((int64_t)s * p.m + mrow) * p.n + r);
        const int64_t o = (int64_t)mrow * p.n + r;
        if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(total);
        else reinterpret_cast<float*>(p.out)[o] = total;
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;
}

template <int MT>
int launch_small_m(const SmallMParams& p, cudaStream_t stream) {
    const size_t smem = (size_t)MT * p.slice_blocks * sizeof(uint4);
    auto kernel = nq_w4a4_small_m_kernel<MT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            nq_set_error("nq_w4a4_gemm: shared memory: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    dim3 grid((unsigned)(p.n / kRowsPerCta), (unsigned)p.ksplit);
    kernel<<<grid, kThreads, smem, stream>>>(p);
    NQ_CHECK_LAUNCH("nq_w4a4_gemm(small-M)");
    return NQ_OK;
}

}  // namespace

// K-slice policy of the small-M path: 64 blocks (512 features) per slice keeps
// > 50 warps per SM in flight on the 1B shapes; capped so ksplit <= 64.
static void small_m_split(int64_t k, int* slice_blocks, int* ksplit) {
    const int bpr = (int)(k / 8);
    int slice = 64;
    while ((bpr + slice - 1) / slice > 64) slice *= 2;
    if (slice > bpr) slice = (bpr + 31) / 32 * 32;
    *slice_blocks = slice;
    *ksplit = (bpr + slice - 1) / slice;
}

size_t nq_small_m_partial_bytes(int64_t m, int64_t n, int64_t k) {
    int slice, ksplit;
    small_m_split(k, &slice, &ksplit);
    return ksplit > 1 ? (size_t)ksplit * m * n * sizeof(float) : 0;
}

// a_dec: bf16 [m,k]; counters: >= n/8 zeroed words; partial: nq_small_m_partial_bytes.
int nq_launch_small_m(const void* a_dec, const uint8_t* w_codes, const uint8_t* w_beta_ids,
                      const float* w_norms, const float* w_betas, int64_t m, int64_t n, int64_t k,
                      int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                      float* partial, unsigned* counters, cudaStream_t stream, const NqDitherSegments* segments) {
    SmallMParams p;
    p.a_dec = reinterpret_cast<const __nv_bfloat16*>(a_dec);
    p.w_codes = reinterpret_cast<const uint32_t*>(w_codes);
    p.w_beta_ids = w_beta_ids;
    p.w_norms = w_norms;
    p.w_betas = w_betas;
    p.m = (int)m; p.n = (int)n; p.k = (int)k;
    small_m_split(k, &p.slice_blocks, &p.ksplit);
    p.seg = segments ? *segments : nq_one_segment(w_block_offset, seed);
    p.sqrt_k = (float)sqrt((double)k);
    p.partial = partial;
    p.counters = counters;
    p.out = out;
    p.out_bf16 = out_dtype == NQ_BF16;
    if (m == 1) return launch_small_m<1>(p, stream);
    if (m == 2) return launch_small_m<2>(p, stream);
    if (m <= 4) return launch_small_m<4>(p, stream);
    if (m <= 8) return launch_small_m<8>(p, stream);
    return launch_small_m<16>(p, stream);
}
