// Small-token projection on a weight that is kept DECODED in HBM (BF16 [n, k],
// the output of nq_w4_decode): a streaming GEMV.  A warp owns one output
// channel, or one of up to eight K ranges of it when the row is longer than
// one burst; every lane issues up to eight 16-byte weight loads before it uses
// the first, so 2048 features are in flight as one burst of 4 KB per warp and
// a long row (8192, 28672 features) is spread over the warps of the CTA instead
// of being walked burst after burst by one.  The K ranges of a row are added
// in range order by one thread.  The weights are read once with a streaming
// hint; the few activation rows are re-read by every warp and stay in L1.
// FP32 accumulation per lane in feature order, then a shuffle tree: the result
// does not depend on scheduling.
//
// This is the opt-in "resident decoded weights" mode: the operands are the very
// BF16 values the packed kernels regenerate on every call (eight dither hashes
// and two E8 searches per block), so the projection trades 4x the weight bytes
// in HBM for a kernel that is bound by HBM instead of by decode instructions.
// The reference has no counterpart: its kernels always decode in the loop
// (runtime/nqrt4_w4a4_mma.cu:901-1061).
#include "nq_common.cuh"

namespace {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kUnroll = 8;  // 16-byte loads in flight per lane

__device__ __forceinline__ uint4 nq_ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int MT>
__global__ void __launch_bounds__(kGemvThreads) nq_bf16_gemv_kernel(const uint4* __restrict__ w,
                                                                    const uint4* __restrict__ a, int m, int n,
                                                                    int bpr, int ksplit, int chunk, void* out,
                                                                    int out_bf16) {
    __shared__ float s_part[kGemvWarps][MT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows_per_cta = kGemvWarps / ksplit;
    const int part = warp % ksplit;
    const int row = blockIdx.x * rows_per_cta + warp / ksplit;
    const bool live = row < n;
    const int b_begin = part * chunk, b_end = min(bpr, b_begin + chunk);

    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;

    if (live) {
        const uint4* wr = w + (int64_t)row * bpr;
        for (int b0 = b_begin + lane; b0 < b_end; b0 += 32 * kUnroll) {
            uint4 wv[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int b = b0 + 32 * u;
                wv[u] = b < b_end ? nq_ld_stream(wr + b) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int b = b0 + 32 * u;
                if (b >= b_end) break;
                float wf[8];
                nq_unpack_bf16x8(wv[u], wf);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    if (i < m) {
                        float af[8];
                        nq_unpack_bf16x8(__ldg(a + (int64_t)i * bpr + b), af);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[i] = fmaf(af[j], wf[j], acc[i]);
                    }
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    if (ksplit > 1) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i) s_part[warp][i] = acc[i];
        }
        __syncthreads();
        if (part != 0) return;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            float total = 0.0f;
            for (int q = 0; q < ksplit; ++q) total += s_part[warp + q][i];
            acc[i] = total;
        }
    }
    if (lane == 0 && live) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            if (i < m) {
                const int64_t o = (int64_t)i * n + row;
                if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(acc[i]);
                else reinterpret_cast<float*>(out)[o] = acc[i];
            }
        }
    }
}

}  // namespace

// Rows per launch of the streaming GEMV; the caller loops over larger m.
int nq_bf16_gemv_max_rows() { return 4; }

// a_dec: bf16 [m, k], w_dec: bf16 [n, k], both 16-byte aligned; m <= 4.
int nq_launch_bf16_gemv(const void* a_dec, const void* w_dec, int64_t m, int64_t n, int64_t k, void* out,
                        int out_dtype, cudaStream_t stream) {
    const uint4* w = reinterpret_cast<const uint4*>(w_dec);
    const uint4* a = reinterpret_cast<const uint4*>(a_dec);
    const int bpr = (int)(k / 8);
    // one burst = 32 lanes x 8 loads = 256 blocks; longer rows are shared by 2, 4 or 8 warps
    int ksplit = 1;
    while (ksplit < kGemvWarps && bpr > 256 * ksplit) ksplit *= 2;
    const int chunk = ((bpr + ksplit - 1) / ksplit + 31) / 32 * 32;
    const int rows_per_cta = kGemvWarps / ksplit;
    const unsigned grid = (unsigned)((n + rows_per_cta - 1) / rows_per_cta);
    const int out_bf16 = out_dtype == NQ_BF16;
    if (m == 1)
        nq_bf16_gemv_kernel<1><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, ksplit, chunk, out, out_bf16);
    else if (m == 2)
        nq_bf16_gemv_kernel<2><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, ksplit, chunk, out, out_bf16);
    else
        nq_bf16_gemv_kernel<4><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, ksplit, chunk, out, out_bf16);
    NQ_CHECK_LAUNCH("nq_w4a4_gemm_resident(gemv)");
    return NQ_OK;
}
