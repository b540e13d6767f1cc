// Small-token projection on a weight that is kept DECODED in HBM (BF16 [n, k],
// the output of nq_w4_decode): a streaming GEMV.  One warp owns one output
// channel; every lane issues up to eight 16-byte weight loads before it uses
// the first, so a row of 2048 features is in flight as one burst of 4 KB per
// warp.  The weights are read once with a streaming hint; the few activation
// rows are re-read by every warp and stay in L1.  FP32 accumulation per lane
// in feature order, then a shuffle tree: the result does not depend on
// scheduling.
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
                                                                    int bpr, void* out, int out_bf16) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kGemvWarps + (threadIdx.x >> 5);
    if (row >= n) return;
    const uint4* wr = w + (int64_t)row * bpr;

    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;

    for (int b0 = lane; b0 < bpr; b0 += 32 * kUnroll) {
        uint4 wv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int b = b0 + 32 * u;
            wv[u] = b < bpr ? nq_ld_stream(wr + b) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int b = b0 + 32 * u;
            if (b >= bpr) break;
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

#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    if (lane == 0) {
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
    const unsigned grid = (unsigned)((n + kGemvWarps - 1) / kGemvWarps);
    const int out_bf16 = out_dtype == NQ_BF16;
    if (m == 1) nq_bf16_gemv_kernel<1><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, out, out_bf16);
    else if (m == 2) nq_bf16_gemv_kernel<2><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, out, out_bf16);
    else nq_bf16_gemv_kernel<4><<<grid, kGemvThreads, 0, stream>>>(w, a, (int)m, (int)n, bpr, out, out_bf16);
    NQ_CHECK_LAUNCH("nq_w4a4_gemm_resident(gemv)");
    return NQ_OK;
}
