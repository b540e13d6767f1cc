// Rotate-then-encode in one launch: the normalised Hadamard transform of every activation row
// (what FusedNQRTLinear applies to its input, models/fused_linear.py:287-290) followed by the A4
// row encoder, without the round trip of the rotated rows through HBM and without a second
// launch.  The rows are transformed in shared memory with the arithmetic of nq_hadamard
// (per-stage rounding to the tensor dtype, IEEE division by sqrt(n)) and the encoder body reads
// them from there, so codes, beta ids, norms and reconstruction are bit-identical to
// nq_hadamard followed by nq_a4_encode.
//
// hadamard_block < k applies the transform to consecutive blocks of that size (the
// block-diagonal rotation of a tensor-parallel K shard).
//
// Two more entries put the elementwise work that PRECEDES the rotation into the same launch
// (module-level fusion at the plugin boundary): the Llama RMS norm in front of q/k/v and
// gate/up, and SiLU(gate) * up in front of down_proj.  Both compute exactly what the separate
// launches compute (nq_rmsnorm with its fixed reduction order; the tensor ops silu and mul with
// their roundings to the tensor dtype), so the streams stay bit-identical.
#include <math.h>

#include "nq_common.cuh"
#include "nq_encode_core.cuh"
#include "nq_rotate_core.cuh"

namespace {

enum { kPlain = 0, kRmsNorm = 1, kSiluMul = 2 };  // what produces the rows that are rotated

// kRmsNorm: x2 = the norm's weight [k]; kSiluMul: x = gate, x2 = up (both with row stride `stride`).
template <typename T, int MODE>
__global__ void __launch_bounds__(NQ_ENC_THREADS, 5)
nq_encode_rotated_kernel(const T* __restrict__ x, const T* __restrict__ x2, int64_t stride, float eps, int64_t rows,
                         int k, int hadamard_block, float root, float inv_root,
                         const float* __restrict__ beta_table, float sqrt_k, uint32_t* __restrict__ codes,
                         uint8_t* __restrict__ beta_ids, float* __restrict__ norms,
                         __nv_bfloat16* __restrict__ decoded, int blocks_per_split, int rpc, int four_lanes) {
    extern __shared__ __align__(16) float smem[];
    float* rotated = smem;                       // [rpc][k] float32 values of dtype T
    float* encoder_smem = smem + (size_t)rpc * k;
    const int bpr = k >> 3;
    const int64_t row0 = (int64_t)blockIdx.x * rpc;
    const int nrows = (int)min((int64_t)rpc, rows - row0);
    const int total = nrows * k;
    // 16-bit dtypes: packed butterflies on the rows in their own dtype, held at the end of `rotated` until they
    // are handed to the encoder as float32 (nq_fwht_packed_to_floats)
    const bool packed = sizeof(T) == 2 && hadamard_block >= 16;
    uint32_t* words = nq_fwht_words_in_place(rotated, total);
    if (MODE == kPlain) {
        if constexpr (sizeof(T) == 2) {
            if (packed) nq_fwht_rows_packed<T>(x + row0 * k, words, total, hadamard_block);
        }
        if (!packed) nq_fwht_rows_to_smem<T>(x + row0 * k, rotated, total, hadamard_block);
    } else if (MODE == kRmsNorm) {
        // 1 / rms of every row of this CTA, with nq_rmsnorm's reduction order: 128 threads take the row's groups
        // of 8 in strides, FMA chains, butterfly over the warp, the four warps in order
        __shared__ float s_part[NQ_ENC_THREADS / 32];
        float* row_scale = encoder_smem;  // nrows floats; the encoder body overwrites its scratch later
        const int groups = k >> 3;
        for (int r = 0; r < nrows; ++r) {
            const T* src = x + (row0 + r) * stride;
            float acc = 0.0f;
            for (int g = threadIdx.x; g < groups; g += NQ_ENC_THREADS) {
                float v[8];
                nq_load8<T>(src + g * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc = fmaf(v[j], v[j], acc);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < NQ_ENC_THREADS / 32; ++w) sum += s_part[w];
                row_scale[r] = rsqrtf(sum / (float)k + eps);
            }
            __syncthreads();
        }
        auto normalised = [&](int g, float v[8]) {
            const int r = (g * 8) / k, col = g * 8 - r * k;
            float w[8];
            nq_load8<T>(x + (row0 + r) * stride + col, v);
            nq_load8<T>(x2 + col, w);
            const float scale = row_scale[r];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = nq_round_to<T>(nq_mul(w[j], nq_round_to<T>(nq_mul(v[j], scale))));
        };
        if constexpr (sizeof(T) == 2) {
            if (packed)
                nq_fwht_groups_packed<T>([&](int g) { float v[8]; normalised(g, v); return nq_pack_exact8<T>(v); },
                                         words, total, hadamard_block);
        }
        if (!packed) nq_fwht_groups_to_smem<T>(normalised, rotated, total, hadamard_block);
    } else {
        auto product = [&](int g, float v[8]) {
            const int r = (g * 8) / k, col = g * 8 - r * k;
            float u[8];
            nq_load8<T>(x + (row0 + r) * stride + col, v);
            nq_load8<T>(x2 + (row0 + r) * stride + col, u);
            nq_silu_mul8<T>(v, u);
        };
        if constexpr (sizeof(T) == 2) {
            if (packed)
                nq_fwht_groups_packed<T>([&](int g) { float v[8]; product(g, v); return nq_pack_exact8<T>(v); },
                                         words, total, hadamard_block);
        }
        if (!packed) nq_fwht_groups_to_smem<T>(product, rotated, total, hadamard_block);
    }
    if constexpr (sizeof(T) == 2) {
        if (packed) nq_fwht_packed_to_floats<T>(rotated, total, root, inv_root);
    }
    if (!packed) {
        for (int i = threadIdx.x; i < total; i += NQ_ENC_THREADS)
            rotated[i] = nq_round_to<T>(nq_div_by(rotated[i], root, inv_root));
        __syncthreads();
    }
    const int64_t g0 = row0 * bpr;
    const int blk_begin = (int)blockIdx.y * blocks_per_split;
    nq_encode_rows_cta<float, false, false>(rotated, k, nrows, nrows, k, beta_table, sqrt_k, codes + g0,
                                            beta_ids + (g0 >> 2), norms + row0,
                                            decoded ? decoded + g0 * 8 : nullptr, 0u, encoder_smem, blk_begin,
                                            blk_begin + blocks_per_split, blockIdx.y == 0, rpc, four_lanes != 0);
}

template <typename T, int MODE = kPlain>
int launch_encode_rotated(const void* x, int64_t rows, int64_t k, int64_t hadamard_block, const float* beta_table,
                          uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms, void* out_decoded,
                          cudaStream_t stream, const void* x2 = nullptr, int64_t stride = 0, float eps = 0.0f) {
    NqEncodePlan plan = nq_encode_plan(rows, (int)k, false);
    {
        // Every CTA a row is split over repeats the load, the producer and the transform of the whole row, so
        // (unlike the plain encoder) more CTAs than SMs only add work: long rows are split just far enough to
        // give every SM one CTA, and the four-lanes-per-block latency mode is kept for CTAs with at most 64 blocks
        // (measured on 8 / 64 / 256 rows of 2048 and 8192 features).
        const int bpr = (int)k / 8;
        if (nq_encode_rows_per_cta((int)k) == 1) {
            const int sms = nq_sm_count();
            int splits = rows < sms ? (int)(sms / rows) : 1;
            if (splits > bpr / 32) splits = bpr / 32;
            if (splits < 1) splits = 1;
            plan.rpc = 1;
            plan.blocks_per_split = ((bpr + splits - 1) / splits + 31) / 32 * 32;
            plan.splits = (bpr + plan.blocks_per_split - 1) / plan.blocks_per_split;
            plan.four_lanes = plan.blocks_per_split <= 64;
            if (plan.splits == 1) plan.blocks_per_split = 0x40000000;
        }
    }
    const int rpc = plan.rpc, splits = plan.splits, blocks_per_split = plan.blocks_per_split;
    const size_t smem = ((size_t)rpc * k + nq_encode_smem_floats((int)k, rpc)) * sizeof(float);
    auto kernel = nq_encode_rotated_kernel<T, MODE>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            nq_set_error("nq_a4_encode_rotated: cannot reserve %zu bytes of shared memory: %s", smem,
                         cudaGetErrorString(e));
            return (int)e;
        }
    }
    const int64_t grid = (rows + rpc - 1) / rpc;
    const float root = (float)sqrt((double)hadamard_block);
    kernel<<<dim3((unsigned)grid, (unsigned)splits), NQ_ENC_THREADS, smem, stream>>>(
        reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(x2), stride ? stride : k, eps, rows, (int)k,
        (int)hadamard_block, root, 1.0f / root, beta_table,
        (float)sqrt((double)k), reinterpret_cast<uint32_t*>(out_codes), out_beta_ids, out_norms,
        reinterpret_cast<__nv_bfloat16*>(out_decoded), blocks_per_split, rpc, plan.four_lanes ? 1 : 0);
    NQ_CHECK_LAUNCH("nq_a4_encode_rotated");
    return NQ_OK;
}

}  // namespace

extern "C" int nq_a4_encode_rotated(const void* x, int x_dtype, int64_t rows, int64_t k, int64_t hadamard_block,
                                    const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                                    float* out_norms, void* out_decoded, nq_stream_t stream) {
    NQ_RANGE("nq_a4_encode_rotated");
    NQ_REQUIRE(x && beta_table && out_codes && out_beta_ids && out_norms, NQ_ERR_ARG,
               "nq_a4_encode_rotated: null pointer");
    NQ_REQUIRE(rows >= 1 && k % 32 == 0 && k >= 32 && k <= NQ_ROTATED_MAX_K, NQ_ERR_ARG,
               "nq_a4_encode_rotated: k=%lld must be a multiple of 32 in [32, %d]", (long long)k, NQ_ROTATED_MAX_K);
    NQ_REQUIRE(hadamard_block >= 8 && (hadamard_block & (hadamard_block - 1)) == 0 && k % hadamard_block == 0,
               NQ_ERR_ARG, "nq_a4_encode_rotated: hadamard_block=%lld must be a power of two >= 8 dividing k",
               (long long)hadamard_block);
    NQ_REQUIRE(nq_aligned16(x) && (!out_decoded || nq_aligned16(out_decoded)) && nq_aligned16(out_codes), NQ_ERR_ALIGN,
               "nq_a4_encode_rotated: 16-byte alignment required");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case NQ_F32: return launch_encode_rotated<float>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        case NQ_BF16: return launch_encode_rotated<__nv_bfloat16>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        case NQ_F16: return launch_encode_rotated<__half>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        default: nq_set_error("nq_a4_encode_rotated: unknown dtype %d", x_dtype); return NQ_ERR_ARG;
    }
}

// ---- elementwise producers in the same launch -------------------------------------------------

static int check_fused_args(const char* name, const void* a, const void* b, const float* beta_table,
                            const void* out_codes, const void* out_beta_ids, const void* out_norms,
                            const void* out_decoded, int dtype, int64_t rows, int64_t k, int64_t stride,
                            int64_t hadamard_block) {
    NQ_REQUIRE(a && b && beta_table && out_codes && out_beta_ids && out_norms, NQ_ERR_ARG, "%s: null pointer", name);
    NQ_REQUIRE(dtype == NQ_F32 || dtype == NQ_BF16 || dtype == NQ_F16, NQ_ERR_ARG, "%s: unknown dtype %d", name, dtype);
    NQ_REQUIRE(rows >= 1 && k % 32 == 0 && k >= 32 && k <= NQ_ROTATED_MAX_K && stride >= k, NQ_ERR_ARG,
               "%s: k=%lld must be a multiple of 32 in [32, %d] and the row stride at least k", name, (long long)k,
               NQ_ROTATED_MAX_K);
    NQ_REQUIRE(hadamard_block >= 8 && (hadamard_block & (hadamard_block - 1)) == 0 && k % hadamard_block == 0,
               NQ_ERR_ARG, "%s: hadamard_block=%lld must be a power of two >= 8 dividing k", name,
               (long long)hadamard_block);
    const int64_t esize = dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(nq_aligned16(a) && nq_aligned16(b) && (stride * esize) % 16 == 0 && nq_aligned16(out_codes) &&
                   (!out_decoded || nq_aligned16(out_decoded)),
               NQ_ERR_ALIGN, "%s: 16-byte alignment of pointers and row stride required", name);
    return NQ_OK;
}

extern "C" int nq_a4_encode_rmsnorm_rotated(const void* x, const void* weight, float eps, int dtype, int64_t rows,
                                            int64_t k, int64_t row_stride, int64_t hadamard_block,
                                            const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                                            float* out_norms, void* out_decoded, nq_stream_t stream) {
    NQ_RANGE("nq_a4_encode_rmsnorm_rotated");
    int rc = check_fused_args("nq_a4_encode_rmsnorm_rotated", x, weight, beta_table, out_codes, out_beta_ids, out_norms,
                              out_decoded, dtype, rows, k, row_stride, hadamard_block);
    if (rc) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_encode_rotated<float, kRmsNorm>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, weight, row_stride, eps);
        case NQ_BF16: return launch_encode_rotated<__nv_bfloat16, kRmsNorm>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, weight, row_stride, eps);
        default: return launch_encode_rotated<__half, kRmsNorm>(x, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, weight, row_stride, eps);
    }
}

extern "C" int nq_a4_encode_silu_mul_rotated(const void* gate, const void* up, int dtype, int64_t rows, int64_t k,
                                             int64_t row_stride, int64_t hadamard_block, const float* beta_table,
                                             uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms,
                                             void* out_decoded, nq_stream_t stream) {
    NQ_RANGE("nq_a4_encode_silu_mul_rotated");
    int rc = check_fused_args("nq_a4_encode_silu_mul_rotated", gate, up, beta_table, out_codes, out_beta_ids, out_norms,
                              out_decoded, dtype, rows, k, row_stride, hadamard_block);
    if (rc) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_encode_rotated<float, kSiluMul>(gate, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, up, row_stride, 0.0f);
        case NQ_BF16: return launch_encode_rotated<__nv_bfloat16, kSiluMul>(gate, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, up, row_stride, 0.0f);
        default: return launch_encode_rotated<__half, kSiluMul>(gate, rows, k, hadamard_block, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s, up, row_stride, 0.0f);
    }
}
