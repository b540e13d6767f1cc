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
// SILU_MUL: the rows that are transformed are SiLU(x) * x2 (the tensor ops' arithmetic and roundings), the
// input of a Llama down_proj, produced while the rows are loaded.
template <typename T, bool SILU_MUL>
__global__ void __launch_bounds__(1024)
nq_hadamard_kernel(const T* __restrict__ x, const T* __restrict__ x2, int64_t in_stride, T* __restrict__ out,
                   int64_t rows, int n, int rows_per_cta, float root, float inv_root) {
    extern __shared__ __align__(16) float buf[];
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    const int nrows = (int)min((int64_t)rows_per_cta, rows - row0);
    const int total = nrows * n;           // elements of this CTA (rows are independent, n >= 8)
    if constexpr (sizeof(T) == 2) {
        if (n >= 16) {  // 16-bit dtypes: packed butterflies, the rows stay in shared memory in their own dtype
            uint32_t* words = reinterpret_cast<uint32_t*>(buf);
            if constexpr (SILU_MUL) {
                nq_fwht_groups_packed<T>(
                    [&](int g) {
                        float v[8], u[8];
                        const int r = (g * 8) / n;
                        const int64_t at = (row0 + r) * in_stride + (g * 8 - r * n);
                        nq_load8<T>(x + at, v);
                        nq_load8<T>(x2 + at, u);
                        nq_silu_mul8<T>(v, u);
                        return nq_pack_exact8<T>(v);
                    },
                    words, total, n);
            } else {
                nq_fwht_rows_packed<T>(x + row0 * n, words, total, n);
            }
            for (int g = threadIdx.x; g < (total >> 3); g += blockDim.x) {
                float v[8];
                nq_fwht_packed_group<T>(words, g, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = nq_div_by(v[j], root, inv_root);
                nq_store8<T>(out + row0 * n + (int64_t)g * 8, v);
            }
            return;
        }
    }
    if constexpr (SILU_MUL) {
        nq_fwht_groups_to_smem<T>(
            [&](int g, float v[8]) {
                float u[8];
                const int r = (g * 8) / n;
                const int64_t at = (row0 + r) * in_stride + (g * 8 - r * n);
                nq_load8<T>(x + at, v);
                nq_load8<T>(x2 + at, u);
                nq_silu_mul8<T>(v, u);
            },
            buf, total, n);
    } else {
        nq_fwht_rows_to_smem<T>(x + row0 * n, buf, total, n);
    }
    for (int g = threadIdx.x; g < (total >> 3); g += blockDim.x) {
        const float4 lo = reinterpret_cast<const float4*>(buf + g * 8)[0];
        const float4 hi = reinterpret_cast<const float4*>(buf + g * 8)[1];
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = nq_div_by(v[j], root, inv_root);
        nq_store8<T>(out + row0 * n + (int64_t)g * 8, v);
    }
}

template <typename T, bool SILU_MUL = false>
int launch_hadamard(const void* x, void* out, int64_t rows, int64_t n, cudaStream_t stream, const void* x2 = nullptr,
                    int64_t in_stride = 0) {
    int rpc = (int)(n >= 2048 ? 1 : 2048 / n);
    // rows are held as float32, or (16-bit dtypes, packed path) in their own dtype
    const size_t smem = (sizeof(T) == 2 && n >= 16) ? (size_t)nq_fwht_padded_words(rpc * (int)n) * sizeof(uint32_t)
                                                    : (size_t)rpc * n * sizeof(float);
    auto kernel = nq_hadamard_kernel<T, SILU_MUL>;
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
    unsigned threads = groups >= 1024 ? 1024u : (groups >= 512 ? 512u : 256u);
    if (sizeof(T) == 2 && n >= 16) {
        // the packed path works on two groups per thread and pass; with many CTAs queued small ones overlap
        // their barriers better (8644 rows of 8192: 108 us with 128 threads, 155 us with 512; 64 rows: 6.5 / 4.4 us)
        if (threads > 128u) threads /= 2;
        if (grid >= 8 * (int64_t)nq_sm_count()) threads = 128u;
    }
    kernel<<<(unsigned)grid, threads, smem, stream>>>(reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(x2),
                                                  in_stride, reinterpret_cast<T*>(out), rows, (int)n, rpc, root,
                                                  1.0f / root);
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

// hadamard(silu(gate) * up) in one launch: the input of a Llama down_proj whose rows are too long for the
// rotation inside the encoder.  Same bits as the two tensor ops followed by nq_hadamard.
extern "C" int nq_hadamard_silu_mul(const void* gate, const void* up, int64_t row_stride, void* out, int dtype,
                                    int64_t rows, int64_t n, nq_stream_t stream) {
    NQ_RANGE("nq_hadamard_silu_mul");
    NQ_REQUIRE(gate && up && out, NQ_ERR_ARG, "nq_hadamard_silu_mul: null pointer");
    NQ_REQUIRE(rows >= 1 && n >= 8 && n <= 32768 && (n & (n - 1)) == 0, NQ_ERR_ARG,
               "nq_hadamard_silu_mul: n=%lld must be a power of two in [8, 32768]", (long long)n);
    const int64_t esize = dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(row_stride >= n, NQ_ERR_ARG, "nq_hadamard_silu_mul: row_stride < n");
    NQ_REQUIRE(nq_aligned16(gate) && nq_aligned16(up) && nq_aligned16(out) && (row_stride * esize) % 16 == 0, NQ_ERR_ALIGN,
               "nq_hadamard_silu_mul: 16-byte alignment required (pointers and row stride)");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NQ_F32: return launch_hadamard<float, true>(gate, out, rows, n, s, up, row_stride);
        case NQ_BF16: return launch_hadamard<__nv_bfloat16, true>(gate, out, rows, n, s, up, row_stride);
        case NQ_F16: return launch_hadamard<__half, true>(gate, out, rows, n, s, up, row_stride);
        default: nq_set_error("nq_hadamard_silu_mul: unknown dtype %d", dtype); return NQ_ERR_ARG;
    }
}
