// E8 row encoder (activations and K/V rows) and the decode of undithered and
// dithered packed streams.  HBM-bound by bytes, instruction-bound in practice:
// one thread owns one E8 block (8 values in registers, no shuffles in the
// search), 128-bit loads, one 32-bit codeword store per block.
#include <stdarg.h>
#include <math.h>

#include "nq_common.cuh"
#include "nq_encode_core.cuh"

// ---- error message storage (one per host thread) ---------------------------
static thread_local char g_nq_error[512] = "";

void nq_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_nq_error, sizeof(g_nq_error), fmt, args);
    va_end(args);
}

#include <atomic>
static std::atomic<unsigned long long> g_nq_launches{0};
void nq_count_launch() { g_nq_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" unsigned long long nq_launch_count(void) { return g_nq_launches.load(std::memory_order_relaxed); }

extern "C" const char* nq_last_error(void) { return g_nq_error; }
extern "C" int nq_abi_version(void) { return 1; }

// ---------------------------------------------------------------------------
// Encoder kernel: one CTA per group of rows (see nq_encode_core.cuh).
// ---------------------------------------------------------------------------
template <typename T, bool DITHER>
__global__ void __launch_bounds__(NQ_ENC_THREADS, 5)
nq_encode_rows_kernel(const T* __restrict__ x, int64_t rows, int k, int64_t row_stride,
                      const float* __restrict__ beta_table, float sqrt_k,
                      uint32_t* __restrict__ codes, uint8_t* __restrict__ beta_ids,
                      float* __restrict__ norms, __nv_bfloat16* __restrict__ decoded,
                      uint32_t counter_base, int blocks_per_split, int rpc, int four_lanes) {
    extern __shared__ __align__(16) float smem[];
    const int bpr = k >> 3;
    const int64_t row0 = (int64_t)blockIdx.x * rpc;
    const int nrows = (int)min((int64_t)rpc, rows - row0);
    const int64_t g0 = row0 * bpr;
    // gridDim.y > 1: a few long rows are split over several CTAs so the launch fills the GPU
    const int blk_begin = (int)blockIdx.y * blocks_per_split;
    nq_encode_rows_cta<T, DITHER>(x + row0 * row_stride, row_stride, nrows, nrows, k, beta_table, sqrt_k, codes + g0,
                          beta_ids + (g0 >> 2), norms + row0, decoded ? decoded + g0 * 8 : nullptr,
                          counter_base + (uint32_t)g0 * 8u, smem, blk_begin, blk_begin + blocks_per_split,
                          blockIdx.y == 0, rpc, four_lanes != 0);
}

// ---------------------------------------------------------------------------
// Decode of an undithered packed stream (activations / KV pages): one thread
// per block, exact reference arithmetic.
// ---------------------------------------------------------------------------
// Row of flat block g: a 32-bit division whenever the stream has fewer than 2^31 blocks (every real
// tensor), the 64-bit one costs several times as many instructions per thread.
__device__ __forceinline__ int64_t nq_row_of_block(int64_t g, int64_t blocks, int bpr) {
    return blocks <= 0x7fffffff ? (int64_t)((uint32_t)g / (uint32_t)bpr) : g / bpr;
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
nq_a4_decode_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ beta_ids,
                    const float* __restrict__ norms, const float* __restrict__ beta_table,
                    int64_t blocks, int bpr, float sqrt_k, void* __restrict__ out) {
    const int64_t g = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= blocks) return;
    const int64_t row = nq_row_of_block(g, blocks, bpr);
    float r[8];
    nq_decode_codeword_undithered(__ldg(codes + g), r);
    const float beta = __ldg(beta_table + nq_beta_id(beta_ids, g));
    const float ds = nq_div_by(__ldg(norms + row), sqrt_k, nq_rcp(sqrt_k));  // = IEEE division, fewer instructions
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_mul(nq_mul(r[j], beta), ds);
    if (OUT_BF16) {
        reinterpret_cast<uint4*>(out)[g] = nq_pack_bf16x8(r);
    } else {
        float4* o = reinterpret_cast<float4*>(out) + 2 * g;
        o[0] = make_float4(r[0], r[1], r[2], r[3]);
        o[1] = make_float4(r[4], r[5], r[6], r[7]);
    }
}

// Decode of a dithered weight stream to bf16 [n,k]; the dither of block g is a
// pure function of (w_block_offset + g, seed).
__global__ void __launch_bounds__(256)
nq_w4_decode_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ beta_ids,
                    const float* __restrict__ norms, const float* __restrict__ beta_table,
                    int64_t blocks, int bpr, float sqrt_k, const NqDitherSegments seg,
                    uint4* __restrict__ out) {
    const int64_t g = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= blocks) return;
    const int64_t row = nq_row_of_block(g, blocks, bpr);
    float r[8];
    nq_decode_weight_block(__ldg(codes + g), nq_segment_base(seg, (int)row) + (uint32_t)g * 8u, r);
    const float beta = __ldg(beta_table + nq_beta_id(beta_ids, g));
    const float ds = nq_div_by(__ldg(norms + row), sqrt_k, nq_rcp(sqrt_k));  // = IEEE division, fewer instructions
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_mul(nq_mul(r[j], beta), ds);
    out[g] = nq_pack_bf16x8(r);
}

// ---- C ABI ------------------------------------------------------------------


template <typename T>
static int launch_encode(const void* x, int64_t rows, int64_t k, int64_t row_stride,
                         const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                         float* out_norms, void* out_decoded, cudaStream_t stream,
                         int use_dither = 0, uint32_t counter_base = 0) {
    const NqEncodePlan plan = nq_encode_plan(rows, (int)k, use_dither != 0);
    const int rpc = plan.rpc, splits = plan.splits, blocks_per_split = plan.blocks_per_split;
    const size_t smem = nq_encode_smem_floats((int)k, rpc) * sizeof(float);
    auto kernel = use_dither ? nq_encode_rows_kernel<T, true> : nq_encode_rows_kernel<T, false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            nq_set_error("nq_a4_encode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
    }
    const int64_t grid = (rows + rpc - 1) / rpc;
    kernel<<<dim3((unsigned)grid, (unsigned)splits), NQ_ENC_THREADS, smem, stream>>>(
        reinterpret_cast<const T*>(x), rows, (int)k, row_stride, beta_table,
        (float)sqrt((double)k), reinterpret_cast<uint32_t*>(out_codes), out_beta_ids, out_norms,
        reinterpret_cast<__nv_bfloat16*>(out_decoded), counter_base, blocks_per_split, rpc, plan.four_lanes ? 1 : 0);
    NQ_CHECK_LAUNCH("nq_a4_encode");
    return NQ_OK;
}

extern "C" int nq_a4_encode(const void* x, int x_dtype, int64_t rows, int64_t k, int64_t row_stride,
                            const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                            float* out_norms, void* out_decoded, nq_stream_t stream) {
    NQ_RANGE("nq_a4_encode");
    NQ_REQUIRE(x && beta_table && out_codes && out_beta_ids && out_norms, NQ_ERR_ARG,
               "nq_a4_encode: null pointer");
    NQ_REQUIRE(rows >= 1 && rows <= (int64_t)1 << 31, NQ_ERR_ARG, "nq_a4_encode: rows=%lld out of range", (long long)rows);
    NQ_REQUIRE(k >= 32 && k <= 32768 && k % 32 == 0, NQ_ERR_ARG,
               "nq_a4_encode: k=%lld must be a multiple of 32 in [32, 32768]", (long long)k);
    NQ_REQUIRE(row_stride >= k, NQ_ERR_ARG, "nq_a4_encode: row_stride < k");
    const int64_t esize = x_dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(nq_aligned16(x) && (row_stride * esize) % 16 == 0, NQ_ERR_ALIGN,
               "nq_a4_encode: x and its row stride must be 16-byte aligned");
    NQ_REQUIRE(nq_aligned16(out_codes) && (!out_decoded || nq_aligned16(out_decoded)), NQ_ERR_ALIGN,
               "nq_a4_encode: outputs must be 16-byte aligned");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case NQ_F32: return launch_encode<float>(x, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        case NQ_BF16: return launch_encode<__nv_bfloat16>(x, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        case NQ_F16: return launch_encode<__half>(x, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, out_decoded, s);
        default: nq_set_error("nq_a4_encode: unknown dtype %d", x_dtype); return NQ_ERR_ARG;
    }
}

extern "C" int nq_w4_encode(const void* w, int w_dtype, int64_t rows, int64_t k, int64_t row_stride,
                            const float* beta_table, int64_t seed, int64_t w_block_offset,
                            uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms, nq_stream_t stream) {
    NQ_RANGE("nq_w4_encode");
    NQ_REQUIRE(w && beta_table && out_codes && out_beta_ids && out_norms, NQ_ERR_ARG, "nq_w4_encode: null pointer");
    NQ_REQUIRE(rows >= 1 && k >= 32 && k <= 32768 && k % 32 == 0 && row_stride >= k, NQ_ERR_ARG,
               "nq_w4_encode: bad shape rows=%lld k=%lld", (long long)rows, (long long)k);
    NQ_REQUIRE(seed >= 0 && seed < ((int64_t)1 << 31) && w_block_offset >= 0 &&
                   w_block_offset + rows * (k / 8) <= ((int64_t)1 << 28),
               NQ_ERR_ARG, "nq_w4_encode: dither seed / block range outside the 31-bit counter space");
    const int64_t esize = w_dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(nq_aligned16(w) && (row_stride * esize) % 16 == 0 && nq_aligned16(out_codes), NQ_ERR_ALIGN,
               "nq_w4_encode: 16-byte alignment required");
    const uint32_t base = (uint32_t)((uint64_t)w_block_offset * 8u + (uint64_t)seed);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case NQ_F32: return launch_encode<float>(w, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, nullptr, s, 1, base);
        case NQ_BF16: return launch_encode<__nv_bfloat16>(w, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, nullptr, s, 1, base);
        case NQ_F16: return launch_encode<__half>(w, rows, k, row_stride, beta_table, out_codes, out_beta_ids, out_norms, nullptr, s, 1, base);
        default: nq_set_error("nq_w4_encode: unknown dtype %d", w_dtype); return NQ_ERR_ARG;
    }
}

extern "C" int nq_a4_decode(const uint8_t* codes, const uint8_t* beta_ids, const float* norms,
                            const float* beta_table, int64_t rows, int64_t k, void* out, int out_dtype,
                            nq_stream_t stream) {
    NQ_RANGE("nq_a4_decode");
    NQ_REQUIRE(codes && beta_ids && norms && beta_table && out, NQ_ERR_ARG, "nq_a4_decode: null pointer");
    NQ_REQUIRE(rows >= 1 && k >= 8 && k % 8 == 0, NQ_ERR_ARG, "nq_a4_decode: bad shape");
    NQ_REQUIRE(out_dtype == NQ_F32 || out_dtype == NQ_BF16, NQ_ERR_ARG, "nq_a4_decode: out_dtype must be f32 or bf16");
    NQ_REQUIRE(nq_aligned16(out) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0, NQ_ERR_ALIGN,
               "nq_a4_decode: out must be 16-byte and codes 4-byte aligned");
    const int64_t blocks = rows * (k / 8);
    const unsigned grid = (unsigned)((blocks + 255) / 256);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const float sqrt_k = (float)sqrt((double)k);
    if (out_dtype == NQ_BF16)
        nq_a4_decode_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(codes), beta_ids, norms, beta_table, blocks, (int)(k / 8), sqrt_k, out);
    else
        nq_a4_decode_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(codes), beta_ids, norms, beta_table, blocks, (int)(k / 8), sqrt_k, out);
    NQ_CHECK_LAUNCH("nq_a4_decode");
    return NQ_OK;
}

// Shared by the plain and the grouped entry: the dither counters come as segments.
int nq_w4_decode_segments(const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                          const float* w_betas, int64_t n, int64_t k, const NqDitherSegments& seg, void* out_bf16,
                          cudaStream_t stream) {
    const int64_t blocks = n * (k / 8);
    const unsigned grid = (unsigned)((blocks + 255) / 256);
    nq_w4_decode_kernel<<<grid, 256, 0, stream>>>(
        reinterpret_cast<const uint32_t*>(w_codes), w_beta_ids, w_norms, w_betas, blocks, (int)(k / 8),
        (float)sqrt((double)k), seg, reinterpret_cast<uint4*>(out_bf16));
    NQ_CHECK_LAUNCH("nq_w4_decode");
    return NQ_OK;
}

extern "C" int nq_w4_decode(const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                            const float* w_betas, int64_t n, int64_t k, int64_t w_block_offset,
                            int64_t seed, void* out_bf16, nq_stream_t stream) {
    NQ_RANGE("nq_w4_decode");
    NQ_REQUIRE(w_codes && w_beta_ids && w_norms && w_betas && out_bf16, NQ_ERR_ARG, "nq_w4_decode: null pointer");
    NQ_REQUIRE(n >= 1 && k >= 8 && k % 8 == 0, NQ_ERR_ARG, "nq_w4_decode: bad shape");
    NQ_REQUIRE(seed >= 0 && seed < ((int64_t)1 << 31) && w_block_offset >= 0, NQ_ERR_ARG, "nq_w4_decode: bad seed/offset");
    NQ_REQUIRE(w_block_offset + n * (k / 8) <= ((int64_t)1 << 28), NQ_ERR_ARG,
               "nq_w4_decode: block range exceeds the dither counter space");
    NQ_REQUIRE(nq_aligned16(out_bf16) && (reinterpret_cast<uintptr_t>(w_codes) & 3u) == 0, NQ_ERR_ALIGN,
               "nq_w4_decode: alignment");
    return nq_w4_decode_segments(w_codes, w_beta_ids, w_norms, w_betas, n, k, nq_one_segment(w_block_offset, seed),
                                 out_bf16, reinterpret_cast<cudaStream_t>(stream));
}
