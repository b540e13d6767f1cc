// nq_w4a4_gemm: regime selection and workspace carving for the packed W4A4
// projection.  M <= 16 runs the split-K CUDA-core kernel (nq_gemv.cu); larger
// M decodes both operands to BF16 once and runs the tcgen05 GEMM
// (nq_gemm_tc.cu).  Native tails: any M >= 1 is one call, no padding rows.
#include "nq_common.cuh"

size_t nq_small_m_partial_bytes(int64_t m, int64_t n, int64_t k);
int nq_launch_small_m(const void* a_dec, const uint8_t* w_codes, const uint8_t* w_beta_ids,
                      const float* w_norms, const float* w_betas, int64_t m, int64_t n, int64_t k,
                      int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                      float* partial, unsigned* counters, cudaStream_t stream, const NqDitherSegments* segments);
int nq_w4_decode_segments(const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                          const float* w_betas, int64_t n, int64_t k, const NqDitherSegments& seg, void* out_bf16,
                          cudaStream_t stream);
// tcgen05 path (nq_gemm_tc.cu)
bool nq_tc_supported(int64_t m, int64_t n, int64_t k);
size_t nq_tc_workspace_bytes(int64_t m, int64_t n, int64_t k);
int nq_launch_tc_gemm(const void* a_dec, const void* w_dec, int64_t m, int64_t n, int64_t k, void* out,
                      int out_dtype, void* status_word, void* partial, unsigned* counters, cudaStream_t stream);

int nq_launch_fused_gemm(const void* a_dec, const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                         const float* w_betas, const NqDitherSegments& seg, void* w_scratch, int64_t m, int64_t n,
                         int64_t k, void* out, int out_dtype, void* status_word, void* partial, unsigned* counters,
                         cudaStream_t stream);

// streaming GEMV on a resident BF16 weight (nq_gemv_bf16.cu)
int nq_bf16_gemv_max_rows();
int nq_launch_bf16_gemv(const void* a_dec, const void* w_dec, int64_t m, int64_t n, int64_t k, void* out,
                        int out_dtype, cudaStream_t stream);

namespace {

constexpr int64_t kSmallMMax = 16;  // rows handled by one launch of the CUDA-core kernel
constexpr int64_t kTcMinM = 8;     // from here on decode-once + tcgen05 is faster than the per-row GEMV

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Carve {
    size_t a_dec, w_dec, partial, tc, total;
};

Carve carve(int64_t m, int64_t n, int64_t k) {
    Carve c;
    size_t off = NQ_WS_COUNTER_BYTES;
    c.a_dec = off;
    off += align256((size_t)m * k * 2);
    const bool tc = m >= kTcMinM && nq_tc_supported(m, n, k);
    c.w_dec = off;
    if (tc) off += align256((size_t)n * k * 2);
    c.partial = off;
    off += align256(nq_small_m_partial_bytes(m < kSmallMMax ? m : kSmallMMax, n, k));
    c.tc = off;
    if (tc) off += align256(nq_tc_workspace_bytes(m, n, k));
    c.total = off;
    return c;
}

}  // namespace

extern "C" size_t nq_w4a4_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m < 1 || n < 1 || k < 8) return 0;
    return carve(m, n, k).total;
}

namespace {

// One projection; `seg` carries the dither counters of the (possibly stacked) weight.
int w4a4_gemm_impl(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                   const float* act_betas, const void* act_decoded,
                   const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                   const float* w_betas, int64_t m, int64_t n, int64_t k, const NqDitherSegments& seg,
                   void* out, int out_dtype, void* workspace, size_t workspace_bytes, nq_stream_t stream,
                   bool fused = false) {
    NQ_REQUIRE(w_codes && w_beta_ids && w_norms && w_betas && out, NQ_ERR_ARG, "nq_w4a4_gemm: null pointer");
    NQ_REQUIRE(act_decoded || (act_codes && act_beta_ids && act_norms && act_betas), NQ_ERR_ARG,
               "nq_w4a4_gemm: activation streams missing");
    NQ_REQUIRE(m >= 1 && n >= 8 && n % 8 == 0 && n <= 131064, NQ_ERR_ARG,
               "nq_w4a4_gemm: m=%lld n=%lld unsupported (n must be a multiple of 8, <= 131064)",
               (long long)m, (long long)n);
    NQ_REQUIRE(k >= 32 && k % 32 == 0, NQ_ERR_ARG, "nq_w4a4_gemm: k=%lld must be a multiple of 32", (long long)k);
    NQ_REQUIRE(out_dtype == NQ_F32 || out_dtype == NQ_BF16, NQ_ERR_ARG, "nq_w4a4_gemm: out_dtype must be f32 or bf16");
    const Carve c = carve(m, n, k);
    NQ_REQUIRE(workspace && workspace_bytes >= c.total, NQ_ERR_WORKSPACE,
               "nq_w4a4_gemm: workspace of %zu bytes needed, %zu given", c.total, workspace_bytes);
    NQ_REQUIRE(nq_aligned16(workspace) && nq_aligned16(out) && nq_aligned16(w_codes) &&
                   (!act_decoded || nq_aligned16(act_decoded)),
               NQ_ERR_ALIGN, "nq_w4a4_gemm: workspace, out, w_codes and act_decoded must be 16-byte aligned");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    char* ws = reinterpret_cast<char*>(workspace);
    unsigned* counters = reinterpret_cast<unsigned*>(ws);

    const void* a_dec = act_decoded;
    if (!a_dec) {
        int rc = nq_a4_decode(act_codes, act_beta_ids, act_norms, act_betas, m, k, ws + c.a_dec, NQ_BF16, stream);
        if (rc) return rc;
        a_dec = ws + c.a_dec;
    }

    if (m >= kTcMinM && nq_tc_supported(m, n, k)) {
        if (fused)  // one launch: the weight decode runs beside the MMAs of the same kernel
            return nq_launch_fused_gemm(a_dec, w_codes, w_beta_ids, w_norms, w_betas, seg, ws + c.w_dec, m, n, k, out,
                                        out_dtype, ws + NQ_WS_STATUS_OFFSET, ws + c.tc, counters, s);
        int rc = nq_w4_decode_segments(w_codes, w_beta_ids, w_norms, w_betas, n, k, seg, ws + c.w_dec, s);
        if (rc) return rc;
        return nq_launch_tc_gemm(a_dec, ws + c.w_dec, m, n, k, out, out_dtype, ws + NQ_WS_STATUS_OFFSET, ws + c.tc,
                                 counters, s);
    }

    // CUDA-core path; rows beyond 16 are processed 16 at a time
    const size_t out_elem = out_dtype == NQ_BF16 ? 2 : 4;
    for (int64_t m0 = 0; m0 < m; m0 += kSmallMMax) {
        const int64_t mc = (m - m0) < kSmallMMax ? (m - m0) : kSmallMMax;
        int rc = nq_launch_small_m(reinterpret_cast<const char*>(a_dec) + (size_t)m0 * k * 2, w_codes, w_beta_ids,
                                   w_norms, w_betas, mc, n, k, 0, 0,
                                   reinterpret_cast<char*>(out) + (size_t)m0 * n * out_elem, out_dtype,
                                   reinterpret_cast<float*>(ws + c.partial), counters, s, &seg);
        if (rc) return rc;
    }
    return NQ_OK;
}

}  // namespace

extern "C" int nq_w4a4_gemm(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                            const float* act_betas, const void* act_decoded,
                            const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                            const float* w_betas, int64_t m, int64_t n, int64_t k,
                            int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                            void* workspace, size_t workspace_bytes, nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_gemm");
    NQ_REQUIRE(k >= 32 && k % 32 == 0 && n >= 8, NQ_ERR_ARG, "nq_w4a4_gemm: bad shape");
    NQ_REQUIRE(seed >= 0 && seed < ((int64_t)1 << 31) && w_block_offset >= 0 &&
                   w_block_offset + n * (k / 8) <= ((int64_t)1 << 28),
               NQ_ERR_ARG, "nq_w4a4_gemm: dither seed / block range outside the 31-bit counter space");
    return w4a4_gemm_impl(act_codes, act_beta_ids, act_norms, act_betas, act_decoded, w_codes, w_beta_ids, w_norms,
                          w_betas, m, n, k, nq_one_segment(w_block_offset, seed), out, out_dtype, workspace,
                          workspace_bytes, stream);
}

// The same projection as ONE launch: the kernel's decode warps turn the packed weight into BF16 tiles (written to
// the scratch, counted per channel tile) while its tensor pipe multiplies the tiles that are already there.  It runs
// the same MMAs on the same decoded values as nq_w4a4_gemm, so the results are identical bit for bit.  Measured on
// B200 it does not beat the two launches of nq_w4a4_gemm yet (the decode runs slower inside the persistent kernel
// than alone, and the MMAs slow down while it runs), which is why it is a separate entry and not the default.
extern "C" int nq_w4a4_gemm_fused(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                                  const float* act_betas, const void* act_decoded,
                                  const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                                  const float* w_betas, int64_t m, int64_t n, int64_t k,
                                  int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                                  void* workspace, size_t workspace_bytes, nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_gemm_fused");
    NQ_REQUIRE(k >= 32 && k % 32 == 0 && n >= 8, NQ_ERR_ARG, "nq_w4a4_gemm_fused: bad shape");
    NQ_REQUIRE(seed >= 0 && seed < ((int64_t)1 << 31) && w_block_offset >= 0 &&
                   w_block_offset + n * (k / 8) <= ((int64_t)1 << 28),
               NQ_ERR_ARG, "nq_w4a4_gemm_fused: dither seed / block range outside the 31-bit counter space");
    return w4a4_gemm_impl(act_codes, act_beta_ids, act_norms, act_betas, act_decoded, w_codes, w_beta_ids, w_norms,
                          w_betas, m, n, k, nq_one_segment(w_block_offset, seed), out, out_dtype, workspace,
                          workspace_bytes, stream, true);
}

extern "C" int nq_w4a4_gemm_grouped(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                                    const float* act_betas, const void* act_decoded,
                                    const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                                    const float* w_betas, int64_t m, int64_t n, int64_t k, int segments,
                                    const int64_t* seg_first_row, const int64_t* seg_block_offset,
                                    const int64_t* seg_seed, void* out, int out_dtype,
                                    void* workspace, size_t workspace_bytes, nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_gemm_grouped");
    NQ_REQUIRE(segments >= 1 && segments <= NQ_MAX_SEGMENTS && seg_first_row && seg_block_offset && seg_seed,
               NQ_ERR_ARG, "nq_w4a4_gemm_grouped: 1..%d segments with their tables", NQ_MAX_SEGMENTS);
    NQ_REQUIRE(k >= 32 && k % 32 == 0 && n >= 8, NQ_ERR_ARG, "nq_w4a4_gemm_grouped: bad shape");
    NqDitherSegments seg = {};
    seg.count = segments;
    const int64_t bpr = k / 8;
    for (int i = 0; i < segments; ++i) {
        const int64_t first = seg_first_row[i], end = i + 1 < segments ? seg_first_row[i + 1] : n;
        NQ_REQUIRE((i == 0 ? first == 0 : first > seg_first_row[i - 1]) && first < end && end <= n, NQ_ERR_ARG,
                   "nq_w4a4_gemm_grouped: segment rows must start at 0, increase and stay below n");
        NQ_REQUIRE(seg_seed[i] >= 0 && seg_seed[i] < ((int64_t)1 << 31) && seg_block_offset[i] >= 0 &&
                       seg_block_offset[i] + (end - first) * bpr <= ((int64_t)1 << 28),
                   NQ_ERR_ARG, "nq_w4a4_gemm_grouped: dither seed / block range outside the 31-bit counter space");
        seg.first_row[i] = (int)first;
        // block g of the stacked weight is block g - first * bpr of tensor i
        seg.base[i] = (uint32_t)((uint64_t)(seg_block_offset[i] - first * bpr) * 8u + (uint64_t)seg_seed[i]);
    }
    return w4a4_gemm_impl(act_codes, act_beta_ids, act_norms, act_betas, act_decoded, w_codes, w_beta_ids, w_norms,
                          w_betas, m, n, k, seg, out, out_dtype, workspace, workspace_bytes, stream);
}

// ---- resident decoded weights ---------------------------------------------------------------
namespace {

// From this many rows on the tcgen05 GEMM is used on a resident weight; below, the streaming GEMV.
constexpr int64_t kResidentTcMinM = 5;

struct ResidentCarve {
    size_t a_dec, tc, total;
};

ResidentCarve carve_resident(int64_t m, int64_t n, int64_t k) {
    ResidentCarve c;
    size_t off = NQ_WS_COUNTER_BYTES;
    c.a_dec = off;
    off += align256((size_t)m * k * 2);
    c.tc = off;
    if (m >= kResidentTcMinM && nq_tc_supported(m, n, k)) off += align256(nq_tc_workspace_bytes(m, n, k));
    c.total = off;
    return c;
}

}  // namespace

extern "C" size_t nq_w4a4_resident_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m < 1 || n < 1 || k < 8) return 0;
    return carve_resident(m, n, k).total;
}

extern "C" int nq_w4a4_gemm_resident(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                                     const float* act_betas, const void* act_decoded, const void* w_decoded,
                                     int64_t m, int64_t n, int64_t k, void* out, int out_dtype,
                                     void* workspace, size_t workspace_bytes, nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_gemm_resident");
    NQ_REQUIRE(w_decoded && out, NQ_ERR_ARG, "nq_w4a4_gemm_resident: null pointer");
    NQ_REQUIRE(act_decoded || (act_codes && act_beta_ids && act_norms && act_betas), NQ_ERR_ARG,
               "nq_w4a4_gemm_resident: activation streams missing");
    NQ_REQUIRE(m >= 1 && n >= 8 && n % 8 == 0 && n <= 131064, NQ_ERR_ARG,
               "nq_w4a4_gemm_resident: m=%lld n=%lld unsupported (n must be a multiple of 8, <= 131064)",
               (long long)m, (long long)n);
    NQ_REQUIRE(k >= 32 && k % 32 == 0, NQ_ERR_ARG, "nq_w4a4_gemm_resident: k=%lld must be a multiple of 32",
               (long long)k);
    NQ_REQUIRE(out_dtype == NQ_F32 || out_dtype == NQ_BF16, NQ_ERR_ARG,
               "nq_w4a4_gemm_resident: out_dtype must be f32 or bf16");
    const ResidentCarve c = carve_resident(m, n, k);
    NQ_REQUIRE(workspace && workspace_bytes >= c.total, NQ_ERR_WORKSPACE,
               "nq_w4a4_gemm_resident: workspace of %zu bytes needed, %zu given", c.total, workspace_bytes);
    NQ_REQUIRE(nq_aligned16(workspace) && nq_aligned16(out) && nq_aligned16(w_decoded) &&
                   (!act_decoded || nq_aligned16(act_decoded)),
               NQ_ERR_ALIGN, "nq_w4a4_gemm_resident: workspace, out, w_decoded and act_decoded must be 16-byte aligned");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    char* ws = reinterpret_cast<char*>(workspace);

    const void* a_dec = act_decoded;
    if (!a_dec) {
        int rc = nq_a4_decode(act_codes, act_beta_ids, act_norms, act_betas, m, k, ws + c.a_dec, NQ_BF16, stream);
        if (rc) return rc;
        a_dec = ws + c.a_dec;
    }
    if (m >= kResidentTcMinM && nq_tc_supported(m, n, k))
        return nq_launch_tc_gemm(a_dec, w_decoded, m, n, k, out, out_dtype, ws + NQ_WS_STATUS_OFFSET, ws + c.tc,
                                 reinterpret_cast<unsigned*>(ws), s);

    const size_t out_elem = out_dtype == NQ_BF16 ? 2 : 4;
    const int64_t step = nq_bf16_gemv_max_rows();
    for (int64_t m0 = 0; m0 < m; m0 += step) {
        const int64_t mc = (m - m0) < step ? (m - m0) : step;
        int rc = nq_launch_bf16_gemv(reinterpret_cast<const char*>(a_dec) + (size_t)m0 * k * 2, w_decoded, mc, n, k,
                                     reinterpret_cast<char*>(out) + (size_t)m0 * n * out_elem, out_dtype, s);
        if (rc) return rc;
    }
    return NQ_OK;
}

extern "C" int nq_w4a4_status(const void* workspace, uint32_t* status_host, nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_status");
    NQ_REQUIRE(workspace && status_host, NQ_ERR_ARG, "nq_w4a4_status: null pointer");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(status_host, reinterpret_cast<const char*>(workspace) + NQ_WS_STATUS_OFFSET,
                                    sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        nq_set_error("nq_w4a4_status: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return NQ_OK;
}

// Building block of the large-M path, exposed for measurement and tests: the
// tcgen05 GEMM alone on already decoded BF16 operands.
extern "C" int nq_bf16_gemm_tc(const void* a_bf16, const void* w_bf16, int64_t m, int64_t n, int64_t k,
                               void* out, int out_dtype, void* workspace, size_t workspace_bytes,
                               nq_stream_t stream) {
    NQ_RANGE("nq_bf16_gemm_tc");
    NQ_REQUIRE(a_bf16 && w_bf16 && out && workspace, NQ_ERR_ARG, "nq_bf16_gemm_tc: null pointer");
    NQ_REQUIRE(nq_tc_supported(m, n, k), NQ_ERR_ARG, "nq_bf16_gemm_tc: needs n %% 128 == 0 and k %% 64 == 0");
    NQ_REQUIRE(out_dtype == NQ_F32 || out_dtype == NQ_BF16, NQ_ERR_ARG, "nq_bf16_gemm_tc: out_dtype");
    NQ_REQUIRE(workspace_bytes >= NQ_WS_COUNTER_BYTES, NQ_ERR_WORKSPACE, "nq_bf16_gemm_tc: workspace too small");
    NQ_REQUIRE(nq_aligned16(a_bf16) && nq_aligned16(w_bf16) && nq_aligned16(out), NQ_ERR_ALIGN,
               "nq_bf16_gemm_tc: 16-byte alignment required");
    char* ws = reinterpret_cast<char*>(workspace);
    const bool room = workspace_bytes >= NQ_WS_COUNTER_BYTES + nq_tc_workspace_bytes(m, n, k);
    return nq_launch_tc_gemm(a_bf16, w_bf16, m, n, k, out, out_dtype, ws + NQ_WS_STATUS_OFFSET,
                             room ? ws + NQ_WS_COUNTER_BYTES : nullptr, reinterpret_cast<unsigned*>(ws),
                             reinterpret_cast<cudaStream_t>(stream));
}
