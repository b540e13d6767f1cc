// nq_w4a4_gemv_static: the small-M packed W4A4 projection for callers that
// cannot provide (or allocate) a workspace.
//
// Who needs this: hosts that call into this library from a place where device
// allocation is off the table -- a plugin slot that is only handed its input
// and output buffers, a serving thread whose memory is fully budgeted by an
// outer pool, or a latency-critical decode loop that must never reach
// cudaMalloc (which can block on the whole device).  Such a caller passes
// inputs and outputs only; the scratch the split-K kernel needs (decoded
// activation rows, per-slice partial sums, arrival counters) lives in a
// fixed-size array in device global memory that is part of this library's
// image.  Every GPU that loads the library carries that array (about 8.6 MiB)
// until the process exits.
//
// Consequences the caller must know:
//   * Limits: m <= 16, n <= 8192, k <= 8192 (larger shapes are rejected).
//   * The FIRST call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and caches it; make
//     that first call during set-up, before any stream capture.
//   * All calls share the one array: two calls whose kernels overlap on the
//     GPU (different streams, or different host threads) race on it.  Issue
//     them on one stream, or order them yourself.
//   * The array keeps whatever the previous call left; the arrival counters
//     are cleared at the start of every call, everything else is overwritten
//     before it is read.
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#include <math.h>

#include "nq_common.cuh"

size_t nq_small_m_partial_bytes(int64_t m, int64_t n, int64_t k);
int nq_launch_small_m(const void* a_dec, const uint8_t* w_codes, const uint8_t* w_beta_ids,
                      const float* w_norms, const float* w_betas, int64_t m, int64_t n, int64_t k,
                      int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                      float* partial, unsigned* counters, cudaStream_t stream, const NqDitherSegments* segments);

namespace {

constexpr int64_t kStaticMaxM = NQ_STATIC_MAX_M;
constexpr int64_t kStaticMaxN = NQ_STATIC_MAX_N;
constexpr int64_t kStaticMaxK = NQ_STATIC_MAX_K;
constexpr size_t kCounterBytes = 4096;                                   // n / 8 <= 1024 words
constexpr size_t kDecodedBytes = (size_t)kStaticMaxM * kStaticMaxK * 2;  // BF16 activation rows
constexpr size_t kPartialBytes = (size_t)8 << 20;                        // split-K partial sums
constexpr size_t kScratchBytes = kCounterBytes + kDecodedBytes + kPartialBytes;

// In host code this name is only a handle for the runtime, never a device
// address: the address is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_address[kMaxDevices] = {nullptr};

// Device address of the scratch array on the CURRENT device (looked up once per device).
int static_scratch(unsigned char** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        nq_set_error("nq_w4a4_gemv_static: cannot identify the current device (%s)", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : NQ_ERR_DEVICE;
    }
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, g_static_scratch);
        if (e != cudaSuccess || address == nullptr) {
            nq_set_error("nq_w4a4_gemv_static: cudaGetSymbolAddress failed on device %d: %s", device,
                         cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : NQ_ERR_DEVICE;
        }
        g_scratch_address[device] = static_cast<unsigned char*>(address);
    }
    *out = g_scratch_address[device];
    return NQ_OK;
}

}  // namespace

extern "C" int nq_w4a4_gemv_static(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                                   const float* act_betas, const uint8_t* w_codes, const uint8_t* w_beta_ids,
                                   const float* w_norms, const float* w_betas, int64_t m, int64_t n, int64_t k,
                                   int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                                   nq_stream_t stream) {
    NQ_RANGE("nq_w4a4_gemv_static");
    NQ_REQUIRE(act_codes && act_beta_ids && act_norms && act_betas && w_codes && w_beta_ids && w_norms && w_betas && out,
               NQ_ERR_ARG, "nq_w4a4_gemv_static: null pointer");
    NQ_REQUIRE(m >= 1 && m <= kStaticMaxM && n >= 8 && n % 8 == 0 && n <= kStaticMaxN && k >= 32 && k % 32 == 0 &&
                   k <= kStaticMaxK,
               NQ_ERR_ARG,
               "nq_w4a4_gemv_static: shape m=%lld n=%lld k=%lld is outside the built-in scratch "
               "(m <= %lld, n <= %lld multiple of 8, k <= %lld multiple of 32); use nq_w4a4_gemm with a workspace",
               (long long)m, (long long)n, (long long)k, (long long)kStaticMaxM, (long long)kStaticMaxN,
               (long long)kStaticMaxK);
    NQ_REQUIRE(out_dtype == NQ_F32 || out_dtype == NQ_BF16, NQ_ERR_ARG, "nq_w4a4_gemv_static: out_dtype must be f32 or bf16");
    NQ_REQUIRE(seed >= 0 && seed < ((int64_t)1 << 31) && w_block_offset >= 0 &&
                   w_block_offset + n * (k / 8) <= ((int64_t)1 << 28),
               NQ_ERR_ARG, "nq_w4a4_gemv_static: dither seed / block range outside the 31-bit counter space");
    NQ_REQUIRE(nq_small_m_partial_bytes(m, n, k) <= kPartialBytes, NQ_ERR_ARG,
               "nq_w4a4_gemv_static: split-K partial sums do not fit the built-in scratch");
    NQ_REQUIRE(nq_aligned16(out) && nq_aligned16(w_codes), NQ_ERR_ALIGN,
               "nq_w4a4_gemv_static: out and w_codes must be 16-byte aligned");
    unsigned char* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    unsigned* counters = reinterpret_cast<unsigned*>(scratch);
    void* decoded = scratch + kCounterBytes;
    float* partial = reinterpret_cast<float*>(scratch + kCounterBytes + kDecodedBytes);
    // The counters must start at zero; the previous call normally leaves them so, but clear them anyway.
    cudaError_t e = cudaMemsetAsync(counters, 0, kCounterBytes, s);
    if (e != cudaSuccess) {
        nq_set_error("nq_w4a4_gemv_static: clearing the counters failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    rc = nq_a4_decode(act_codes, act_beta_ids, act_norms, act_betas, m, k, decoded, NQ_BF16, stream);
    if (rc) return rc;
    return nq_launch_small_m(decoded, w_codes, w_beta_ids, w_norms, w_betas, m, n, k, w_block_offset, seed, out,
                             out_dtype, partial, counters, s, nullptr);
}
