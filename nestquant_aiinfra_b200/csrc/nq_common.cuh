// Shared host/device helpers of the C-ABI library: error reporting, dtype
// tags, 128-bit vector loads of one E8 block, bf16 packing.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/nq_b200.h"
#include "nq_e8.cuh"

// ---- host-side error plumbing --------------------------------------------
void nq_set_error(const char* fmt, ...);
void nq_count_launch();  // bumps the process-wide kernel-launch counter (nq_launch_count)

#define NQ_REQUIRE(cond, code, ...)          \
    do {                                     \
        if (!(cond)) {                       \
            nq_set_error(__VA_ARGS__);       \
            return (code);                   \
        }                                    \
    } while (0)

#define NQ_CHECK_LAUNCH(name)                                                  \
    do {                                                                       \
        cudaError_t nq_e_ = cudaGetLastError();                                \
        if (nq_e_ != cudaSuccess) {                                            \
            nq_set_error("%s: %s", (name), cudaGetErrorString(nq_e_));         \
            return (int)nq_e_;                                                 \
        }                                                                      \
        nq_count_launch();                                                     \
    } while (0)

static inline bool nq_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// NVTX range around every C-ABI entry (host side only; a no-op call when no profiling tool is attached).
#include <nvtx3/nvToolsExt.h>
struct NqRange {
    explicit NqRange(const char* name) { nvtxRangePushA(name); }
    ~NqRange() { nvtxRangePop(); }
    NqRange(const NqRange&) = delete;
    NqRange& operator=(const NqRange&) = delete;
};
#define NQ_RANGE(name) NqRange nq_range_guard_(name)

// Per-device facts, looked up once per device (a process may drive several GPUs): the current
// device's index (or -1) and its SM count.  The tables only ever receive the same value for the same
// slot, so unsynchronised writers are harmless.
#define NQ_MAX_DEVICES 64
inline int nq_current_device() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NQ_MAX_DEVICES) return -1;
    return device;
}
inline int nq_sm_count() {
    static int counts[NQ_MAX_DEVICES] = {0};
    const int device = nq_current_device();
    if (device < 0) return 148;
    if (counts[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            count = 148;
        counts[device] = count;
    }
    return counts[device];
}

// ---- device helpers --------------------------------------------------------
#if defined(__CUDACC__)

// Dither counters of a weight that stacks the rows of several tensors (q/k/v, gate/up): rows from
// first_row[i] on belong to tensor i, whose block g (index in the stacked weight) has the counter
// base[i] + 8 g.  A plain weight is one segment.
#define NQ_MAX_SEGMENTS 4
struct NqDitherSegments {
    int count;
    int first_row[NQ_MAX_SEGMENTS];
    uint32_t base[NQ_MAX_SEGMENTS];
};
__host__ __device__ inline uint32_t nq_segment_base(const NqDitherSegments& seg, int row) {
    uint32_t base = seg.base[0];
#pragma unroll
    for (int i = 1; i < NQ_MAX_SEGMENTS; ++i)
        if (i < seg.count && row >= seg.first_row[i]) base = seg.base[i];
    return base;
}
inline NqDitherSegments nq_one_segment(int64_t w_block_offset, int64_t seed) {
    NqDitherSegments seg = {};
    seg.count = 1;
    seg.base[0] = (uint32_t)((uint64_t)w_block_offset * 8u + (uint64_t)seed);
    return seg;
}

// Load the 8 consecutive elements of one E8 block (16-byte aligned) as float32.
template <typename T>
__device__ __forceinline__ void nq_load8(const T* p, float v[8]);

template <>
__device__ __forceinline__ void nq_load8<float>(const float* p, float v[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void nq_unpack_bf16x8(const uint4 q, float v[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <>
__device__ __forceinline__ void nq_load8<__nv_bfloat16>(const __nv_bfloat16* p, float v[8]) {
    nq_unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p)), v);
}

template <>
__device__ __forceinline__ void nq_load8<__half>(const __half* p, float v[8]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        const float2 f = __half22float2(h);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// Round 8 floats to bf16 and pack them into one 16-byte vector.
__device__ __forceinline__ uint4 nq_pack_bf16x8(const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);  // one cvt.rn.bf16x2.f32
        w[i] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// 2-bit beta id of flat block g from the packed id stream.
__device__ __forceinline__ int nq_beta_id(const uint8_t* beta_ids, int64_t g) {
    return (beta_ids[g >> 2] >> ((int)(g & 3) * 2)) & 3;
}

#endif  // __CUDACC__
