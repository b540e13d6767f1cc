// Device-side storage of the decode table of undithered codewords (nq_e8.cuh,
// "table-driven decode").
//
// The 106 entries are computed ONCE per device by nq_lut_init_kernel -- with the
// device's own float32 operations: they ARE the roundings the straight decode
// would perform -- into a small array in global memory.  A kernel that decodes
// copies them into shared memory, replicated once per lane: entry i of lane l
// lives at word offset (i * 32 + l) * 2, i.e. always in the lane's own pair of
// banks, so the eight lookups of a block are conflict-free whatever the
// codewords are.  The tie squares (read by a few percent of the blocks) are
// kept once.
#pragma once

#include <cuda_runtime.h>

#include "nq_common.cuh"
#include "nq_e8.cuh"

struct NqLutShared {
    uint2 entries[NQ_LUT_ENTRIES * 32];
    float4 tie[NQ_LUT_ENTRIES];
};

struct NqLutGlobal {
    uint2 entries[NQ_LUT_ENTRIES];
    float4 tie[NQ_LUT_ENTRIES];
};

// one copy per translation unit that includes this header (and per device)
static __device__ NqLutGlobal g_nq_lut;

static __global__ void __launch_bounds__(128) nq_lut_init_kernel() {
    __shared__ NqLutCoord coord[NQ_LUT_ENTRIES];
    for (int i = threadIdx.x; i < NQ_LUT_ENTRIES; i += blockDim.x) nq_lut_coordinate(i - NQ_LUT_BIAS, coord[i]);
    __syncthreads();
    for (int i = threadIdx.x; i < NQ_LUT_ENTRIES; i += blockDim.x) {
        uint32_t k, o;
        nq_lut_pack(coord, i, k, o);
        g_nq_lut.entries[i] = make_uint2(k, o);
        g_nq_lut.tie[i] = make_float4(coord[i].q[0], coord[i].q[1], coord[i].q[2], coord[i].q[3]);
    }
}

// Makes sure the table of the current device is filled before work queued on `stream` after this
// call reads it.  The first call per device launches the init kernel and waits for it once (other
// streams may follow without any ordering against this one); while `stream` is being captured the
// kernel is recorded into the graph instead and nothing is remembered.
inline cudaError_t nq_lut_ensure(cudaStream_t stream) {
    static bool ready[NQ_MAX_DEVICES] = {false};
    const int device = nq_current_device();
    if (device >= 0 && ready[device]) return cudaSuccess;
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    cudaError_t err = cudaStreamIsCapturing(stream, &capture);
    if (err != cudaSuccess) return err;
    nq_lut_init_kernel<<<1, 128, 0, stream>>>();
    nq_count_launch();
    err = cudaGetLastError();
    if (err != cudaSuccess || capture != cudaStreamCaptureStatusNone) return err;
    err = cudaStreamSynchronize(stream);
    if (err == cudaSuccess && device >= 0) ready[device] = true;
    return err;
}

// Copies the table into shared memory; every thread of the CTA must call it (it ends with a barrier).
__device__ __forceinline__ void nq_lut_load(NqLutShared* s) {
    for (int i = threadIdx.x; i < NQ_LUT_ENTRIES; i += blockDim.x) {
        const uint2 e = g_nq_lut.entries[i];
#pragma unroll 8
        for (int l = 0; l < 32; ++l) s->entries[i * 32 + l] = e;
        s->tie[i] = g_nq_lut.tie[i];
    }
    __syncthreads();
}

// The phases of nq_decode_codeword_lut on the shared-memory table; `lane` = threadIdx.x & 31.
__device__ __forceinline__ void nq_lut_begin_shared(uint32_t word, const NqLutShared* s, int lane, NqLutBlock& blk) {
    const char* base = reinterpret_cast<const char*>(s->entries) + lane * 8;
    nq_lut_begin(word,
                 [&](uint32_t packed, int i, uint32_t& k, uint32_t& o) {
                     // byte i of `packed` moved to bits 8..15: the entry's byte offset (index * 32 lanes * 8 bytes)
                     const uint32_t off = __byte_perm(packed, 0u, 0x4404u | ((uint32_t)i << 4));
                     const uint2 v = *reinterpret_cast<const uint2*>(base + off);
                     k = v.x;
                     o = v.y;
                 },
                 blk);
}

__device__ __forceinline__ bool nq_lut_resolve_tie_shared(const NqLutBlock& blk, const NqLutShared* s) {
    const char* tie_base = reinterpret_cast<const char*>(s->tie);
    return nq_lut_resolve_tie(blk, [&](uint32_t packed, int i, float q[4]) {
        const uint32_t off = __byte_perm(packed, 0u, 0x4440u | (uint32_t)i) << 4;
        const float4 v = *reinterpret_cast<const float4*>(tie_base + off);
        q[0] = v.x; q[1] = v.y; q[2] = v.z; q[3] = v.w;
    });
}

// nq_decode_codeword_undithered(word, r) from the table.
__device__ __forceinline__ void nq_decode_codeword_shared(uint32_t word, const NqLutShared* s, int lane, float r[8]) {
    NqLutBlock blk;
    nq_lut_begin_shared(word, s, lane, blk);
    bool integer_coset = blk.delta < 0;
    if (blk.delta == 0) integer_coset = nq_lut_resolve_tie_shared(blk, s);
    nq_lut_finish(blk, integer_coset, r);
}
