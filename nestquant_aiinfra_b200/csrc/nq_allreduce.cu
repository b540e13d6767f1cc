// Sum of the tensor-parallel ranks' partial projection outputs (after o_proj / down_proj), read straight
// out of the peers' memory over NVLink: one launch per rank, no library collective.
//
// Every rank keeps, in memory that all ranks of the group have mapped (symmetric / IPC memory):
//   * its partial output (BF16, `count` values), written by its own GEMM before this launch;
//   * a flag pad of 32 words: [0..7] "rank r has its partial of call e ready", [8..15] "rank r has read
//     everyone's partial of call e", [16] the number of calls completed (local), [17] a CTA ticket (local),
//     [18] status (local; non-zero: a bounded wait gave up).
// Call e on every rank:  announce my partial to all pads  ->  wait until my pad shows all ranks at e  ->
// sum the `world` partials in rank order in float32 (the same order on every rank: identical results), one
// rounding to BF16  ->  the last CTA announces "done reading" to all pads and waits until all ranks have,
// so that no GEMM overwrites a partial a slower rank is still reading.  Flags only ever grow (call numbers),
// nothing is reset between calls.  Peer memory is read with volatile 16-byte loads (never through TMA or
// multicast) and every wait is bounded: after 2^22 polls the kernel records a status and carries on.
//
// The reference is single-GPU: no counterpart.  Replaces dist.all_reduce in RowParallelNQRTLinear when the
// group shares one node.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nq_common.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kArThreads = 256;
constexpr uint32_t kPollLimit = 1u << 22;

struct ArParams {
    const uint4* partial[kMaxRanks];  // every rank's partial, as mapped in THIS process
    uint32_t* pad[kMaxRanks];         // every rank's flag pad, as mapped in this process
    int rank, world;
    uint4* out;                       // [count] BF16, local
    int64_t vecs;                     // count / 8
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_volatile_16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// waits until all `world` words at `flags` have reached call number e; false when the poll limit (one budget
// for the whole wait, a few seconds) ran out
__device__ __forceinline__ bool wait_all(const uint32_t* flags, int world, uint32_t e) {
    uint32_t polls = 0;
    for (int r = 0; r < world; ++r) {
        while ((int32_t)(ld_acquire_sys(flags + r) - e) < 0) {
            if (++polls > kPollLimit) return false;
            __nanosleep(64);
        }
    }
    return true;
}

__global__ void __launch_bounds__(kArThreads) nq_tp_allreduce_kernel(const ArParams p) {
    uint32_t* mine = p.pad[p.rank];
    __shared__ int s_last;
    // the call number: every CTA reads it before the last CTA of this launch advances it
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(mine + 16) + 1u;
    // once a wait has given up, the group is out of step for good: later calls do not wait again (fail fast,
    // the status stays set for the host to see)
    const bool broken = *reinterpret_cast<volatile uint32_t*>(mine + 18) != 0u;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();  // my partial was written by the previous kernel of this stream
        st_release_sys(p.pad[threadIdx.x] + p.rank, e);
    }
    if (threadIdx.x == 0 && !broken && !wait_all(mine, p.world, e)) atomicCAS(mine + 18, 0u, 1u);
    __syncthreads();

    for (int64_t i = (int64_t)blockIdx.x * kArThreads + threadIdx.x; i < p.vecs; i += (int64_t)gridDim.x * kArThreads) {
        uint4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.world) v[r] = ld_volatile_16(p.partial[r] + i);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.world) {
                float f[8];
                nq_unpack_bf16x8(v[r], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += f[j];
            }
        }
        p.out[i] = nq_pack_bf16x8(acc);
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(mine + 17, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        // every CTA of this rank has finished reading: tell the others, and leave only when all of them have
        if (threadIdx.x < p.world) st_release_sys(p.pad[threadIdx.x] + 8 + p.rank, e);
        if (threadIdx.x == 0) {
            if (!broken && !wait_all(mine + 8, p.world, e)) atomicCAS(mine + 18, 0u, 2u);
            mine[17] = 0u;
            *reinterpret_cast<volatile uint32_t*>(mine + 16) = e;
        }
    }
}

// Two-shot form for four ranks and more: a rank first sums ITS slice (1 / world of the values) of all partials
// and writes the rounded result back into its own partial buffer (nobody else reads that slice in this phase),
// then every rank copies the other ranks' finished slices.  Per rank 2 * (world - 1) / world of the buffer
// crosses NVLink instead of world - 1 buffers; the price is a third flag round between the two phases, for
// which every CTA of the launch has to be resident (the grid is at most one CTA per SM, and a CTA only ever
// waits for flags that CTAs which have already started will set).  Flag words 20..27: "rank r has reduced its
// slice of call e"; word 19: CTA ticket of the first phase.  Same sums in the same order as the one-shot form.
__global__ void __launch_bounds__(kArThreads) nq_tp_allreduce_two_shot_kernel(const ArParams p) {
    uint32_t* mine = p.pad[p.rank];
    __shared__ int s_last;
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(mine + 16) + 1u;
    const bool broken = *reinterpret_cast<volatile uint32_t*>(mine + 18) != 0u;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();
        st_release_sys(p.pad[threadIdx.x] + p.rank, e);
    }
    if (threadIdx.x == 0 && !broken && !wait_all(mine, p.world, e)) atomicCAS(mine + 18, 0u, 1u);
    __syncthreads();

    // phase 1: my slice of every partial -> reduced, into my own buffer (peers fetch it in phase 2) and into out
    const int64_t slice = p.vecs / p.world, begin = slice * p.rank;
    uint4* my_partial = const_cast<uint4*>(p.partial[p.rank]);
    for (int64_t i = (int64_t)blockIdx.x * kArThreads + threadIdx.x; i < slice; i += (int64_t)gridDim.x * kArThreads) {
        uint4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.world) v[r] = ld_volatile_16(p.partial[r] + begin + i);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.world) {
                float f[8];
                nq_unpack_bf16x8(v[r], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += f[j];
            }
        }
        const uint4 packed = nq_pack_bf16x8(acc);
        my_partial[begin + i] = packed;
        p.out[begin + i] = packed;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // the reduced slice before the flag
        s_last = atomicAdd(mine + 19, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last && threadIdx.x < p.world) st_release_sys(p.pad[threadIdx.x] + 20 + p.rank, e);
    if (s_last && threadIdx.x == 0) mine[19] = 0u;
    if (threadIdx.x == 0 && !broken && !wait_all(mine + 20, p.world, e)) atomicCAS(mine + 18, 0u, 3u);
    __syncthreads();

    // phase 2: the other ranks' reduced slices
    const int64_t others = slice * (p.world - 1);
    for (int64_t i = (int64_t)blockIdx.x * kArThreads + threadIdx.x; i < others; i += (int64_t)gridDim.x * kArThreads) {
        const int hop = (int)(i / slice);                      // 0 .. world - 2
        const int src = (p.rank + 1 + hop) % p.world;          // every rank starts with another peer
        const int64_t at = slice * src + (i - (int64_t)hop * slice);
        p.out[at] = ld_volatile_16(p.partial[src] + at);
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(mine + 17, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        if (threadIdx.x < p.world) st_release_sys(p.pad[threadIdx.x] + 8 + p.rank, e);
        if (threadIdx.x == 0) {
            if (!broken && !wait_all(mine + 8, p.world, e)) atomicCAS(mine + 18, 0u, 2u);
            mine[17] = 0u;
            *reinterpret_cast<volatile uint32_t*>(mine + 16) = e;
        }
    }
}

}  // namespace

extern "C" int nq_tp_allreduce_bf16(const void* const* partials_host, void* const* pads_host, int rank, int world,
                                    void* out_bf16, int64_t count, nq_stream_t stream) {
    NQ_RANGE("nq_tp_allreduce_bf16");
    NQ_REQUIRE(partials_host && pads_host && out_bf16, NQ_ERR_ARG, "nq_tp_allreduce_bf16: null pointer");
    NQ_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, NQ_ERR_ARG,
               "nq_tp_allreduce_bf16: 1 <= world <= %d and 0 <= rank < world required", kMaxRanks);
    NQ_REQUIRE(count >= 8 && count % 8 == 0, NQ_ERR_ARG, "nq_tp_allreduce_bf16: count must be a positive multiple of 8");
    ArParams p;
    for (int r = 0; r < kMaxRanks; ++r) {
        p.partial[r] = nullptr;
        p.pad[r] = nullptr;
    }
    for (int r = 0; r < world; ++r) {
        NQ_REQUIRE(partials_host[r] && pads_host[r] && nq_aligned16(partials_host[r]) && nq_aligned16(pads_host[r]),
                   NQ_ERR_ALIGN, "nq_tp_allreduce_bf16: every rank's partial and flag pad must be mapped and 16-byte aligned");
        p.partial[r] = reinterpret_cast<const uint4*>(partials_host[r]);
        p.pad[r] = reinterpret_cast<uint32_t*>(pads_host[r]);
    }
    NQ_REQUIRE(nq_aligned16(out_bf16), NQ_ERR_ALIGN, "nq_tp_allreduce_bf16: out must be 16-byte aligned");
    p.rank = rank;
    p.world = world;
    p.out = reinterpret_cast<uint4*>(out_bf16);
    p.vecs = count / 8;
    const int64_t wanted = (p.vecs + kArThreads - 1) / kArThreads;
    const int sms = nq_sm_count();
    const unsigned grid = (unsigned)(wanted < sms ? wanted : sms);
    if (world >= 4 && p.vecs % world == 0) {
        // the two-shot kernel waits between its phases: never more CTAs than can be resident at once
        const int64_t per_phase = (p.vecs / world * (world - 1) + kArThreads - 1) / kArThreads;
        const unsigned two_shot_grid = (unsigned)(per_phase < sms ? per_phase : sms);
        nq_tp_allreduce_two_shot_kernel<<<two_shot_grid, kArThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    } else {
        nq_tp_allreduce_kernel<<<grid, kArThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    }
    NQ_CHECK_LAUNCH("nq_tp_allreduce_bf16");
    return NQ_OK;
}
