// Large-M packed W4A4 projection: tcgen05 GEMM over the BF16 reconstructions
// of both operands (the weight is decoded once per call by nq_w4_decode, the
// activation by the encoder or nq_a4_decode).
//
//   out[t, n] = sum_k A^[t, k] * W^[n, k]        (both operands K-major BF16)
//
// Mapping ("swap-AB"): the 128 output channels of a tile are the UMMA M side
// (TMEM lanes), the tokens are the UMMA N side (up to 256 TMEM columns), so a
// short token tile does not waste tensor-core rows.
//
// Persistent, warp-specialised CTA (one per SM, 192 threads):
//   warp 0      TMA producer: 128B-swizzled [rows x 64] BF16 tiles of W^ and A^
//               into a multi-stage shared-memory ring (no multicast)
//   warp 1      allocates TMEM, then one elected thread issues tcgen05.mma
//               (4 x K16 per stage) and tcgen05.commit to recycle stages
//   warps 2..5  epilogue: tcgen05.ld of one accumulator buffer while the next
//               tile's MMAs fill the other one (2 x 256 TMEM columns)
// Every mbarrier wait is bounded; on a time-out the role records a code in
// the status word, raises the CTA abort flag, in-flight copies are drained and
// TMEM is released before the CTA returns.
//
// FUSED variant (one launch for the whole projection): sixteen more warps per CTA
// decode the packed NQRT4 weight -- codeword, regenerated dither, two E8 searches,
// beta and row scale -- on the ALU pipes while the tensor pipe of the same SM runs
// the MMAs.  Decode work is cut into units of 128 channels x 64 features that the
// CTAs take round-robin in channel-tile order; a unit's BF16 values go to the W^
// scratch (L2-resident for the shapes of interest), every warp bumps the channel
// tile's arrival counter when its share of a unit is written, and a TMA producer
// waits (bounded) until the counter of ITS channel tile says all features are
// there before it starts loading that tile.  Output tiles are ordered channel-tile
// major, so the first tiles become ready after 1/n_tiles of the decode and the MMAs
// trail the decode instead of waiting for all of it.  Decode warps never wait for
// anything, so no CTA can block another one: the kernel needs no co-residency.
// The weight is still decoded exactly once per call.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include "nq_common.cuh"
#include "nq_sm100.cuh"

namespace {

using namespace nq100;

constexpr int kTileN = 128;      // output channels per tile (UMMA M)
constexpr int kTileK = 64;       // K elements per stage (one 128-byte swizzle row)
constexpr int kThreadsTc = 192;  // 6 warps
constexpr int kAccCols = 256;    // TMEM columns per accumulator buffer
constexpr int kMaxStages = 8;
constexpr int kPairMinK = 2048;   // paired channel tiles: measured from 32 k-steps per item upwards
constexpr int kDecodeWarps = 16;                              // FUSED: warps 6..21 decode the weight
constexpr int kThreadsFused = kThreadsTc + kDecodeWarps * 32;  // 704 threads at 80 registers
constexpr int kUnitBlocks = kTileN * (kTileK / 8);            // E8 blocks per decode unit (128 channels x 64 features)

struct TcParams {
    int m, n, k;        // tokens, channels, features
    int tile_t;         // tokens per tile (32, 64, 128 or 256)
    int stages;
    int n_tiles, t_tiles;
    void* out;          // [m, n]
    int out_bf16;
    unsigned* status;   // 0 = ok
    int group_n;        // output tiles are visited in bands of group_n channel tiles: within a band token-tile major
                        // (group_n = n_tiles: plain token-tile-major order)
    int pair;           // 1: a work item covers TWO adjacent channel tiles (256 channels) that share the token tile in
                        // shared memory; both 256-column accumulators belong to the item, n_tiles counts pairs
    int splits;         // K splits per output tile (1 = none); work item = tile * splits + split
    float* partial;     // [splits, m, n] float32 partial sums when splits > 1
    unsigned* counters; // unused
};

// Operands of the decode warps (FUSED only).
struct FusedParams {
    const uint32_t* codes;   // packed NQRT4 streams of the weight
    const uint8_t* beta_ids;
    const float* norms;
    const float* betas;
    NqDitherSegments seg;
    float sqrt_k;
    uint4* w_dec;            // [n, k] BF16 scratch: written by the decode warps, read by the TMA loads of map_w
    unsigned* ready;         // [n_tiles] warp arrivals per channel tile; zero on entry, zero again on exit
    unsigned* exit_count;    // CTAs that have finished; the last one clears `ready`
};

struct __align__(8) TcBarriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    unsigned ticket;
};

// Channel and token offset of output tile `tile` (see TcParams::group_n).
template <bool PAIR = false>
__device__ __forceinline__ void tc_tile_origin(const TcParams& p, int tile, int& n0, int& t0) {
    const int per_band = p.group_n * p.t_tiles;
    const int band = tile / per_band, r = tile - band * per_band;
    const int width = min(p.group_n, p.n_tiles - band * p.group_n);
    const int t_tile = r / width;
    n0 = (band * p.group_n + (r - t_tile * width)) * (PAIR ? 2 * kTileN : kTileN);
    t0 = t_tile * p.tile_t;
}

__device__ __forceinline__ void tc_fail(const TcParams& p, TcBarriers* bars, unsigned code) {
    atomicCAS(p.status, 0u, code);
    *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
}

template <bool FUSED, bool PAIR = false>
__global__ void __launch_bounds__(FUSED ? kThreadsFused : kThreadsTc, 1)
nq_w4a4_tc_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                       const TcParams p, const FusedParams f) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment required by the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t w_tile_bytes = kTileN * kTileK * 2;
    const uint32_t w_bytes = PAIR ? 2 * w_tile_bytes : w_tile_bytes;
    const uint32_t a_bytes = (uint32_t)p.tile_t * kTileK * 2;
    const uint32_t stage_bytes = w_bytes + a_bytes;
    TcBarriers* bars = reinterpret_cast<TcBarriers*>(smem + (size_t)p.stages * stage_bytes);
    // PAIR: four private 32 x 32 BF16 tiles behind the barriers, one per epilogue warp
    uint8_t* epilogue_stage = reinterpret_cast<uint8_t*>(bars) + ((sizeof(TcBarriers) + 15) & ~(size_t)15);
    (void)epilogue_stage;
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_steps_all = p.k / kTileK;
    const int total_tiles = p.n_tiles * p.t_tiles * p.splits;  // work items

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->acc_full[b], 1);
            mbar_init(&bars->acc_empty[b], 4);  // one arrival per epilogue warp
        }
        bars->abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, 2 * kAccCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t fill = 0;  // running stage-fill counter
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const int tile = item / p.splits, split = item - tile * p.splits;
                int n0, t0;
                tc_tile_origin<PAIR>(p, tile, n0, t0);
                const int ks0 = split * k_steps_all / p.splits, ks1 = (split + 1) * k_steps_all / p.splits;
                if (FUSED) {
                    // every decode warp adds one arrival per unit of this channel tile
                    const uint32_t target = (uint32_t)k_steps_all * kDecodeWarps;
                    const uint32_t* flag = f.ready + n0 / kTileN;
                    bool there = false;
                    for (uint32_t poll = 0; poll < (1u << 19) && !there; ++poll) {
                        there = ld_acquire_gpu(flag) >= target;
                        if (!there) {
                            if (*abort_flag) break;
                            __nanosleep(200);
                        }
                    }
                    if (!there) {
                        tc_fail(p, bars, 5);
                        ok = false;
                        break;
                    }
                    fence_proxy_async_all();  // the decoded values were written with plain stores
                }
                for (int ks = ks0; ks < ks1; ++ks, ++fill) {
                    const int s = fill % p.stages;
                    const uint32_t use = fill / p.stages;
                    if (use > 0 && !mbar_wait_bounded(&bars->empty[s], (use - 1) & 1, abort_flag)) {
                        tc_fail(p, bars, 1);
                        ok = false;
                        break;
                    }
                    uint8_t* dst = smem + (size_t)s * stage_bytes;
                    mbar_arrive_expect_tx(&bars->full[s], stage_bytes);
                    tma_load_2d(dst, &map_w, ks * kTileK, n0, &bars->full[s]);
                    if (PAIR) tma_load_2d(dst + w_tile_bytes, &map_w, ks * kTileK, n0 + kTileN, &bars->full[s]);
                    tma_load_2d(dst + w_bytes, &map_a, ks * kTileK, t0, &bars->full[s]);
                }
            }
            if (*abort_flag) {
                // drain: wait (bounded) for every copy this thread armed
                for (int s = 0; s < p.stages && (uint32_t)s < fill; ++s) {
                    const uint32_t uses = (fill - 1 - s) / p.stages + 1;
                    mbar_wait_limit(&bars->full[s], (uses - 1) & 1, 1u << 16);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kTileN, (uint32_t)p.tile_t);
            uint32_t fill = 0, local_tile = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++local_tile) {
                // paired items own both accumulator buffers: nothing to alternate, the epilogue has to drain first
                const uint32_t buf = PAIR ? 0u : (local_tile & 1), use = PAIR ? local_tile : (local_tile >> 1);
                if (use > 0 && !mbar_wait_bounded(&bars->acc_empty[buf], (use - 1) & 1, abort_flag)) {
                    tc_fail(p, bars, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * kAccCols;
                const int split = item % p.splits;
                const int ks0 = split * k_steps_all / p.splits, ks1 = (split + 1) * k_steps_all / p.splits;
                for (int ks = ks0; ks < ks1; ++ks, ++fill) {
                    const int s = fill % p.stages;
                    if (!mbar_wait_bounded(&bars->full[s], (fill / p.stages) & 1, abort_flag)) {
                        tc_fail(p, bars, 3);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + (size_t)s * stage_bytes);
                    const uint64_t desc_w = umma_desc_sw128(base);
                    const uint64_t desc_w1 = umma_desc_sw128(base + w_tile_bytes);
                    const uint64_t desc_a = umma_desc_sw128(base + w_bytes);
#pragma unroll
                    for (int kk = 0; kk < kTileK / 16; ++kk) {
                        // +32 bytes per K16 step inside the 128-byte swizzle row (16-byte units)
                        umma_bf16(acc, desc_w + (uint64_t)(kk * 2), desc_a + (uint64_t)(kk * 2), idesc,
                                  (ks > ks0 || kk > 0) ? 1u : 0u);
                        if (PAIR)
                            umma_bf16(acc + kAccCols, desc_w1 + (uint64_t)(kk * 2), desc_a + (uint64_t)(kk * 2), idesc,
                                      (ks > ks0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&bars->empty[s]);
                }
                if (ok) umma_commit(&bars->acc_full[buf]);
            }
        }
    } else if (FUSED && warp >= kThreadsTc / 32) {
        // ------------------------------------------------------------ weight decode (ALU pipes)
        // A unit is 128 channels x 64 features = 1024 blocks, two per decode thread; eight consecutive threads
        // write the 128 contiguous bytes of one channel's 64 features.  When a warp has written its share of a
        // unit, every lane makes its stores visible device-wide and lane 0 counts the warp in.
        // (Measured alternatives that were slower: 26 decode warps at 64 registers, fetching the next block's
        // operands ahead, counting with a release one iteration late instead of the fence.)
        const int dt = (int)threadIdx.x - kThreadsTc;
        const int bpr = p.k >> 3;
        const int units = p.n_tiles * k_steps_all;
        const float rcp_sqrt_k = nq_rcp(f.sqrt_k);
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int n_tile = u / k_steps_all, kc = u - n_tile * k_steps_all;
#pragma unroll 1
            for (int i = dt; i < kUnitBlocks; i += kDecodeWarps * 32) {
                const int row = n_tile * kTileN + (i >> 3);
                const int64_t g = (int64_t)row * bpr + kc * (kTileK / 8) + (i & 7);
                float r[8];
                nq_decode_weight_block(__ldg(f.codes + g), nq_segment_base(f.seg, row) + (uint32_t)g * 8u, r);
                const float beta = __ldg(f.betas + nq_beta_id(f.beta_ids, g));
                const float ds = nq_div_by(__ldg(f.norms + row), f.sqrt_k, rcp_sqrt_k);  // = IEEE division
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = nq_mul(nq_mul(r[j], beta), ds);
                f.w_dec[g] = nq_pack_bf16x8(r);
            }
            fence_proxy_async_all();
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(f.ready + n_tile, 1u);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        uint32_t local_tile = 0;
        for (int item = blockIdx.x; item < total_tiles; item += gridDim.x, ++local_tile) {
            const uint32_t buf = PAIR ? 0u : (local_tile & 1), use = PAIR ? local_tile : (local_tile >> 1);
            const int tile = item / p.splits, split = item - tile * p.splits;
            int n0, t0;
            tc_tile_origin<PAIR>(p, tile, n0, t0);
            const bool ready = mbar_wait_bounded(&bars->acc_full[buf], use & 1, abort_flag);
            if (!ready) {
                if (lane == 0) tc_fail(p, bars, 4);
                break;
            }
            tc_fence_after();
            for (int half = 0; half < (PAIR ? 2 : 1); ++half) {
            const int channel = n0 + half * kTileN + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (buf + half) * kAccCols + ((uint32_t)(quarter * 32) << 16);
            for (int c = 0; c < p.tile_t; c += 32) {
                if (t0 + c >= p.m) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + (uint32_t)c, r);
                tmem_ld_wait();
                if constexpr (PAIR) {
                    if (p.out_bf16) {
                        // The pair's epilogue is not hidden behind the next item's MMAs, so it is worth doing
                        // properly: the warp's 32 tokens x 32 channels go through a private 2 KB tile of shared
                        // memory and leave as 16-byte stores (four per lane instead of 32 two-byte ones).
                        __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(epilogue_stage) + (warp - 2) * (32 * 32);
#pragma unroll
                        for (int j = 0; j < 32; ++j) tile[j * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        __syncwarp();
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)(t0 + c) * p.n + n0 +
                                           half * kTileN + quarter * 32;
#pragma unroll
                        for (int round = 0; round < 4; ++round) {
                            const int row = round * 8 + (lane >> 2), piece = lane & 3;
                            const uint4 v = *reinterpret_cast<const uint4*>(tile + row * 32 + piece * 8);
                            if (t0 + c + row < p.m) *reinterpret_cast<uint4*>(o + (int64_t)row * p.n + piece * 8) = v;
                        }
                        __syncwarp();
                        continue;
                    }
                }
                if (p.splits > 1) {
                    float* o = p.partial + ((int64_t)split * p.m + t0 + c) * p.n + channel;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (t0 + c + j < p.m) o[(int64_t)j * p.n] = __uint_as_float(r[j]);
                } else if (p.out_bf16) {
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)(t0 + c) * p.n + channel;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (t0 + c + j < p.m) o[(int64_t)j * p.n] = __float2bfloat16_rn(__uint_as_float(r[j]));
                } else {
                    float* o = reinterpret_cast<float*>(p.out) + (int64_t)(t0 + c) * p.n + channel;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (t0 + c + j < p.m) o[(int64_t)j * p.n] = __uint_as_float(r[j]);
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * kAccCols);
    }
    if (FUSED) {
        // the last CTA to finish puts the arrival counters back to zero for the next call
        if (threadIdx.x == 0) {
            __threadfence();
            bars->ticket = atomicAdd(f.exit_count, 1u);
        }
        __syncthreads();
        if (bars->ticket == gridDim.x - 1) {
            for (int i = threadIdx.x; i < p.n_tiles; i += blockDim.x) f.ready[i] = 0u;
            if (threadIdx.x == 0) *f.exit_count = 0u;
        }
    }
}

// Sum the K-split partial tiles in split order (deterministic) and cast to the output dtype.
__global__ void __launch_bounds__(256)
nq_tc_splitk_reduce_kernel(const float4* __restrict__ partial, int splits, int64_t quads, void* __restrict__ out,
                           int out_bf16) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= quads) return;
    float4 acc = __ldcg(partial + i);
    for (int s = 1; s < splits; ++s) {
        const float4 v = __ldcg(partial + (int64_t)s * quads + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (out_bf16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo),
                                                      *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        reinterpret_cast<float4*>(out)[i] = acc;
    }
}

// ---- host side -----------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [rows, k] BF16 row-major matrix, box = [box_rows, 64], 128-byte swizzle, zero fill out of bounds.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    NQ_REQUIRE(fn != nullptr, NQ_ERR_DEVICE, "nq_w4a4_gemm: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NQ_REQUIRE(r == CUDA_SUCCESS, NQ_ERR_ARG, "nq_w4a4_gemm: cuTensorMapEncodeTiled failed with %d", (int)r);
    return NQ_OK;
}

int sm_count() { return nq_sm_count(); }

}  // namespace

bool nq_tc_supported(int64_t m, int64_t n, int64_t k) {
    return m >= 1 && n % kTileN == 0 && k % kTileK == 0 && k >= kTileK;
}

namespace {
// K splits for grids that would leave most SMs idle (few output tiles, long K).
int tc_splits(int64_t m, int64_t n, int64_t k) {
    const int tile_t = m > 128 ? 256 : (m > 64 ? 128 : (m > 32 ? 64 : 32));
    const int tiles = (int)(n / kTileN) * (int)((m + tile_t - 1) / tile_t);
    const int k_steps = (int)(k / kTileK);
    int splits = sm_count() / tiles;
    if (splits > k_steps / 4) splits = k_steps / 4;
    if (splits > 16) splits = 16;
    return splits < 2 ? 1 : splits;
}
}  // namespace

// float32 partial sums of the split-K variant
size_t nq_tc_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    const int splits = tc_splits(m, n, k);
    return splits > 1 ? (size_t)splits * m * n * sizeof(float) : 256;
}

namespace {

struct TcPlan {
    TcParams p;
    CUtensorMap map_w, map_a;
    size_t smem;
    int total;  // output work items (tiles x splits)
};

int tc_plan(TcPlan& plan, const void* a_dec, const void* w_dec, int64_t m, int64_t n, int64_t k, void* out,
            int out_dtype, void* status_word, void* partial, unsigned* counters, bool allow_pair = false) {
    TcParams& p = plan.p;
    p.splits = partial ? tc_splits(m, n, k) : 1;
    p.partial = reinterpret_cast<float*>(partial);
    p.counters = counters;
    p.m = (int)m; p.n = (int)n; p.k = (int)k;
    p.tile_t = m > 128 ? 256 : (m > 64 ? 128 : (m > 32 ? 64 : 32));
    p.n_tiles = (int)(n / kTileN);
    p.t_tiles = (int)((m + p.tile_t - 1) / p.tile_t);
    // Two channel tiles per work item when that still gives every SM an item: the token tile is loaded once for 256
    // channels (64 KB instead of 96 KB of shared-memory fill for the same MMAs), at the price of an epilogue that
    // the next item's MMAs cannot overlap (both accumulator buffers belong to the item) -- which is why the paired
    // epilogue leaves through shared memory as 16-byte stores.  Measured on M = 8192 (GEMM alone): down_proj
    // (K = 8192) 224 -> 178 us, gate/up (K = 2048) 207 -> 180 us, q/o 55 -> 41 us.  The pairing is a template
    // parameter: as a run-time flag it slowed the unpaired kernel by 20 %.
    p.pair = (allow_pair && p.tile_t == 256 && p.splits == 1 && n % (2 * kTileN) == 0 && k >= kPairMinK &&
              (n / (2 * kTileN)) * p.t_tiles >= sm_count()) ? 1 : 0;
    if (p.pair) p.n_tiles /= 2;
    p.group_n = p.n_tiles;
    const size_t stage_bytes = (size_t)(kTileN * (p.pair ? 2 : 1) + p.tile_t) * kTileK * 2;
    int stages = (int)((200 * 1024) / stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    p.stages = stages;
    p.out = out;
    p.out_bf16 = out_dtype == NQ_BF16;
    p.status = reinterpret_cast<unsigned*>(status_word);
    int rc = make_map(&plan.map_w, w_dec, n, k, kTileN);
    if (rc) return rc;
    rc = make_map(&plan.map_a, a_dec, m, k, p.tile_t);
    if (rc) return rc;
    plan.smem = (size_t)stages * stage_bytes + sizeof(TcBarriers) + 1024 + (p.pair ? 16 + 4 * 32 * 32 * 2 : 0);
    plan.total = p.n_tiles * p.t_tiles * p.splits;
    return NQ_OK;
}

// the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of each kernel
template <bool FUSED, bool PAIR = false>
int tc_configure() {
    static bool configured[NQ_MAX_DEVICES] = {false};
    const int device = nq_current_device();
    if (device < 0 || !configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(nq_w4a4_tc_gemm_kernel<FUSED, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) {
            nq_set_error("nq_w4a4_gemm: cannot reserve shared memory: %s", cudaGetErrorString(e));
            return (int)e;
        }
        if (device >= 0) configured[device] = true;
    }
    return NQ_OK;
}

int tc_reduce(const TcParams& p, int64_t m, int64_t n, void* out, cudaStream_t stream) {
    if (p.splits > 1) {
        const int64_t quads = m * n / 4;  // n % 128 == 0
        nq_tc_splitk_reduce_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<const float4*>(p.partial), p.splits, quads, out, p.out_bf16);
        NQ_CHECK_LAUNCH("nq_w4a4_gemm(split-K reduce)");
    }
    return NQ_OK;
}

}  // namespace

int nq_launch_tc_gemm(const void* a_dec, const void* w_dec, int64_t m, int64_t n, int64_t k, void* out,
                      int out_dtype, void* status_word, void* partial, unsigned* counters, cudaStream_t stream) {
    TcPlan plan;
    int rc = tc_plan(plan, a_dec, w_dec, m, n, k, out, out_dtype, status_word, partial, counters, true);
    if (rc) return rc;
    const int grid = plan.total < sm_count() ? plan.total : sm_count();
    if (plan.p.pair) {
        if ((rc = tc_configure<false, true>())) return rc;
        nq_w4a4_tc_gemm_kernel<false, true><<<grid, kThreadsTc, plan.smem, stream>>>(plan.map_w, plan.map_a, plan.p, FusedParams{});
    } else {
        if ((rc = tc_configure<false>())) return rc;
        nq_w4a4_tc_gemm_kernel<false><<<grid, kThreadsTc, plan.smem, stream>>>(plan.map_w, plan.map_a, plan.p, FusedParams{});
    }
    NQ_CHECK_LAUNCH("nq_w4a4_gemm(tcgen05)");
    return tc_reduce(plan.p, m, n, out, stream);
}

// The whole projection in one launch: the packed weight is decoded into w_scratch by the decode warps
// of the same kernel that multiplies it (see the header of this file).  counters: at least
// n / 128 + 1 zeroed words, left zero.
int nq_launch_fused_gemm(const void* a_dec, const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                         const float* w_betas, const NqDitherSegments& seg, void* w_scratch, int64_t m, int64_t n,
                         int64_t k, void* out, int out_dtype, void* status_word, void* partial, unsigned* counters,
                         cudaStream_t stream) {
    TcPlan plan;
    int rc = tc_plan(plan, a_dec, w_scratch, m, n, k, out, out_dtype, status_word, partial, counters);
    if (rc) return rc;
    if ((rc = tc_configure<true>())) return rc;
    // Tile order: narrow bands of channel tiles, so that the first tiles only need the first band of the weight
    // (the MMAs then trail the decode) -- but every band streams the whole activation matrix once more, so when
    // that matrix is larger than about half of the L2 the bands are widened to keep it to four passes over HBM.
    const size_t a_bytes = (size_t)m * k * 2;
    plan.p.group_n = a_bytes <= ((size_t)64 << 20) ? 2 : (plan.p.n_tiles + 3) / 4;
    if (plan.p.group_n < 2) plan.p.group_n = 2;
    if (plan.p.group_n > plan.p.n_tiles) plan.p.group_n = plan.p.n_tiles;
    FusedParams f;
    f.codes = reinterpret_cast<const uint32_t*>(w_codes);
    f.beta_ids = w_beta_ids;
    f.norms = w_norms;
    f.betas = w_betas;
    f.seg = seg;
    f.sqrt_k = (float)sqrt((double)k);
    f.w_dec = reinterpret_cast<uint4*>(w_scratch);
    f.ready = counters;
    f.exit_count = counters + plan.p.n_tiles;
    const int units = plan.p.n_tiles * (int)(k / kTileK);
    const int work = plan.total > units ? plan.total : units;
    const int grid = work < sm_count() ? work : sm_count();
    nq_w4a4_tc_gemm_kernel<true><<<grid, kThreadsFused, plan.smem, stream>>>(plan.map_w, plan.map_a, plan.p, f);
    NQ_CHECK_LAUNCH("nq_w4a4_gemm(fused decode + tcgen05)");
    return tc_reduce(plan.p, m, n, out, stream);
}
