// Paged GQA attention that reads NQKV4 pages directly (decode and chunked
// causal prefill).  One CTA owns one (query token or tile of query tokens, KV
// head, page-range split): every K/V vector is decoded ONCE for all query rows
// of the CTA -- the heads of its GQA group, times the tokens of a prefill
// tile -- with the exact codec arithmetic (undithered streams have real Voronoi
// ties, see the table-driven decode in nq_e8.cuh), FP32 online softmax, and a
// BF16 hot tail as the last "page".  No page-count cap.
//
// Lane mapping: one cached token per lane (a warp covers 32 consecutive token
// positions per step); the kernel's own comment below describes the passes.
// Split partials (m, l, acc[D]) are merged by a second small kernel (skipped
// when there is a single split).
//
// Replaces runtime/nqkv_attention_k1.py:243-471 (page / hot / reduce Triton
// kernels, 127-page cap at :807-809) and adds the page-reading prefill the
// reference only has as materialise + SDPA (runtime/nqkv_hf_backend.py:127-150).
#include <math.h>

#include "nq_common.cuh"
#include "nq_lut.cuh"

namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;

struct AttnParams {
    const void* query;  // [B, Tq, Hq, D]
    int q_dtype;
    int batch, q_tokens, q_heads, kv_heads, dim, page_size;
    const int32_t* slot_ids;      // [B]
    const uint8_t* active_mask;   // [B] or null (all active)
    const int32_t* q_lens;        // [B] or null (decode: one token, full context)
    const uint8_t* cache_active;  // [S]
    const int32_t* sequence_lengths;
    const int32_t* page_indices;  // [S, max_pages]
    const int32_t* page_counts;
    const int32_t* last_page_lens;
    const int32_t* hot_lengths;
    const uint8_t *key_codes, *key_betas, *value_codes, *value_betas;
    const float *key_norms, *value_norms, *key_beta_table, *value_beta_table;
    const void *hot_keys, *hot_values;  // [S, P, H, D] bf16
    const int8_t *key_lattice, *value_lattice;  // optional decoded shadow of the pool (doubled coordinates as int8)
    int max_sequences, max_pages, pool_capacity;
    float scale_log2e;  // attention scale * log2(e)
    float sqrt_dim, inv_sqrt_dim;
    int splits;
    int per_slots;  // page slots (cold pages + hot tail) per split
    int q_tiles;    // query tiles per batch row (a CTA of the tiled instantiations owns QT consecutive query tokens)
    float* partial;  // [B*Tq, Hq, splits, D + 2]
    void* out;       // [B, Tq, Hq, D]
    int out_dtype;
};

__device__ __forceinline__ void store_out(void* out, int out_dtype, int64_t index, const float v[8]) {
    if (out_dtype == NQ_BF16) {
        reinterpret_cast<uint4*>(out)[index] = nq_pack_bf16x8(v);
    } else {
        float4* o = reinterpret_cast<float4*>(out) + 2 * index;
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// Resolve the query row: returns false when the row is inactive (output zero).
__device__ __forceinline__ bool resolve_query(const AttnParams& p, int qi, int& slot, int& limit, int& total_slots,
                                              int& page_count, int& last_len, int& hot_len) {
    const int b = qi / p.q_tokens, i = qi - b * p.q_tokens;
    const int requested = p.slot_ids[b];
    const bool in_range = requested >= 0 && requested < p.max_sequences;
    slot = min(max(requested, 0), p.max_sequences - 1);
    bool active = in_range && p.cache_active[slot] != 0 && p.sequence_lengths[slot] > 0;
    if (p.active_mask) active = active && p.active_mask[b] != 0;
    page_count = min(max(p.page_counts[slot], 0), p.max_pages);
    last_len = p.last_page_lens[slot];
    hot_len = min(max(p.hot_lengths[slot], 0), p.page_size);
    const int cold = page_count > 0 ? (page_count - 1) * p.page_size + last_len : 0;
    const int total = cold + hot_len;
    limit = total;
    if (p.q_lens) {
        const int ql = p.q_lens[b];
        active = active && i < ql;
        limit = total - ql + i + 1;  // causal: query i of the chunk sees the first `limit` tokens
    }
    total_slots = page_count + (hot_len > 0 ? 1 : 0);
    return active && limit > 0;
}

// The same for a tile of QT consecutive query tokens of batch row b, first token i0.  `limit0` is the causal
// limit of the first token (token i0 + r sees the first limit0 + r positions), `nrows` the number of tokens of
// the tile that are queries at all, `limit` the limit of the last of them.  Returns false when no token of the
// tile sees anything.
template <int QT>
__device__ __forceinline__ bool resolve_tile(const AttnParams& p, int b, int i0, int& slot, int& limit0, int& nrows,
                                             int& limit, int& total_slots, int& page_count, int& last_len,
                                             int& hot_len) {
    const int requested = p.slot_ids[b];
    const bool in_range = requested >= 0 && requested < p.max_sequences;
    slot = min(max(requested, 0), p.max_sequences - 1);
    bool active = in_range && p.cache_active[slot] != 0 && p.sequence_lengths[slot] > 0;
    if (p.active_mask) active = active && p.active_mask[b] != 0;
    page_count = min(max(p.page_counts[slot], 0), p.max_pages);
    last_len = p.last_page_lens[slot];
    hot_len = min(max(p.hot_lengths[slot], 0), p.page_size);
    const int cold = page_count > 0 ? (page_count - 1) * p.page_size + last_len : 0;
    const int total = cold + hot_len;
    nrows = min(QT, p.q_tokens - i0);
    limit0 = total;
    if (p.q_lens) {
        const int ql = p.q_lens[b];
        nrows = min(nrows, ql - i0);
        limit0 = total - ql + i0 + 1;
    }
    // without query lengths every token sees the whole context: one limit for all rows
    limit = p.q_lens ? limit0 + nrows - 1 : total;
    total_slots = page_count + (hot_len > 0 ? 1 : 0);
    return active && nrows > 0 && limit > 0;
}

// Register budget: the exact E8 decode leaves issue slots idle at 12 warps per SM (168 registers), so the
// kernel is built for 4 resident CTAs (128 registers; a few spilled words cost less than the lost warps).
// Eight doubled lattice coordinates (int8) -> the float coordinates the packed decode yields: each byte,
// offset by 128, is dropped into the mantissa of 1.5 * 2^23 and one FMA removes the offsets and halves.
__device__ __forceinline__ void nq_lattice_block(const uint2 raw, float v[8]) {
    const uint32_t lo = raw.x ^ 0x80808080u, hi = raw.y ^ 0x80808080u;
    const float bias = -0.5f * (NQ_MAGIC + 128.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = fmaf(__uint_as_float(__byte_perm(lo, 0x4B400000u, 0x7650u | (uint32_t)j)), 0.5f, bias);
        v[j + 4] = fmaf(__uint_as_float(__byte_perm(hi, 0x4B400000u, 0x7650u | (uint32_t)j)), 0.5f, bias);
    }
}

// Sum of v[0..N) over the 32 lanes by recursive halving: in every round a lane keeps one half of its values and
// hands the other half to the partner lane^M.  With N >= 32 a lane ends up owning the totals of the N / 32
// values [lane * N/32, (lane + 1) * N/32) in v[0..N/32); with N < 32 value lane / (32 / N) in v[0] (the lanes of
// one group all hold it).
template <int N, int M>
__device__ __forceinline__ void reduce_scatter(float* v, int lane) {
    if constexpr (M >= 1) {
        if constexpr (N >= 2) {
            const bool up = (lane & M) != 0;
#pragma unroll
            for (int i = 0; i < N / 2; ++i) {
                const float send = up ? v[i] : v[i + N / 2];
                const float keep = up ? v[i + N / 2] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, M);
            }
            reduce_scatter<N / 2, M / 2>(v, lane);
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], M);
            reduce_scatter<1, M / 2>(v, lane);
        }
    }
}

// a[c] of a small register array with a run-time index (a chain of selects: the array stays in registers)
template <typename T, int N>
__device__ __forceinline__ T pick_step(const T (&a)[N], int c) {
    T v = a[0];
#pragma unroll
    for (int i = 1; i < N; ++i) v = (c == i) ? a[i] : v;
    return v;
}

// 2-bit beta ids of the BPR blocks of one row (block b in bits 2b, 2b+1).
template <int BPR>
struct RowIds {
    using type = uint32_t;
};
template <>
struct RowIds<32> {
    using type = uint64_t;
};
template <int BPR>
__device__ __forceinline__ typename RowIds<BPR>::type load_row_ids(const uint8_t* ids, int64_t row) {
    const uint8_t* src = ids + row * (BPR / 4);
    if constexpr (BPR == 4) return __ldg(src);
    else if constexpr (BPR == 8) return __ldg(reinterpret_cast<const uint16_t*>(src));
    else if constexpr (BPR == 16) return __ldg(reinterpret_cast<const uint32_t*>(src));
    else return __ldg(reinterpret_cast<const unsigned long long*>(src));
}

// One CTA = one (query token, KV head, page-range split); its four warps take turns on steps of 32 consecutive
// token positions of the range, ONE TOKEN PER LANE.  A warp works in chunks of CH of its steps:
//   pass 1  every lane decodes the K blocks of its token one after the other and accumulates the scores of the
//           G query heads (query in shared memory, read as broadcasts): no cross-lane traffic at all;
//   softmax chunk maximum per head over the warp (the reference point only moves when it is exceeded by more
//           than 8, i.e. a factor 256), one exp2 per (token, head);
//   pass 2  block by block of V: every lane decodes the block of its CH tokens and accumulates the G x 8
//           products p * v; ONE recursive-halving reduction per block and chunk then leaves each lane with the
//           chunk's total of one output feature, which it adds to its running output.
// K/V blocks are decoded once for all query heads of the GQA group.
// Compile-time layout of one instantiation: steps per chunk and the shared-memory regions
// [decode table of the packed pages | scaled query | scores / probabilities | per-step values]; the merge buffer of
// the epilogue reuses the same storage once every warp has left the page loop.
template <int G, int BPR, bool LAT>
struct AttnLayout {
    using Ids = typename RowIds<BPR>::type;
    static constexpr int D = BPR * 8;
    // steps per chunk; four for the widest GQA group too were measured no faster (651 against 656 us on the 70B
    // shard shape, slower with one KV head per rank)
    static constexpr int CH = G <= 4 ? 4 : 2;
    static constexpr size_t kMergeBytes = sizeof(float) * kAttnWarps * G * (D + 2);
    static constexpr size_t kTableBytes = LAT ? 0 : sizeof(NqLutShared);
    static constexpr size_t kQueryBytes = sizeof(float) * G * D;
    static constexpr size_t kProbBytes = sizeof(float) * CH * kAttnThreads * G;
    // per-step values that pass 2 reads once per (block, step pair): in shared memory (indexed by a run-time step
    // there, a chain of selects on the busiest pipe otherwise), every thread its own column.  Measured: pays for
    // four steps per chunk on packed pages (268 -> 258 us); with two steps per chunk or on the cheap lattice pages
    // the extra shared-memory reads cost more than the selects.
    static constexpr size_t kStateBytes = (size_t)CH * kAttnThreads * (sizeof(int64_t) + sizeof(Ids) + sizeof(float)) + 32;
    static constexpr bool kStateInShared = !LAT && CH == 4;
    static constexpr size_t kLoopBytes = kTableBytes + kQueryBytes + kProbBytes + (kStateInShared ? kStateBytes : 0);
    static constexpr size_t kSharedBytes = kMergeBytes > kLoopBytes ? kMergeBytes : kLoopBytes;
    static_assert(kTableBytes % 16 == 0 && kQueryBytes % 16 == 0 && kProbBytes % 16 == 0,
                  "shared-memory regions must stay 16-byte aligned");
};

//
// QT > 1 (chunk prefill): the G rows of the CTA are QT consecutive query tokens x G / QT query heads, row
// r = token * (G / QT) + head.  A K/V block is then decoded once for all of them; query token r of the tile sees
// the first limit0 + r positions, which is a per-row mask on the scores.
template <int G, int BPR, bool LAT, int QT = 1>
__global__ void __launch_bounds__(kAttnThreads, (G <= 4 ? 4 : 3)) nq_attn_paged_kernel(const AttnParams p) {
    static_assert(G % QT == 0, "rows = query tokens x heads of the GQA group");
    constexpr int GH = G / QT;  // query heads per KV head
    using Layout = AttnLayout<G, BPR, LAT>;
    using Ids = typename Layout::Ids;
    constexpr int D = BPR * 8;
    constexpr int NV = G * 8;                      // products of one V block
    constexpr int NVL = NV >= 32 ? NV / 32 : 1;    // totals a lane owns after the reduction
    constexpr int CH = Layout::CH;
    constexpr size_t kTableBytes = Layout::kTableBytes, kQueryBytes = Layout::kQueryBytes, kProbBytes = Layout::kProbBytes;
    constexpr bool kStateInShared = Layout::kStateInShared;
    extern __shared__ __align__(16) unsigned char s_raw[];  // Layout::kSharedBytes
    float (*s_merge)[G][D + 2] = reinterpret_cast<float (*)[G][D + 2]>(s_raw);
    const NqLutShared* lut = reinterpret_cast<const NqLutShared*>(s_raw);
    float* s_q = reinterpret_cast<float*>(s_raw + kTableBytes);
    // scores, then probabilities, of my token of each step
    float (*s_prob)[kAttnThreads][G] = reinterpret_cast<float (*)[kAttnThreads][G]>(s_raw + kTableBytes + kQueryBytes);
    unsigned char* s_state = s_raw + kTableBytes + kQueryBytes + kProbBytes;
    int64_t (*s_row)[kAttnThreads] = reinterpret_cast<int64_t (*)[kAttnThreads]>(s_state);
    Ids (*s_vid)[kAttnThreads] = reinterpret_cast<Ids (*)[kAttnThreads]>(s_state + (size_t)CH * kAttnThreads * sizeof(int64_t));
    float (*s_vds)[kAttnThreads] = reinterpret_cast<float (*)[kAttnThreads]>(
        s_state + (size_t)CH * kAttnThreads * (sizeof(int64_t) + sizeof(Ids)));
    float* s_vbeta = reinterpret_cast<float*>(s_state + (size_t)CH * kAttnThreads * (sizeof(int64_t) + sizeof(Ids) + sizeof(float)));
    (void)s_row; (void)s_vid; (void)s_vds; (void)s_vbeta;

    // qi: the (first) query token of this CTA, as an index into [B * Tq]
    const int tile = blockIdx.x / p.kv_heads, h = blockIdx.x - tile * p.kv_heads;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int qi, slot, limit, total_slots, page_count, last_len, hot_len;
    int limit0 = 0, nrows = 1, rows_in_tensor = 1;  // of the tile
    bool active;
    if constexpr (QT == 1) {
        qi = tile;
        active = resolve_query(p, qi, slot, limit, total_slots, page_count, last_len, hot_len);
    } else {
        const int b = tile / p.q_tiles, i0 = (tile - b * p.q_tiles) * QT;
        qi = b * p.q_tokens + i0;
        rows_in_tensor = min(QT, p.q_tokens - i0);
        active = resolve_tile<QT>(p, b, i0, slot, limit0, nrows, limit, total_slots, page_count, last_len, hot_len);
    }
    (void)limit0; (void)nrows; (void)rows_in_tensor;
    const int cold = page_count > 0 ? (page_count - 1) * p.page_size + last_len : 0;
    // row r of the CTA -> row of the [B * Tq, Hq] output (only rows with r / GH < rows_in_tensor exist)
    auto out_row = [&](int r) { return (int64_t)(qi + r / GH) * p.q_heads + h * GH + (r % GH); };

    // A split that starts past the sequence's end (or past the causal limit) has nothing to add: it leaves the
    // neutral partial and returns before the table is loaded.
    if (p.splits > 1 && !(active && split * p.per_slots < total_slots && split * p.per_slots * p.page_size < limit)) {
        for (int item = threadIdx.x; item < G * (D + 2); item += kAttnThreads) {
            const int g = item / (D + 2), f = item - g * (D + 2);
            if (g / GH < rows_in_tensor) p.partial[(out_row(g) * p.splits + split) * (D + 2) + f] = f == D ? -INFINITY : 0.0f;
        }
        return;
    }

    // the query heads of this KV head are contiguous per token: [qi + token][h * GH .. h * GH + GH)[D]; they are
    // pre-multiplied by scale * log2(e)
    for (int i = threadIdx.x; i < G * D / 8; i += kAttnThreads) {
        const int r = (i * 8) / D;
        const int64_t qoff = out_row(r) * D + (i * 8 - r * D);
        float v[8];
        if (r / GH >= rows_in_tensor) {  // a tile that reaches past the last query token
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        } else if (p.q_dtype == NQ_BF16) nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.query) + qoff, v);
        else if (p.q_dtype == NQ_F16) nq_load8<__half>(reinterpret_cast<const __half*>(p.query) + qoff, v);
        else nq_load8<float>(reinterpret_cast<const float*>(p.query) + qoff, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) s_q[i * 8 + j] = v[j] * p.scale_log2e;
    }
    if constexpr (!LAT) nq_lut_load(reinterpret_cast<NqLutShared*>(s_raw));  // ends with a barrier
    else __syncthreads();

    float m[G], l[G], out[BPR][NVL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
    }
#pragma unroll
    for (int b = 0; b < BPR; ++b)
#pragma unroll
        for (int i = 0; i < NVL; ++i) out[b][i] = 0.0f;
    // the head whose totals this lane owns after a reduction
    const int my_head = (NV >= 32 ? lane * NVL : lane / (32 / (NV < 32 ? NV : 32))) >> 3;

    if (active) {
        const int P = p.page_size;
        const int s_begin = split * p.per_slots, s_end = min(total_slots, s_begin + p.per_slots);
        const int tok_begin = s_begin * P, tok_end = s_end * P;
        const int steps = tok_end > tok_begin ? (tok_end - tok_begin + 31) >> 5 : 0;
        const int rows = P * p.kv_heads;
        const uint32_t* kcodes = reinterpret_cast<const uint32_t*>(p.key_codes);
        const uint32_t* vcodes = reinterpret_cast<const uint32_t*>(p.value_codes);

        float kbeta[4], vbeta[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            kbeta[i] = __ldg(p.key_beta_table + i);
            vbeta[i] = __ldg(p.value_beta_table + i);
        }
        if constexpr (kStateInShared) {
            // every thread writes the same four values: no ordering needed beyond the warp's own
            if (lane < 4) s_vbeta[lane] = __ldg(p.value_beta_table + lane);
            __syncwarp();
        }
        for (int st0 = warp; st0 < steps; st0 += kAttnWarps * CH) {
            // ---- where is my token of each step?  (all loads of the chunk's bookkeeping go out together) ----
            int64_t row[CH];       // row of the pool (cold) or of the hot tail
            unsigned hot_mask = 0, valid_mask = 0, any_mask = 0;   // bit c: this lane's token of step c
            unsigned first_rows = 0;  // QT > 1, four bits per step: the first query token of the tile that sees my token
            Ids kid[CH], vid[CH];
            float kds[CH], vds[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int st = st0 + c * kAttnWarps;
                row[c] = 0;
                kid[c] = 0;
                vid[c] = 0;
                kds[c] = 0.0f;
                vds[c] = 0.0f;
                bool valid = false, hot = false;
                if (st < steps) {
                    const int tau = tok_begin + st * 32 + lane;
                    const int ps = tau / P, t = tau - ps * P;
                    if (tau < tok_end) {
                        hot = ps >= page_count;
                        const int tlimit = hot ? hot_len : (ps == page_count - 1 ? last_len : P);
                        const int base_token = hot ? cold : ps * P;
                        valid = t < tlimit && base_token + t < limit;
                        if constexpr (QT > 1) first_rows |= (unsigned)min(max(base_token + t - limit0 + 1, 0), QT) << (4 * c);
                        if (valid && !hot) {
                            const int page_id = p.page_indices[(int64_t)slot * p.max_pages + ps];
                            valid = page_id >= 0 && page_id < p.pool_capacity;  // defensive: never read outside the pool
                            if (valid) {
                                row[c] = (int64_t)page_id * rows + t * p.kv_heads + h;
                                kid[c] = load_row_ids<BPR>(p.key_betas, row[c]);
                                vid[c] = load_row_ids<BPR>(p.value_betas, row[c]);
                                kds[c] = __ldg(p.key_norms + row[c]);
                                vds[c] = __ldg(p.value_norms + row[c]);
                                // pull the code rows towards L1: the first use is a few hundred instructions away
                                if constexpr (LAT) {
                                    asm volatile("prefetch.global.L1 [%0];" ::"l"(p.key_lattice + row[c] * D));
                                    asm volatile("prefetch.global.L1 [%0];" ::"l"(p.value_lattice + row[c] * D));
                                } else {
                                    asm volatile("prefetch.global.L1 [%0];" ::"l"(kcodes + row[c] * BPR));
                                    asm volatile("prefetch.global.L1 [%0];" ::"l"(vcodes + row[c] * BPR));
                                }
                            }
                        } else if (valid) {
                            row[c] = ((int64_t)slot * P + t) * p.kv_heads + h;
                        }
                    }
                }
                const bool any = __any_sync(0xffffffffu, valid);
                valid_mask |= (valid ? 1u : 0u) << c;
                hot_mask |= (hot ? 1u : 0u) << c;
                any_mask |= (any ? 1u : 0u) << c;
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                kds[c] = nq_div_by(kds[c], p.sqrt_dim, p.inv_sqrt_dim);
                vds[c] = nq_div_by(vds[c], p.sqrt_dim, p.inv_sqrt_dim);
                if constexpr (kStateInShared) {
                    s_row[c][threadIdx.x] = row[c];
                    s_vid[c][threadIdx.x] = vid[c];
                    s_vds[c][threadIdx.x] = vds[c];
                }
            }
            // The step loops below stay rolled (ONE copy of the block decode per pass: laid out once per
            // step the kernel text no longer fits the instruction cache), so the per-step values are
            // picked out of their registers by index.
            // ---- pass 1: scores of my token against the G heads, two blocks at a time ----
#pragma unroll 1
            for (int c = 0; c < CH; ++c) {
                const bool valid = (valid_mask >> c) & 1u, hot = (hot_mask >> c) & 1u;
                const bool cold_row = valid && !hot;
                const int64_t my_row = pick_step(row, c);
                const Ids my_ids = pick_step(kid, c);
                const float my_ds = pick_step(kds, c);
                float sc[G];
#pragma unroll
                for (int g = 0; g < G; ++g) sc[g] = 0.0f;
                if ((any_mask >> c) & 1u) {
                    // the operands of the NEXT pair of blocks are fetched before this pair is decoded
                    uint2 next_words = make_uint2(0, 0);
                    uint4 next_lat = make_uint4(0, 0, 0, 0);
                    if (cold_row) {
                        if constexpr (LAT) next_lat = __ldg(reinterpret_cast<const uint4*>(p.key_lattice) + my_row * (BPR / 2));
                        else next_words = __ldg(reinterpret_cast<const uint2*>(kcodes + my_row * BPR));
                    }
#pragma unroll 1
                    for (int b = 0; b < BPR; b += 2) {
                        float kv0[8], kv1[8], ksc0 = 0.0f, ksc1 = 0.0f;
                        const uint2 words = next_words;
                        const uint4 lat = next_lat;
                        if (cold_row && b + 2 < BPR) {
                            if constexpr (LAT) next_lat = __ldg(reinterpret_cast<const uint4*>(p.key_lattice) + my_row * (BPR / 2) + (b >> 1) + 1);
                            else next_words = __ldg(reinterpret_cast<const uint2*>(kcodes + my_row * BPR + b + 2));
                        }
                        if constexpr (LAT) {
                            nq_lattice_block(make_uint2(lat.x, lat.y), kv0);  // zero words (inactive lane) decode to finite values
                            nq_lattice_block(make_uint2(lat.z, lat.w), kv1);
                        } else {
                            NqLutBlock b0, b1;
                            nq_lut_begin_shared(words.x, lut, lane, b0);
                            nq_lut_begin_shared(words.y, lut, lane, b1);
                            bool ic0 = b0.delta < 0, ic1 = b1.delta < 0;
                            if (b0.delta == 0) ic0 = nq_lut_resolve_tie_shared(b0, lut);
                            if (b1.delta == 0) ic1 = nq_lut_resolve_tie_shared(b1, lut);
                            nq_lut_finish(b0, ic0, kv0);
                            nq_lut_finish(b1, ic1, kv1);
                        }
                        if (cold_row) {
                            ksc0 = pick_step(kbeta, (int)((my_ids >> (2 * b)) & 3)) * my_ds;
                            ksc1 = pick_step(kbeta, (int)((my_ids >> (2 * b + 2)) & 3)) * my_ds;
                        } else if (valid) {  // hot tail: BF16 rows
                            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.hot_keys) + my_row * D + b * 8;
                            nq_load8<__nv_bfloat16>(src, kv0);
                            nq_load8<__nv_bfloat16>(src + 8, kv1);
                            ksc0 = ksc1 = 1.0f;
                        }
                        const float4* qrow = reinterpret_cast<const float4*>(s_q + b * 8);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            const float4 q0 = qrow[g * (D / 4)], q1 = qrow[g * (D / 4) + 1];
                            const float4 q2 = qrow[g * (D / 4) + 2], q3 = qrow[g * (D / 4) + 3];
                            float d0 = q0.x * kv0[0], d1 = q2.x * kv1[0];
                            d0 = fmaf(q0.y, kv0[1], d0); d1 = fmaf(q2.y, kv1[1], d1);
                            d0 = fmaf(q0.z, kv0[2], d0); d1 = fmaf(q2.z, kv1[2], d1);
                            d0 = fmaf(q0.w, kv0[3], d0); d1 = fmaf(q2.w, kv1[3], d1);
                            d0 = fmaf(q1.x, kv0[4], d0); d1 = fmaf(q3.x, kv1[4], d1);
                            d0 = fmaf(q1.y, kv0[5], d0); d1 = fmaf(q3.y, kv1[5], d1);
                            d0 = fmaf(q1.z, kv0[6], d0); d1 = fmaf(q3.z, kv1[6], d1);
                            d0 = fmaf(q1.w, kv0[7], d0); d1 = fmaf(q3.w, kv1[7], d1);
                            sc[g] = fmaf(ksc0, d0, sc[g]);
                            sc[g] = fmaf(ksc1, d1, sc[g]);
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) s_prob[c][threadIdx.x][g] = valid ? sc[g] : -INFINITY;
            }

            // ---- softmax of the chunk (every thread only touches its own column of s_prob) ----
            bool rescale = false;
            float my_corr = 1.0f;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float sv[CH];
#pragma unroll
                for (int c = 0; c < CH; ++c) sv[c] = s_prob[c][threadIdx.x][g];
                if constexpr (QT > 1) {  // causal mask of this row's query token (rows past the chunk see nothing)
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        const int first = (int)((first_rows >> (4 * c)) & 15u);
                        if (g / GH < first || g / GH >= nrows) sv[c] = -INFINITY;
                    }
                }
                float cm = sv[0];
#pragma unroll
                for (int c = 1; c < CH; ++c) cm = fmaxf(cm, sv[c]);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, off));
                // The reference point m[g] of the running softmax only moves when a score exceeds it by more
                // than 8 (a factor 256): until then the terms are added unscaled, which saves rescaling the
                // running output on almost every chunk and changes no sum mathematically.
                if (cm > m[g] + 8.0f) {
                    const float corr = exp2f(m[g] - cm);  // exp2(-inf) = 0 on the first chunk
                    l[g] *= corr;
                    if (g == my_head) my_corr = corr;
                    m[g] = cm;
                    rescale = true;
                }
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const float pr = (((valid_mask >> c) & 1u) && (QT == 1 || sv[c] != -INFINITY)) ? exp2f(sv[c] - m[g]) : 0.0f;
                    s_prob[c][threadIdx.x][g] = pr;
                    l[g] += pr;
                }
            }
            if (rescale) {
#pragma unroll
                for (int b = 0; b < BPR; ++b)
#pragma unroll
                    for (int i = 0; i < NVL; ++i) out[b][i] *= my_corr;
            }

            // ---- pass 2: p * V, one block of features at a time, two steps at a time ----
#pragma unroll 1
            for (int b = 0; b < BPR; ++b) {
                float acc[NV];
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[i] = 0.0f;
#pragma unroll 1
                for (int c = 0; c < CH; c += 2) {
                    if (!((any_mask >> c) & 3u)) continue;  // warp-uniform: neither step has a token
                    const bool valid0 = (valid_mask >> c) & 1u, valid1 = (valid_mask >> (c + 1)) & 1u;
                    const bool cold0 = valid0 && !((hot_mask >> c) & 1u), cold1 = valid1 && !((hot_mask >> (c + 1)) & 1u);
                    int64_t row0, row1;
                    if constexpr (kStateInShared) {
                        row0 = s_row[c][threadIdx.x];
                        row1 = s_row[c + 1][threadIdx.x];
                    } else {
                        row0 = pick_step(row, c);
                        row1 = pick_step(row, c + 1);
                    }
                    float vv0[8], vv1[8], vsc0 = 0.0f, vsc1 = 0.0f;
                    if constexpr (LAT) {
                        const uint2 z = make_uint2(0, 0);
                        nq_lattice_block(cold0 ? __ldg(reinterpret_cast<const uint2*>(p.value_lattice) + row0 * BPR + b) : z, vv0);
                        nq_lattice_block(cold1 ? __ldg(reinterpret_cast<const uint2*>(p.value_lattice) + row1 * BPR + b) : z, vv1);
                    } else {
                        const uint32_t w0 = cold0 ? __ldg(vcodes + row0 * BPR + b) : 0u;
                        const uint32_t w1 = cold1 ? __ldg(vcodes + row1 * BPR + b) : 0u;
                        NqLutBlock b0, b1;
                        nq_lut_begin_shared(w0, lut, lane, b0);
                        nq_lut_begin_shared(w1, lut, lane, b1);
                        bool ic0 = b0.delta < 0, ic1 = b1.delta < 0;
                        if (b0.delta == 0) ic0 = nq_lut_resolve_tie_shared(b0, lut);
                        if (b1.delta == 0) ic1 = nq_lut_resolve_tie_shared(b1, lut);
                        nq_lut_finish(b0, ic0, vv0);
                        nq_lut_finish(b1, ic1, vv1);
                    }
                    if (cold0) {
                        if constexpr (kStateInShared) vsc0 = s_vbeta[(int)((s_vid[c][threadIdx.x] >> (2 * b)) & 3)] * s_vds[c][threadIdx.x];
                        else vsc0 = pick_step(vbeta, (int)((pick_step(vid, c) >> (2 * b)) & 3)) * pick_step(vds, c);
                    }
                    else if (valid0) {
                        nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.hot_values) + row0 * D + b * 8, vv0);
                        vsc0 = 1.0f;
                    }
                    if (cold1) {
                        if constexpr (kStateInShared) vsc1 = s_vbeta[(int)((s_vid[c + 1][threadIdx.x] >> (2 * b)) & 3)] * s_vds[c + 1][threadIdx.x];
                        else vsc1 = pick_step(vbeta, (int)((pick_step(vid, c + 1) >> (2 * b)) & 3)) * pick_step(vds, c + 1);
                    }
                    else if (valid1) {
                        nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.hot_values) + row1 * D + b * 8, vv1);
                        vsc1 = 1.0f;
                    }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        // an inactive lane has probability 0 and scale 0 against finite decoded values
                        const float pv0 = s_prob[c][threadIdx.x][g] * vsc0, pv1 = s_prob[c + 1][threadIdx.x][g] * vsc1;
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[g * 8 + j] = fmaf(pv1, vv1[j], fmaf(pv0, vv0[j], acc[g * 8 + j]));
                    }
                }
                reduce_scatter<NV, 16>(acc, lane);
                // out[b] is indexed with the loop variable of a rolled loop: keep it in registers with a switch
#pragma unroll
                for (int bb = 0; bb < BPR; ++bb) {
                    if (bb == b) {
#pragma unroll
                        for (int i = 0; i < NVL; ++i) out[bb][i] += acc[i];
                    }
                }
            }
        }
    }

    // the lanes' partial denominators
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) l[g] += __shfl_xor_sync(0xffffffffu, l[g], off);
    }
    __syncthreads();  // the loop's storage becomes the merge buffer
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            s_merge[warp][g][D] = m[g];
            s_merge[warp][g][D + 1] = l[g];
        }
    }
    {
        constexpr int kGroup = NV >= 32 ? 1 : 32 / NV;  // lanes holding the same total
        if (lane % kGroup == 0) {
            const int first = NV >= 32 ? lane * NVL : lane / kGroup;  // index g * 8 + j of the lane's first total
#pragma unroll
            for (int b = 0; b < BPR; ++b)
#pragma unroll
                for (int i = 0; i < NVL; ++i) s_merge[warp][(first + i) >> 3][b * 8 + ((first + i) & 7)] = out[b][i];
        }
    }
    __syncthreads();

    // merge the warps; thread (g, blk) handles 8 output features
    for (int item = threadIdx.x; item < G * BPR; item += kAttnThreads) {
        const int g = item / BPR, b8 = item - g * BPR;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_merge[w][g][D]);
        float ll = 0.0f, a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float c = mm == -INFINITY ? 0.0f : exp2f(s_merge[w][g][D] - mm);
            ll += s_merge[w][g][D + 1] * c;
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] += s_merge[w][g][b8 * 8 + j] * c;
        }
        if (g / GH >= rows_in_tensor) continue;  // a tile that reaches past the last query token
        if (p.splits == 1) {
            const float inv = (active && ll > 0.0f) ? 1.0f / ll : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] *= inv;
            store_out(p.out, p.out_dtype, out_row(g) * BPR + b8, a);
        } else {
            float* dst = p.partial + (out_row(g) * p.splits + split) * (D + 2);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[b8 * 8 + j] = a[j];
            if (b8 == 0) {
                dst[D] = mm;
                dst[D + 1] = ll;
            }
        }
    }
}

// Merge the split partials of one (query, head): log-sum-exp weights, inactive rows -> 0.
__global__ void __launch_bounds__(128) nq_attn_reduce_kernel(const AttnParams p) {
    const int row = blockIdx.x;  // qi * q_heads + head
    const int D = p.dim, bpr = D >> 3;
    const float* src = p.partial + (int64_t)row * p.splits * (D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, src[(int64_t)s * (D + 2) + D]);
    for (int b8 = threadIdx.x; b8 < bpr; b8 += blockDim.x) {
        float ll = 0.0f, a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < p.splits; ++s) {
            const float* ps = src + (int64_t)s * (D + 2);
            const float c = mm == -INFINITY ? 0.0f : exp2f(ps[D] - mm);
            ll += ps[D + 1] * c;
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] += ps[b8 * 8 + j] * c;
        }
        const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] *= inv;
        store_out(p.out, p.out_dtype, (int64_t)row * bpr + b8, a);
    }
}

// One instantiation: the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel.
template <int G, int BPR, bool LAT, int QT = 1>
int launch_attn_one(const AttnParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t bytes = AttnLayout<G, BPR, LAT>::kSharedBytes;
    if (bytes > 48 * 1024) {
        static bool configured[NQ_MAX_DEVICES] = {false};
        const int device = nq_current_device();
        if (device < 0 || !configured[device]) {
            const cudaError_t e = cudaFuncSetAttribute(nq_attn_paged_kernel<G, BPR, LAT, QT>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) {
                nq_set_error("nq_kv_attention: cannot reserve %zu bytes of shared memory: %s", bytes, cudaGetErrorString(e));
                return (int)e;
            }
            if (device >= 0) configured[device] = true;
        }
    }
    nq_attn_paged_kernel<G, BPR, LAT, QT><<<grid, kAttnThreads, bytes, s>>>(p);
    return NQ_OK;
}

template <int G, bool LAT>
int launch_attn_dim(const AttnParams& p, dim3 grid, cudaStream_t s) {
    if (p.dim == 64) return launch_attn_one<G, 8, LAT>(p, grid, s);
    if (p.dim == 128) return launch_attn_one<G, 16, LAT>(p, grid, s);
    if (p.dim == 32) return launch_attn_one<G, 4, LAT>(p, grid, s);
    if (p.dim == 256) return launch_attn_one<G, 32, LAT>(p, grid, s);
    nq_set_error("nq_kv_attention: head_dim must be 32, 64, 128 or 256");
    return NQ_ERR_ARG;
}

template <int G>
int launch_attn(const AttnParams& p, dim3 grid, cudaStream_t s) {
    return p.key_lattice ? launch_attn_dim<G, true>(p, grid, s) : launch_attn_dim<G, false>(p, grid, s);
}

// Chunk prefill: a CTA takes `tile` consecutive query tokens so that its eight rows (tile x heads of the GQA
// group) share every decoded K/V block.  Built for the two common head sizes; everything else (and a group of
// eight, which fills the rows by itself) runs one query token per CTA.
constexpr int kTileRows = 8;
int query_tile(int q_tokens, int group, int dim) {
    return (q_tokens > 1 && group < kTileRows && (dim == 64 || dim == 128)) ? kTileRows / group : 1;
}

template <int BPR, bool LAT>
int launch_attn_tiled_dim(const AttnParams& p, dim3 grid, cudaStream_t s, int tile) {
    if (tile == 2) return launch_attn_one<kTileRows, BPR, LAT, 2>(p, grid, s);
    if (tile == 4) return launch_attn_one<kTileRows, BPR, LAT, 4>(p, grid, s);
    return launch_attn_one<kTileRows, BPR, LAT, 8>(p, grid, s);
}

int launch_attn_tiled(const AttnParams& p, dim3 grid, cudaStream_t s, int tile) {
    if (p.dim == 64)
        return p.key_lattice ? launch_attn_tiled_dim<8, true>(p, grid, s, tile) : launch_attn_tiled_dim<8, false>(p, grid, s, tile);
    return p.key_lattice ? launch_attn_tiled_dim<16, true>(p, grid, s, tile) : launch_attn_tiled_dim<16, false>(p, grid, s, tile);
}

// Page-range splits per (query token, KV head).  Every CTA of a launch owns the SAME number of page slots
// (`per_slots`, from the cache's maximum length), so a short sequence occupies few CTAs instead of being cut
// into slivers, and the CTAs past a sequence's end return at once.  A warp works best on chunks of
// CH x 32 tokens, a CTA therefore on kAttnWarps x CH x 32: that is the range, as long as it still yields
// about two resident sets of CTAs; small batches take shorter ranges (down to one step per warp) to fill the
// machine, very large grids longer ones (at most ~8 resident sets).  The plan only depends on what
// nq_kv_attention_workspace_bytes is told; pages count as 16 tokens in it (any page size is correct).
struct SplitPlan {
    int splits, per_slots;
};
SplitPlan plan_splits(int queries, int kv_heads, int max_pages, int group) {
    const long base = (long)queries * kv_heads;
    const long resident = 148L * (group <= 4 ? 4 : 3);
    const int max_slots = max_pages + 1;  // cold pages + the hot tail
    const int steps_per_chunk = group <= 4 ? 4 : 2;
    const int slots_full = kAttnWarps * steps_per_chunk * 32 / 16;
    const int slots_min = kAttnWarps * 32 / 16;
    const int splits_fill = (int)((2 * resident + base - 1) / base);
    int per = slots_full;
    int splits = (max_slots + per - 1) / per;
    if (splits >= splits_fill) {
        while (splits > 1 && base * splits > 8 * resident) {
            per += slots_full;
            splits = (max_slots + per - 1) / per;
        }
    } else {
        // not enough sequences to fill the machine with full ranges: one resident set of shorter ones
        const int one_set = (int)((resident + base - 1) / base);
        const int finest = (max_slots + slots_min - 1) / slots_min;
        splits = one_set < finest ? one_set : finest;
        if (splits < (max_slots + slots_full - 1) / slots_full) splits = (max_slots + slots_full - 1) / slots_full;
    }
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    SplitPlan plan;
    plan.per_slots = (max_slots + splits - 1) / splits;
    plan.splits = (max_slots + plan.per_slots - 1) / plan.per_slots;
    return plan;
}

}  // namespace

extern "C" size_t nq_kv_attention_workspace_bytes(int batch, int q_tokens, int q_heads, int kv_heads, int dim,
                                                  int max_pages) {
    if (batch < 1 || q_tokens < 1 || q_heads < 1 || kv_heads < 1) return 0;
    const int group = q_heads / kv_heads;
    const int tile = query_tile(q_tokens, group, dim);
    const int splits = plan_splits(batch * ((q_tokens + tile - 1) / tile), kv_heads, max_pages,
                                   tile > 1 ? kTileRows : group).splits;
    return (size_t)batch * q_tokens * q_heads * splits * (dim + 2) * sizeof(float) + 256;
}

static int kv_attention_impl(const void* query, int q_dtype, int batch, int q_tokens, int q_heads,
                               const int32_t* slot_ids, const uint8_t* active_mask, const int32_t* q_lens,
                               const uint8_t* cache_active, const int32_t* sequence_lengths,
                               const int32_t* page_indices, const int32_t* page_counts,
                               const int32_t* last_page_lens, const int32_t* hot_lengths,
                               const uint8_t* key_codes, const uint8_t* key_betas, const float* key_norms,
                               const uint8_t* value_codes, const uint8_t* value_betas, const float* value_norms,
                               const float* key_beta_table, const float* value_beta_table,
                               const void* hot_keys, const void* hot_values, int max_sequences, int max_pages,
                               int pool_capacity, int page_size, int kv_heads, int dim, float scale,
                               void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                               const int8_t* key_lattice, const int8_t* value_lattice, nq_stream_t stream) {
    NQ_REQUIRE(query && slot_ids && cache_active && sequence_lengths && page_indices && page_counts &&
                   last_page_lens && hot_lengths && key_codes && key_betas && key_norms && value_codes &&
                   value_betas && value_norms && key_beta_table && value_beta_table && hot_keys && hot_values && out,
               NQ_ERR_ARG, "nq_kv_attention: null pointer");
    NQ_REQUIRE(batch >= 1 && q_tokens >= 1 && q_heads >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0, NQ_ERR_ARG,
               "nq_kv_attention: query_heads must be a positive multiple of num_kv_heads");
    NQ_REQUIRE(max_sequences >= 1 && max_pages >= 1 && pool_capacity >= 1 && page_size >= 1, NQ_ERR_ARG,
               "nq_kv_attention: bad cache geometry");
    NQ_REQUIRE(out_dtype == NQ_BF16 || out_dtype == NQ_F32, NQ_ERR_ARG, "nq_kv_attention: out_dtype must be bf16 or f32");
    NQ_REQUIRE(nq_aligned16(query) && nq_aligned16(out) && nq_aligned16(hot_keys) && nq_aligned16(hot_values) &&
                   nq_aligned16(key_codes) && nq_aligned16(value_codes),
               NQ_ERR_ALIGN, "nq_kv_attention: 16-byte alignment required");
    const int group = q_heads / kv_heads;
    NQ_REQUIRE(group == 1 || group == 2 || group == 4 || group == 8, NQ_ERR_ARG,
               "nq_kv_attention: GQA group size must be 1, 2, 4 or 8");
    AttnParams p;
    p.query = query; p.q_dtype = q_dtype; p.batch = batch; p.q_tokens = q_tokens; p.q_heads = q_heads;
    p.kv_heads = kv_heads; p.dim = dim; p.page_size = page_size;
    p.slot_ids = slot_ids; p.active_mask = active_mask; p.q_lens = q_lens; p.cache_active = cache_active;
    p.sequence_lengths = sequence_lengths; p.page_indices = page_indices; p.page_counts = page_counts;
    p.last_page_lens = last_page_lens; p.hot_lengths = hot_lengths;
    p.key_codes = key_codes; p.key_betas = key_betas; p.value_codes = value_codes; p.value_betas = value_betas;
    p.key_norms = key_norms; p.value_norms = value_norms;
    p.key_beta_table = key_beta_table; p.value_beta_table = value_beta_table;
    p.hot_keys = hot_keys; p.hot_values = hot_values;
    p.key_lattice = key_lattice; p.value_lattice = value_lattice;
    p.max_sequences = max_sequences; p.max_pages = max_pages; p.pool_capacity = pool_capacity;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.sqrt_dim = (float)sqrt((double)dim);
    p.inv_sqrt_dim = 1.0f / p.sqrt_dim;
    const int tile = query_tile(q_tokens, group, dim);
    p.q_tiles = (q_tokens + tile - 1) / tile;
    // same with or without the shadow: same sums
    const SplitPlan plan = plan_splits(batch * p.q_tiles, kv_heads, max_pages, tile > 1 ? kTileRows : group);
    p.splits = plan.splits;
    p.per_slots = plan.per_slots;
    p.out = out; p.out_dtype = out_dtype;
    p.partial = reinterpret_cast<float*>(workspace);
    if (p.splits > 1) {
        const size_t need = (size_t)batch * q_tokens * q_heads * p.splits * (dim + 2) * sizeof(float);
        NQ_REQUIRE(workspace && workspace_bytes >= need && nq_aligned16(workspace), NQ_ERR_WORKSPACE,
                   "nq_kv_attention: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!key_lattice) {
        const cudaError_t err = nq_lut_ensure(s);
        NQ_REQUIRE(err == cudaSuccess, (int)err, "nq_kv_attention: decode table: %s", cudaGetErrorString(err));
    }
    dim3 grid((unsigned)(batch * p.q_tiles * kv_heads), (unsigned)p.splits);
    int rc;
    if (tile > 1) rc = launch_attn_tiled(p, grid, s, tile);
    else switch (group) {
        case 1: rc = launch_attn<1>(p, grid, s); break;
        case 2: rc = launch_attn<2>(p, grid, s); break;
        case 4: rc = launch_attn<4>(p, grid, s); break;
        default: rc = launch_attn<8>(p, grid, s); break;
    }
    if (rc) return rc;
    NQ_CHECK_LAUNCH("nq_kv_attention");
    if (p.splits > 1) {
        nq_attn_reduce_kernel<<<(unsigned)(batch * q_tokens * q_heads), 128, 0, s>>>(p);
        NQ_CHECK_LAUNCH("nq_kv_attention(reduce)");
    }
    return NQ_OK;
}

extern "C" int nq_kv_attention(const void* query, int q_dtype, int batch, int q_tokens, int q_heads,
                               const int32_t* slot_ids, const uint8_t* active_mask, const int32_t* q_lens,
                               const uint8_t* cache_active, const int32_t* sequence_lengths,
                               const int32_t* page_indices, const int32_t* page_counts,
                               const int32_t* last_page_lens, const int32_t* hot_lengths,
                               const uint8_t* key_codes, const uint8_t* key_betas, const float* key_norms,
                               const uint8_t* value_codes, const uint8_t* value_betas, const float* value_norms,
                               const float* key_beta_table, const float* value_beta_table,
                               const void* hot_keys, const void* hot_values, int max_sequences, int max_pages,
                               int pool_capacity, int page_size, int kv_heads, int dim, float scale,
                               void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                               nq_stream_t stream) {
    NQ_RANGE("nq_kv_attention");
    return kv_attention_impl(query, q_dtype, batch, q_tokens, q_heads, slot_ids, active_mask, q_lens, cache_active,
                             sequence_lengths, page_indices, page_counts, last_page_lens, hot_lengths, key_codes,
                             key_betas, key_norms, value_codes, value_betas, value_norms, key_beta_table,
                             value_beta_table, hot_keys, hot_values, max_sequences, max_pages, pool_capacity,
                             page_size, kv_heads, dim, scale, workspace, workspace_bytes, out, out_dtype, nullptr,
                             nullptr, stream);
}

extern "C" int nq_kv_attention_lattice(const void* query, int q_dtype, int batch, int q_tokens, int q_heads,
                                       const int32_t* slot_ids, const uint8_t* active_mask, const int32_t* q_lens,
                                       const uint8_t* cache_active, const int32_t* sequence_lengths,
                                       const int32_t* page_indices, const int32_t* page_counts,
                                       const int32_t* last_page_lens, const int32_t* hot_lengths,
                                       const uint8_t* key_codes, const uint8_t* key_betas, const float* key_norms,
                                       const uint8_t* value_codes, const uint8_t* value_betas,
                                       const float* value_norms, const float* key_beta_table,
                                       const float* value_beta_table, const void* hot_keys, const void* hot_values,
                                       int max_sequences, int max_pages, int pool_capacity, int page_size,
                                       int kv_heads, int dim, float scale, void* workspace, size_t workspace_bytes,
                                       void* out, int out_dtype, const int8_t* key_lattice,
                                       const int8_t* value_lattice, nq_stream_t stream) {
    NQ_RANGE("nq_kv_attention_lattice");
    NQ_REQUIRE(key_lattice && value_lattice && nq_aligned16(key_lattice) && nq_aligned16(value_lattice), NQ_ERR_ARG,
               "nq_kv_attention_lattice: 16-byte aligned lattice pages required");
    return kv_attention_impl(query, q_dtype, batch, q_tokens, q_heads, slot_ids, active_mask, q_lens, cache_active,
                             sequence_lengths, page_indices, page_counts, last_page_lens, hot_lengths, key_codes,
                             key_betas, key_norms, value_codes, value_betas, value_norms, key_beta_table,
                             value_beta_table, hot_keys, hot_values, max_sequences, max_pages, pool_capacity,
                             page_size, kv_heads, dim, scale, workspace, workspace_bytes, out, out_dtype, key_lattice,
                             value_lattice, stream);
}
