// Row encoder shared by the activation / weight encoder and the KV page
// writers.  One CTA of NQ_ENC_THREADS threads owns `nrows` consecutive rows of k features
// (NQ_ENC_THREADS / (k/8) rows for short rows, one or a few rows otherwise).  Small CTAs (five
// per SM) keep other CTAs issuing while one waits at a barrier.
//   phase 1  every thread squares its blocks into shared memory, transposed so that the
//            elements j, j+8, j+16, ... of a row (one "lane sequence") are contiguous
//   phase 2  8 threads per row run the reference's 8-lane strided accumulation
//            (the order PyTorch's CPU vector_norm uses; it decides the last
//            bit of the norm and therefore the emitted codes)
//   phase 3  every thread runs the 4-beta search on its blocks; codeword, optional BF16
//            reconstruction and four 2-bit beta ids per byte are written out.
// All pointers address the CTA's first row.  Rows >= valid_rows read as zero
// (partially filled KV pages).  Shared memory: nq_encode_smem_floats() floats.
#pragma once

#include "nq_common.cuh"

#ifndef NQ_ENC_THREADS
#define NQ_ENC_THREADS 128
#endif
#ifndef NQ_ENC_ROUNDS
#define NQ_ENC_ROUNDS 4      /* rounds of NQ_ENC_THREADS blocks per batch of the undithered search */
#endif
#ifndef NQ_ENC_QUEUE_CAP
#define NQ_ENC_QUEUE_CAP 256 /* queued boundary candidates per batch; overflow is evaluated in place */
#endif
// Batch results and the queue of the slow path (per CTA).  They ALIAS the squares buffer of the
// norm phase, which is dead once the row scales are known.
#define NQ_ENCODE_STAGE_FLOATS (NQ_ENC_THREADS * NQ_ENC_ROUNDS * (2 + 4 + 1) + NQ_ENC_QUEUE_CAP * (8 + 8 + 1) + 4)
#define NQ_ENC_MAX_LAYOUT_FLOATS 8192 /* squares buffer of a CTA that takes several long rows */

// Rows per CTA: short rows fill the CTA's threads once; long rows default to one per CTA and a
// launch with many rows may ask for more (nq_encode_rows_per_cta_many) to fill the batches.
__host__ __device__ inline int nq_encode_rows_per_cta(int k) {
    const int bpr = k / 8;
    return bpr >= NQ_ENC_THREADS ? 1 : NQ_ENC_THREADS / bpr;
}
__host__ __device__ inline int nq_encode_rows_per_cta_many(int k) {
    const int base = nq_encode_rows_per_cta(k);
    const int wide = NQ_ENC_MAX_LAYOUT_FLOATS / k;
    return wide > base ? wide : base;
}
__host__ __device__ inline size_t nq_encode_smem_floats(int k, int rows_layout = 0) {
    const int rpc = rows_layout > 0 ? rows_layout : nq_encode_rows_per_cta(k);
    const size_t squares = (size_t)rpc * (k + 40);  // per row: 8 lane sequences of k/8 + 4 floats, + 8
    const size_t body = squares > (size_t)NQ_ENCODE_STAGE_FLOATS ? squares : (size_t)NQ_ENCODE_STAGE_FLOATS;
    return body + (size_t)rpc * 10 + 4;
}

// Launch geometry of an encoder launch over `rows` rows of k features.
//   rpc               rows per CTA (also the shared-memory layout)
//   splits            CTAs per row (gridDim.y); each takes blocks_per_split blocks of phase 3
//   four_lanes        latency mode of small launches: the four candidates of a block on four lanes
struct NqEncodePlan {
    int rpc, splits, blocks_per_split;
    bool four_lanes;
};
inline NqEncodePlan nq_encode_plan(int64_t rows, int k, bool dither) {
    NqEncodePlan plan;
    const int bpr = k / 8;
    const int sms = nq_sm_count();
    const int slots = sms * 5;  // resident CTAs of the current device
    plan.rpc = nq_encode_rows_per_cta(k);
    plan.four_lanes = !dither && rows * bpr <= (int64_t)slots * (NQ_ENC_THREADS / 4);
    if (plan.four_lanes) {
        if (bpr < NQ_ENC_THREADS / 4) plan.rpc = (NQ_ENC_THREADS / 4) / bpr;  // one round of blocks per CTA
        else plan.rpc = 1;
    } else if (!dither) {
        // many long rows: several per CTA, so that a batch of the search queue fills up
        const int many = nq_encode_rows_per_cta_many(k);
        if (many > plan.rpc && rows / many >= slots) plan.rpc = many;
    }
    const int64_t grid = (rows + plan.rpc - 1) / plan.rpc;
    // Few long rows (decode-time activations): split each row's blocks over several CTAs, every
    // one of which repeats the cheap norm of its row.
    const bool splittable = plan.rpc == 1 && bpr > 32;
    plan.splits = 1;
    if (splittable && plan.four_lanes) {
        plan.splits = bpr / 32;
    } else if (splittable && bpr >= NQ_ENC_THREADS && grid < sms) {
        plan.splits = (int)((2 * sms + grid - 1) / grid);
        if (plan.splits > bpr / 32) plan.splits = bpr / 32;
    }
    if (plan.splits < 1) plan.splits = 1;
    plan.blocks_per_split = ((bpr + plan.splits - 1) / plan.splits + 31) / 32 * 32;
    if (plan.splits == 1) plan.blocks_per_split = 0x40000000;
    else plan.splits = (bpr + plan.blocks_per_split - 1) / plan.blocks_per_split;
    return plan;
}

// Block load of the encoder: from global memory in the tensor dtype, or (GLOBAL_IN = false)
// float32 values that an earlier phase of the same kernel left in shared memory.
template <typename T, bool GLOBAL_IN>
__device__ __forceinline__ void nq_encode_load8(const T* p, float v[8]) {
    if (GLOBAL_IN) {
        nq_load8<T>(p, v);
    } else {
        const float4 a = reinterpret_cast<const float4*>(p)[0];
        const float4 b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// DITHER selects the weight path (subtractive dither, straight search) at compile time, so that
// each kernel carries only the code of its own search.
template <typename T, bool DITHER = false, bool GLOBAL_IN = true>
__device__ __forceinline__ void nq_encode_rows_cta(
    const T* __restrict__ x, int64_t row_stride, int nrows, int valid_rows, int k,
    const float* __restrict__ beta_table, float sqrt_k, uint32_t* __restrict__ codes,
    uint8_t* __restrict__ beta_ids, float* __restrict__ norms, __nv_bfloat16* __restrict__ decoded,
    uint32_t counter_base, float* smem, int blk_begin = 0, int blk_end = 0x7fffffff,
    bool write_norms = true, int rows_layout = 0, bool four_lanes = false) {
    static_assert(GLOBAL_IN || sizeof(T) == 4, "shared-memory input is float32");
    const int rows_per_cta = rows_layout > 0 ? rows_layout : nq_encode_rows_per_cta(k);
    const int bpr = k >> 3;
    const int lane_pitch = bpr + 4;    // k/8 squares per lane sequence; +4 keeps the 16-byte chain reads conflict-free
    const int pitch = 8 * lane_pitch + 8;  // floats per row; +8 spreads the rows of one warp over the banks
    float* partial = smem;
    float* scale = partial + rows_per_cta * 8;
    float* dscale = scale + rows_per_cta;
    // 16-byte aligned body: squares during the norm phase, staging arrays afterwards
    float* sq = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(dscale + rows_per_cta) + 15) & ~(uintptr_t)15);
    const int tid = threadIdx.x;
    const int nblocks = nrows * bpr;

    for (int b = tid; b < nblocks; b += NQ_ENC_THREADS) {
        const int r = b / bpr, bb = b - r * bpr;
        float v[8];
        if (r < valid_rows) {
            nq_encode_load8<T, GLOBAL_IN>(x + (int64_t)r * row_stride + (int64_t)bb * 8, v);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        // transposed: lane sequence j of row r (elements j, j+8, j+16, ...) is contiguous
        float* dst = sq + (size_t)r * pitch + bb;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j * lane_pitch] = nq_mul(v[j], v[j]);
    }
    __syncthreads();

    for (int t = tid; t < nrows * 8; t += NQ_ENC_THREADS) {
        const int r = t >> 3, l = t & 7;
        const float4* p = reinterpret_cast<const float4*>(sq + (size_t)r * pitch + l * lane_pitch);
        float acc = 0.0f;
#pragma unroll 4
        for (int i = 0; i < (bpr >> 2); ++i) {
            const float4 q = p[i];
            acc = nq_add(nq_add(nq_add(nq_add(acc, q.x), q.y), q.z), q.w);
        }
        partial[t] = acc;
    }
    __syncthreads();

    for (int t = tid; t < nrows; t += NQ_ENC_THREADS) {
        float total = partial[t * 8];
#pragma unroll
        for (int l = 1; l < 8; ++l) total = nq_add(total, partial[t * 8 + l]);
        const float norm = nq_sqrt(total);
        if (write_norms) norms[t] = norm;
        // sqrt(K)/norm is evaluated as reciprocal(norm) * sqrt(K) by the reference.
        scale[t] = norm > 0.0f ? nq_mul(nq_rcp(norm), sqrt_k) : 0.0f;
        dscale[t] = nq_div(norm, sqrt_k);
    }
    __syncthreads();

    // Phase 3 covers blocks [blk_begin, blk_end) of the CTA's rows (a long row can be split over
    // several CTAs, each recomputing the cheap norm); blk_begin is a multiple of 32.
    const int enc_end = min(nblocks, blk_end);
    const int padded = blk_begin + ((max(enc_end - blk_begin, 0) + 31) & ~31);
    if (DITHER) {
        // weights: straight per-thread search with the subtractive dither of the global block
        for (int b = blk_begin + tid; b < padded; b += NQ_ENC_THREADS) {
            const bool valid = b < enc_end;
            int bid = 0;
            if (valid) {
                const int r = b / bpr, bb = b - r * bpr;
                float v[8], recon[8], d[8];
                if (r < valid_rows) {
                    nq_encode_load8<T, GLOBAL_IN>(x + (int64_t)r * row_stride + (int64_t)bb * 8, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                }
                const float s = scale[r];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = nq_mul(v[j], s);
                nq_dither_block(counter_base + (uint32_t)b * 8u, d);
                codes[b] = nq_encode_block(v, beta_table, d, bid, recon);
                if (decoded != nullptr) {
                    const float ds = dscale[r];
#pragma unroll
                    for (int j = 0; j < 8; ++j) recon[j] = nq_mul(recon[j], ds);
                    *reinterpret_cast<uint4*>(decoded + (int64_t)b * 8) = nq_pack_bf16x8(recon);
                }
            }
            unsigned merged = (unsigned)bid;
            merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 1) << 2;
            merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 2) << 4;
            merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 3) << 6;
            if (valid && (tid & 3) == 0) beta_ids[b >> 2] = (uint8_t)merged;
        }
        return;
    }

    // Undithered rows (activations, K/V).  Work proceeds in batches of NQ_ENC_ROUNDS rounds of
    // NQ_ENC_THREADS blocks.  Every thread classifies the four candidates of its block with the
    // cheap exact tests and posts a provisional result (codeword, scaled reconstruction, search
    // key) in shared memory.  Candidates whose lattice point lies ON the boundary of 14*V(E8)
    // -- about one block in seven on Gaussian rows -- need the full evaluation: they are queued
    // with their lattice point and evaluated densely by the whole CTA once per batch, so no warp
    // idles behind one slow lane and the barriers are paid once per batch.  The search rule is
    // the minimum of nq_candidate_key(), taken with a shared-memory atomic.
    constexpr int NT = NQ_ENC_THREADS;
    constexpr int BATCH = NT * NQ_ENC_ROUNDS;
    constexpr int CAP = NQ_ENC_QUEUE_CAP;
    float* stage = sq;  // the squares are dead: every row scale has been computed (barrier above)
    unsigned long long* out_key = reinterpret_cast<unsigned long long*>(stage);  // [BATCH]
    uint4* out_dec = reinterpret_cast<uint4*>(out_key + BATCH);                  // [BATCH]
    float* item_x = reinterpret_cast<float*>(out_dec + BATCH);                   // [CAP][8]; after evaluation: key, word
    float* item_lam = item_x + CAP * 8;                                          // [CAP][8]; after evaluation: BF16 reconstruction
    uint32_t* out_word = reinterpret_cast<uint32_t*>(item_lam + CAP * 8);        // [BATCH]
    unsigned short* item_meta = reinterpret_cast<unsigned short*>(out_word + BATCH);  // [CAP] (slot << 2) | beta
    unsigned* queue_count = reinterpret_cast<unsigned*>(item_meta + CAP);
    const bool want_dec = decoded != nullptr;
    // Latency mode for small launches (four_lanes): the four candidates of a block go to four
    // neighbouring lanes, so a block costs one candidate evaluation of latency instead of four.
    // A batch then holds at most CAP / 4 blocks, which the queue can always take.
    const int batch_cap = four_lanes ? CAP / 4 : BATCH;
    for (int base = blk_begin; base < enc_end; base += batch_cap) {
        if (tid == 0) *queue_count = 0u;
        __syncthreads();  // also: the previous batch has been written out
        const int batch_n = min(batch_cap, enc_end - base);
        if (four_lanes) {
            for (int slot0 = 0; slot0 < batch_n; slot0 += NT / 4) {
                const int slot = slot0 + (tid >> 2), c = tid & 3;
                const bool valid = slot < batch_n;
                const int b = base + (valid ? slot : 0);
                const int row_r = b / bpr, bb = b - row_r * bpr;
                float v[8];
                if (row_r < valid_rows) {
                    nq_encode_load8<T, GLOBAL_IN>(x + (int64_t)row_r * row_stride + (int64_t)bb * 8, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                }
                const float s = scale[row_r], ds = dscale[row_r];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = nq_mul(v[j], s);
                const float bt = beta_table[c];
                float lam[8], asif;
                const int cls = nq_classify_candidate(v, bt, lam, asif);
                const unsigned long long mine = (valid && cls > 0) ? nq_candidate_key(asif, c) : ~0ull;
                unsigned long long best_key = mine;
#pragma unroll
                for (int off = 1; off < 4; off <<= 1) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best_key, off);
                    best_key = other < best_key ? other : best_key;
                }
                if (valid) {
                    const bool have_best = best_key != ~0ull;
                    const float best_err = nq_bits_float((uint32_t)(best_key >> 8));
                    if (cls > 0 && mine == best_key) {  // keys of one block differ in the beta index: one winner
                        out_key[slot] = mine;
                        out_word[slot] = nq_lattice_to_codeword(lam);
                        uint4 dec = make_uint4(0, 0, 0, 0);
                        if (want_dec) {
                            float recon[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) recon[j] = nq_mul(nq_mul(lam[j], bt), ds);
                            dec = nq_pack_bf16x8(recon);
                        }
                        out_dec[slot] = dec;
                    } else if (!have_best && c == 0) {
                        out_key[slot] = ~0ull;
                        out_word[slot] = 0u;
                        out_dec[slot] = make_uint4(0, 0, 0, 0);
                    }
                    // boundary: error >= asif; outside: error > 353 beta^2 -- queued unless the best inside candidate rules it out
                    const bool queue_it = cls == 0 ? !(have_best && asif > best_err)
                                                   : (cls < 0 && !(have_best && 353.0f * bt * bt > best_err));
                    if (queue_it) {
                        const unsigned idx = atomicAdd(queue_count, 1u);  // at most 4 * batch_cap = CAP entries
                        float4* dx = reinterpret_cast<float4*>(item_x + idx * 8);
                        dx[0] = make_float4(v[0], v[1], v[2], v[3]);
                        dx[1] = make_float4(v[4], v[5], v[6], v[7]);
                        float4* dl = reinterpret_cast<float4*>(item_lam + idx * 8);
                        dl[0] = make_float4(lam[0], lam[1], lam[2], lam[3]);
                        dl[1] = make_float4(lam[4], lam[5], lam[6], lam[7]);
                        item_meta[idx] = (unsigned short)((slot << 2) | c);
                    }
                }
            }
        } else
        for (int slot = tid; slot < batch_n; slot += NT) {
            const int b = base + slot;
            const int row_r = b / bpr, bb = b - row_r * bpr;
            float v[8];
            if (row_r < valid_rows) {
                nq_encode_load8<T, GLOBAL_IN>(x + (int64_t)row_r * row_stride + (int64_t)bb * 8, v);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            }
            const float s = scale[row_r], ds = dscale[row_r];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = nq_mul(v[j], s);
            int best;
            float best_err, best_lam[8];
            unsigned pending, overflow = 0;
            nq_encode_block_fastpass_push(v, beta_table, best, best_err, best_lam, pending,
                                          [&](int c, const float* lam) {
                const unsigned idx = atomicAdd(queue_count, 1u);
                if (idx < (unsigned)CAP) {
                    float4* dx = reinterpret_cast<float4*>(item_x + idx * 8);
                    dx[0] = make_float4(v[0], v[1], v[2], v[3]);
                    dx[1] = make_float4(v[4], v[5], v[6], v[7]);
                    float4* dl = reinterpret_cast<float4*>(item_lam + idx * 8);
                    dl[0] = make_float4(lam[0], lam[1], lam[2], lam[3]);
                    dl[1] = make_float4(lam[4], lam[5], lam[6], lam[7]);
                    item_meta[idx] = (unsigned short)((slot << 2) | c);
                } else {
                    overflow |= 1u << c;  // queue full (degenerate inputs): generic evaluation below
                }
            });
            pending |= overflow;
            uint32_t word = 0;
            uint4 dec = make_uint4(0, 0, 0, 0);
            unsigned long long key = ~0ull;
            if (best >= 0) {
                word = nq_lattice_to_codeword(best_lam);
                key = nq_candidate_key(best_err, best);
                if (want_dec) {
                    const float bt = beta_table[best];
                    float recon[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) recon[j] = nq_mul(nq_mul(best_lam[j], bt), ds);
                    dec = nq_pack_bf16x8(recon);
                }
            }
            if (pending) {  // rare: candidates outside the cell that nothing rules out, or a full queue
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    if (!((pending >> c) & 1u)) continue;
                    float r[8], err;
                    const uint32_t w = nq_encode_candidate_exact(v, beta_table[c], nullptr, r, err);
                    const unsigned long long k2 = nq_candidate_key(err, c);
                    if (k2 < key) {
                        key = k2;
                        word = w;
#pragma unroll
                        for (int j = 0; j < 8; ++j) r[j] = nq_mul(r[j], ds);
                        dec = nq_pack_bf16x8(r);
                    }
                }
            }
            out_key[slot] = key;
            out_word[slot] = word;
            out_dec[slot] = dec;
        }
        __syncthreads();
        const int items = (int)min(*queue_count, (unsigned)CAP);
        for (int it = tid; it < items; it += NT) {
            const int slot = item_meta[it] >> 2, c = item_meta[it] & 3;
            float v[8], lam[8], r[8], err;
            float4 lo = reinterpret_cast<const float4*>(item_x + it * 8)[0];
            float4 hi = reinterpret_cast<const float4*>(item_x + it * 8)[1];
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            lo = reinterpret_cast<const float4*>(item_lam + it * 8)[0];
            hi = reinterpret_cast<const float4*>(item_lam + it * 8)[1];
            lam[0] = lo.x; lam[1] = lo.y; lam[2] = lo.z; lam[3] = lo.w; lam[4] = hi.x; lam[5] = hi.y; lam[6] = hi.z; lam[7] = hi.w;
            const uint32_t word = nq_eval_candidate_from_lam(v, lam, beta_table[c], r, err);
            const unsigned long long key = nq_candidate_key(err, c);
            const float ds = dscale[(base + slot) / bpr];
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = nq_mul(r[j], ds);
            // the item's inputs are in registers: its storage now holds the result
            *reinterpret_cast<unsigned long long*>(item_x + it * 8) = key;
            *reinterpret_cast<uint32_t*>(item_x + it * 8 + 2) = word;
            *reinterpret_cast<uint4*>(item_lam + it * 8) = nq_pack_bf16x8(r);
            atomicMin(out_key + slot, key);
        }
        __syncthreads();
        for (int it = tid; it < items; it += NT) {
            const int slot = item_meta[it] >> 2;
            // keys of one block differ in the beta index: at most one item equals the minimum
            if (out_key[slot] == *reinterpret_cast<const unsigned long long*>(item_x + it * 8)) {
                out_word[slot] = *reinterpret_cast<const uint32_t*>(item_x + it * 8 + 2);
                out_dec[slot] = *reinterpret_cast<const uint4*>(item_lam + it * 8);
            }
        }
        __syncthreads();
        for (int slot = tid; slot < batch_n; slot += NT) {
            codes[base + slot] = out_word[slot];
            if (want_dec) *reinterpret_cast<uint4*>(decoded + (int64_t)(base + slot) * 8) = out_dec[slot];
        }
        // four neighbouring blocks share one beta byte (block i -> bits 2i..2i+1); batch_n is a multiple of 4
        for (int q4 = tid; q4 < (batch_n >> 2); q4 += NT) {
            unsigned merged = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) merged |= ((unsigned)out_key[q4 * 4 + i] & 3u) << (2 * i);
            beta_ids[(base >> 2) + q4] = (uint8_t)merged;
        }
    }
}
