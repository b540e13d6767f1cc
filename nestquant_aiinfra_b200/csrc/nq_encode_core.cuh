// Row encoder shared by the activation / weight encoder and the KV page
// writers.  One CTA of NQ_ENC_THREADS threads owns `nrows` consecutive rows of k features
// (NQ_ENC_THREADS / (k/8) rows for short rows, one row otherwise).  Small CTAs (six per SM)
// keep other CTAs issuing while one waits at a barrier of its compaction rounds.
//   phase 1  every thread squares its blocks into shared memory
//   phase 2  8 threads per row run the reference's 8-lane strided accumulation
//            (the order PyTorch's CPU vector_norm uses; it decides the last
//            bit of the norm and therefore the emitted codes)
//   phase 3  every thread runs the 4-beta search on its blocks and stores the
//            codeword; beta ids of 4 neighbouring blocks are merged by shuffle.
// All pointers address the CTA's first row.  Rows >= valid_rows read as zero
// (partially filled KV pages).  Shared memory: nq_encode_smem_floats() floats.
#pragma once

#include "nq_common.cuh"

#define NQ_ENC_THREADS 128
// Staging area of the compacted slow path (per CTA): normalised blocks, per-(thread, beta) results
// of the full evaluation, the work queue and its counter.  It ALIASES the squares buffer of the
// norm phase, which is dead once the row scales are known.
#define NQ_ENCODE_STAGE_FLOATS (NQ_ENC_THREADS * 8 + NQ_ENC_THREADS * 4 * 2 + NQ_ENC_THREADS * 4 * 4 + NQ_ENC_THREADS * 2 + 4)

__host__ __device__ inline int nq_encode_rows_per_cta(int k) {
    const int bpr = k / 8;
    return bpr >= NQ_ENC_THREADS ? 1 : NQ_ENC_THREADS / bpr;
}
__host__ __device__ inline size_t nq_encode_smem_floats(int k) {
    const int rpc = nq_encode_rows_per_cta(k);
    const size_t squares = (size_t)rpc * (k + 8);
    const size_t body = squares > (size_t)NQ_ENCODE_STAGE_FLOATS ? squares : (size_t)NQ_ENCODE_STAGE_FLOATS;
    return body + (size_t)rpc * 10 + 4;
}

template <typename T>
__device__ __forceinline__ void nq_encode_rows_cta(
    const T* __restrict__ x, int64_t row_stride, int nrows, int valid_rows, int k,
    const float* __restrict__ beta_table, float sqrt_k, uint32_t* __restrict__ codes,
    uint8_t* __restrict__ beta_ids, float* __restrict__ norms, __nv_bfloat16* __restrict__ decoded,
    int use_dither, uint32_t counter_base, float* smem, int blk_begin = 0, int blk_end = 0x7fffffff,
    bool write_norms = true) {
    const int rows_per_cta = nq_encode_rows_per_cta(k);
    const int bpr = k >> 3;
    const int pitch = k + 8;  // de-conflicts the strided chain reads of neighbouring rows
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
            nq_load8<T>(x + (int64_t)r * row_stride + (int64_t)bb * 8, v);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        float4 lo = make_float4(nq_mul(v[0], v[0]), nq_mul(v[1], v[1]), nq_mul(v[2], v[2]), nq_mul(v[3], v[3]));
        float4 hi = make_float4(nq_mul(v[4], v[4]), nq_mul(v[5], v[5]), nq_mul(v[6], v[6]), nq_mul(v[7], v[7]));
        float4* dst = reinterpret_cast<float4*>(sq + (size_t)r * pitch + bb * 8);
        dst[0] = lo;
        dst[1] = hi;
    }
    __syncthreads();

    for (int t = tid; t < nrows * 8; t += NQ_ENC_THREADS) {
        const int r = t >> 3, l = t & 7;
        const float* p = sq + (size_t)r * pitch + l;
        float acc = 0.0f;
#pragma unroll 8
        for (int i = 0; i < bpr; ++i) acc = nq_add(acc, p[8 * i]);
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
    // several CTAs, each recomputing the cheap norm); blk_begin is a multiple of the CTA size.
    const int enc_end = min(nblocks, blk_end);
    const int padded = blk_begin + ((max(enc_end - blk_begin, 0) + 31) & ~31);
    if (use_dither) {
        // weights: straight per-thread search with the subtractive dither of the global block
        for (int b = blk_begin + tid; b < padded; b += NQ_ENC_THREADS) {
            const bool valid = b < enc_end;
            int bid = 0;
            if (valid) {
                const int r = b / bpr, bb = b - r * bpr;
                float v[8], recon[8], d[8];
                if (r < valid_rows) {
                    nq_load8<T>(x + (int64_t)r * row_stride + (int64_t)bb * 8, v);
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

    // Undithered rows (activations, K/V): every thread classifies its four candidates with the
    // cheap exact tests; the few (thread, beta) pairs that need the full evaluation are queued in
    // shared memory and evaluated densely by the whole CTA, so no warp idles behind one slow lane.
    float* stage = sq;  // the squares are dead: every row scale has been computed (barrier above)
    constexpr int NT = NQ_ENC_THREADS;
    float* xs = stage;                                                    // [NT][8] normalised blocks
    uint4* res_dec = reinterpret_cast<uint4*>(xs + NT * 8);               // [NT][4] scaled BF16 reconstruction
    float* res_err = reinterpret_cast<float*>(res_dec + NT * 4);          // [NT][4]
    uint32_t* res_word = reinterpret_cast<uint32_t*>(res_err + NT * 4);   // [NT][4]
    unsigned short* queue = reinterpret_cast<unsigned short*>(res_word + NT * 4);  // [4 NT] (thread << 2) | beta
    unsigned* queue_count = reinterpret_cast<unsigned*>(queue + NT * 4);
    for (int base = blk_begin; base < padded; base += NQ_ENC_THREADS) {
        const int b = base + tid;
        const bool valid = b < enc_end;
        if (tid == 0) *queue_count = 0u;
        __syncthreads();
        int best = 0, row_r = 0;
        float best_err = 0.0f, best_lam[8];
        unsigned pending = 0;
        if (valid) {
            row_r = b / bpr;
            const int bb = b - row_r * bpr;
            float v[8];
            if (row_r < valid_rows) {
                nq_load8<T>(x + (int64_t)row_r * row_stride + (int64_t)bb * 8, v);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            }
            const float s = scale[row_r];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = nq_mul(v[j], s);
            float4* dst = reinterpret_cast<float4*>(xs + tid * 8);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            nq_encode_block_fastpass(v, beta_table, best, best_err, best_lam, pending);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if ((pending >> c) & 1u) queue[atomicAdd(queue_count, 1u)] = (unsigned short)((tid << 2) | c);
        }
        __syncthreads();
        const int items = (int)*queue_count;
        for (int it = tid; it < items; it += NQ_ENC_THREADS) {
            const int owner = queue[it] >> 2, c = queue[it] & 3;
            float v[8], r[8], err;
            const float4 lo = reinterpret_cast<const float4*>(xs + owner * 8)[0];
            const float4 hi = reinterpret_cast<const float4*>(xs + owner * 8)[1];
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            res_word[owner * 4 + c] = nq_encode_candidate_exact(v, beta_table[c], nullptr, r, err);
            res_err[owner * 4 + c] = err;
            const float ds = dscale[(base + owner) / bpr];
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = nq_mul(r[j], ds);
            res_dec[owner * 4 + c] = nq_pack_bf16x8(r);
        }
        __syncthreads();
        int bid = 0;
        if (valid) {
            uint32_t word = 0;
            uint4 dec = make_uint4(0, 0, 0, 0);
            bool from_queue = false;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (!((pending >> c) & 1u)) continue;
                const float err = res_err[tid * 4 + c];
                if (nq_candidate_wins(c, err, best, best_err)) {
                    best = c;
                    best_err = err;
                    word = res_word[tid * 4 + c];
                    dec = res_dec[tid * 4 + c];
                    from_queue = true;
                }
            }
            if (!from_queue) {
                word = nq_lattice_to_codeword(best_lam);
                if (decoded != nullptr) {
                    const float bt = beta_table[best], ds = dscale[row_r];
                    float recon[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) recon[j] = nq_mul(nq_mul(best_lam[j], bt), ds);
                    dec = nq_pack_bf16x8(recon);
                }
            }
            bid = best;
            codes[b] = word;
            if (decoded != nullptr) *reinterpret_cast<uint4*>(decoded + (int64_t)b * 8) = dec;
        }
        // four neighbouring blocks share one beta byte (block i -> bits 2i..2i+1)
        unsigned merged = (unsigned)bid;
        merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 1) << 2;
        merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 2) << 4;
        merged |= __shfl_down_sync(0xffffffffu, (unsigned)bid, 3) << 6;
        if (valid && (tid & 3) == 0) beta_ids[b >> 2] = (uint8_t)merged;
    }
}
