// Paged GQA attention that reads NQKV4 pages directly (decode and chunked
// causal prefill).  One CTA owns one (query token, KV head, page-range split):
// every K/V vector is decoded ONCE for all query heads of its GQA group, with
// the exact codec arithmetic (undithered streams have real Voronoi ties), FP32
// online softmax, and a BF16 hot tail as the last "page".  No page-count cap.
//
// Lane mapping: a warp covers 32 / (D/8) tokens per step; lane = (token, E8
// block of the head vector).  Score = shuffle-reduced dot over the D/8 lanes of
// a token.  Split partials (m, l, acc[D]) are merged by a second small kernel
// (skipped when there is a single split).
//
// Replaces runtime/nqkv_attention_k1.py:243-471 (page / hot / reduce Triton
// kernels, 127-page cap at :807-809) and adds the page-reading prefill the
// reference only has as materialise + SDPA (runtime/nqkv_hf_backend.py:127-150).
#include <math.h>

#include "nq_common.cuh"

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

template <int G, int BPR, bool LAT>
__global__ void __launch_bounds__(kAttnThreads, (G <= 4 ? 4 : 3)) nq_attn_paged_kernel(const AttnParams p) {
    constexpr int TPW = 32 / BPR;  // tokens per warp step
    constexpr int D = BPR * 8;
    __shared__ float s_merge[kAttnWarps][G][D + 2];

    const int qi = blockIdx.x / p.kv_heads, h = blockIdx.x - qi * p.kv_heads;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = lane % BPR, tsub = lane / BPR;

    int slot, limit, total_slots, page_count, last_len, hot_len;
    const bool active = resolve_query(p, qi, slot, limit, total_slots, page_count, last_len, hot_len);
    const int cold = page_count > 0 ? (page_count - 1) * p.page_size + last_len : 0;

    float m[G], l[G], acc[G][8], q[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
        const int64_t qoff = ((int64_t)qi * p.q_heads + h * G + g) * D + blk * 8;
        if (p.q_dtype == NQ_BF16) nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.query) + qoff, q[g]);
        else if (p.q_dtype == NQ_F16) nq_load8<__half>(reinterpret_cast<const __half*>(p.query) + qoff, q[g]);
        else nq_load8<float>(reinterpret_cast<const float*>(p.query) + qoff, q[g]);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[g][j] *= p.scale_log2e;
    }

    if (active) {
        const int per = (total_slots + p.splits - 1) / p.splits;
        const int s_begin = split * per, s_end = min(total_slots, s_begin + per);
        const int rows = p.page_size * p.kv_heads;
        const int64_t code_bytes = (int64_t)rows * D / 2, beta_bytes = (int64_t)rows * D / 32;
        // scores of one token against the G query heads and the running-softmax update (lane = one E8 block)
        auto update = [&](const float kvec[8], const float vvec[8], float kscale, float vscale, bool valid) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float s = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) s = fmaf(q[g][j], kvec[j], s);
                s *= kscale;  // the beta of this lane's block, the norm of its row
#pragma unroll
                for (int off = 1; off < BPR; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                if (valid) {
                    // The reference point m[g] of the running softmax only moves when a score exceeds it
                    // by more than 8 (a factor 256): until then the terms are added unscaled, which saves
                    // the rescaling of the accumulator on almost every token and changes no sum mathematically.
                    if (s > m[g] + 8.0f) {
                        const float corr = exp2f(m[g] - s);  // exp2(-inf) = 0 on the first token
                        l[g] *= corr;
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[g][j] *= corr;
                        m[g] = s;
                    }
                    const float pr = exp2f(s - m[g]);
                    l[g] += pr;
                    const float pv = pr * vscale;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(pv, vvec[j], acc[g][j]);
                }
            }
        };
        if constexpr (LAT) {
            // Decoded shadow: a page costs a few hundred instructions per warp, so the loads are what has to be
            // hidden.  The warp walks its cold pages as a stream of half-page items and fetches item i + 1
            // (lattice coordinates, beta ids, norms) before it computes item i; token order is unchanged, so
            // the sums are those of the packed kernel.
            constexpr int CH = 2;                  // token steps per item
            constexpr int kItemTokens = CH * TPW;
            const int items_per_page = (p.page_size + kItemTokens - 1) / kItemTokens;
            const int cold_end = min(s_end, page_count);
            uint2 nk[CH], nv[CH];
            int nid[CH];
            float nkn[CH], nvn[CH];
            // returns the page id of the item, -1 past the end of the warp's work, -2 for a page to skip
            auto fetch_item = [&](int item) -> int {
                const int ps = s_begin + warp + (item / items_per_page) * kAttnWarps;
                if (ps >= cold_end || ps * p.page_size >= limit) return -1;
                const int page_id = p.page_indices[(int64_t)slot * p.max_pages + ps];
                if (page_id < 0 || page_id >= p.pool_capacity) return -2;
                const int t_base = (item % items_per_page) * kItemTokens + tsub;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int row = min(t_base + i * TPW, p.page_size - 1) * p.kv_heads + h;
                    const int64_t g = (int64_t)row * BPR + blk;
                    const int64_t gl = (int64_t)page_id * rows * BPR + g;
                    nk[i] = __ldg(reinterpret_cast<const uint2*>(p.key_lattice) + gl);
                    nv[i] = __ldg(reinterpret_cast<const uint2*>(p.value_lattice) + gl);
                    nid[i] = nq_beta_id(p.key_betas + page_id * beta_bytes, g) |
                             (nq_beta_id(p.value_betas + page_id * beta_bytes, g) << 2);
                    nkn[i] = __ldg(p.key_norms + (int64_t)page_id * rows + row);
                    nvn[i] = __ldg(p.value_norms + (int64_t)page_id * rows + row);
                }
                return page_id;
            };
            int item = 0;
            int next_page = fetch_item(0);
            while (next_page != -1) {
                uint2 ck[CH], cv[CH];
                int cid[CH];
                float ckn[CH], cvn[CH];
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    ck[i] = nk[i]; cv[i] = nv[i]; cid[i] = nid[i]; ckn[i] = nkn[i]; cvn[i] = nvn[i];
                }
                const int this_page = next_page, this_item = item;
                ++item;
                next_page = fetch_item(item);
                if (this_page < 0) continue;
                const int ps = s_begin + warp + (this_item / items_per_page) * kAttnWarps;
                const int tlimit = ps == page_count - 1 ? last_len : p.page_size;
                const int base_token = ps * p.page_size;
                const int t_first = (this_item % items_per_page) * kItemTokens;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    if (t_first + i * TPW >= tlimit) break;  // warp-uniform
                    const int t = t_first + i * TPW + tsub;
                    const bool valid = t < tlimit && base_token + t < limit;
                    const float kb = __ldg(p.key_beta_table + (cid[i] & 3));
                    const float vb = __ldg(p.value_beta_table + (cid[i] >> 2));
                    const float kds = nq_div_by(ckn[i], p.sqrt_dim, p.inv_sqrt_dim);
                    const float vds = nq_div_by(cvn[i], p.sqrt_dim, p.inv_sqrt_dim);
                    float kvec[8], vvec[8];
                    nq_lattice_block(ck[i], kvec);
                    nq_lattice_block(cv[i], vvec);
                    update(kvec, vvec, kb * kds, vb * vds, valid);
                }
            }
        }
        for (int ps = s_begin + warp; ps < s_end; ps += kAttnWarps) {
            const bool is_hot = ps >= page_count;
            if (LAT && !is_hot) continue;  // cold pages were streamed above
            const int base_token = is_hot ? cold : ps * p.page_size;
            if (base_token >= limit) break;  // warp-uniform: later slots are later tokens
            const int tlimit = is_hot ? hot_len : (ps == page_count - 1 ? last_len : p.page_size);
            int page_id = 0;
            if (!is_hot) {
                page_id = p.page_indices[(int64_t)slot * p.max_pages + ps];
                if (page_id < 0 || page_id >= p.pool_capacity) continue;  // defensive: never read outside the pool
            }
            // pull the codes of this warp's NEXT page towards L1 while this one is decoded: lane l asks for
            // the code row of token l & 15 (keys on lanes 0..15, values on lanes 16..31)
            {
                const int nps = ps + kAttnWarps;
                if (nps < s_end && nps < page_count && (lane & 15) < p.page_size) {
                    const int next_id = p.page_indices[(int64_t)slot * p.max_pages + nps];
                    if (next_id >= 0 && next_id < p.pool_capacity) {
                        const int row = (lane & 15) * p.kv_heads + h;
                        if (LAT) {  // the row's decoded coordinates: D bytes
                            const int8_t* src = (lane < 16 ? p.key_lattice : p.value_lattice) +
                                                ((int64_t)next_id * rows + row) * D;
                            asm volatile("prefetch.global.L1 [%0];" ::"l"(src));
                            if (D > 128) asm volatile("prefetch.global.L1 [%0];" ::"l"(src + 128));
                        } else {
                            const uint8_t* src = (lane < 16 ? p.key_codes : p.value_codes) + next_id * code_bytes +
                                                 (int64_t)row * BPR * 4;
                            asm volatile("prefetch.global.L1 [%0];" ::"l"(src));
                            if (BPR * 4 > 128) asm volatile("prefetch.global.L1 [%0];" ::"l"(src + 128));
                        }
                    }
                }
            }
            if (is_hot) {
                for (int t0 = 0; t0 < tlimit; t0 += TPW) {
                    const int t = t0 + tsub;
                    const bool valid = t < tlimit && base_token + t < limit;
                    float kvec[8], vvec[8];
                    const int64_t off = (((int64_t)slot * p.page_size + min(t, p.page_size - 1)) * p.kv_heads + h) * D + blk * 8;
                    nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.hot_keys) + off, kvec);
                    nq_load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.hot_values) + off, vvec);
                    update(kvec, vvec, 1.0f, 1.0f, valid);
                }
            } else {
                // The packed operands of the NEXT token step are fetched before this step is decoded: the
                // decode is a few hundred instructions long, enough to cover the loads' latency.
                const uint32_t* kcodes = reinterpret_cast<const uint32_t*>(p.key_codes + page_id * code_bytes);
                const uint32_t* vcodes = reinterpret_cast<const uint32_t*>(p.value_codes + page_id * code_bytes);
                const uint8_t* kbetas = p.key_betas + page_id * beta_bytes;
                const uint8_t* vbetas = p.value_betas + page_id * beta_bytes;
                const float* knorms = p.key_norms + (int64_t)page_id * rows;
                const float* vnorms = p.value_norms + (int64_t)page_id * rows;
                uint32_t kw = 0, vw = 0;
                uint2 klat = make_uint2(0, 0), vlat = make_uint2(0, 0);
                int kid, vid;
                float kn, vn;
                auto fetch = [&](int t) {
                    const int row = min(t, p.page_size - 1) * p.kv_heads + h;
                    const int64_t g = (int64_t)row * BPR + blk;
                    if (LAT) {
                        const int64_t gl = (int64_t)page_id * rows * BPR + g;
                        klat = __ldg(reinterpret_cast<const uint2*>(p.key_lattice) + gl);
                        vlat = __ldg(reinterpret_cast<const uint2*>(p.value_lattice) + gl);
                    } else {
                        kw = __ldg(kcodes + g);
                        vw = __ldg(vcodes + g);
                    }
                    kid = nq_beta_id(kbetas, g);
                    vid = nq_beta_id(vbetas, g);
                    kn = __ldg(knorms + row);
                    vn = __ldg(vnorms + row);
                };
                fetch(tsub);
                for (int t0 = 0; t0 < tlimit; t0 += TPW) {
                    const int t = t0 + tsub;
                    const bool valid = t < tlimit && base_token + t < limit;
                    const uint32_t kw_now = kw, vw_now = vw;
                    const uint2 klat_now = klat, vlat_now = vlat;
                    const float kb = __ldg(p.key_beta_table + kid), vb = __ldg(p.value_beta_table + vid);
                    const float kds = nq_div_by(kn, p.sqrt_dim, p.inv_sqrt_dim);
                    const float vds = nq_div_by(vn, p.sqrt_dim, p.inv_sqrt_dim);
                    if (t0 + TPW < tlimit) fetch(t + TPW);
                    float kvec[8], vvec[8];
                    if (LAT) {
                        // the pages' decoded shadow: same coordinates, read instead of searched
                        nq_lattice_block(klat_now, kvec);
                        nq_lattice_block(vlat_now, vvec);
                    } else {
                        nq_decode_codeword_undithered(kw_now, kvec);
                        nq_decode_codeword_undithered(vw_now, vvec);
                    }
                    update(kvec, vvec, kb * kds, vb * vds, valid);
                }
            }
        }
    }

    // merge the token sub-groups of the warp (same block index, different tokens)
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int off = BPR; off < 32; off <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
            const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
            const float mn = fmaxf(m[g], mo);
            const float c0 = mn == -INFINITY ? 0.0f : exp2f(m[g] - mn);
            const float c1 = mn == -INFINITY ? 0.0f : exp2f(mo - mn);
            l[g] = l[g] * c0 + lo * c1;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][j], off);
                acc[g][j] = acc[g][j] * c0 + ao * c1;
            }
            m[g] = mn;
        }
        if (tsub == 0) {
            if (blk == 0) {
                s_merge[warp][g][D] = m[g];
                s_merge[warp][g][D + 1] = l[g];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) s_merge[warp][g][blk * 8 + j] = acc[g][j];
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
        const int head = h * G + g;
        if (p.splits == 1) {
            const float inv = (active && ll > 0.0f) ? 1.0f / ll : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] *= inv;
            store_out(p.out, p.out_dtype, ((int64_t)qi * p.q_heads + head) * BPR + b8, a);
        } else {
            float* dst = p.partial + (((int64_t)qi * p.q_heads + head) * p.splits + split) * (D + 2);
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

template <int G, bool LAT>
int launch_attn_dim(const AttnParams& p, dim3 grid, cudaStream_t s) {
    if (p.dim == 64) nq_attn_paged_kernel<G, 8, LAT><<<grid, kAttnThreads, 0, s>>>(p);
    else if (p.dim == 128) nq_attn_paged_kernel<G, 16, LAT><<<grid, kAttnThreads, 0, s>>>(p);
    else if (p.dim == 32) nq_attn_paged_kernel<G, 4, LAT><<<grid, kAttnThreads, 0, s>>>(p);
    else if (p.dim == 256) nq_attn_paged_kernel<G, 32, LAT><<<grid, kAttnThreads, 0, s>>>(p);
    else {
        nq_set_error("nq_kv_attention: head_dim must be 32, 64, 128 or 256");
        return NQ_ERR_ARG;
    }
    return NQ_OK;
}

template <int G>
int launch_attn(const AttnParams& p, dim3 grid, cudaStream_t s) {
    return p.key_lattice ? launch_attn_dim<G, true>(p, grid, s) : launch_attn_dim<G, false>(p, grid, s);
}

// Page-range splits per (query token, KV head).  The grid should fill whole waves of the CTAs that are
// resident at once (148 SMs x 4, or x 3 for the widest GQA group): 256 CTAs x 3 splits used to run as 1.3
// waves, i.e. the time of 2.  Among the split counts that leave every split >= 4 page slots and the grid
// within 8 waves, take the smallest whose last wave is (nearly) full.
int choose_splits(int queries, int kv_heads, int max_pages, int group) {
    const long ctas = (long)queries * kv_heads;
    const long resident = 148L * (group <= 4 ? 4 : 3);
    int cap = (max_pages + 1 + 3) / 4;
    if (cap > 64) cap = 64;
    if (cap < 1) cap = 1;
    double best = 0.0;
    double score[65];
    for (int s = 1; s <= cap; ++s) {
        const long total = ctas * s;
        if (s > 1 && total > 8 * resident) {
            cap = s - 1;
            break;
        }
        const long waves = (total + resident - 1) / resident;
        score[s] = (double)total / (double)(waves * resident);
        if (score[s] > best) best = score[s];
    }
    for (int s = 1; s <= cap; ++s)
        if (score[s] >= best - 0.02) return s;
    return 1;
}

}  // namespace

extern "C" size_t nq_kv_attention_workspace_bytes(int batch, int q_tokens, int q_heads, int kv_heads, int dim,
                                                  int max_pages) {
    if (batch < 1 || q_tokens < 1 || q_heads < 1 || kv_heads < 1) return 0;
    const int splits = choose_splits(batch * q_tokens, kv_heads, max_pages, q_heads / kv_heads);
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
    p.splits = choose_splits(batch * q_tokens, kv_heads, max_pages, group);  // same split with or without the shadow: same sums
    p.out = out; p.out_dtype = out_dtype;
    p.partial = reinterpret_cast<float*>(workspace);
    if (p.splits > 1) {
        const size_t need = (size_t)batch * q_tokens * q_heads * p.splits * (dim + 2) * sizeof(float);
        NQ_REQUIRE(workspace && workspace_bytes >= need && nq_aligned16(workspace), NQ_ERR_WORKSPACE,
                   "nq_kv_attention: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)(batch * q_tokens * kv_heads), (unsigned)p.splits);
    int rc;
    switch (group) {
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
    NQ_REQUIRE(key_lattice && value_lattice && nq_aligned16(key_lattice) && nq_aligned16(value_lattice), NQ_ERR_ARG,
               "nq_kv_attention_lattice: 16-byte aligned lattice pages required");
    return kv_attention_impl(query, q_dtype, batch, q_tokens, q_heads, slot_ids, active_mask, q_lens, cache_active,
                             sequence_lengths, page_indices, page_counts, last_page_lens, hot_lengths, key_codes,
                             key_betas, key_norms, value_codes, value_betas, value_norms, key_beta_table,
                             value_beta_table, hot_keys, hot_values, max_sequences, max_pages, pool_capacity,
                             page_size, kv_heads, dim, scale, workspace, workspace_bytes, out, out_dtype, key_lattice,
                             value_lattice, stream);
}
