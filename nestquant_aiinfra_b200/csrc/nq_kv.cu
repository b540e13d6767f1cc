// NQKV4 writers: hot-tail append (K1 / ragged / segment), full-page
// encode-and-publish into the SoA page pool, and the eager single-page
// quantiser.  The page payload is produced by the same row encoder as the
// activations (rows = page_size * kv_heads, k = head_dim), so it is
// bit-identical to PackedNQKVPage.from_tensors (core/kv_format.py:71-131).
//
// Replaces runtime/nqkv_graph_writer.py:15-252 (six Triton kernels),
// runtime/nqkv_graph_pack.py:19-193 (encode of every slot + ~12 torch packing
// ops + 6 masked copies + publish) and runtime/nqkv_page.py:241-329.
#include <math.h>

#include "nq_common.cuh"
#include "nq_encode_core.cuh"

namespace {

// ----------------------------------------------------------------- append ----
struct AppendParams {
    const uint4* key;    // [B, T, H, D] as 16-byte vectors
    const uint4* value;
    int batch, tokens, mode;  // 0 = one token per row, 1 = prefix write mask, 2 = (start, count) segment
    const int32_t* slot_ids;
    const uint8_t* mask;             // mode 0: [B]; mode 1: [B, T]
    const int32_t* source_starts;    // mode 2
    const int32_t* segment_counts;   // mode 2
    const uint8_t* cache_active;     // [S]
    uint4* hot_keys;                 // [S, P, H, D]
    uint4* hot_values;
    int32_t* hot_lengths;
    int32_t* sequence_lengths;
    int max_sequences, page_size, vec_per_token;  // vec_per_token = H * D * elem / 16
    int64_t key_row_vecs, value_row_vecs;         // 16-byte vectors between the rows b and b + 1 of key / value
};

__global__ void __launch_bounds__(256) nq_kv_append_kernel(const AppendParams p) {
    const int b = blockIdx.x;
    const int requested = p.slot_ids[b];
    const bool in_range = requested >= 0 && requested < p.max_sequences;
    const int slot = min(max(requested, 0), p.max_sequences - 1);
    const bool cache_ok = in_range && p.cache_active[slot] != 0;
    const int hot_len = p.hot_lengths[slot];
    __syncthreads();  // every thread has read the old length before thread 0 may change it

    int count = 0;       // tokens the metadata update accounts for
    bool commit = false;
    if (p.mode == 0) {
        commit = cache_ok && p.mask[b] != 0 && hot_len < p.page_size;
        count = 1;
    } else if (p.mode == 1) {
        for (int t = 0; t < p.tokens; ++t) count += p.mask[(int64_t)b * p.tokens + t] != 0;
        commit = cache_ok && count > 0 && hot_len + count <= p.page_size;
    } else {
        count = p.segment_counts[b];
        commit = cache_ok && count > 0 && hot_len + count <= p.page_size;
    }

    const int start = p.mode == 2 ? p.source_starts[b] : 0;
    const int64_t work = (int64_t)p.tokens * p.vec_per_token;
    for (int64_t i = threadIdx.x; i < work; i += blockDim.x) {
        const int local = (int)(i / p.vec_per_token), v = (int)(i - (int64_t)local * p.vec_per_token);
        int src = local;
        bool ok;
        if (p.mode == 0) {
            ok = local == 0 && cache_ok && p.mask[b] != 0 && hot_len < p.page_size;
        } else if (p.mode == 1) {
            ok = cache_ok && p.mask[(int64_t)b * p.tokens + local] != 0;
        } else {
            src = start + local;
            ok = cache_ok && local < count && src < p.tokens;
        }
        const int dst = hot_len + local;
        if (!ok || dst >= p.page_size) continue;
        const int64_t in_row = (int64_t)src * p.vec_per_token + v;
        const int64_t d_off = ((int64_t)slot * p.page_size + dst) * p.vec_per_token + v;
        p.hot_keys[d_off] = __ldg(p.key + b * p.key_row_vecs + in_row);
        p.hot_values[d_off] = __ldg(p.value + b * p.value_row_vecs + in_row);
    }
    if (threadIdx.x == 0 && commit) {
        p.hot_lengths[slot] = hot_len + count;
        p.sequence_lengths[slot] += count;
    }
}

// ------------------------------------------------------------ pack + publish --
struct PackParams {
    const void* hot_keys;    // [S, P, H, D]
    const void* hot_values;
    const int32_t* hot_lengths;
    const uint8_t* boundary_mask;    // [S]
    const int32_t* target_page_ids;  // [S], or null: static ids slot * max_pages + page_counts[slot]
    uint8_t *key_codes, *key_betas, *value_codes, *value_betas;  // pool streams [capacity, bytes per page]
    float *key_norms, *value_norms;                                // [capacity, P*H]
    const float *key_beta_table, *value_beta_table;
    int32_t* page_indices;  // [S, max_pages]
    int32_t* page_counts;
    int32_t* last_page_lens;
    int32_t* hot_lengths_rw;
    int max_sequences, max_pages, page_size, heads, dim, pool_capacity, ctas_per_stream;
    float sqrt_dim;
    int8_t *key_lattice, *value_lattice;  // optional decoded shadow of the pool, [capacity, P*H*D]
};

// A slot's hot page is packed and published only when all of this holds: the slot is selected, its hot tail
// is full, its page table has room, and the target id lies inside the pool.  The three kernels of a
// pack-and-publish call use this one predicate, so a page is never written without being published
// (a slot whose table is full must not touch the pool: with caller-computed ids its "next" id may
// belong to another sequence) and never published without having been written.
// The page a slot packs into: the caller's id, or (no id array) the slot's own next page of a pool that is a fixed
// partition of max_pages per slot.  page_counts only changes in the publish kernel, after every reader.
__device__ __forceinline__ int nq_pack_target(const PackParams& p, int slot) {
    return p.target_page_ids ? p.target_page_ids[slot] : slot * p.max_pages + p.page_counts[slot];
}

__device__ __forceinline__ bool nq_pack_selected(const PackParams& p, int slot) {
    const int page_id = nq_pack_target(p, slot);
    return p.boundary_mask[slot] != 0 && p.hot_lengths[slot] == p.page_size && p.page_counts[slot] < p.max_pages &&
           page_id >= 0 && page_id < p.pool_capacity;
}

// Decoded shadow of a page ("lattice page"): every E8 block of the code stream decoded once to its eight
// minimum-energy coordinates, stored doubled as int8 (half-integers in [-14, 14] -> integers in [-28, 28]).
// It is a pure function of the code stream, kept beside it by callers that trade HBM for attention time.
__device__ __forceinline__ void nq_expand_block(const uint32_t* codes, int8_t* lattice, int64_t g) {
    float r[8];
    nq_decode_codeword_undithered(__ldg(codes + g), r);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        lo |= ((uint32_t)(int)(2.0f * r[j]) & 0xffu) << (8 * j);
        hi |= ((uint32_t)(int)(2.0f * r[j + 4]) & 0xffu) << (8 * j);
    }
    reinterpret_cast<uint2*>(lattice)[g] = make_uint2(lo, hi);
}

// Shadow of the pages that nq_kv_pack_pages_kernel has just written (same predicate, before the publish).
__global__ void __launch_bounds__(256) nq_kv_expand_packed_kernel(const PackParams p) {
    const int slot = blockIdx.x;
    if (!nq_pack_selected(p, slot)) return;
    const int page_id = nq_pack_target(p, slot);
    const int blocks = p.page_size * p.heads * (p.dim >> 3);
    const bool is_value = blockIdx.y != 0;
    const uint32_t* codes = reinterpret_cast<const uint32_t*>(is_value ? p.value_codes : p.key_codes) +
                            (int64_t)page_id * blocks;
    int8_t* lattice = (is_value ? p.value_lattice : p.key_lattice) + (int64_t)page_id * blocks * 8;
    for (int g = threadIdx.x; g < blocks; g += blockDim.x) nq_expand_block(codes, lattice, g);
}

// Shadow of an explicit list of pages (eager writers, conversion of an existing pool).
__global__ void __launch_bounds__(256) nq_kv_expand_pages_kernel(const uint32_t* codes, int8_t* lattice,
                                                                 const int32_t* page_ids, int blocks,
                                                                 int pool_capacity) {
    const int page_id = page_ids[blockIdx.x];
    if (page_id < 0 || page_id >= pool_capacity) return;
    const uint32_t* src = codes + (int64_t)page_id * blocks;
    int8_t* dst = lattice + (int64_t)page_id * blocks * 8;
    for (int g = blockIdx.y * blockDim.x + threadIdx.x; g < blocks; g += gridDim.y * blockDim.x)
        nq_expand_block(src, dst, g);
}

template <typename T>
__global__ void __launch_bounds__(NQ_ENC_THREADS, 5) nq_kv_pack_pages_kernel(const PackParams p) {
    extern __shared__ __align__(16) float smem[];
    const int slot = blockIdx.x;
    if (!nq_pack_selected(p, slot)) return;  // CTA-uniform
    const int page_id = nq_pack_target(p, slot);
    const int is_value = blockIdx.y / p.ctas_per_stream;
    const int chunk = blockIdx.y - is_value * p.ctas_per_stream;
    const int rows = p.page_size * p.heads, rpc = nq_encode_rows_per_cta(p.dim), bpr = p.dim >> 3;
    const int r0 = chunk * rpc;
    const int nrows = min(rpc, rows - r0);
    if (nrows <= 0) return;
    const T* src = reinterpret_cast<const T*>(is_value ? p.hot_values : p.hot_keys) +
                   ((int64_t)slot * rows + r0) * p.dim;
    const int64_t code_bytes = (int64_t)rows * p.dim / 2, beta_bytes = (int64_t)rows * p.dim / 32;
    uint8_t* codes = (is_value ? p.value_codes : p.key_codes) + page_id * code_bytes + (int64_t)r0 * p.dim / 2;
    uint8_t* betas = (is_value ? p.value_betas : p.key_betas) + page_id * beta_bytes + (int64_t)r0 * bpr / 4;
    float* norms = (is_value ? p.value_norms : p.key_norms) + (int64_t)page_id * rows + r0;
    nq_encode_rows_cta<T>(src, p.dim, nrows, nrows, p.dim, is_value ? p.value_beta_table : p.key_beta_table,
                          p.sqrt_dim, reinterpret_cast<uint32_t*>(codes), betas, norms, nullptr, 0u, smem);
}

__global__ void __launch_bounds__(256) nq_kv_publish_kernel(const PackParams p) {
    const int slot = blockIdx.x * blockDim.x + threadIdx.x;
    if (slot >= p.max_sequences) return;
    if (!nq_pack_selected(p, slot)) return;
    const int count = p.page_counts[slot];
    p.page_indices[(int64_t)slot * p.max_pages + count] = nq_pack_target(p, slot);
    p.page_counts[slot] = count + 1;
    p.last_page_lens[slot] = p.page_size;
    p.hot_lengths_rw[slot] = 0;
}

// ------------------------------------------------------ device-side page allocator --
// The free pages of a pool are a stack in device memory: free_ids[0 .. *free_count).  Kernels of one stream pop
// and push it without the host: no per-step read of the hot lengths, no host reservation, and the pool need not be
// a fixed partition of max_pages per slot.  Admission control (the host never admits more requests than the pool
// can hold at their maximum lengths) is what guarantees that a pop finds a page; a pop from an empty stack
// yields -1, which the pack kernels treat as "do not pack" (the slot's hot tail stays full).

// One target page for every slot that is about to pack: same predicate as nq_pack_selected, minus the id.
__global__ void __launch_bounds__(256) nq_kv_alloc_targets_kernel(const int32_t* hot_lengths, const uint8_t* boundary_mask,
                                                                  const int32_t* page_counts, const int32_t* free_ids,
                                                                  int32_t* free_count, int32_t* target_page_ids,
                                                                  int max_sequences, int max_pages, int page_size) {
    const int slot = blockIdx.x * blockDim.x + threadIdx.x;
    if (slot >= max_sequences) return;
    int id = -1;
    if (boundary_mask[slot] != 0 && hot_lengths[slot] == page_size && page_counts[slot] < max_pages) {
        const int old = atomicSub(free_count, 1);
        if (old > 0) id = free_ids[old - 1];
        else atomicAdd(free_count, 1);  // empty: put the count back
    }
    target_page_ids[slot] = id;
}

// `count` pages at once (bulk writers): out_ids[i] for i < count, -1 where the stack ran dry.
__global__ void __launch_bounds__(256) nq_kv_alloc_pages_kernel(int count, const int32_t* free_ids, int32_t* free_count,
                                                                int32_t* out_ids) {
    __shared__ int s_old;
    if (threadIdx.x == 0) {
        const int old = atomicSub(free_count, count);
        if (old < count) atomicAdd(free_count, count - max(old, 0));  // only max(old, 0) pages were there
        s_old = old;
    }
    __syncthreads();
    const int old = s_old;
    for (int i = threadIdx.x; i < count; i += blockDim.x) out_ids[i] = i < old ? free_ids[old - 1 - i] : -1;
}

// Give the pages of the selected slots back and empty those slots (one CTA per slot).
__global__ void __launch_bounds__(128) nq_kv_release_pages_kernel(const uint8_t* slot_mask, int32_t* page_indices,
                                                                  int32_t* page_counts, int32_t* last_page_lens,
                                                                  int32_t* hot_lengths, int32_t* sequence_lengths,
                                                                  int32_t* free_ids, int32_t* free_count, int max_pages,
                                                                  int pool_capacity) {
    __shared__ int s_base;
    const int slot = blockIdx.x;
    if (slot_mask[slot] == 0) return;
    const int count = min(max(page_counts[slot], 0), max_pages);
    if (threadIdx.x == 0) s_base = count > 0 ? atomicAdd(free_count, count) : 0;
    __syncthreads();
    for (int i = threadIdx.x; i < max_pages; i += blockDim.x) {
        int32_t* entry = page_indices + (int64_t)slot * max_pages + i;
        if (i < count) {
            const int id = *entry;
            // a table entry is always a page this allocator handed out; the range check guards the stack anyway
            if (s_base + i < pool_capacity) free_ids[s_base + i] = (id >= 0 && id < pool_capacity) ? id : 0;
        }
        *entry = -1;
    }
    if (threadIdx.x == 0) {
        page_counts[slot] = 0;
        last_page_lens[slot] = 0;
        hot_lengths[slot] = 0;
        sequence_lengths[slot] = 0;
    }
}

// ------------------------------------------------------------- eager one page --
struct PageParams {
    const void *key, *value;  // [valid, H, D]
    int valid_tokens, page_size, heads, dim, ctas_per_stream;
    const float *key_beta_table, *value_beta_table;
    uint8_t *key_codes, *key_betas, *value_codes, *value_betas;
    float *key_norms, *value_norms;
    float sqrt_dim;
};

template <typename T>
__global__ void __launch_bounds__(NQ_ENC_THREADS, 5) nq_kv_quantize_page_kernel(const PageParams p) {
    extern __shared__ __align__(16) float smem[];
    const int is_value = blockIdx.x / p.ctas_per_stream;
    const int chunk = blockIdx.x - is_value * p.ctas_per_stream;
    const int rows = p.page_size * p.heads, rpc = nq_encode_rows_per_cta(p.dim), bpr = p.dim >> 3;
    const int r0 = chunk * rpc;
    const int nrows = min(rpc, rows - r0);
    if (nrows <= 0) return;
    const int valid_rows = min(max(p.valid_tokens * p.heads - r0, 0), nrows);  // later rows are zero padding
    const T* src = reinterpret_cast<const T*>(is_value ? p.value : p.key) + (int64_t)r0 * p.dim;
    uint8_t* codes = (is_value ? p.value_codes : p.key_codes) + (int64_t)r0 * p.dim / 2;
    uint8_t* betas = (is_value ? p.value_betas : p.key_betas) + (int64_t)r0 * bpr / 4;
    float* norms = (is_value ? p.value_norms : p.key_norms) + r0;
    nq_encode_rows_cta<T>(src, p.dim, nrows, valid_rows, p.dim, is_value ? p.value_beta_table : p.key_beta_table,
                          p.sqrt_dim, reinterpret_cast<uint32_t*>(codes), betas, norms, nullptr, 0u, smem);
}

template <typename K>
int set_smem(K kernel, size_t smem, const char* name) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            nq_set_error("%s: shared memory: %s", name, cudaGetErrorString(e));
            return (int)e;
        }
    }
    return NQ_OK;
}

bool dims_ok(int page_size, int heads, int dim) {
    return page_size >= 1 && heads >= 1 && dim >= 32 && dim % 32 == 0 && dim <= 1024 &&
           ((int64_t)page_size * heads) % 1 == 0;
}

}  // namespace

extern "C" int nq_kv_append(const void* key, const void* value, int kv_dtype, int batch, int tokens, int mode,
                            const int32_t* slot_ids, const uint8_t* mask, const int32_t* source_starts,
                            const int32_t* segment_counts, const uint8_t* cache_active, void* hot_keys,
                            void* hot_values, int32_t* hot_lengths, int32_t* sequence_lengths, int max_sequences,
                            int page_size, int heads, int dim, int64_t key_row_stride, int64_t value_row_stride,
                            nq_stream_t stream) {
    NQ_RANGE("nq_kv_append");
    NQ_REQUIRE(key && value && slot_ids && cache_active && hot_keys && hot_values && hot_lengths && sequence_lengths,
               NQ_ERR_ARG, "nq_kv_append: null pointer");
    NQ_REQUIRE(mode >= 0 && mode <= 2, NQ_ERR_ARG, "nq_kv_append: mode must be 0 (K1), 1 (write mask) or 2 (segment)");
    NQ_REQUIRE((mode == 2) ? (source_starts && segment_counts) : (mask != nullptr), NQ_ERR_ARG,
               "nq_kv_append: mask / segment arrays missing for mode %d", mode);
    NQ_REQUIRE(batch >= 1 && tokens >= 1 && (mode != 0 || tokens == 1), NQ_ERR_ARG, "nq_kv_append: bad batch/tokens");
    NQ_REQUIRE(max_sequences >= 1 && dims_ok(page_size, heads, dim), NQ_ERR_ARG, "nq_kv_append: bad cache geometry");
    const int esize = kv_dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(((int64_t)heads * dim * esize) % 16 == 0, NQ_ERR_ALIGN, "nq_kv_append: token size must be a multiple of 16 bytes");
    NQ_REQUIRE(nq_aligned16(key) && nq_aligned16(value) && nq_aligned16(hot_keys) && nq_aligned16(hot_values),
               NQ_ERR_ALIGN, "nq_kv_append: 16-byte alignment required");
    AppendParams p;
    p.key = reinterpret_cast<const uint4*>(key);
    p.value = reinterpret_cast<const uint4*>(value);
    p.batch = batch; p.tokens = tokens; p.mode = mode;
    p.slot_ids = slot_ids; p.mask = mask; p.source_starts = source_starts; p.segment_counts = segment_counts;
    p.cache_active = cache_active;
    p.hot_keys = reinterpret_cast<uint4*>(hot_keys);
    p.hot_values = reinterpret_cast<uint4*>(hot_values);
    p.hot_lengths = hot_lengths; p.sequence_lengths = sequence_lengths;
    p.max_sequences = max_sequences; p.page_size = page_size;
    p.vec_per_token = heads * dim * esize / 16;
    const int64_t dense = (int64_t)tokens * heads * dim;  // elements of one row [T, H, D]
    NQ_REQUIRE((key_row_stride == 0 || key_row_stride >= dense) && (value_row_stride == 0 || value_row_stride >= dense),
               NQ_ERR_ARG, "nq_kv_append: a row stride is smaller than a row");
    NQ_REQUIRE((key_row_stride * esize) % 16 == 0 && (value_row_stride * esize) % 16 == 0, NQ_ERR_ALIGN,
               "nq_kv_append: row strides must be multiples of 16 bytes");
    p.key_row_vecs = (key_row_stride ? key_row_stride : dense) * esize / 16;
    p.value_row_vecs = (value_row_stride ? value_row_stride : dense) * esize / 16;
    nq_kv_append_kernel<<<batch, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    NQ_CHECK_LAUNCH("nq_kv_append");
    return NQ_OK;
}

static int kv_pack_publish_impl(const void* hot_keys, const void* hot_values, int kv_dtype, int32_t* hot_lengths,
                                const uint8_t* boundary_mask, const int32_t* target_page_ids,
                                uint8_t* key_codes, uint8_t* key_betas, float* key_norms, uint8_t* value_codes,
                                uint8_t* value_betas, float* value_norms, const float* key_beta_table,
                                const float* value_beta_table, int32_t* page_indices, int32_t* page_counts,
                                int32_t* last_page_lens, int max_sequences, int max_pages, int pool_capacity,
                                int page_size, int heads, int dim, int8_t* key_lattice, int8_t* value_lattice,
                                nq_stream_t stream) {
    NQ_REQUIRE(hot_keys && hot_values && hot_lengths && boundary_mask && key_codes && key_betas &&
                   key_norms && value_codes && value_betas && value_norms && key_beta_table && value_beta_table &&
                   page_indices && page_counts && last_page_lens,
               NQ_ERR_ARG, "nq_kv_pack_publish: null pointer");
    NQ_REQUIRE(max_sequences >= 1 && max_pages >= 1 && pool_capacity >= 1 && dims_ok(page_size, heads, dim),
               NQ_ERR_ARG, "nq_kv_pack_publish: bad cache geometry");
    NQ_REQUIRE(kv_dtype == NQ_BF16 || kv_dtype == NQ_F16, NQ_ERR_ARG, "nq_kv_pack_publish: hot tail must be bf16 or f16");
    NQ_REQUIRE(nq_aligned16(hot_keys) && nq_aligned16(hot_values) && nq_aligned16(key_codes) && nq_aligned16(value_codes),
               NQ_ERR_ALIGN, "nq_kv_pack_publish: 16-byte alignment required");
    PackParams p;
    p.hot_keys = hot_keys; p.hot_values = hot_values; p.hot_lengths = hot_lengths; p.hot_lengths_rw = hot_lengths;
    p.boundary_mask = boundary_mask; p.target_page_ids = target_page_ids;
    p.key_codes = key_codes; p.key_betas = key_betas; p.key_norms = key_norms;
    p.value_codes = value_codes; p.value_betas = value_betas; p.value_norms = value_norms;
    p.key_beta_table = key_beta_table; p.value_beta_table = value_beta_table;
    p.page_indices = page_indices; p.page_counts = page_counts; p.last_page_lens = last_page_lens;
    p.max_sequences = max_sequences; p.max_pages = max_pages; p.page_size = page_size; p.heads = heads; p.dim = dim;
    p.pool_capacity = pool_capacity;
    p.key_lattice = key_lattice; p.value_lattice = value_lattice;
    const int rpc = nq_encode_rows_per_cta(dim);
    p.ctas_per_stream = (page_size * heads + rpc - 1) / rpc;
    p.sqrt_dim = (float)sqrt((double)dim);
    const size_t smem = nq_encode_smem_floats(dim) * sizeof(float);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)max_sequences, (unsigned)(2 * p.ctas_per_stream));
    if (kv_dtype == NQ_BF16) {
        int rc = set_smem(nq_kv_pack_pages_kernel<__nv_bfloat16>, smem, "nq_kv_pack_publish");
        if (rc) return rc;
        nq_kv_pack_pages_kernel<__nv_bfloat16><<<grid, NQ_ENC_THREADS, smem, s>>>(p);
    } else {
        int rc = set_smem(nq_kv_pack_pages_kernel<__half>, smem, "nq_kv_pack_publish");
        if (rc) return rc;
        nq_kv_pack_pages_kernel<__half><<<grid, NQ_ENC_THREADS, smem, s>>>(p);
    }
    NQ_CHECK_LAUNCH("nq_kv_pack_publish(pack)");
    if (key_lattice) {
        nq_kv_expand_packed_kernel<<<dim3((unsigned)max_sequences, 2), 256, 0, s>>>(p);
        NQ_CHECK_LAUNCH("nq_kv_pack_publish(lattice shadow)");
    }
    nq_kv_publish_kernel<<<(max_sequences + 255) / 256, 256, 0, s>>>(p);
    NQ_CHECK_LAUNCH("nq_kv_pack_publish(publish)");
    return NQ_OK;
}

extern "C" int nq_kv_pack_publish(const void* hot_keys, const void* hot_values, int kv_dtype, int32_t* hot_lengths,
                                  const uint8_t* boundary_mask, const int32_t* target_page_ids,
                                  uint8_t* key_codes, uint8_t* key_betas, float* key_norms, uint8_t* value_codes,
                                  uint8_t* value_betas, float* value_norms, const float* key_beta_table,
                                  const float* value_beta_table, int32_t* page_indices, int32_t* page_counts,
                                  int32_t* last_page_lens, int max_sequences, int max_pages, int pool_capacity,
                                  int page_size, int heads, int dim, nq_stream_t stream) {
    NQ_RANGE("nq_kv_pack_publish");
    return kv_pack_publish_impl(hot_keys, hot_values, kv_dtype, hot_lengths, boundary_mask, target_page_ids, key_codes,
                                key_betas, key_norms, value_codes, value_betas, value_norms, key_beta_table,
                                value_beta_table, page_indices, page_counts, last_page_lens, max_sequences, max_pages,
                                pool_capacity, page_size, heads, dim, nullptr, nullptr, stream);
}

extern "C" int nq_kv_pack_publish_lattice(const void* hot_keys, const void* hot_values, int kv_dtype,
                                          int32_t* hot_lengths, const uint8_t* boundary_mask,
                                          const int32_t* target_page_ids, uint8_t* key_codes, uint8_t* key_betas,
                                          float* key_norms, uint8_t* value_codes, uint8_t* value_betas,
                                          float* value_norms, const float* key_beta_table,
                                          const float* value_beta_table, int32_t* page_indices, int32_t* page_counts,
                                          int32_t* last_page_lens, int max_sequences, int max_pages,
                                          int pool_capacity, int page_size, int heads, int dim, int8_t* key_lattice,
                                          int8_t* value_lattice, nq_stream_t stream) {
    NQ_RANGE("nq_kv_pack_publish_lattice");
    NQ_REQUIRE(key_lattice && value_lattice && nq_aligned16(key_lattice) && nq_aligned16(value_lattice), NQ_ERR_ARG,
               "nq_kv_pack_publish_lattice: 16-byte aligned lattice pages required");
    return kv_pack_publish_impl(hot_keys, hot_values, kv_dtype, hot_lengths, boundary_mask, target_page_ids, key_codes,
                                key_betas, key_norms, value_codes, value_betas, value_norms, key_beta_table,
                                value_beta_table, page_indices, page_counts, last_page_lens, max_sequences, max_pages,
                                pool_capacity, page_size, heads, dim, key_lattice, value_lattice, stream);
}

extern "C" int nq_kv_alloc_targets(const int32_t* hot_lengths, const uint8_t* boundary_mask, const int32_t* page_counts,
                                   const int32_t* free_ids, int32_t* free_count, int32_t* target_page_ids,
                                   int max_sequences, int max_pages, int page_size, nq_stream_t stream) {
    NQ_RANGE("nq_kv_alloc_targets");
    NQ_REQUIRE(hot_lengths && boundary_mask && page_counts && free_ids && free_count && target_page_ids, NQ_ERR_ARG,
               "nq_kv_alloc_targets: null pointer");
    NQ_REQUIRE(max_sequences >= 1 && max_pages >= 1 && page_size >= 1, NQ_ERR_ARG, "nq_kv_alloc_targets: bad geometry");
    nq_kv_alloc_targets_kernel<<<(max_sequences + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        hot_lengths, boundary_mask, page_counts, free_ids, free_count, target_page_ids, max_sequences, max_pages,
        page_size);
    NQ_CHECK_LAUNCH("nq_kv_alloc_targets");
    return NQ_OK;
}

extern "C" int nq_kv_alloc_pages(int count, const int32_t* free_ids, int32_t* free_count, int32_t* out_ids,
                                 nq_stream_t stream) {
    NQ_RANGE("nq_kv_alloc_pages");
    NQ_REQUIRE(free_ids && free_count && (out_ids || count == 0), NQ_ERR_ARG, "nq_kv_alloc_pages: null pointer");
    NQ_REQUIRE(count >= 0, NQ_ERR_ARG, "nq_kv_alloc_pages: negative count");
    if (count == 0) return NQ_OK;
    nq_kv_alloc_pages_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(count, free_ids, free_count, out_ids);
    NQ_CHECK_LAUNCH("nq_kv_alloc_pages");
    return NQ_OK;
}

extern "C" int nq_kv_release_pages(const uint8_t* slot_mask, int32_t* page_indices, int32_t* page_counts,
                                   int32_t* last_page_lens, int32_t* hot_lengths, int32_t* sequence_lengths,
                                   int32_t* free_ids, int32_t* free_count, int max_sequences, int max_pages,
                                   int pool_capacity, nq_stream_t stream) {
    NQ_RANGE("nq_kv_release_pages");
    NQ_REQUIRE(slot_mask && page_indices && page_counts && last_page_lens && hot_lengths && sequence_lengths &&
                   free_ids && free_count,
               NQ_ERR_ARG, "nq_kv_release_pages: null pointer");
    NQ_REQUIRE(max_sequences >= 1 && max_pages >= 1 && pool_capacity >= 1, NQ_ERR_ARG, "nq_kv_release_pages: bad geometry");
    nq_kv_release_pages_kernel<<<max_sequences, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        slot_mask, page_indices, page_counts, last_page_lens, hot_lengths, sequence_lengths, free_ids, free_count,
        max_pages, pool_capacity);
    NQ_CHECK_LAUNCH("nq_kv_release_pages");
    return NQ_OK;
}

extern "C" int nq_kv_expand_pages(const uint8_t* codes, int8_t* lattice, const int32_t* page_ids, int64_t count,
                                  int pool_capacity, int page_size, int heads, int dim, nq_stream_t stream) {
    NQ_RANGE("nq_kv_expand_pages");
    NQ_REQUIRE(codes && lattice && page_ids, NQ_ERR_ARG, "nq_kv_expand_pages: null pointer");
    NQ_REQUIRE(count >= 0 && count <= 0x7fffffff && pool_capacity >= 1 && dims_ok(page_size, heads, dim), NQ_ERR_ARG,
               "nq_kv_expand_pages: bad geometry");
    NQ_REQUIRE(nq_aligned16(codes) && nq_aligned16(lattice), NQ_ERR_ALIGN, "nq_kv_expand_pages: 16-byte alignment required");
    if (count == 0) return NQ_OK;
    const int blocks = page_size * heads * (dim >> 3);
    const unsigned chunks = (unsigned)((blocks + 1023) / 1024);
    nq_kv_expand_pages_kernel<<<dim3((unsigned)count, chunks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(codes), lattice, page_ids, blocks, pool_capacity);
    NQ_CHECK_LAUNCH("nq_kv_expand_pages");
    return NQ_OK;
}

extern "C" int nq_kv_quantize_page(const void* key, const void* value, int kv_dtype, int valid_tokens, int page_size,
                                   int heads, int dim, const float* key_beta_table, const float* value_beta_table,
                                   uint8_t* key_codes, uint8_t* key_betas, float* key_norms, uint8_t* value_codes,
                                   uint8_t* value_betas, float* value_norms, nq_stream_t stream) {
    NQ_RANGE("nq_kv_quantize_page");
    NQ_REQUIRE(key && value && key_beta_table && value_beta_table && key_codes && key_betas && key_norms &&
                   value_codes && value_betas && value_norms,
               NQ_ERR_ARG, "nq_kv_quantize_page: null pointer");
    NQ_REQUIRE(dims_ok(page_size, heads, dim) && valid_tokens >= 1 && valid_tokens <= page_size, NQ_ERR_ARG,
               "nq_kv_quantize_page: token count must be in [1, page_size] and head_dim a multiple of 32");
    NQ_REQUIRE(nq_aligned16(key) && nq_aligned16(value) && nq_aligned16(key_codes) && nq_aligned16(value_codes),
               NQ_ERR_ALIGN, "nq_kv_quantize_page: 16-byte alignment required");
    PageParams p;
    p.key = key; p.value = value; p.valid_tokens = valid_tokens; p.page_size = page_size; p.heads = heads; p.dim = dim;
    p.key_beta_table = key_beta_table; p.value_beta_table = value_beta_table;
    p.key_codes = key_codes; p.key_betas = key_betas; p.key_norms = key_norms;
    p.value_codes = value_codes; p.value_betas = value_betas; p.value_norms = value_norms;
    const int rpc = nq_encode_rows_per_cta(dim);
    p.ctas_per_stream = (page_size * heads + rpc - 1) / rpc;
    p.sqrt_dim = (float)sqrt((double)dim);
    const size_t smem = nq_encode_smem_floats(dim) * sizeof(float);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)(2 * p.ctas_per_stream);
    int rc = NQ_OK;
    switch (kv_dtype) {
        case NQ_BF16:
            if ((rc = set_smem(nq_kv_quantize_page_kernel<__nv_bfloat16>, smem, "nq_kv_quantize_page"))) return rc;
            nq_kv_quantize_page_kernel<__nv_bfloat16><<<grid, NQ_ENC_THREADS, smem, s>>>(p);
            break;
        case NQ_F16:
            if ((rc = set_smem(nq_kv_quantize_page_kernel<__half>, smem, "nq_kv_quantize_page"))) return rc;
            nq_kv_quantize_page_kernel<__half><<<grid, NQ_ENC_THREADS, smem, s>>>(p);
            break;
        case NQ_F32:
            if ((rc = set_smem(nq_kv_quantize_page_kernel<float>, smem, "nq_kv_quantize_page"))) return rc;
            nq_kv_quantize_page_kernel<float><<<grid, NQ_ENC_THREADS, smem, s>>>(p);
            break;
        default:
            nq_set_error("nq_kv_quantize_page: unknown dtype %d", kv_dtype);
            return NQ_ERR_ARG;
    }
    NQ_CHECK_LAUNCH("nq_kv_quantize_page");
    return NQ_OK;
}
