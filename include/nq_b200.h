/*
 * C ABI of the B200 (sm_100a) implementation of NestQuant's W4A4KV4 hot path.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes, no framework types; every pointer is a DEVICE
 *     pointer unless its name ends in _host;
 *   - the caller owns every buffer, passes the CUDA stream explicitly and
 *     supplies workspaces; nothing here allocates device memory or synchronises
 *     the host (nq_w4a4_status and the first nq_kv_attention call per device
 *     excepted).  Host-side state is limited to
 *     per-device look-ups made on first use (SM count, the opt-in of a kernel
 *     to large shared memory, the driver entry point that builds tensor maps,
 *     whether the page-decode table of nq_kv_attention has been filled)
 *     and, for nq_w4a4_gemv_static only, the address of its built-in scratch;
 *     launches go to the CURRENT device, which must be the stream's device;
 *   - every entry point opens an NVTX range of its own name around its launches
 *     (visible to profiling tools, otherwise a no-op);
 *   - return value 0 = success, negative = argument error (NQ_ERR_*), positive
 *     = cudaError_t of the failed launch; nq_last_error() describes the last
 *     failure of the calling thread;
 *   - q = 14, 4-bit residues, four betas (2-bit ids): the NQRT4 / NQA4 / NQKV4
 *     formats of the reference (core/packing.py:137-208: value i of width w in
 *     byte floor(i*w/8), bit offset (i*w) mod 8, LSB first).
 *
 * Each declaration cites the reference interface it replaces
 * (file:line inside the reference project).
 */
#ifndef NQ_B200_H
#define NQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* nq_stream_t; /* cudaStream_t */

enum { NQ_F32 = 0, NQ_BF16 = 1, NQ_F16 = 2 };

enum {
    NQ_OK = 0,
    NQ_ERR_ARG = -1,       /* null pointer, bad size, unsupported shape */
    NQ_ERR_ALIGN = -2,     /* pointer or stride not 16-byte aligned */
    NQ_ERR_WORKSPACE = -3, /* workspace missing or too small */
    NQ_ERR_DEVICE = -4     /* not an sm_100 device / driver entry point missing */
};

int nq_abi_version(void);
const char* nq_last_error(void);
/* Number of kernels this library has launched in the process so far (host-side
 * counter; benchmarks report the difference over their timed region). */
unsigned long long nq_launch_count(void);

/* -------------------------------------------------------------------------
 * On-the-fly E8 encoder (activations, and K/V rows with k = head_dim).
 * Replaces quantize_activation_cuda (runtime/triton_w4a4_linear.py:581-617) =
 * torch vector_norm + _nqkv_encode_kernel (runtime/nqkv_page.py:97-185,332-372)
 * + two _pack_unsigned_cuda chains (runtime/nqkv_page.py:446-456), in ONE launch.
 * Bit-exact with quantize_rows + pack_nestquant_indices on the CPU
 * (core/quantizer.py:214-301, core/packing.py:137-171).
 *
 *   x            [rows, k] of x_dtype, row r at x + r*row_stride elements
 *   beta_table   4 floats
 *   out_codes    rows*k/2 bytes, out_beta_ids rows*k/32 bytes, out_norms rows floats
 *   out_decoded  optional (may be NULL): bf16 [rows, k] reconstruction
 *                bf16(((t - 14 Q(t/14)) * beta) * (norm / sqrt(k)))
 * Requirements: k % 32 == 0, 32 <= k <= 32768, 16-byte aligned x and stride. */
int nq_a4_encode(const void* x, int x_dtype, int64_t rows, int64_t k, int64_t row_stride,
                 const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                 float* out_norms, void* out_decoded, nq_stream_t stream);

/* Rotate-then-encode: the normalised Hadamard transform FusedNQRTLinear applies to its input
 * (models/fused_linear.py:287-290 -> core/rotation.py:12-27) and nq_a4_encode in one launch.
 * Outputs are bit-identical to nq_hadamard(x) followed by nq_a4_encode; the rotated rows are
 * not written out.  hadamard_block = k rotates whole rows; a smaller power of two dividing k
 * rotates consecutive blocks of that size (block-diagonal rotation of a tensor-parallel K
 * shard).  x is [rows, k] contiguous.  No counterpart in the reference, which runs the
 * transform as separate tensor ops.
 * Requirements: k % 32 == 0, 32 <= k <= NQ_ROTATED_MAX_K, 16-byte aligned pointers. */
#define NQ_ROTATED_MAX_K 16384
int nq_a4_encode_rotated(const void* x, int x_dtype, int64_t rows, int64_t k, int64_t hadamard_block,
                         const float* beta_table, uint8_t* out_codes, uint8_t* out_beta_ids,
                         float* out_norms, void* out_decoded, nq_stream_t stream);

/* Module-level fusion at the plugin boundary: the elementwise producer of a projection's input, the rotation and
 * the A4 encode in ONE launch.  Outputs are bit-identical to the separate launches.
 *   nq_a4_encode_rmsnorm_rotated   rows = weight * dtype(x * rsqrt(mean(x^2) + eps)), i.e. nq_rmsnorm (same fixed
 *                                  reduction order), in front of q/k/v and gate/up (models/fused_linear.py:287-306
 *                                  receives the normalised hidden state from the model's LlamaRMSNorm)
 *   nq_a4_encode_silu_mul_rotated  rows = dtype(dtype(silu(gate)) * up), the tensor ops of the Llama MLP in front of
 *                                  down_proj
 * x / gate / up are [rows, k] with row stride `row_stride` elements (gate and up may be column ranges of one
 * stacked projection output); weight is [k].  Other arguments as nq_a4_encode_rotated.  The reference leaves both
 * producers to the model's tensor ops: no counterpart. */
int nq_a4_encode_rmsnorm_rotated(const void* x, const void* weight, float eps, int dtype, int64_t rows, int64_t k,
                                 int64_t row_stride, int64_t hadamard_block, const float* beta_table,
                                 uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms, void* out_decoded,
                                 nq_stream_t stream);
int nq_a4_encode_silu_mul_rotated(const void* gate, const void* up, int dtype, int64_t rows, int64_t k,
                                  int64_t row_stride, int64_t hadamard_block, const float* beta_table,
                                  uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms, void* out_decoded,
                                  nq_stream_t stream);

/* Weight encoder: the same search with the stateless subtractive dither of
 * global block  w_block_offset + row*k/8 + block  ("lcg31_mix_v1",
 * core/codec.py:176-224).  Bit-exact with quantize_rows(W, 14, betas,
 * dither=generate_e8_dither_stateless(...)) + pack_nestquant_indices, i.e. with
 * the streams PackedNestQuantTensor.from_quantized_rows stores
 * (core/tensor_checkpoint.py:59-118).  Replaces the CPU-only offline encode of
 * models/quantization.py for synthetic / re-sharded weights. */
int nq_w4_encode(const void* w, int w_dtype, int64_t rows, int64_t k, int64_t row_stride,
                 const float* beta_table, int64_t seed, int64_t w_block_offset,
                 uint8_t* out_codes, uint8_t* out_beta_ids, float* out_norms, nq_stream_t stream);

/* Diagnostic / operand decode of a packed undithered stream.
 * Replaces decode_packed_a4_m16 (runtime/cuda_w4a4_mma.py:688-696, kernel
 * nqrt4_w4a4_mma.cu:83-93) and dequantize_nqkv_page_triton
 * (runtime/nqkv_page.py:494-537).  Output is bit-identical to
 * QuantizedRows.dequantize (core/quantizer.py:39-51), then cast to out_dtype
 * (NQ_F32 or NQ_BF16). */
int nq_a4_decode(const uint8_t* codes, const uint8_t* beta_ids, const float* norms,
                 const float* beta_table, int64_t rows, int64_t k, void* out, int out_dtype,
                 nq_stream_t stream);

/* -------------------------------------------------------------------------
 * Packed W4A4 projection  Y[m,n] = sum_k bf16(A^[m,k]) * bf16(W^[n,k]).
 * One entry for every M regime; replaces the pybind family run_m1 / run_small_m /
 * run_m16 / run_large_m_staged (runtime/nqrt4_w4a4_mma_binding.cpp:51-69) and the
 * Python chunk+pad wrapper (runtime/cuda_w4a4_mma.py:393-484).
 *
 *   act_*      packed activation streams of m rows (from nq_a4_encode)
 *   act_decoded optional bf16 [m,k] produced by nq_a4_encode; NULL = decode here
 *   w_*        NQRT4 streams of n rows: codes n*k/2 bytes, beta ids n*k/32, norms n, betas 4
 *   w_block_offset  global index of the weight's first E8 block in its record
 *              (the dither counter of block b of row r is w_block_offset + r*k/8 + b);
 *              the reference always passes 0 (runtime/cuda_w4a4_mma.py:243)
 *   seed       stateless dither seed of the record, in [0, 2^31)
 *   out        [m, n] of out_dtype (NQ_F32 = accumulator before rounding, NQ_BF16)
 *   workspace  at least nq_w4a4_workspace_bytes(m,n,k) bytes; its first
 *              NQ_WS_COUNTER_BYTES bytes must be zero before the FIRST use and are
 *              left zero by every call.
 * Requirements: k % 32 == 0, n % 8 == 0, n <= 131064.  The tcgen05 path is taken for
 * m >= 8 when n % 128 == 0 and k % 64 == 0 (split-K with a deterministic reduction when few tiles):
 * the weight is decoded once per call into the BF16 scratch of the workspace, then multiplied. */
#define NQ_WS_COUNTER_BYTES 65536
#define NQ_WS_STATUS_OFFSET 65532 /* last word of the counter area: device status, 0 = ok */
size_t nq_w4a4_workspace_bytes(int64_t m, int64_t n, int64_t k);
int nq_w4a4_gemm(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                 const float* act_betas, const void* act_decoded,
                 const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                 const float* w_betas, int64_t m, int64_t n, int64_t k,
                 int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                 void* workspace, size_t workspace_bytes, nq_stream_t stream);

/* nq_w4a4_gemm as ONE launch for m >= 8 (n % 128 == 0, k % 64 == 0; other shapes take nq_w4a4_gemm's path): the
 * kernel's decode warps turn the packed weight into BF16 tiles on the ALU pipes (dither regenerated, two E8
 * searches per block) while the tensor pipe of the same SM multiplies the tiles that are already there; a TMA
 * producer waits (bounded; status code 5 when it gives up) for the arrival counter of its channel tile.  This is the
 * shape of the reference's large-M kernel, which decodes inside its MMA loop (runtime/nqrt4_w4a4_mma.cu:606-723),
 * with the weight still decoded once per call.  Same arguments and workspace as nq_w4a4_gemm, same result bit for
 * bit.  On B200 it does not beat nq_w4a4_gemm's two launches yet, so it is a separate entry, not the default. */
int nq_w4a4_gemm_fused(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                       const float* act_betas, const void* act_decoded,
                       const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                       const float* w_betas, int64_t m, int64_t n, int64_t k,
                       int64_t w_block_offset, int64_t seed, void* out, int out_dtype,
                       void* workspace, size_t workspace_bytes, nq_stream_t stream);

/* The same projection for a weight that stacks the rows of several tensors sharing one input
 * (q/k/v, gate/up): one launch sequence instead of one per tensor.  The packed streams are the
 * tensors' streams one after the other (rows of tensor i from seg_first_row[i] on; n = all rows);
 * every tensor keeps its own dither counters (seg_block_offset[i], seg_seed[i]), so each output
 * column has the operands nq_w4a4_gemm uses for its tensor alone (identical on the CUDA-core path;
 * on the tensor-core path the split of K follows the tile count, i.e. the order of the sums may differ).  segments in [1, 4]; the three
 * tables are host arrays read during the call.  The reference launches each projection on its own
 * (runtime/cuda_w4a4_mma.py:230-484): no counterpart there. */
int nq_w4a4_gemm_grouped(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                         const float* act_betas, const void* act_decoded,
                         const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                         const float* w_betas, int64_t m, int64_t n, int64_t k, int segments,
                         const int64_t* seg_first_row, const int64_t* seg_block_offset,
                         const int64_t* seg_seed, void* out, int out_dtype,
                         void* workspace, size_t workspace_bytes, nq_stream_t stream);

/* Small-M projection for callers that cannot allocate or pass a workspace (a plugin slot that
 * only receives inputs and outputs, a thread that must never reach cudaMalloc): same result as
 * nq_w4a4_gemm for m <= NQ_STATIC_MAX_M, but the scratch (decoded activation rows, split-K
 * partial sums, arrival counters) is a fixed array inside the library's device image, about
 * 8.6 MiB held by every GPU that loads the library until the process exits.  Shapes beyond
 * the limits below are rejected with NQ_ERR_ARG.  The first call on a device resolves the
 * array's address for the CURRENT device, which must be the device of `stream` (do it during
 * set-up, before any stream capture).  All calls share the one array: calls that overlap on the
 * GPU race on it.  Allocates nothing.
 * This entry point has no counterpart in the reference. */
#define NQ_STATIC_MAX_M 16
#define NQ_STATIC_MAX_N 8192
#define NQ_STATIC_MAX_K 8192
int nq_w4a4_gemv_static(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                        const float* act_betas, const uint8_t* w_codes, const uint8_t* w_beta_ids,
                        const float* w_norms, const float* w_betas, int64_t m, int64_t n, int64_t k,
                        int64_t w_block_offset, int64_t seed, void* out, int out_dtype, nq_stream_t stream);

/* The tcgen05 GEMM of the large-M path alone: out[m,n] = A[m,k] * W[n,k]^T on
 * BF16 row-major operands that were already decoded (nq_a4_encode's
 * out_decoded / nq_w4_decode).  Building block exposed for measurement and
 * tests; the reference has no counterpart (its large-M kernel decodes in the
 * MMA loop, runtime/nqrt4_w4a4_mma.cu:606-723).  workspace as for nq_w4a4_gemm
 * (only the status word is used).  Requires n % 128 == 0, k % 64 == 0. */
int nq_bf16_gemm_tc(const void* a_bf16, const void* w_bf16, int64_t m, int64_t n, int64_t k,
                    void* out, int out_dtype, void* workspace, size_t workspace_bytes, nq_stream_t stream);

/* Copy the device status word of a workspace to the host and synchronise the
 * stream (the only entry point that synchronises).  Non-zero means a bounded
 * wait inside the tcgen05 kernel gave up: 1 = producer waiting for a free
 * stage, 2 = MMA waiting for a free accumulator, 3 = MMA waiting for a TMA
 * stage, 4 = epilogue waiting for the accumulator, 5 = (nq_w4a4_gemm_fused) producer
 * waiting for the decode warps to finish a channel tile of the weight.  No counterpart in the
 * reference (its kernels have no device-side waits). */
int nq_w4a4_status(const void* workspace, uint32_t* status_host, nq_stream_t stream);

/* Decode a packed NQRT4 weight to bf16 [n,k] (dither regenerated on the fly);
 * bit-identical to bf16(QuantizedRows.dequantize) of the record
 * (core/quantizer.py:39-51, dither core/codec.py:176-224).  Used by the
 * large-M path and by parity tests. */
int nq_w4_decode(const uint8_t* w_codes, const uint8_t* w_beta_ids, const float* w_norms,
                 const float* w_betas, int64_t n, int64_t k, int64_t w_block_offset,
                 int64_t seed, void* out_bf16, nq_stream_t stream);

/* The projection on a weight that the caller keeps DECODED in device memory (w_decoded = the
 * bf16 [n,k] output of nq_w4_decode, 4x the packed bytes): an opt-in trade of HBM capacity for
 * time.  The operands are exactly the values nq_w4a4_gemm regenerates on every call, so the
 * result agrees with it up to the order of the FP32 sums; m < 5 runs a streaming GEMV bound by
 * HBM (one warp per output channel), larger m the tcgen05 GEMM without the per-call weight
 * decode.  Activation arguments, out, out_dtype and the zero-initialised workspace (size from
 * nq_w4a4_resident_workspace_bytes) as for nq_w4a4_gemm.  The reference never keeps a decoded
 * weight (models/fused_linear.py:130-137 states that as the module's purpose): no counterpart. */
size_t nq_w4a4_resident_workspace_bytes(int64_t m, int64_t n, int64_t k);
int nq_w4a4_gemm_resident(const uint8_t* act_codes, const uint8_t* act_beta_ids, const float* act_norms,
                          const float* act_betas, const void* act_decoded, const void* w_decoded,
                          int64_t m, int64_t n, int64_t k, void* out, int out_dtype,
                          void* workspace, size_t workspace_bytes, nq_stream_t stream);

/* -------------------------------------------------------------------------
 * NQKV4 paged cache.  Device data model (unchanged from the reference):
 *   pool   key_codes/value_codes u8[capacity, P*H*D/2], key_betas/value_betas u8[capacity, P*H*D/32],
 *          key_norms/value_norms f32[capacity, P*H]            (runtime/nqkv_pool.py:100-110)
 *   tables page_indices i32[S, max_pages] (-1 = empty), page_counts, last_page_lens, hot_lengths,
 *          sequence_lengths i32[S], cache_active bool[S]        (runtime/paged_nqkv_cache.py:26-79)
 *   hot    hot_keys/hot_values [S, P, H, D] in the KV dtype, target_page_ids i32[S]
 *                                                               (runtime/nqkv_hot_cache.py:22-35)
 * S = max_sequences, P = page_size, H = kv heads, D = head_dim (multiple of 32).
 * Masks are 1-byte booleans.
 *
 * nq_kv_append: write new K/V tokens into the hot tail and bump hot/sequence lengths, one launch.
 *   mode 0  one token per row, key/value [B, H, D], mask = active_mask[B]
 *           (_launch_append_hot_k1_graph_safe, runtime/nqkv_graph_writer.py:291-332)
 *   mode 1  key/value [B, T, H, D], mask = prefix write_mask[B, T]  (:373-419)
 *   mode 2  key/value [B, T, H, D], per-row (source_starts, segment_counts)  (:422-473)
 * Active slot ids must be unique (the reference's control plane guarantees it).
 * key_row_stride / value_row_stride: elements between the batch rows b and b + 1 of key / value, 0 = dense
 * (T * H * D); a row itself is contiguous.  With a stride the V rows of a stacked q/k/v projection result are
 * read where they are. */
int nq_kv_append(const void* key, const void* value, int kv_dtype, int batch, int tokens, int mode,
                 const int32_t* slot_ids, const uint8_t* mask, const int32_t* source_starts,
                 const int32_t* segment_counts, const uint8_t* cache_active, void* hot_keys,
                 void* hot_values, int32_t* hot_lengths, int32_t* sequence_lengths, int max_sequences,
                 int page_size, int heads, int dim, int64_t key_row_stride, int64_t value_row_stride,
                 nq_stream_t stream);

/* For every slot with boundary_mask[s] && hot_lengths[s] == P: encode its hot page, store the six
 * payload rows at pool[target_page_ids[s]], append the page id to the page table, set
 * last_page_lens = P and hot_lengths = 0.  A slot whose page table is full (page_counts ==
 * max_pages) or whose target id lies outside [0, pool_capacity) is left untouched: nothing is
 * written to the pool and nothing is published, its hot tail stays full.  Only the selected slots
 * are encoded.  target_page_ids may be null for a pool that is a fixed partition of max_pages pages
 * per slot: slot s then packs into page s * max_pages + page_counts[s] (no id array to refresh per
 * step).  Payload bytes equal PackedNQKVPage.from_tensors
 * (core/kv_format.py:71-131).  Replaces launch_pack_full_hot_pages_graph_safe
 * (runtime/nqkv_graph_pack.py:76-135: encode of all slots + 6 copies + publish). */
int nq_kv_pack_publish(const void* hot_keys, const void* hot_values, int kv_dtype, int32_t* hot_lengths,
                       const uint8_t* boundary_mask, const int32_t* target_page_ids,
                       uint8_t* key_codes, uint8_t* key_betas, float* key_norms, uint8_t* value_codes,
                       uint8_t* value_betas, float* value_norms, const float* key_beta_table,
                       const float* value_beta_table, int32_t* page_indices, int32_t* page_counts,
                       int32_t* last_page_lens, int max_sequences, int max_pages, int pool_capacity,
                       int page_size, int heads, int dim, nq_stream_t stream);

/* Device-side page allocation.  The free pages of a pool are a stack in device memory, free_ids[0 .. *free_count),
 * that kernels pop and push in stream order, so a decode step needs no host read of the hot lengths and no host
 * reservation, and the pool need not be a fixed partition of max_pages per slot.  The reference allocates on the
 * host and reads hot_lengths every step (runtime/nqkv_batched_runner.py:344-359); its notes sketch a device-side
 * scheme without building it (docs/nqkv_gpu_page_ring_research.md:148-186): no counterpart.
 *   nq_kv_alloc_targets  before nq_kv_pack_publish: writes target_page_ids[s] = a popped page for every slot that
 *                        will pack (boundary_mask[s], hot_lengths[s] == P, page_counts[s] < max_pages), -1 for the
 *                        others and when the stack is empty (such a slot is then not packed);
 *   nq_kv_alloc_pages    pops `count` pages into out_ids (bulk writers; -1 where the stack ran dry);
 *   nq_kv_release_pages  pushes the pages of the slots selected by slot_mask back, sets their page-table rows to -1
 *                        and their page_counts / last_page_lens / hot_lengths / sequence_lengths to 0.
 * The host's admission control must keep the sum of the admitted requests' maximum page counts within the pool. */
int nq_kv_alloc_targets(const int32_t* hot_lengths, const uint8_t* boundary_mask, const int32_t* page_counts,
                        const int32_t* free_ids, int32_t* free_count, int32_t* target_page_ids,
                        int max_sequences, int max_pages, int page_size, nq_stream_t stream);
int nq_kv_alloc_pages(int count, const int32_t* free_ids, int32_t* free_count, int32_t* out_ids, nq_stream_t stream);
int nq_kv_release_pages(const uint8_t* slot_mask, int32_t* page_indices, int32_t* page_counts,
                        int32_t* last_page_lens, int32_t* hot_lengths, int32_t* sequence_lengths,
                        int32_t* free_ids, int32_t* free_count, int max_sequences, int max_pages,
                        int pool_capacity, nq_stream_t stream);

/* Quantise and bit-pack one NHD page prefix key/value [valid_tokens, H, D] (rows after the prefix
 * are zero) into six caller-provided payload buffers of one page.  Replaces
 * quantize_nqkv_page_cuda (runtime/nqkv_page.py:241-329). */
int nq_kv_quantize_page(const void* key, const void* value, int kv_dtype, int valid_tokens, int page_size,
                        int heads, int dim, const float* key_beta_table, const float* value_beta_table,
                        uint8_t* key_codes, uint8_t* key_betas, float* key_norms, uint8_t* value_codes,
                        uint8_t* value_betas, float* value_norms, nq_stream_t stream);

/* Paged GQA attention over NQKV4 pages plus the BF16 hot tail.
 *   query  [B, Tq, Hq, D]; out [B, Tq, Hq, D] (NQ_BF16 or NQ_F32); rows that are inactive are zero.
 *   decode q_lens = NULL, Tq = 1: every active row attends to its whole sequence
 *          (nqkv_decode_attention_batched_k1, runtime/nqkv_attention_k1.py:763-942; no 127-page cap)
 *   prefill q_lens[b] <= Tq new tokens per row whose K/V are already appended: query i attends to
 *          the first  total - q_lens[b] + i + 1  tokens (causal), reading pages directly
 *          (semantic of NQKVLlamaCache.prefill, runtime/nqkv_hf_backend.py:127-150).
 * K/V of cold pages are the float32 reconstruction; softmax and accumulation in float32.
 * The hot tail (hot_keys / hot_values) is read as BF16 whatever dtype the pages were packed from.
 * workspace: nq_kv_attention_workspace_bytes(...) bytes (split partials).
 * The pages are decoded through a 106-entry table that the library keeps in a fixed array of
 * its own image (no allocation): the FIRST call on a device fills it with a one-CTA kernel on
 * `stream` and waits for that kernel once; while `stream` is being captured the fill is
 * recorded into the graph instead. */
size_t nq_kv_attention_workspace_bytes(int batch, int q_tokens, int q_heads, int kv_heads, int dim, int max_pages);
int nq_kv_attention(const void* query, int q_dtype, int batch, int q_tokens, int q_heads,
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
                    nq_stream_t stream);

/* Decoded shadow of the page pool ("lattice pages"), an opt-in trade of HBM for attention time.
 * Decoding a K/V block (a nearest-point search in E8) is a pure function of its 32-bit codeword, and
 * the paged attention above is bound by those searches, not by HBM.  A caller with memory to spare
 * keeps, beside each code stream, key_lattice / value_lattice int8[capacity, P*H*D]: the eight
 * minimum-energy coordinates of every block, doubled (half-integers in [-14, 14] -> [-28, 28]);
 * 8 bits per entry beside the 4.25 of the page itself.  The NQKV4 streams stay the record (and what
 * is compared with the reference); the shadow is derived from them on the device:
 *   nq_kv_expand_pages         shadow of the listed pages of ONE code stream (page_ids[i] < 0 skipped),
 *                              for eager writers and for converting a pool that is already filled;
 *   nq_kv_pack_publish_lattice nq_kv_pack_publish that also writes the shadow of the pages it publishes;
 *   nq_kv_attention_lattice    nq_kv_attention reading the shadow instead of searching: the same
 *                              coordinates enter the same float32 arithmetic, so the output is
 *                              bit-identical to nq_kv_attention.
 * The reference always decodes in the attention kernel (runtime/nqkv_attention_k1.py:50-81): no counterpart. */
int nq_kv_expand_pages(const uint8_t* codes, int8_t* lattice, const int32_t* page_ids, int64_t count,
                       int pool_capacity, int page_size, int heads, int dim, nq_stream_t stream);
int nq_kv_pack_publish_lattice(const void* hot_keys, const void* hot_values, int kv_dtype,
                               int32_t* hot_lengths, const uint8_t* boundary_mask,
                               const int32_t* target_page_ids, uint8_t* key_codes, uint8_t* key_betas,
                               float* key_norms, uint8_t* value_codes, uint8_t* value_betas,
                               float* value_norms, const float* key_beta_table,
                               const float* value_beta_table, int32_t* page_indices, int32_t* page_counts,
                               int32_t* last_page_lens, int max_sequences, int max_pages,
                               int pool_capacity, int page_size, int heads, int dim, int8_t* key_lattice,
                               int8_t* value_lattice, nq_stream_t stream);
int nq_kv_attention_lattice(const void* query, int q_dtype, int batch, int q_tokens, int q_heads,
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
                            const int8_t* value_lattice, nq_stream_t stream);

/* -------------------------------------------------------------------------
 * Normalised Sylvester Hadamard along the last axis of a contiguous [rows, n]
 * tensor, n a power of two in [8, 32768], computed in the tensor's dtype exactly as
 * hadamard() does (core/rotation.py:12-27): every butterfly stage rounded to
 * the dtype, final IEEE division by float32(sqrt(n)).  x may equal out. */
int nq_hadamard(const void* x, void* out, int dtype, int64_t rows, int64_t n, nq_stream_t stream);

/* hadamard(silu(gate) * up) in one launch: the rotated input of a Llama down_proj
 * (models/fused_linear.py:287-290 applied to the MLP's `act_fn(gate_proj(x)) * up_proj(x)`) for rows too long
 * for nq_a4_encode_silu_mul_rotated.  gate and up are [rows, n] tensors of `dtype` whose rows lie row_stride
 * elements apart (column ranges of one stacked gate/up result need no copy), out is contiguous [rows, n]; the
 * product is formed with the tensor ops' arithmetic (x / (1 + exp(-x)) in float32 rounded to the dtype, then
 * the product rounded to the dtype), so the result equals nq_hadamard of that product bit for bit. */
int nq_hadamard_silu_mul(const void* gate, const void* up, int64_t row_stride, void* out, int dtype, int64_t rows,
                         int64_t n, nq_stream_t stream);

/* Rotary position embedding of query or key heads and, with apply_hadamard != 0, the float32
 * Hadamard rotation the KV backend applies to them afterwards, in one launch:
 *   rope     (x * cos) + (rotate_half(x) * sin), every product and the sum rounded to `dtype`
 *            (the model's apply_rotary_pos_emb on tensors of that dtype)
 *   rotation dtype(hadamard(float32(rope)))   (runtime/nqkv_batched_hf_backend.py:381,549)
 * Result for result identical to that sequence of tensor ops.  The reference leaves the rope to the
 * model and runs the rotation as tensor ops: no counterpart there.
 *   x    [batch, heads, tokens, dim] with element strides stride_b/h/t and unit stride along dim
 *   cos, sin [batch, tokens, dim] contiguous;  out [batch, heads, tokens, dim] contiguous
 *   dim a power of two in [16, 1024]; pointers and strides 16-byte aligned. */
int nq_rope_hadamard(const void* x, int dtype, int64_t batch, int64_t heads, int64_t tokens, int64_t dim,
                     int64_t stride_b, int64_t stride_h, int64_t stride_t, const void* cos, const void* sin,
                     int apply_hadamard, void* out, nq_stream_t stream);

/* The same for the query heads and the key heads of one attention layer in ONE launch: q [B, Hq, T, D] and
 * k [B, Hk, T, D] of one dtype with their own element strides ({batch, head, token}, 16-byte multiples) and
 * their own contiguous outputs; cos / sin [B, T, D] are shared. */
int nq_rope_hadamard_pair(const void* q, const void* k, int dtype, int64_t batch, int64_t q_heads, int64_t k_heads,
                          int64_t tokens, int64_t dim, const int64_t* q_strides, const int64_t* k_strides,
                          const void* cos, const void* sin, int apply_hadamard, void* q_out, void* k_out,
                          nq_stream_t stream);

/* RMS normalisation of rows as Hugging Face's LlamaRMSNorm computes it, in one launch:
 *   out = weight * dtype(x * rsqrt(mean(x^2) + eps))      (mean and product in float32)
 * It precedes every rotate-then-encode launch of a decoder layer; the reference leaves it to
 * the model's tensor ops, so there is no counterpart in the reference.  The sum of squares has
 * a fixed order of its own: deterministic, not bit-identical to the tensor-op reduction.
 *   x, out [rows, n] contiguous, weight [n], all of `dtype`; n % 8 == 0; 16-byte aligned. */
int nq_rmsnorm(const void* x, const void* weight, int dtype, int64_t rows, int64_t n, float eps, void* out,
               nq_stream_t stream);

/* -------------------------------------------------------------------------
 * Tensor-parallel sum of the ranks' partial projection outputs over peer memory (one node).
 * No counterpart in the reference (single GPU); replaces the NCCL all-reduce after o_proj /
 * down_proj of a tensor-parallel shard (one launch per rank, partials read over NVLink with
 * plain 16-byte loads, summed in rank order in float32 on every rank: identical results).
 *   partials_host  HOST array of `world` device pointers: every rank's BF16 partial [count]
 *                  as mapped in THIS process (symmetric / IPC memory); entry `rank` is local
 *   pads_host      HOST array of `world` device pointers: every rank's flag pad of
 *                  NQ_TP_PAD_BYTES bytes, mapped the same way, zeroed once before the first
 *                  call of the group (words 0..15 are written by the peers, 16..18 are local:
 *                  calls completed, CTA ticket, status: non-zero = a bounded wait gave up)
 *   out_bf16       local result [count]; count % 8 == 0
 * All ranks must issue the same sequence of calls with the same count; a rank's partial must
 * not be rewritten before ITS call has completed (stream order on the rank is enough: the
 * call returns only after every rank has finished reading).  world <= NQ_TP_MAX_RANKS. */
#define NQ_TP_MAX_RANKS 8
#define NQ_TP_PAD_BYTES 128
int nq_tp_allreduce_bf16(const void* const* partials_host, void* const* pads_host, int rank, int world,
                         void* out_bf16, int64_t count, nq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NQ_B200_H */
