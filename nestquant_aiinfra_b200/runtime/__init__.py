"""Operator layer: the reference's ``nestquant.runtime`` names for the W4A4KV4 path."""

from .w4a4 import (  # noqa: F401
    PreparedNQA4Activation, PreparedNQRTLinear, prepare_fused_linear, quantize_activation_cuda, quantize_weight_cuda, can_rotate_in_encoder, prefer_rotation_in_encoder, prefer_producer_in_encoder, group_prepared_linears,
    can_use_w4a4, can_use_w4a4_gemv_m1, can_use_w4a4_mma_small_m, can_use_w4a4_mma_m16,
    can_use_w4a4_mma_large_m_staged, can_use_w4a4_mma_chunked_staged,
    linear_packed_w4a4, linear_packed_w4a4_fp32, linear_packed_w4a4_fused_fp32, linear_packed_w4a4_gemv_m1,
    linear_packed_w4a4_gemv_m1_fp32_probe, linear_packed_w4a4_mma_small_m, linear_packed_w4a4_mma_m16,
    linear_packed_w4a4_mma_large_m_staged, linear_packed_w4a4_mma_chunked_staged,
    decode_packed_a4, decode_packed_a4_m16, decode_packed_weight, keep_decoded_weight, workspace_for, read_status, gemm_bf16_tc, launch_count,
)
from .kv import (  # noqa: F401,E402
    NQKVPagePool, NQKVHotColdCache, PreparedNQKVPage, quantize_nqkv_page_cuda,
    _launch_append_hot_k1_graph_safe, _launch_append_hot_ragged_subpage_graph_safe,
    _launch_append_hot_ragged_segment_graph_safe, append_hot_k1_graph_safe,
    launch_pack_full_hot_pages_graph_safe, BatchedNQKVAttentionWorkspace,
    nqkv_decode_attention_batched_k1, _launch_nqkv_decode_attention_batched_k1, nqkv_prefill_attention,
    cache_arrays,
)
