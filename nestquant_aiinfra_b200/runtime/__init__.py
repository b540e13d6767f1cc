"""Operator layer: the reference's ``nestquant.runtime`` names for the W4A4KV4 path."""

from .w4a4 import (  # noqa: F401
    PreparedNQA4Activation, PreparedNQRTLinear, prepare_fused_linear, quantize_activation_cuda, quantize_weight_cuda,
    can_use_w4a4, can_use_w4a4_gemv_m1, can_use_w4a4_mma_small_m, can_use_w4a4_mma_m16,
    can_use_w4a4_mma_large_m_staged, can_use_w4a4_mma_chunked_staged,
    linear_packed_w4a4, linear_packed_w4a4_fp32, linear_packed_w4a4_gemv_m1,
    linear_packed_w4a4_gemv_m1_fp32_probe, linear_packed_w4a4_mma_small_m, linear_packed_w4a4_mma_m16,
    linear_packed_w4a4_mma_large_m_staged, linear_packed_w4a4_mma_chunked_staged,
    decode_packed_a4, decode_packed_a4_m16, decode_packed_weight, workspace_for, read_status, gemm_bf16_tc, launch_count,
)
