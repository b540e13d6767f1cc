"""GPU parity of the A4 encoder, the packed decode and the W4A4 projection (through the C ABI).

Bit-exact gates: packed code / beta-id streams and row norms against the CPU
checker and the committed reference vectors.  Tolerance gates (projection):
max abs <= 1e-2 and relative Frobenius <= 1e-3 against the product of the
BF16-rounded dequantised operands accumulated in float64.
"""

import numpy as np
import pytest
import torch

from helpers import (ACT_BETAS, KEY_BETAS, MAX_ABS_TOL, REL_FRO_TOL, UNIT_BETAS, W_BETAS, make_weight_record,
                     max_abs, rel_fro, rng)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import nestquant_aiinfra_b200.runtime as runtime

    return runtime


def _encode(rt, x: torch.Tensor, betas):
    act = rt.quantize_activation_cuda(x.cuda(), q=14, betas=betas, keep_decoded=True)
    torch.cuda.synchronize()
    return act


@pytest.mark.parametrize("name,betas", [("a4_2048", ACT_BETAS), ("a4_8192_bf16", ACT_BETAS), ("kv_64_bf16", KEY_BETAS),
                                        ("unit_betas_256", UNIT_BETAS), ("zero_row_64", KEY_BETAS)])
def test_encoder_matches_reference_vectors(rt, golden, name, betas):
    x = torch.from_numpy(golden[f"{name}_x"])
    if name.endswith("bf16"):
        x = x.bfloat16()
    act = _encode(rt, x, betas)
    assert np.array_equal(act.code_payload.cpu().numpy(), golden[f"{name}_codes"])
    assert np.array_equal(act.beta_payload.cpu().numpy(), golden[f"{name}_beta_ids"])
    assert np.array_equal(act.row_norms.cpu().numpy(), golden[f"{name}_norms"])
    decoded = rt.decode_packed_a4(act, dtype=torch.float32).cpu().numpy()
    assert np.array_equal(decoded, golden[f"{name}_dequant"])
    # the BF16 reconstruction emitted by the encoder itself is the rounded decode
    assert torch.equal(act.decoded.cpu(), torch.from_numpy(golden[f"{name}_dequant"]).bfloat16())


@pytest.mark.parametrize("rows,k,dtype", [(1, 2048, torch.bfloat16), (17, 2048, torch.bfloat16), (128, 8192, torch.bfloat16),
                                          (1000, 64, torch.bfloat16), (33, 128, torch.float16), (16, 2048, torch.float32),
                                          (300, 32, torch.float32), (5, 3584, torch.bfloat16)])
def test_encoder_bit_exact_against_checker(rt, oracle, rows, k, dtype):
    x = (torch.randn(rows, k, generator=rng(rows * 7 + k)) * 1.7).to(dtype)
    act = _encode(rt, x, ACT_BETAS)
    codes, beta_ids, norms = oracle.encode_packed(x.float().numpy(), ACT_BETAS)
    mism = int((act.code_payload.cpu().numpy() != codes).sum())
    assert mism == 0, f"{mism} code bytes differ"
    assert np.array_equal(act.beta_payload.cpu().numpy(), beta_ids)
    assert np.array_equal(act.row_norms.cpu().numpy(), norms)


def test_encoder_strided_rows_and_leading_dims(rt, oracle):
    base = torch.randn(4, 6, 4096, generator=rng(5)).bfloat16().cuda()
    view = base[..., :2048]  # row stride 4096, 16-byte aligned
    act = rt.quantize_activation_cuda(view, q=14, betas=ACT_BETAS)
    codes, beta_ids, norms = oracle.encode_packed(view.float().cpu().reshape(-1, 2048).numpy(), ACT_BETAS)
    assert act.original_shape == (4, 6, 2048) and act.token_count == 24
    assert np.array_equal(act.code_payload.cpu().numpy(), codes)
    assert np.array_equal(act.row_norms.cpu().numpy(), norms)


@pytest.mark.parametrize("rows,k,block,dtype", [
    (1, 2048, 2048, torch.bfloat16), (5, 8192, 8192, torch.bfloat16), (64, 2048, 2048, torch.bfloat16),
    (3000, 2048, 2048, torch.bfloat16), (300, 64, 64, torch.float32), (33, 4096, 4096, torch.float16),
    (16, 14336, 2048, torch.bfloat16), (7, 3584, 512, torch.bfloat16), (2, 16384, 16384, torch.float32)])
def test_rotation_inside_the_encoder_equals_two_launches(rt, rows, k, block, dtype):
    """nq_a4_encode_rotated == nq_hadamard then nq_a4_encode, bit for bit (whole-row and block-diagonal rotation)."""
    from nestquant_aiinfra_b200.rotation import hadamard

    x = torch.randn(rows, k, generator=rng(600 + rows)).to(dtype).cuda()
    rotated = hadamard(x.reshape(rows, k // block, block)).reshape(rows, k)
    two = rt.quantize_activation_cuda(rotated, q=14, betas=ACT_BETAS, keep_decoded=True)
    one = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, hadamard_block=block, keep_decoded=True)
    torch.cuda.synchronize()
    assert torch.equal(one.code_payload, two.code_payload) and torch.equal(one.beta_payload, two.beta_payload)
    assert torch.equal(one.row_norms, two.row_norms) and torch.equal(one.decoded, two.decoded)


def test_rotation_inside_the_encoder_argument_errors(rt):
    x = torch.zeros(4, 2048, dtype=torch.bfloat16, device="cuda")
    assert rt.can_rotate_in_encoder(2048, 2048) and rt.can_rotate_in_encoder(14336, 2048)
    assert not rt.can_rotate_in_encoder(32768, 32768) and not rt.can_rotate_in_encoder(2048, 96)
    with pytest.raises(ValueError):
        rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, hadamard_block=96)
    with pytest.raises(ValueError):
        rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, hadamard_block=4096)


def test_activation_decoder_boundary_codewords_exact(rt, oracle):
    # mirrors reference tests/unit/runtime/test_cuda_w4a4_mma.py:78-97
    k = 32
    codes = np.zeros((16, k // 8, 8), dtype=np.uint8)
    codes[0, 0] = [5, 12, 3, 0, 7, 3, 9, 2]
    codes[5, 1] = [5, 5, 2, 7, 2, 4, 10, 2]
    codes[10, 2] = [3, 0, 2, 12, 4, 9, 7, 2]
    act = rt.PreparedNQA4Activation(
        code_payload=torch.from_numpy(oracle.pack(codes, 4)).cuda(),
        beta_payload=torch.zeros(16 * k // 32, dtype=torch.uint8, device="cuda"),
        row_norms=torch.ones(16, dtype=torch.float32, device="cuda"),
        beta_table=torch.tensor(UNIT_BETAS, dtype=torch.float32, device="cuda"),
        original_shape=(16, k), q=14, code_width=4, beta_width=2, output_dtype=torch.bfloat16)
    actual = rt.decode_packed_a4_m16(act)
    expected = oracle.dequantize_rows(oracle.pack(codes, 4), np.zeros(16 * k // 32, np.uint8), np.ones(16, np.float32),
                                      UNIT_BETAS, 16, k)
    assert torch.equal(actual.cpu(), torch.from_numpy(expected).bfloat16())


def test_weight_decode_bit_exact(rt, oracle):
    record, deq = make_weight_record(oracle, 64, 512, seed=1000, dither_seed=20261029)
    weight = rt.prepare_fused_linear(record)
    got = rt.decode_packed_weight(weight).cpu()
    assert torch.equal(got, torch.from_numpy(deq).bfloat16())


@pytest.mark.parametrize("n,k,dtype", [(96, 512, torch.float32), (64, 2048, torch.float32), (40, 8192, torch.bfloat16)])
def test_weight_encoder_bit_exact(rt, oracle, golden, n, k, dtype):
    if (n, k) == (96, 512):
        w = torch.from_numpy(golden["w_x"])
    else:
        w = torch.from_numpy(oracle.hadamard((0.02 * torch.randn(n, k, generator=rng(n + k))).numpy())).to(dtype)
    seed = int(golden["dither_seed"][0])
    prepared = rt.quantize_weight_cuda(w.cuda(), betas=W_BETAS, dither_seed=seed)
    codes, beta_ids, norms = oracle.encode_packed(w.float().numpy(), W_BETAS, seed=seed)
    assert np.array_equal(prepared.code_payload.cpu().numpy(), codes)
    assert np.array_equal(prepared.beta_payload.cpu().numpy(), beta_ids)
    assert np.array_equal(prepared.row_norms.cpu().numpy(), norms)
    if (n, k) == (96, 512):
        assert np.array_equal(codes, golden["w_codes"]) and np.array_equal(beta_ids, golden["w_beta_ids"])
    deq = oracle.dequantize_rows(codes, beta_ids, norms, W_BETAS, n, k, seed=seed)
    assert torch.equal(rt.decode_packed_weight(prepared).cpu(), torch.from_numpy(deq).bfloat16())


SHAPES = [(64, 256), (512, 2048), (2048, 2048), (256, 8192), (96, 96 * 32)]


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 13, 16, 17, 40])
@pytest.mark.parametrize("n,k", SHAPES[:3])
def test_projection_small_shapes(rt, oracle, m, n, k):
    _projection_case(rt, oracle, m, n, k)


@pytest.mark.parametrize("m,n,k", [(1, 256, 8192), (16, 256, 8192), (1, 96, 4096), (64, 512, 2048), (128, 2048, 2048),
                                   (200, 512, 2048), (512, 512, 2048), (384, 256, 8192)])
def test_projection_more_shapes(rt, oracle, m, n, k):
    _projection_case(rt, oracle, m, n, k)


def _projection_case(rt, oracle, m, n, k):
    record, w_deq = make_weight_record(oracle, n, k, seed=1000 + n + k, dither_seed=777 + n)
    weight = rt.prepare_fused_linear(record)
    x = torch.from_numpy(oracle.hadamard(torch.randn(m, k, generator=rng(2000 + m)).bfloat16().float().numpy(),
                                          round_bf16=True)).bfloat16()
    act = rt.quantize_activation_cuda(x.cuda(), q=14, betas=ACT_BETAS)
    ac, ab, an = oracle.encode_packed(x.float().numpy(), ACT_BETAS)
    assert np.array_equal(act.code_payload.cpu().numpy(), ac)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
    expected = oracle.gemm_bf16_operands(a_deq, w_deq)
    actual = rt.linear_packed_w4a4_fp32(act, weight).cpu().numpy()
    assert actual.shape == (m, n)
    assert rt.read_status() == 0
    assert max_abs(actual, expected) <= MAX_ABS_TOL, (max_abs(actual, expected), rel_fro(actual, expected))
    assert rel_fro(actual, expected) <= REL_FRO_TOL, rel_fro(actual, expected)
    # same result when the kernel decodes the packed activation itself
    from dataclasses import replace
    again = rt.linear_packed_w4a4_fp32(replace(act, decoded=None), weight).cpu().numpy()
    assert np.array_equal(again, actual)
    # output-dtype path: bf16 rounding of the same accumulator
    out = rt.linear_packed_w4a4(act, weight)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n)
    assert torch.equal(out.cpu(), torch.from_numpy(actual).bfloat16())


def test_projection_is_deterministic_and_leaves_counters_zero(rt, oracle):
    record, _ = make_weight_record(oracle, 256, 8192, seed=5, dither_seed=9)
    weight = rt.prepare_fused_linear(record)
    x = torch.randn(2, 8192, generator=rng(1)).bfloat16().cuda()
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
    first = rt.linear_packed_w4a4_fp32(act, weight)
    for _ in range(3):
        assert torch.equal(rt.linear_packed_w4a4_fp32(act, weight), first)
    ws = rt.workspace_for(x.device, 1)
    torch.cuda.synchronize()
    assert int(ws[:65536].count_nonzero()) == 0


def test_regime_entry_points_and_errors(rt, oracle):
    record, _ = make_weight_record(oracle, 64, 256, seed=3, dither_seed=4)
    weight = rt.prepare_fused_linear(record)
    x = torch.randn(1, 256, generator=rng(2)).bfloat16().cuda()
    act1 = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
    act2 = rt.quantize_activation_cuda(x.repeat(2, 1), q=14, betas=ACT_BETAS)
    assert rt.can_use_w4a4_gemv_m1(act1, weight) and not rt.can_use_w4a4_gemv_m1(act2, weight)
    y1 = rt.linear_packed_w4a4_gemv_m1(act1, weight)
    y2 = rt.linear_packed_w4a4_mma_small_m(act2, weight)
    assert torch.equal(y2[0], y1[0]) and torch.equal(y2[1], y1[0])
    with pytest.raises(ValueError):
        rt.linear_packed_w4a4_gemv_m1(act2, weight)
    with pytest.raises(TypeError):
        rt.linear_packed_w4a4(x, weight)
    bad = rt.quantize_activation_cuda(torch.randn(1, 512).bfloat16().cuda(), q=14, betas=ACT_BETAS)
    with pytest.raises(ValueError):
        rt.linear_packed_w4a4(bad, weight)
    with pytest.raises(ValueError):
        rt.quantize_activation_cuda(torch.randn(1, 40).cuda(), q=14, betas=ACT_BETAS)


@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (2, 512, 2048), (3, 256, 8192), (4, 96, 4096), (5, 256, 2048),
                                   (7, 96, 4096), (9, 512, 2048), (64, 2048, 2048), (300, 512, 2048)])
def test_resident_decoded_weight_projection(rt, oracle, m, n, k):
    """Opt-in mode: the decoded BF16 weight stays in device memory; same operands, so the same parity gate."""
    record, w_deq = make_weight_record(oracle, n, k, seed=1500 + n + k, dither_seed=321 + n)
    packed = rt.prepare_fused_linear(record)
    weight = rt.keep_decoded_weight(packed)
    assert weight.decoded is not None and tuple(weight.decoded.shape) == (n, k)
    assert torch.equal(weight.decoded.cpu(), torch.from_numpy(w_deq).bfloat16())
    assert rt.keep_decoded_weight(weight) is weight
    x = torch.randn(m, k, generator=rng(2500 + m)).bfloat16()
    act = rt.quantize_activation_cuda(x.cuda(), q=14, betas=ACT_BETAS)
    ac, ab, an = oracle.encode_packed(x.float().numpy(), ACT_BETAS)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
    expected = oracle.gemm_bf16_operands(a_deq, w_deq)
    actual = rt.linear_packed_w4a4_fp32(act, weight).cpu().numpy()
    assert actual.shape == (m, n) and rt.read_status() == 0
    assert max_abs(actual, expected) <= MAX_ABS_TOL, (max_abs(actual, expected), rel_fro(actual, expected))
    assert rel_fro(actual, expected) <= REL_FRO_TOL, rel_fro(actual, expected)
    # deterministic, and the packed path (which regenerates the same operands) agrees to summation order
    assert np.array_equal(rt.linear_packed_w4a4_fp32(act, weight).cpu().numpy(), actual)
    per_call = rt.linear_packed_w4a4_fp32(act, packed).cpu().numpy()
    assert rel_fro(actual, per_call) <= 1e-5
    # the kernel can decode the packed activation itself
    from dataclasses import replace
    again = rt.linear_packed_w4a4_fp32(replace(act, decoded=None), weight).cpu().numpy()
    assert np.array_equal(again, actual)
    out = rt.linear_packed_w4a4(act, weight)
    assert out.dtype == torch.bfloat16 and torch.equal(out.cpu(), torch.from_numpy(actual).bfloat16())


def test_resident_decoded_weight_argument_errors(rt, oracle):
    import ctypes

    from nestquant_aiinfra_b200 import _lib

    library = _lib.lib()
    assert library.nq_w4a4_resident_workspace_bytes(ctypes.c_int64(0), ctypes.c_int64(64), ctypes.c_int64(256)) == 0
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    null = ctypes.c_void_p(0)
    args = [null, null, null, null, ctypes.c_void_p(buf.data_ptr()), null, ctypes.c_int64(1), ctypes.c_int64(64),
            ctypes.c_int64(256), ctypes.c_void_p(buf.data_ptr()), ctypes.c_int(0), ctypes.c_void_p(buf.data_ptr()),
            ctypes.c_size_t(buf.numel()), null]
    assert library.nq_w4a4_gemm_resident(*args) < 0      # no decoded weight
    args[5] = ctypes.c_void_p(buf.data_ptr())
    args[8] = ctypes.c_int64(250)
    assert library.nq_w4a4_gemm_resident(*args) < 0      # k not a multiple of 32
    args[8] = ctypes.c_int64(256)
    args[12] = ctypes.c_size_t(16)
    assert library.nq_w4a4_gemm_resident(*args) < 0      # workspace too small
    record, _ = make_weight_record(oracle, 64, 256, seed=3, dither_seed=4)
    with pytest.raises(TypeError):
        rt.keep_decoded_weight(record)



@pytest.mark.parametrize("m,n,k", [(8, 128, 64), (40, 512, 2048), (200, 256, 1024), (520, 2048, 2048), (1300, 1024, 512)])
def test_fused_decode_gemm_equals_the_two_launch_path(rt, oracle, m, n, k):
    """The kernel that decodes the weight beside its own MMAs (nq_w4a4_gemm_fused) and the default decode-then-GEMM
    pair run the same MMAs on the same decoded values: results must be identical bit for bit, the status word
    clean, and a second call on the same workspace (arrival counters back at zero) must reproduce the first."""
    record, w_deq = make_weight_record(oracle, n, k, seed=900 + m, dither_seed=1234 + m)
    weight = rt.prepare_fused_linear(record)
    x = torch.randn(m, k, generator=rng(77 + m)).bfloat16().cuda()
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, keep_decoded=True)
    fused = rt.linear_packed_w4a4_fused_fp32(act, weight)
    again = rt.linear_packed_w4a4_fused_fp32(act, weight)
    two_pass = rt.linear_packed_w4a4_fp32(act, weight)
    assert rt.read_status() == 0
    assert torch.equal(fused, again)
    assert torch.equal(fused, two_pass)
    codes, beta_ids, norms = (t.cpu().numpy() for t in (act.code_payload, act.beta_payload, act.row_norms))
    expected = oracle.gemm_bf16_operands(oracle.dequantize_rows(codes, beta_ids, norms, ACT_BETAS, m, k), w_deq)
    actual = fused.cpu().numpy()
    assert max_abs(actual, expected) <= MAX_ABS_TOL and rel_fro(actual, expected) <= REL_FRO_TOL


@pytest.mark.parametrize("rows,k,dtype", [(5, 2048, torch.bfloat16), (64, 2048, torch.bfloat16), (1, 4096, torch.bfloat16),
                                          (3, 8192, torch.bfloat16), (70, 8192, torch.bfloat16), (9, 1024, torch.float16),
                                          (4, 512, torch.float32)])
def test_producers_inside_the_encoder_equal_the_separate_launches(rt, rows, k, dtype):
    """RMS norm -> rotate -> encode and SiLU(gate) * up -> rotate -> encode as ONE launch each: the same streams,
    norms and reconstruction as the producer's own launch(es) followed by the rotate-and-encode launch."""
    from nestquant_aiinfra_b200.norm import rms_norm

    def same(one, two):
        assert torch.equal(one.code_payload, two.code_payload) and torch.equal(one.beta_payload, two.beta_payload)
        assert torch.equal(one.row_norms, two.row_norms) and torch.equal(one.decoded, two.decoded)

    x = (3.0 * torch.randn(rows, k, generator=rng(900 + rows))).to(dtype).cuda()
    weight = (1.0 + 0.1 * torch.randn(k, generator=rng(901))).to(dtype).cuda()
    one = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, hadamard_block=k, keep_decoded=True, rmsnorm=(weight, 1e-5))
    two = rt.quantize_activation_cuda(rms_norm(x, weight, 1e-5), q=14, betas=ACT_BETAS, hadamard_block=k, keep_decoded=True)
    same(one, two)
    # gate and up as the two column ranges of one stacked projection output (row stride 2k)
    stacked = torch.randn(rows, 2 * k, generator=rng(902 + rows)).to(dtype).cuda()
    gate, up = stacked[:, :k], stacked[:, k:]
    one = rt.quantize_activation_cuda(gate, q=14, betas=ACT_BETAS, hadamard_block=k, keep_decoded=True, silu_mul_with=up)
    two = rt.quantize_activation_cuda(torch.nn.functional.silu(gate) * up, q=14, betas=ACT_BETAS, hadamard_block=k,
                                      keep_decoded=True)
    same(one, two)
    with pytest.raises(ValueError):
        rt.quantize_activation_cuda(gate, q=14, betas=ACT_BETAS, silu_mul_with=up)             # needs hadamard_block
    with pytest.raises(ValueError):
        rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, hadamard_block=k, rmsnorm=(weight[:8], 1e-5))
