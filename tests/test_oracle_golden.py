"""The CPU checker against vectors produced by the reference's own CPU code.

These tests pin the restatement in oracle/nq_oracle.c; the GPU parity tests
then compare the CUDA kernels with the checker.
"""

import hashlib

import numpy as np
import pytest

from helpers import ACT_BETAS, KEY_BETAS, VALUE_BETAS, W_BETAS

ENCODE_CASES = ["a4_2048", "a4_8192_bf16", "kv_64_bf16", "kv_128_bf16", "unit_betas_256", "zero_row_64"]


def test_nearest_e8_matches_reference_including_ties(oracle, golden):
    assert np.array_equal(oracle.nearest_e8(golden["e8_in"]), golden["e8_out"])


def test_tie_goes_to_half_integer_coset(oracle):
    # reference tests/unit/core/test_lattice.py:29-52: equal distance -> half coset
    x = np.array([[0.25] * 8], dtype=np.float32)
    assert np.array_equal(oracle.nearest_e8(x), np.full((1, 8), 0.5, dtype=np.float32))


def test_stateless_dither_known_answers(oracle, golden):
    seed = int(golden["dither_seed"][0])
    assert list(oracle.lcg31_hash(0, 8, seed)) == [542997489, 1008614140, 626638871, 764041742,
                                                    232696865, 790416531, 975085482, 1139066079]
    assert np.array_equal(oracle.dither(0, 64, seed), golden["dither_blocks_0_64"])
    assert np.array_equal(oracle.dither(1_000_003, 32, 12345), golden["dither_blocks_off"])


def test_decode_nested_boundary_codewords(oracle, golden):
    out = oracle.decode_nested(golden["decode_codes"])
    assert np.array_equal(out, golden["decode_out"])
    # the three boundary codewords of tests/unit/runtime/test_cuda_w4a4_mma.py:83-85
    assert out[0].tolist() == [6, 3, -3, 1, -2, 2, 3, 8]
    assert out[1].tolist() == [-1, -3, 3, -1, 6, 2, 4, 8]
    assert out[2].tolist() == [0, 6, -2, 2, 3, -4, 1, 8]


def test_packing_byte_order(oracle):
    # reference tests/unit/core/test_packing.py:18-53
    assert oracle.pack(np.array([1, 2, 3, 4], dtype=np.uint8), 4).tolist() == [0x21, 0x43]
    assert oracle.pack(np.array([0, 3, 0, 0], dtype=np.uint8), 2).tolist() == [0b00001100]
    assert oracle.pack(np.array([1, 0, 1], dtype=np.uint8), 1).tolist() == [0b101]
    values = np.arange(14, dtype=np.uint8)
    assert np.array_equal(oracle.unpack(oracle.pack(values, 4), 14, 4), values)


@pytest.mark.parametrize("name", ENCODE_CASES)
def test_row_encoder_bit_exact(oracle, golden, name):
    x, betas = golden[f"{name}_x"], golden[f"{name}_betas"]
    codes, beta_ids, norms = oracle.encode_packed(x, betas)
    assert np.array_equal(codes, golden[f"{name}_codes"])
    assert np.array_equal(beta_ids, golden[f"{name}_beta_ids"])
    assert np.array_equal(norms, golden[f"{name}_norms"])
    deq = oracle.dequantize_rows(codes, beta_ids, norms, betas, *x.shape)
    assert np.array_equal(deq, golden[f"{name}_dequant"])


def test_zero_row_stays_zero(oracle, golden):
    x = golden["zero_row_64_x"]
    codes, beta_ids, norms = oracle.encode_packed(x, KEY_BETAS)
    deq = oracle.dequantize_rows(codes, beta_ids, norms, KEY_BETAS, *x.shape)
    assert norms[2] == 0.0 and not deq[2].any()


def test_weight_encoder_with_dither_bit_exact(oracle, golden):
    x = golden["w_x"]
    seed = int(golden["dither_seed"][0])
    codes, beta_ids, norms = oracle.encode_packed(x, W_BETAS, seed=seed)
    assert np.array_equal(codes, golden["w_codes"])
    assert np.array_equal(beta_ids, golden["w_beta_ids"])
    assert np.array_equal(norms, golden["w_norms"])
    deq = oracle.dequantize_rows(codes, beta_ids, norms, W_BETAS, *x.shape, seed=seed)
    assert np.array_equal(deq, golden["w_dequant"])


def test_config0_product(oracle, golden):
    seed = int(golden["dither_seed"][0])
    a = golden["y_a_x"]
    ac, ab, an = oracle.encode_packed(a, ACT_BETAS)
    ad = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, *a.shape)
    wd = oracle.dequantize_rows(golden["w_codes"], golden["w_beta_ids"], golden["w_norms"], W_BETAS, 96, 512, seed=seed)
    y = oracle.gemm_f32(ad, wd)
    assert np.allclose(y, golden["y"], rtol=0, atol=2e-5 * np.abs(golden["y"]).max())


def test_config0_activation_digest(oracle, golden):
    x = golden["cfg0_a_x"]
    codes, beta_ids, norms = oracle.encode_packed(x, ACT_BETAS)
    assert hashlib.sha256(codes.tobytes()).digest() == golden["cfg0_a_code_sha256"].tobytes()
    assert hashlib.sha256(beta_ids.tobytes()).digest() == golden["cfg0_a_beta_sha256"].tobytes()
    assert hashlib.sha256(codes.tobytes()).hexdigest().startswith("f99a1820ec226dcf")
    assert np.array_equal(norms, golden["cfg0_a_norms"])


@pytest.mark.parametrize("tag", ["page_11x8x64", "page_16x2x128"])
def test_kv_page_bit_exact(oracle, golden, tag):
    out = oracle.kv_pack_page(golden[f"{tag}_key"], golden[f"{tag}_value"], page_size=16,
                              key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    for array, suffix in zip(out, ("_k_codes", "_k_beta", "_k_norms", "_v_codes", "_v_beta", "_v_norms")):
        assert np.array_equal(array, golden[tag + suffix]), suffix
    assert sum(a.nbytes for a in out) == int(golden[f"{tag}_payload_bytes"][0])
    valid, heads, dim = golden[f"{tag}_key"].shape
    dk = oracle.dequantize_rows(out[0], out[1], out[2], KEY_BETAS, 16 * heads, dim).reshape(16, heads, dim)[:valid]
    dv = oracle.dequantize_rows(out[3], out[4], out[5], VALUE_BETAS, 16 * heads, dim).reshape(16, heads, dim)[:valid]
    assert np.array_equal(dk, golden[f"{tag}_dk"]) and np.array_equal(dv, golden[f"{tag}_dv"])


def test_kv_page_is_9728_bytes(oracle, golden):
    assert int(golden["page_11x8x64_payload_bytes"][0]) == 9728


def test_hadamard(oracle, golden):
    assert np.array_equal(oracle.hadamard(golden["had_f32_in"]), golden["had_f32_out"])
    assert np.array_equal(oracle.hadamard(golden["had_64_in"]), golden["had_64_out"])
    assert np.array_equal(oracle.hadamard(golden["had_bf16_in"], round_bf16=True), golden["had_bf16_out"])
    with pytest.raises(ValueError):
        oracle.hadamard(np.zeros((1, 24), dtype=np.float32))
