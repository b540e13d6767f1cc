"""The codec header the kernels include, compiled for the host, against the CPU checker.

csrc/nq_e8.cuh is written once for host and device; building it with g++
(-ffp-contract=off) lets the CPU suite check the very source the GPU runs.
"""

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

from helpers import ACT_BETAS, W_BETAS

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = tmp_path_factory.mktemp("shim") / "libshim.so"
    subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-ffp-contract=off", "-mfma",
                    "-I", str(ROOT / "nestquant_aiinfra_b200" / "csrc"), "-o", str(out),
                    str(ROOT / "tests" / "hostmath" / "e8_host_shim.cpp")], check=True)
    return ctypes.CDLL(str(out))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_nearest_dither_decode(shim, oracle, golden):
    x = golden["e8_in"]
    out = np.empty_like(x)
    shim.shim_nearest_e8(_p(x), _p(out), ctypes.c_long(len(x)))
    assert np.array_equal(out, golden["e8_out"])
    d = np.empty((64, 8), np.float32)
    shim.shim_dither(ctypes.c_long(0), ctypes.c_long(64), ctypes.c_long(int(golden["dither_seed"][0])), _p(d))
    assert np.array_equal(d, golden["dither_blocks_0_64"])
    words = np.ascontiguousarray(oracle.pack(golden["decode_codes"], 4)).view(np.uint32)
    dec = np.empty((len(words), 8), np.float32)
    shim.shim_decode(_p(words), ctypes.c_long(len(words)), _p(dec))
    assert np.array_equal(dec, golden["decode_out"])


@pytest.mark.parametrize("seed,betas", [(-1, ACT_BETAS), (4242, W_BETAS)])
def test_block_encoder_matches_checker(shim, oracle, seed, betas):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((50000, 8)).astype(np.float32)
    betas = np.array(betas, np.float32)
    codes, beta_ids, norms = oracle.quantize_rows(x, betas, seed=seed)
    scale = ((np.float32(1) / norms).astype(np.float32) * np.float32(np.sqrt(8.0))).astype(np.float32)
    xn = (x * scale[:, None]).astype(np.float32)
    words = np.empty(len(x), np.uint32)
    ids = np.empty(len(x), np.int32)
    rec = np.empty_like(x)
    shim.shim_encode_blocks(_p(xn), ctypes.c_long(len(x)), _p(betas), ctypes.c_long(seed), ctypes.c_long(0),
                            _p(words), _p(ids), _p(rec))
    assert np.array_equal(np.ascontiguousarray(oracle.pack(codes, 4)).view(np.uint32), words)
    assert np.array_equal(beta_ids.reshape(-1), ids.astype(np.uint8))


def test_bf16_rounding(shim, oracle):
    shim.shim_bf16_round.restype = ctypes.c_float
    values = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 1e-20, 65504.0], np.float32)
    got = np.array([shim.shim_bf16_round(ctypes.c_float(v)) for v in values], np.float32)
    assert np.array_equal(got, oracle.round_bf16(values))


def test_guarded_nearest_equals_exact(shim, oracle, golden):
    x = golden["e8_in"]
    out = np.empty_like(x)
    shim.shim_nearest_e8_guarded(_p(x), _p(out), ctypes.c_long(len(x)))
    assert np.array_equal(out, golden["e8_out"])
    x = (np.random.default_rng(1).standard_normal((500000, 8)) * 2).astype(np.float32)
    out = np.empty_like(x)
    shim.shim_nearest_e8_guarded(_p(x), _p(out), ctypes.c_long(len(x)))
    assert np.array_equal(out, oracle.nearest_e8(x))


def test_weight_block_decode_matches_checker(shim, oracle):
    n = 300000
    codes = np.random.default_rng(2).integers(0, 14, (n, 8)).astype(np.uint8)
    words = np.ascontiguousarray(oracle.pack(codes, 4)).view(np.uint32)
    out = np.empty((n, 8), np.float32)
    shim.shim_decode_weight(_p(words), ctypes.c_long(n), ctypes.c_long(77), ctypes.c_long(4242), _p(out))
    ref = oracle.dequantize_rows(oracle.pack(codes, 4), np.zeros(n // 4, np.uint8),
                                 np.full(1, np.float32(np.sqrt(8 * n))), [1.0] * 4, 1, 8 * n, seed=4242,
                                 block_offset=77)
    assert np.array_equal(out.reshape(-1), ref.reshape(-1))
