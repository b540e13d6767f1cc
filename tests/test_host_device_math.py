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


@pytest.mark.parametrize("entry", ["shim_nearest_e8_guarded", "shim_nearest_e8_guarded_lean"])
def test_guarded_nearest_equals_exact(shim, oracle, golden, entry):
    search = getattr(shim, entry)  # the lean form is the one the encoder's searches use
    x = golden["e8_in"]
    out = np.empty_like(x)
    search(_p(x), _p(out), ctypes.c_long(len(x)))
    assert np.array_equal(out, golden["e8_out"])
    x = (np.random.default_rng(1).standard_normal((500000, 8)) * 2).astype(np.float32)
    out = np.empty_like(x)
    search(_p(x), _p(out), ctypes.c_long(len(x)))
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


def _encode_both(shim, x, betas):
    x = np.ascontiguousarray(x, np.float32)
    betas = np.array(betas, np.float32)
    n = len(x)
    out = []
    for variant in ("full", "pruned", "queued"):
        words, ids, rec = np.empty(n, np.uint32), np.empty(n, np.int32), np.empty_like(x)
        if variant == "pruned":
            shim.shim_encode_blocks_pruned(_p(x), ctypes.c_long(n), _p(betas), _p(words), _p(ids), _p(rec))
        elif variant == "queued":
            shim.shim_encode_blocks_queued(_p(x), ctypes.c_long(n), _p(betas), _p(words), _p(ids), _p(rec), None)
        else:
            shim.shim_encode_blocks(_p(x), ctypes.c_long(n), _p(betas), ctypes.c_long(-1), ctypes.c_long(0),
                                    _p(words), _p(ids), _p(rec))
        out.append((words, ids, rec))
    return out


@pytest.mark.parametrize("case", ["gauss", "heavy", "huge", "tiny", "grid", "boundary"])
def test_pruned_search_equals_full_search(shim, case):
    """The pruned 4-beta searches (interior test + error bounds) must never change a bit."""
    rng = np.random.default_rng(11)
    unit = (0.25, 0.5, 0.75, 1.0)
    if case == "gauss":
        x, betas = rng.standard_normal((300000, 8)), ACT_BETAS
    elif case == "heavy":
        x, betas = rng.standard_t(2, (300000, 8)), ACT_BETAS
    elif case == "huge":
        x, betas = rng.standard_normal((100000, 8)) * 30, ACT_BETAS
    elif case == "tiny":
        x, betas = rng.standard_normal((100000, 8)) * 1e-3, ACT_BETAS
    elif case == "grid":  # inputs on beta * (half-integer grid): dense coset ties and cell-boundary points
        x = np.concatenate([rng.integers(-30, 31, (100000, 8)) * 0.5 * b for b in unit])
        betas = unit
    else:
        a = np.zeros((8, 8)); a[:, 0] = 7; a[:, 1] = 7          # |lam|^2 = 98, on the boundary of 14 V
        b = np.full((8, 8), 3.5)
        x, betas = np.concatenate([a, b, a * 0.5, b * 0.75]), unit
    (w1, i1, r1), *others = _encode_both(shim, x, betas)
    for w2, i2, r2 in others:  # pruned per-thread search, and the search as the kernel's work queue runs it
        assert np.array_equal(w1, w2) and np.array_equal(i1, i2) and np.array_equal(r1, r2)


def test_cell_class_known_points(shim):
    pts = np.array([[0] * 8, [7, 7, 0, 0, 0, 0, 0, 0], [3.5] * 8, [7, 6, 0, 0, 0, 0, 0, 0], [8, 7, 0, 0, 0, 0, 0, 0],
                    [3.5] * 7 + [-3.5], [14, 0, 0, 0, 0, 0, 0, 0], [13, 0, 0, 0, 0, 0, 0, 0], [7, 7, 7, 7, 0, 0, 0, 0]],
                   np.float32)
    out = np.empty(len(pts), np.int32)
    shim.shim_cell_class(_p(pts), ctypes.c_long(len(pts)), _p(out))
    #            origin  root facet  half facet  inside  outside  odd half      (2,0..) facet  inside  norm-4 facet
    assert out.tolist() == [1, 0, 0, 1, -1, 1, 0, 1, 0]


def test_lean_undithered_decode_equals_the_exact_decode(shim, oracle, golden):
    """nq_decode_codeword_undithered (attention, activation decode) is the exact decode with fewer instructions.

    The identity was checked once over all 14^8 codewords (35 s on 8 threads); the suite repeats it on
    every 61st codeword and on the reference's boundary vectors.
    """
    assert shim.shim_div14_exact() == 1
    shim.shim_undithered_mismatches.restype = ctypes.c_long
    assert shim.shim_undithered_mismatches(ctypes.c_long(61)) == 0
    words = np.ascontiguousarray(oracle.pack(golden["decode_codes"], 4)).view(np.uint32)
    dec = np.empty((len(words), 8), np.float32)
    shim.shim_decode_undithered(_p(words), ctypes.c_long(len(words)), _p(dec))
    assert np.array_equal(dec, golden["decode_out"])


def test_table_driven_undithered_decode_equals_the_exact_decode(shim, oracle, golden):
    """nq_decode_codeword_lut (what the paged attention runs) reproduces the exact decode bit for bit.

    Every coordinate of an undithered codeword takes one of 92 values, so the roundings of the search are
    tabulated; coset ties and equal-|residual| parity repairs follow the reference's float32 order through
    tabulated squares and ranks.  The identity was checked once over all 14^8 codewords (25 s on 8 threads);
    the suite repeats it on every 61st codeword and on the reference's boundary vectors.
    """
    assert shim.shim_lut_field_overflows() == 0
    shim.shim_lut_mismatches.restype = ctypes.c_long
    assert shim.shim_lut_mismatches(ctypes.c_long(61), ctypes.c_long(0), ctypes.c_long(14 ** 4)) == 0
    words = np.ascontiguousarray(oracle.pack(golden["decode_codes"], 4)).view(np.uint32)
    dec = np.empty((len(words), 8), np.float32)
    shim.shim_decode_lut(_p(words), ctypes.c_long(len(words)), _p(dec))
    assert np.array_equal(dec, golden["decode_out"])
