"""ctypes front-end of the CPU checker in ``nq_oracle.c``.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module: it exists so that tests, the smoke check and the benchmark's CPU
baseline can compare the CUDA kernels with a CPU restatement of the
reference algorithm.  Parity status of the restatement: pinned against
golden vectors generated from the reference implementation
(``tests/golden/make_golden.py``).

All array arguments are NumPy arrays; float data is float32.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libnq_oracle.so"
_LIB = None

# Default beta tables of the reference (scripts/benchmark_full_nqrt_model.py:36,
# scripts/benchmark_service_workloads.py:39-40, configs/beta_profiles.v1.json:16-22).
ACTIVATION_BETAS = tuple(v / 14.0 for v in (3.47, 4.74, 6.90, 18.11))
WEIGHT_BETAS = tuple(v / 14.0 for v in (4.0, 5.5, 7.0, 18.0))


def build(force: bool = False) -> Path:
    """Compile the C checker next to its source (idempotent)."""
    source = _HERE / "nq_oracle.c"
    if not force and _LIB_PATH.exists() and _LIB_PATH.stat().st_mtime >= source.stat().st_mtime:
        return _LIB_PATH
    # compile beside the target and rename: several processes (test ranks) may build at the same time
    scratch = _LIB_PATH.with_name(f".{_LIB_PATH.name}.{os.getpid()}.tmp")
    base = ["-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-std=c11",
            "-o", str(scratch), str(source), "-lm"]
    compilers = [c for c in ("/usr/bin/gcc", "gcc", "cc") if c]
    last = None
    for compiler in compilers:
        for extra in (["-fopenmp"], []):
            try:
                subprocess.run([compiler, *extra, *base], check=True, capture_output=True)
                os.replace(scratch, _LIB_PATH)
                return _LIB_PATH
            except (OSError, subprocess.CalledProcessError) as error:  # try next variant
                last = error
    if scratch.exists():
        scratch.unlink()
    raise RuntimeError(f"could not build the CPU checker: {last}")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        _LIB = ctypes.CDLL(str(_LIB_PATH))
    return _LIB


def _p(array: np.ndarray):
    return array.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint8))


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


_I64 = ctypes.c_int64
_INT = ctypes.c_int


def nearest_e8(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().nqo_nearest_e8(_p(x), _p(out), _I64(x.size // 8))
    return out


def lcg31_hash(first_counter: int, count: int, seed: int) -> np.ndarray:
    out = np.empty(count, dtype=np.int64)
    lib().nqo_hash(_I64(first_counter), _I64(count), _I64(seed), _p(out))
    return out


def dither(first_block: int, blocks: int, seed: int) -> np.ndarray:
    out = np.empty((blocks, 8), dtype=np.float32)
    lib().nqo_dither(_I64(first_block), _I64(blocks), _I64(seed), _p(out))
    return out


def decode_nested(codes) -> np.ndarray:
    codes = _u8(codes)
    out = np.empty(codes.shape, dtype=np.float32)
    lib().nqo_decode_nested(_p(codes), _I64(codes.size // 8), _p(out))
    return out


def quantize_rows(x, betas, *, seed: int = -1, block_offset: int = 0):
    """Return ``(codes u8 [rows,K/8,8], beta_ids u8 [rows,K/8], norms f32 [rows])``."""
    x = _f32(x)
    rows, k = x.shape
    betas = _f32(betas)
    codes = np.empty((rows, k // 8, 8), dtype=np.uint8)
    beta_ids = np.empty((rows, k // 8), dtype=np.uint8)
    norms = np.empty(rows, dtype=np.float32)
    status = lib().nqo_quantize_rows(_p(x), _I64(rows), _I64(k), _p(betas), _INT(betas.size),
                                     _I64(seed), _I64(block_offset), _p(codes), _p(beta_ids), _p(norms))
    if status:
        raise ValueError("bad arguments to quantize_rows")
    return codes, beta_ids, norms


def pack(values, width: int) -> np.ndarray:
    values = _u8(values).reshape(-1)
    per_byte = 8 // width
    out = np.empty((values.size + per_byte - 1) // per_byte, dtype=np.uint8)
    lib().nqo_pack(_p(values), _I64(values.size), _INT(width), _p(out))
    return out


def unpack(payload, count: int, width: int) -> np.ndarray:
    payload = _u8(payload).reshape(-1)
    out = np.empty(count, dtype=np.uint8)
    lib().nqo_unpack(_p(payload), _I64(count), _INT(width), _p(out))
    return out


def encode_packed(x, betas, *, seed: int = -1, block_offset: int = 0):
    """quantize_rows + NQPK packing: ``(code_payload, beta_payload, norms)``."""
    codes, beta_ids, norms = quantize_rows(x, betas, seed=seed, block_offset=block_offset)
    return pack(codes, 4), pack(beta_ids, 2), norms


def dequantize_rows(code_payload, beta_payload, norms, betas, rows: int, k: int, *,
                    seed: int = -1, block_offset: int = 0) -> np.ndarray:
    code_payload, beta_payload = _u8(code_payload), _u8(beta_payload)
    norms, betas = _f32(norms), _f32(betas)
    out = np.empty((rows, k), dtype=np.float32)
    lib().nqo_dequantize_rows(_p(code_payload), _p(beta_payload), _p(norms), _p(betas),
                              _I64(rows), _I64(k), _I64(seed), _I64(block_offset), _p(out))
    return out


def round_bf16(x) -> np.ndarray:
    out = _f32(x).copy()
    lib().nqo_round_bf16(_p(out), _I64(out.size))
    return out


def gemm_bf16_operands(a, w) -> np.ndarray:
    a, w = _f32(a), _f32(w)
    m, k = a.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    lib().nqo_gemm_bf16_operands(_p(a), _p(w), _I64(m), _I64(n), _I64(k), _p(y))
    return y


def gemm_f32(a, w) -> np.ndarray:
    a, w = _f32(a), _f32(w)
    m, k = a.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    lib().nqo_gemm_f32(_p(a), _p(w), _I64(m), _I64(n), _I64(k), _p(y))
    return y


def hadamard(x, *, round_bf16: bool = False) -> np.ndarray:
    out = _f32(x).copy()
    n = out.shape[-1]
    status = lib().nqo_hadamard(_p(out), _I64(out.size // n), _I64(n), _INT(int(round_bf16)))
    if status:
        raise ValueError("feature dimension must be a positive power of two")
    return out


def kv_pack_page(key, value, *, page_size: int, key_betas, value_betas):
    """key/value float32 ``[valid, H, D]`` -> six payload arrays of one page."""
    key, value = _f32(key), _f32(value)
    valid, heads, dim = key.shape
    rows = page_size * heads
    kc = np.empty(rows * dim // 2, dtype=np.uint8)
    kb = np.empty(rows * dim // 32, dtype=np.uint8)
    kn = np.empty(rows, dtype=np.float32)
    vc, vb, vn = np.empty_like(kc), np.empty_like(kb), np.empty_like(kn)
    kbt, vbt = _f32(key_betas), _f32(value_betas)
    status = lib().nqo_kv_pack_page(_p(key), _p(value), _INT(valid), _INT(page_size), _INT(heads),
                                    _INT(dim), _p(kbt), _p(vbt), _p(kc), _p(kb), _p(kn),
                                    _p(vc), _p(vb), _p(vn))
    if status:
        raise ValueError("bad arguments to kv_pack_page")
    return kc, kb, kn, vc, vb, vn


def _cache_args(cache: dict):
    keep = [
        _i32(cache["page_indices"]), _i32(cache["page_counts"]), _i32(cache["last_page_lens"]),
        _i32(cache["hot_lengths"]),
        _u8(cache["key_codes"]), _u8(cache["key_betas"]), _f32(cache["key_norms"]),
        _u8(cache["value_codes"]), _u8(cache["value_betas"]), _f32(cache["value_norms"]),
        _f32(cache["key_beta_table"]), _f32(cache["value_beta_table"]),
        _f32(cache["hot_keys"]), _f32(cache["hot_values"]),
    ]
    return keep


def attn_decode(query, slot_ids, active, cache: dict, *, scale: float) -> np.ndarray:
    """``cache`` holds the pool / page-table / hot-tail arrays under the reference's names."""
    query = _f32(query)
    batch, q_heads, dim = query.shape
    slot_ids, active = _i32(slot_ids), _u8(active)
    c = _cache_args(cache)
    page, kv_heads = cache["hot_keys"].shape[1], cache["hot_keys"].shape[2]
    out = np.zeros_like(query)
    lib().nqo_attn_decode(
        _p(query), _p(slot_ids), _p(active), _INT(batch), _INT(q_heads), _INT(kv_heads), _INT(dim),
        _INT(page), _p(c[0]), _INT(c[0].shape[1]), _p(c[1]), _p(c[2]), _p(c[3]),
        _p(c[4]), _p(c[5]), _p(c[6]), _p(c[7]), _p(c[8]), _p(c[9]), _p(c[10]), _p(c[11]),
        _p(c[12]), _p(c[13]), ctypes.c_float(scale), _p(out))
    return out


def attn_prefill(query, slot_ids, q_lens, cache: dict, *, scale: float) -> np.ndarray:
    query = _f32(query)
    batch, t_max, q_heads, dim = query.shape
    slot_ids, q_lens = _i32(slot_ids), _i32(q_lens)
    c = _cache_args(cache)
    page, kv_heads = cache["hot_keys"].shape[1], cache["hot_keys"].shape[2]
    out = np.zeros_like(query)
    lib().nqo_attn_prefill(
        _p(query), _p(slot_ids), _p(q_lens), _INT(batch), _INT(t_max), _INT(q_heads), _INT(kv_heads),
        _INT(dim), _INT(page), _p(c[0]), _INT(c[0].shape[1]), _p(c[1]), _p(c[2]), _p(c[3]),
        _p(c[4]), _p(c[5]), _p(c[6]), _p(c[7]), _p(c[8]), _p(c[9]), _p(c[10]), _p(c[11]),
        _p(c[12]), _p(c[13]), ctypes.c_float(scale), _p(out))
    return out


def set_threads(threads: int) -> None:
    """Threads of the checker's parallel loops from now on (overrides OMP_NUM_THREADS)."""
    lib().nqo_set_threads(_INT(int(threads)))


def thread_count() -> int:
    """Threads the C checker uses for its parallel loops right now."""
    return int(lib().nqo_max_threads())
