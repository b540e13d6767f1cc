"""Loader of the C-ABI CUDA library ``libnq_b200.so`` (sources in ``csrc/``).

There is no CPU fallback: if the library cannot be loaded every operator of
this package raises.  ``build_library()`` compiles it in-tree with nvcc for
sm_100a (cross-compilation works on a machine without a GPU).
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
LIB_PATH = _PKG / "libnq_b200.so"
HEADER = _PKG.parent / "include" / "nq_b200.h"
SOURCES = ("nq_encode.cu", "nq_gemv.cu", "nq_gemv_bf16.cu", "nq_gemv_static.cu", "nq_gemm.cu", "nq_gemm_tc.cu", "nq_kv.cu", "nq_attn.cu",
           "nq_rotate.cu", "nq_encode_rotated.cu", "nq_norm.cu", "nq_rope.cu", "nq_allreduce.cu")

NQ_F32, NQ_BF16, NQ_F16 = 0, 1, 2
WS_COUNTER_BYTES = 65536
WS_STATUS_OFFSET = 65532  # NQ_WS_STATUS_OFFSET of the header

_LIB: ctypes.CDLL | None = None


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; cannot build libnq_b200.so")


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a into ``libnq_b200.so`` (in-tree)."""
    sources = [CSRC / name for name in SOURCES if (CSRC / name).exists()]
    deps = sources + list(CSRC.glob("*.cuh")) + [HEADER]
    if not force and LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return LIB_PATH
    # link beside the target and rename: several ranks may find the library stale at the same time
    scratch = LIB_PATH.with_name(f".{LIB_PATH.name}.{os.getpid()}.tmp")
    command = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--threads", "0",
        "-shared", "-Xcompiler", "-fPIC", "-o", str(scratch), *map(str, sources),
    ]
    if verbose:
        command.insert(1, "-Xptxas=-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        if scratch.exists():
            scratch.unlink()
        raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
    os.replace(scratch, LIB_PATH)
    if verbose:
        print(result.stderr)
    return LIB_PATH


def declared_symbols() -> list[str]:
    """Names of every function the public header declares (``nq_*``)."""
    import re

    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nq_[a-z0-9_]+)\s*\(", text)))


def lib() -> ctypes.CDLL:
    """Return the loaded library or raise (never falls back to another path)."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with nestquant_aiinfra_b200.build_library(); "
                "this package has no CPU or library fallback")
        handle = ctypes.CDLL(str(LIB_PATH))
        handle.nq_last_error.restype = ctypes.c_char_p
        handle.nq_w4a4_workspace_bytes.restype = ctypes.c_size_t
        handle.nq_launch_count.restype = ctypes.c_ulonglong
        for name in ("nq_kv_attention_workspace_bytes", "nq_w4a4_resident_workspace_bytes"):
            if hasattr(handle, name):
                getattr(handle, name).restype = ctypes.c_size_t
        _LIB = handle
    return _LIB


class NQError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def check(status: int, what: str) -> None:
    if status == 0:
        return
    message = lib().nq_last_error().decode("utf-8", "replace")
    if status < 0:
        raise ValueError(f"{what}: {message} (status {status})")
    raise NQError(f"{what}: CUDA error {status}: {message}")
