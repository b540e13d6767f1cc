"""Normalised Sylvester Hadamard along the last axis (core/rotation.py:12-27).

The transform precedes every encode (Linear inputs in their own dtype, Q/K in
float32).  ``hadamard`` dispatches to the fused CUDA kernel when the library
exports it and the input is a CUDA tensor; the butterfly fallback below is the
reference's own sequence of tensor ops, kept for CPU tensors (tests, set-up).
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

_DTYPE_TAG = {torch.float32: _lib.NQ_F32, torch.bfloat16: _lib.NQ_BF16, torch.float16: _lib.NQ_F16}


def hadamard_butterflies(x: torch.Tensor) -> torch.Tensor:
    n = x.shape[-1]
    y = x.reshape(-1, n)
    width = 1
    while width < n:
        pairs = y.reshape(-1, n // (2 * width), 2, width)
        left, right = pairs[:, :, 0], pairs[:, :, 1]
        y = torch.stack((left + right, left - right), dim=2).reshape(-1, n)
        width *= 2
    return (y / math.sqrt(n)).reshape(x.shape)


def hadamard(x: torch.Tensor) -> torch.Tensor:
    if x.ndim == 0 or not x.is_floating_point():
        raise ValueError("expected a floating-point tensor with a feature axis")
    n = x.shape[-1]
    if n < 1 or n & (n - 1):
        raise ValueError("feature dimension must be a positive power of two")
    if x.device.type == "cuda" and x.dtype in _DTYPE_TAG and 8 <= n <= 32768 and x.numel() > 0:
        library = _lib.lib()
        if hasattr(library, "nq_hadamard"):
            src = x.contiguous()
            out = torch.empty_like(src)
            status = library.nq_hadamard(
                ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(out.data_ptr()), _DTYPE_TAG[x.dtype],
                ctypes.c_int64(src.numel() // n), ctypes.c_int64(n),
                ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
            _lib.check(status, "hadamard")
            return out
    return hadamard_butterflies(x)


def hadamard_silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``hadamard(silu(gate) * up)`` as one launch on CUDA tensors (same bits as the three tensor steps)."""
    if gate.shape != up.shape or gate.dtype != up.dtype or gate.device != up.device:
        raise ValueError("gate and up must share shape, dtype and device")
    n = gate.shape[-1] if gate.ndim else 0
    if (gate.device.type != "cuda" or gate.dtype not in _DTYPE_TAG or n < 8 or n > 32768 or n & (n - 1)
            or gate.numel() == 0):
        return hadamard(torch.nn.functional.silu(gate) * up)
    # rows a fixed distance apart (column ranges of one stacked gate/up result) are read in place
    esize = gate.element_size()
    try:
        a, b = gate.view(-1, n), up.view(-1, n)
        strided = (a.stride(1) == 1 and b.stride() == a.stride() and (a.shape[0] == 1 or a.stride(0) >= n)
                   and (a.stride(0) * esize) % 16 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)
    except RuntimeError:  # the leading axes do not collapse into rows of one stride
        strided = False
    if not strided:
        a, b = gate.contiguous().view(-1, n), up.contiguous().view(-1, n)
    row_stride = max(int(a.stride(0)), n) if a.shape[0] > 1 else n
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    status = _lib.lib().nq_hadamard_silu_mul(
        ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_int64(row_stride),
        ctypes.c_void_p(out.data_ptr()), _DTYPE_TAG[gate.dtype], ctypes.c_int64(gate.numel() // n), ctypes.c_int64(n),
        ctypes.c_void_p(torch.cuda.current_stream(gate.device).cuda_stream))
    _lib.check(status, "hadamard_silu_mul")
    return out
