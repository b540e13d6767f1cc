"""RMS normalisation in one launch, in front of the rotate-then-encode launches of a decoder layer.

Hugging Face's ``LlamaRMSNorm`` (float32 mean of squares, ``x * rsqrt(mean + eps)`` rounded to the
input dtype, times the weight) runs as six small tensor kernels; at decode batch sizes they cost
more than the arithmetic.  ``FusedRMSNorm`` keeps the module's parameters and formula and calls
``nq_rmsnorm``.  The reference leaves the normalisation to the stock model (its fused scope ends at
the projection input, models/fused_linear.py:280-300), so this has no counterpart there.
"""

from __future__ import annotations

import ctypes

import torch
from torch import nn

from . import _lib

_DTYPE_TAG = {torch.float32: _lib.NQ_F32, torch.bfloat16: _lib.NQ_BF16, torch.float16: _lib.NQ_F16}


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * (x * rsqrt(mean(x^2, -1) + eps)).to(x.dtype)`` along the last axis, one CUDA launch."""
    if not isinstance(x, torch.Tensor) or x.device.type != "cuda" or x.dtype not in _DTYPE_TAG:
        raise ValueError("rms_norm needs a CUDA tensor of float16, bfloat16 or float32")
    n = x.shape[-1]
    if weight.shape != (n,) or weight.dtype != x.dtype or weight.device != x.device:
        raise ValueError("weight must be a vector of the feature size with the dtype and device of the input")
    if n % 8:
        raise ValueError("the feature size must be a multiple of 8")
    src = x.contiguous()
    w = weight.contiguous()
    out = torch.empty_like(src)
    if src.numel() == 0:
        return out
    status = _lib.lib().nq_rmsnorm(
        ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(w.data_ptr()), _DTYPE_TAG[x.dtype],
        ctypes.c_int64(src.numel() // n), ctypes.c_int64(n), ctypes.c_float(float(eps)),
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    _lib.check(status, "rms_norm")
    return out


class FusedRMSNorm(nn.Module):
    """Drop-in for ``LlamaRMSNorm``: same parameter, same formula, one launch."""

    def __init__(self, weight: torch.Tensor, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(weight.detach(), requires_grad=False)
        self.variance_epsilon = float(eps)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return rms_norm(hidden_states, self.weight, self.variance_epsilon)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


def fuse_rmsnorm_(model: nn.Module) -> int:
    """Replace every RMS-norm child that has a ``weight`` and a ``variance_epsilon`` by ``FusedRMSNorm``."""
    replaced = 0
    for module in list(model.modules()):
        for name, child in list(module.named_children()):
            if isinstance(child, FusedRMSNorm) or not type(child).__name__.endswith("RMSNorm"):
                continue
            if not hasattr(child, "variance_epsilon") or not isinstance(getattr(child, "weight", None), torch.Tensor):
                continue
            setattr(module, name, FusedRMSNorm(child.weight, child.variance_epsilon))
            replaced += 1
    return replaced
