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
    """Drop-in for ``LlamaRMSNorm``: same parameter, same formula, one launch.

    ``defer=True`` is for a norm whose ONLY consumers are ``FusedNQRTLinear`` modules (Llama's
    ``input_layernorm`` in front of q/k/v and ``post_attention_layernorm`` in front of gate/up): the
    module then launches nothing and returns a view of its input that carries the pending
    normalisation; the first projection that receives it normalises, rotates and encodes in one
    launch (bit-identical to this module's kernel followed by the rotate-and-encode), the others reuse
    that encoding.  A consumer that cannot fuse materialises the normalised tensor once.
    """

    def __init__(self, weight: torch.Tensor, eps: float, *, defer: bool = False) -> None:
        super().__init__()
        self.weight = nn.Parameter(weight.detach(), requires_grad=False)
        self.variance_epsilon = float(eps)
        self.defer = bool(defer)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self.defer and not torch.is_grad_enabled() and hidden_states.is_cuda:
            pending = hidden_states.view(hidden_states.shape)  # a new tensor object on the same storage, no launch
            pending._nq_pending_norm = (self.weight, self.variance_epsilon)
            return pending
        return rms_norm(hidden_states, self.weight, self.variance_epsilon)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


def _feeds_only_packed_projections(layer: nn.Module, norm_name: str) -> bool:
    """Llama decoder layer: ``input_layernorm`` feeds q/k/v, ``post_attention_layernorm`` feeds gate/up."""
    from .fused_linear import FusedNQRTLinear

    owner, leaves = {"input_layernorm": ("self_attn", ("q_proj", "k_proj", "v_proj")),
                     "post_attention_layernorm": ("mlp", ("gate_proj", "up_proj"))}.get(norm_name, (None, ()))
    block = getattr(layer, owner, None) if owner else None
    return block is not None and all(isinstance(getattr(block, leaf, None), FusedNQRTLinear) for leaf in leaves)


def fuse_rmsnorm_(model: nn.Module, *, defer_into_projections: bool = False) -> int:
    """Replace every RMS-norm child that has a ``weight`` and a ``variance_epsilon`` by ``FusedRMSNorm``.

    ``defer_into_projections`` lets the two norms of a Llama decoder layer whose consumers are all packed
    projections hand their work to the projections' encoder launch (see ``FusedRMSNorm``).
    """
    replaced = 0
    for module in list(model.modules()):
        for name, child in list(module.named_children()):
            if isinstance(child, FusedRMSNorm) or not type(child).__name__.endswith("RMSNorm"):
                continue
            if not hasattr(child, "variance_epsilon") or not isinstance(getattr(child, "weight", None), torch.Tensor):
                continue
            defer = defer_into_projections and _feeds_only_packed_projections(module, name)
            setattr(module, name, FusedRMSNorm(child.weight, child.variance_epsilon, defer=defer))
            replaced += 1
    return replaced


class FusedSiluMLP(nn.Module):
    """Llama's gated MLP ``down(silu(gate(x)) * up(x))`` with the elementwise part inside down_proj's encoder launch.

    Keeps the three projection modules of the MLP it replaces (same attribute names).  The reference leaves SiLU
    and the product to the model's tensor ops (two launches) in front of ``FusedNQRTLinear``'s own Hadamard and
    encode (models/fused_linear.py:287-306); no counterpart there.
    """

    def __init__(self, gate_proj: nn.Module, up_proj: nn.Module, down_proj: nn.Module) -> None:
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.down_proj.forward_silu_mul(self.gate_proj(hidden_states), self.up_proj(hidden_states))


def fuse_silu_mlp_(model: nn.Module) -> int:
    """Replace every Llama-style MLP (``act_fn`` = SiLU, three bias-free packed projections) by ``FusedSiluMLP``."""
    from .fused_linear import FusedNQRTLinear

    replaced = 0
    for module in list(model.modules()):
        for name, child in list(module.named_children()):
            if isinstance(child, FusedSiluMLP) or not all(hasattr(child, a) for a in ("gate_proj", "up_proj", "down_proj", "act_fn")):
                continue
            if not isinstance(child.act_fn, nn.SiLU) and getattr(child.act_fn, "__name__", "") != "silu" \
                    and type(child.act_fn).__name__ not in {"SiLUActivation", "SiLU"}:
                continue
            if not isinstance(child.down_proj, FusedNQRTLinear):
                continue
            setattr(module, name, FusedSiluMLP(child.gate_proj, child.up_proj, child.down_proj))
            replaced += 1
    return replaced
