"""Rotary embedding and the Q/K Hadamard rotation of the KV backend in one launch.

``rope_hadamard`` computes what Hugging Face's ``apply_rotary_pos_emb`` followed by the backend's
``hadamard(x.float()).to(dtype)`` (runtime/nqkv_batched_hf_backend.py:381,549) compute, bit for
bit, for one of the two tensors.  ``fused_rope_scope`` makes Llama's attention modules use it while a
runner drives the model: inside the scope ``apply_rotary_pos_emb`` returns tensors that are already
Hadamard-rotated and marked so (``rotation_done``), and the cache skips its own rotation for them.
Outside the scope, or for tensors the kernel does not take, the stock function runs.
"""

from __future__ import annotations

import contextlib
import ctypes
import threading

import torch

from . import _lib

_DTYPE_TAG = {torch.float32: _lib.NQ_F32, torch.bfloat16: _lib.NQ_BF16, torch.float16: _lib.NQ_F16}
_MARK = "_nestquant_hadamard_done"
_state = threading.local()
_stock_apply = None


def rotation_done(tensor: torch.Tensor) -> bool:
    """True for a tensor that left ``apply_rotary_pos_emb`` already Hadamard-rotated."""
    return bool(getattr(tensor, _MARK, False))


def _usable(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> bool:
    if x.device.type != "cuda" or x.dtype not in _DTYPE_TAG or x.ndim != 4 or cos.ndim != 3:
        return False
    dim = x.shape[-1]
    if dim < 16 or dim > 1024 or dim & (dim - 1) or x.stride(-1) != 1 or x.numel() == 0:
        return False
    size = x.element_size()
    if x.data_ptr() % 16 or any((x.stride(i) * size) % 16 for i in range(3)):
        return False
    return (cos.dtype == x.dtype and sin.dtype == x.dtype and cos.shape == sin.shape and cos.shape[-1] == dim
            and cos.shape[1] == x.shape[2] and cos.shape[0] in (1, x.shape[0]))


def rope_hadamard(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, rotate: bool = True) -> torch.Tensor:
    """``x [B, H, T, D]`` (any strides over B, H, T), ``cos`` / ``sin`` ``[B or 1, T, D]`` -> contiguous ``[B, H, T, D]``."""
    if not _usable(x, cos, sin):
        raise ValueError("rope_hadamard needs CUDA [B, H, T, D] with a power-of-two D in [16, 1024] and 16-byte aligned strides")
    batch, heads, tokens, dim = x.shape
    cos = cos.expand(batch, tokens, dim).contiguous()
    sin = sin.expand(batch, tokens, dim).contiguous()
    out = torch.empty((batch, heads, tokens, dim), dtype=x.dtype, device=x.device)
    status = _lib.lib().nq_rope_hadamard(
        ctypes.c_void_p(x.data_ptr()), _DTYPE_TAG[x.dtype], ctypes.c_int64(batch), ctypes.c_int64(heads),
        ctypes.c_int64(tokens), ctypes.c_int64(dim), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)),
        ctypes.c_int64(x.stride(2)), ctypes.c_void_p(cos.data_ptr()), ctypes.c_void_p(sin.data_ptr()),
        ctypes.c_int(1 if rotate else 0), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    _lib.check(status, "rope_hadamard")
    return out


def rope_hadamard_pair(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *,
                       rotate: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """``rope_hadamard`` of the query heads and the key heads of one layer as ONE launch."""
    if not (_usable(q, cos, sin) and _usable(k, cos, sin)) or q.dtype != k.dtype or q.shape[0] != k.shape[0] \
            or q.shape[2:] != k.shape[2:] or q.device != k.device:
        raise ValueError("rope_hadamard_pair needs q and k [B, H, T, D] of one dtype, batch, length and head size")
    batch, q_heads, tokens, dim = q.shape
    cos = cos.expand(batch, tokens, dim).contiguous()
    sin = sin.expand(batch, tokens, dim).contiguous()
    q_out = torch.empty((batch, q_heads, tokens, dim), dtype=q.dtype, device=q.device)
    k_out = torch.empty((batch, k.shape[1], tokens, dim), dtype=k.dtype, device=k.device)
    strides = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))  # noqa: E731
    status = _lib.lib().nq_rope_hadamard_pair(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), _DTYPE_TAG[q.dtype], ctypes.c_int64(batch),
        ctypes.c_int64(q_heads), ctypes.c_int64(k.shape[1]), ctypes.c_int64(tokens), ctypes.c_int64(dim), strides(q),
        strides(k), ctypes.c_void_p(cos.data_ptr()), ctypes.c_void_p(sin.data_ptr()), ctypes.c_int(1 if rotate else 0),
        ctypes.c_void_p(q_out.data_ptr()), ctypes.c_void_p(k_out.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    _lib.check(status, "rope_hadamard_pair")
    return q_out, k_out


def _apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
    if (getattr(_state, "depth", 0) > 0 and unsqueeze_dim == 1 and isinstance(q, torch.Tensor)
            and not torch.is_grad_enabled() and _usable(q, cos, sin) and _usable(k, cos, sin)):
        if q.dtype == k.dtype and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:]:
            q_out, k_out = rope_hadamard_pair(q, k, cos, sin)
        else:
            q_out = rope_hadamard(q, cos, sin)
            k_out = rope_hadamard(k, cos, sin)
        setattr(q_out, _MARK, True)
        setattr(k_out, _MARK, True)
        return q_out, k_out
    return _stock_apply(q, k, cos, sin, unsqueeze_dim)


def install_fused_rope() -> None:
    """Route Llama's ``apply_rotary_pos_emb`` through this module (the stock function still serves every call outside a scope)."""
    global _stock_apply
    from transformers.models.llama import modeling_llama

    if modeling_llama.apply_rotary_pos_emb is _apply_rotary_pos_emb:
        return
    _stock_apply = modeling_llama.apply_rotary_pos_emb
    modeling_llama.apply_rotary_pos_emb = _apply_rotary_pos_emb


@contextlib.contextmanager
def fused_rope_scope(enabled: bool = True):
    """Within the scope (per thread) the attention modules get rope + Hadamard rotation from one launch per tensor."""
    if enabled:
        install_fused_rope()
    _state.depth = getattr(_state, "depth", 0) + (1 if enabled else 0)
    try:
        yield
    finally:
        _state.depth -= 1 if enabled else 0
