"""Put this package behind the reference's own module names.

``install()`` rebinds, inside an importable ``nestquant`` package, every symbol of the hot path that
this package implements: the A4 encoder and the prepared-operand dataclasses, the packed W4A4
projection family, the NQKV4 pool / hot tail / writers / attention, the Hugging Face cache with its
attention interface, and the ``FusedNQRTLinear`` module family.  Code that imports those names from
``nestquant.runtime`` or ``nestquant.models.fused_linear`` AFTER the call -- the reference's
``BatchedNQKVLlamaRunner``, its serving script, its continuous-batching engine -- then runs on the
sm_100a kernels through the C ABI without being edited.  ``uninstall()`` restores the originals.

Modules that took their own reference to a symbol with ``from x import y`` before the call are
patched too: every module listed below is scanned for the names, not only the defining one.
"""

from __future__ import annotations

import importlib
import sys
from typing import Any

_ORIGINALS: list[tuple[Any, str, Any]] = []

# modules of the reference that define or re-import hot-path symbols
_TARGET_MODULES = (
    "nestquant.runtime", "nestquant.runtime.triton_w4a4_linear", "nestquant.runtime.triton_fused_linear",
    "nestquant.runtime.cuda_w4a4_mma", "nestquant.runtime.nqkv_page", "nestquant.runtime.nqkv_pool",
    "nestquant.runtime.nqkv_hot_cache", "nestquant.runtime.nqkv_graph_writer", "nestquant.runtime.nqkv_graph_pack",
    "nestquant.runtime.nqkv_attention_k1", "nestquant.runtime.nqkv_batched_hf_backend",
    "nestquant.runtime.nqkv_batched_runner", "nestquant.models.fused_linear",
)


def _replacements() -> dict[str, Any]:
    from . import fused_linear, hf_backend
    from .runtime import kv, w4a4

    names: dict[str, Any] = {}
    for module, wanted in (
        (w4a4, ("PreparedNQA4Activation", "PreparedNQRTLinear", "prepare_fused_linear", "quantize_activation_cuda",
                "can_use_w4a4_gemv_m1", "can_use_w4a4_mma_small_m", "can_use_w4a4_mma_m16",
                "can_use_w4a4_mma_large_m_staged", "can_use_w4a4_mma_chunked_staged",
                "linear_packed_w4a4_gemv_m1", "linear_packed_w4a4_mma_small_m", "linear_packed_w4a4_mma_m16",
                "linear_packed_w4a4_mma_large_m_staged", "linear_packed_w4a4_mma_chunked_staged",
                "linear_packed_w4a4_gemv_m1_fp32_probe", "decode_packed_a4_m16")),
        (kv, ("NQKVPagePool", "NQKVHotColdCache", "PreparedNQKVPage", "quantize_nqkv_page_cuda",
              "_launch_append_hot_k1_graph_safe", "_launch_append_hot_ragged_subpage_graph_safe",
              "_launch_append_hot_ragged_segment_graph_safe", "launch_pack_full_hot_pages_graph_safe",
              "BatchedNQKVAttentionWorkspace", "nqkv_decode_attention_batched_k1",
              "_launch_nqkv_decode_attention_batched_k1")),
        (hf_backend, ("BatchedNQKVLlamaCache", "_batched_nqkv_attention_interface",
                      "install_batched_nqkv_llama_backend", "BATCHED_NQKV_ATTENTION_NAME")),
        (fused_linear, ("FusedNQRTLinear", "SharedHadamardCache", "SharedPackedActivationCache",
                        "FusedNQRTConversionReport", "convert_linears_to_fused_nqrt_")),
    ):
        for name in wanted:
            names[name] = getattr(module, name)
    return names


def install(*, reference_path: str | None = None) -> dict[str, list[str]]:
    """Rebind the reference's hot-path symbols; returns ``{module name: [rebound names]}``.

    ``reference_path`` is put on ``sys.path`` first when ``nestquant`` is not importable yet.
    Raises ``ImportError`` when the reference cannot be imported at all.
    """
    if _ORIGINALS:
        raise RuntimeError("already installed; call uninstall() first")
    if reference_path is not None and reference_path not in sys.path:
        sys.path.insert(0, reference_path)
    names = _replacements()
    rebound: dict[str, list[str]] = {}
    for module_name in _TARGET_MODULES:
        try:
            module = importlib.import_module(module_name)
        except ImportError:
            if module_name == "nestquant.runtime":
                raise
            continue
        for name, value in names.items():
            if name in vars(module) and vars(module)[name] is not value:
                _ORIGINALS.append((module, name, vars(module)[name]))
                setattr(module, name, value)
                rebound.setdefault(module_name, []).append(name)
    return rebound


def uninstall() -> None:
    """Put back every symbol ``install()`` replaced."""
    while _ORIGINALS:
        module, name, value = _ORIGINALS.pop()
        setattr(module, name, value)


def installed() -> bool:
    return bool(_ORIGINALS)
