"""Drop-in surface on the CPU: converter behaviour, the install() rebinding, and signature conformance.

The reference package is imported from oracle/_ref when it is installed there (the tests that need it
are skipped otherwise); nothing here launches a kernel.
"""

import inspect
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch
from torch import nn

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "oracle" / "_ref"
needs_reference = pytest.mark.skipif(not (REF / "nestquant" / "runtime" / "inference_engine.py").exists(),
                                     reason="the reference is not installed under oracle/_ref")


@pytest.fixture()
def reference():
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import nestquant  # noqa: F401

    return nestquant


# --------------------------------------------------------------------------------------------- converter
class _Reader:
    def __init__(self, shapes, rotated):
        self.shapes = shapes
        self.model_metadata = {"hadamard_rotation": {"format": "local_hadamard_linear_v1",
                                                     "converted_linear_names": list(rotated)}}

    def get_entry(self, name):
        return SimpleNamespace(kind="nestquant", shape=self.shapes[name])

    def read_named_record(self, name):
        raise AssertionError("conversion must not read any record (modules prepare lazily)")


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn = nn.Module()
        for leaf, out in (("q_proj", 64), ("k_proj", 32), ("v_proj", 32), ("o_proj", 64)):
            setattr(self.self_attn, leaf, nn.Linear(64, out, bias=False))
        self.mlp = nn.Module()
        self.mlp.gate_proj, self.mlp.up_proj = nn.Linear(64, 128, bias=False), nn.Linear(64, 128, bias=False)
        self.mlp.down_proj = nn.Linear(128, 64, bias=False)


def _model_and_reader():
    model = nn.Module()
    model.layers = nn.ModuleList([_Block()])
    names = [n for n, m in model.named_modules() if isinstance(m, nn.Linear)]
    shapes = {f"{n}.weight": tuple(dict(model.named_modules())[n].weight.shape) for n in names}
    rotated = [n for n in names if not n.endswith("down_proj")]
    return model, _Reader(shapes, rotated), names


BETAS = (0.25, 0.5, 0.75, 1.0)


def test_converter_follows_the_reference_call_and_infers_the_sharing_groups():
    from nestquant_aiinfra_b200.fused_linear import (FusedNQRTConversionReport, FusedNQRTLinear,
                                                     convert_linears_to_fused_nqrt_)

    model, reader, names = _model_and_reader()
    # the call scripts/serve_w4a4kv4.py makes
    report = convert_linears_to_fused_nqrt_(
        model, reader, names, output_dtype=torch.bfloat16, group_qkv=False, compute_backend="packed_w4a4_cuda_mma",
        activation_betas=BETAS, enable_m1_down_splitk=True, m1_down_splitk_fallback_names=("layers.0.mlp.down_proj",))
    assert isinstance(report, FusedNQRTConversionReport)
    assert report.replaced_linear_names == tuple(sorted(names))
    assert "layers.0.mlp.down_proj" not in report.input_hadamard_names   # not listed in the checkpoint metadata
    assert set(map(frozenset, report.shared_hadamard_groups)) == {
        frozenset(f"layers.0.self_attn.{x}_proj" for x in "qkv"),
        frozenset(f"layers.0.mlp.{x}_proj" for x in ("gate", "up"))}
    assert report.m1_down_splitk_fallback_names == ("layers.0.mlp.down_proj",)
    block = model.layers[0]
    q, k, v = block.self_attn.q_proj, block.self_attn.k_proj, block.self_attn.v_proj
    assert all(isinstance(m, FusedNQRTLinear) for m in (q, k, v, block.mlp.down_proj))
    assert q.packed_activation_cache is k.packed_activation_cache is v.packed_activation_cache is not None
    assert q.input_transform_cache is v.input_transform_cache and q.input_transform_cache.uses_per_input == 3
    assert block.mlp.gate_proj.packed_activation_cache is block.mlp.up_proj.packed_activation_cache
    assert block.self_attn.o_proj.packed_activation_cache is None and block.self_attn.o_proj.input_hadamard
    assert not block.mlp.down_proj.input_hadamard and not block.mlp.down_proj.enable_m1_down_splitk
    assert q.output_dtype == torch.bfloat16 and q.enable_m1_down_splitk


def test_converter_rejects_bad_calls_and_leaves_the_model_untouched():
    from nestquant_aiinfra_b200.fused_linear import convert_linears_to_fused_nqrt_

    model, reader, names = _model_and_reader()
    with pytest.raises(TypeError):
        convert_linears_to_fused_nqrt_(model, reader, names, activation_betas=BETAS, share_groups=())  # no stray kwargs
    with pytest.raises(TypeError):
        convert_linears_to_fused_nqrt_(model, reader, "layers.0.mlp.down_proj", activation_betas=BETAS)
    with pytest.raises(ValueError, match="unique"):
        convert_linears_to_fused_nqrt_(model, reader, names + names[:1], activation_betas=BETAS)
    with pytest.raises(ValueError, match="compute_backend"):
        convert_linears_to_fused_nqrt_(model, reader, names, compute_backend="tensor_core_dot", activation_betas=BETAS)
    with pytest.raises(ValueError, match="activation_betas"):
        convert_linears_to_fused_nqrt_(model, reader, names)
    with pytest.raises(ValueError, match="included in include_names"):
        convert_linears_to_fused_nqrt_(model, reader, names[:2], activation_betas=BETAS, w4a4_tiled_fallback_names=names[3:4])
    with pytest.raises(ValueError, match="enable_m1_down_splitk"):
        convert_linears_to_fused_nqrt_(model, reader, names, activation_betas=BETAS, m1_down_splitk_fallback_names=names[:1])
    reader.shapes[f"{names[-1]}.weight"] = (1, 1)   # the LAST module is wrong: nothing may have been replaced
    with pytest.raises(ValueError, match="shape mismatch"):
        convert_linears_to_fused_nqrt_(model, reader, names, activation_betas=BETAS)
    assert all(isinstance(m, nn.Linear) for m in (model.layers[0].self_attn.q_proj, model.layers[0].mlp.down_proj))
    reader.model_metadata = {"hadamard_rotation": {"format": "something else"}}
    with pytest.raises(ValueError, match="Hadamard"):
        convert_linears_to_fused_nqrt_(model, reader, names[:1], activation_betas=BETAS)


def test_shared_caches_serve_every_consumer_once():
    from nestquant_aiinfra_b200.fused_linear import SharedHadamardCache

    cache = SharedHadamardCache(3)
    x = torch.randn(2, 16)
    with torch.no_grad():
        first = cache.transform(x)
        assert cache.transform(x) is first and cache.transform(x) is first
        assert (cache.hits, cache.misses) == (2, 1)
        assert cache.transform(x) is not first and cache.misses == 2   # the entry was dropped after the third use
        other = torch.randn(2, 16)
        assert cache.transform(other) is not first and cache.misses == 3
    with pytest.raises(RuntimeError):
        cache.transform(x)   # grad mode
    with pytest.raises(ValueError):
        SharedHadamardCache(1)


# --------------------------------------------------------------------------------------------- install()
@needs_reference
def test_install_rebinds_the_reference_symbols_and_uninstall_restores_them(reference):
    import nestquant.models.fused_linear as ref_fused
    import nestquant.runtime as ref_rt
    import nestquant.runtime.nqkv_batched_runner as ref_runner

    from nestquant_aiinfra_b200 import fused_linear, hf_backend, install as dropin
    from nestquant_aiinfra_b200.runtime import w4a4

    before = (ref_rt.quantize_activation_cuda, ref_runner.BatchedNQKVLlamaCache, ref_fused.FusedNQRTLinear)
    rebound = dropin.install()
    try:
        assert dropin.installed()
        assert ref_rt.quantize_activation_cuda is w4a4.quantize_activation_cuda
        assert ref_rt.linear_packed_w4a4_mma_chunked_staged is w4a4.linear_packed_w4a4_mma_chunked_staged
        assert ref_runner.BatchedNQKVLlamaCache is hf_backend.BatchedNQKVLlamaCache
        assert ref_fused.FusedNQRTLinear is fused_linear.FusedNQRTLinear
        assert ref_fused.convert_linears_to_fused_nqrt_ is fused_linear.convert_linears_to_fused_nqrt_
        assert "nestquant.runtime.nqkv_batched_hf_backend" in rebound
        with pytest.raises(RuntimeError):
            dropin.install()
    finally:
        dropin.uninstall()
    assert (ref_rt.quantize_activation_cuda, ref_runner.BatchedNQKVLlamaCache, ref_fused.FusedNQRTLinear) == before
    assert not dropin.installed()


# --------------------------------------------------------------------------------------------- signatures
def _parameters(function):
    return [(p.name, p.kind) for p in inspect.signature(function).parameters.values() if p.name != "self"]


def _accepts_the_calls_of(mine, reference) -> bool:
    """Every parameter of the reference function exists here with the same kind and order; anything this
    package adds is keyword-only with a default, so no call written for the reference changes meaning."""
    ours = [p for p in inspect.signature(mine).parameters.values() if p.name != "self"]
    theirs = _parameters(reference)
    if [(p.name, p.kind) for p in ours[:len(theirs)] if (p.name, p.kind) in theirs] != theirs and \
            [(p.name, p.kind) for p in ours if (p.name, p.kind) in theirs] != theirs:
        return False
    extras = [p for p in ours if (p.name, p.kind) not in theirs]
    return all(p.kind is p.KEYWORD_ONLY and p.default is not p.empty for p in extras)


@needs_reference
def test_cache_and_runner_expose_the_reference_protocol(reference):
    from nestquant.runtime.inference_engine import RaggedDecodeBackend
    from nestquant.runtime.nqkv_batched_hf_backend import BatchedNQKVLlamaCache as RefCache
    from nestquant.runtime.nqkv_batched_runner import BatchedNQKVLlamaRunner as RefRunner

    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner
    from nestquant_aiinfra_b200.hf_backend import BatchedNQKVLlamaCache

    for name in ("set_batch_state", "set_decode_execution_state", "set_prefill_execution_state", "enable_graph_decode",
                 "disable_graph_decode", "finish_prefill_page_transaction", "register", "register_batch",
                 "release_slots", "attend"):
        assert _accepts_the_calls_of(getattr(BatchedNQKVLlamaCache, name), getattr(RefCache, name)), name
    for name in ("graph_decode_enabled", "max_cache_len", "batch_size", "is_compileable"):
        assert isinstance(getattr(BatchedNQKVLlamaCache, name), property), name
    assert _accepts_the_calls_of(BatchedNQKVLlamaCache.__init__, RefCache.__init__)
    # every call the engine protocol makes binds against this runner's signatures, with the protocol's keywords
    t = object()
    for name in ("prefill", "prefill_slots", "capture", "decode", "clear_slots"):
        protocol = inspect.signature(getattr(RaggedDecodeBackend, name))
        keywords = {p.name: t for p in protocol.parameters.values() if p.kind is p.KEYWORD_ONLY}
        positional = [t for p in protocol.parameters.values() if p.kind is p.POSITIONAL_OR_KEYWORD and p.name != "self"]
        inspect.signature(getattr(BatchedNQKVLlamaRunner, name)).bind(t, *positional, **keywords)
        assert _parameters(getattr(RefRunner, name))  # the reference runner has the same entry
    assert _parameters(BatchedNQKVLlamaRunner.clear_slots) == _parameters(RefRunner.clear_slots)
    assert _parameters(BatchedNQKVLlamaRunner.capture) == _parameters(RefRunner.capture)


@needs_reference
def test_converter_has_the_reference_signature(reference):
    from nestquant.models.fused_linear import convert_linears_to_fused_nqrt_ as ref_convert

    from nestquant_aiinfra_b200.fused_linear import convert_linears_to_fused_nqrt_

    assert _parameters(convert_linears_to_fused_nqrt_) == _parameters(ref_convert)
