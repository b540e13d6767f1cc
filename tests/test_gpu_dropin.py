"""The reference's own control plane on top of this package's kernels (GPU).

Needs the reference installed under oracle/_ref (tests are skipped otherwise): its
ContinuousBatchInferenceEngine drives this package's runner through the RaggedDecodeBackend protocol,
its BatchedNQKVLlamaRunner drives this package's cache after install(), and a checkpoint written and
read by the reference's NQMC code feeds convert_linears_to_fused_nqrt_.
"""

import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import ACT_BETAS, MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro, rng

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "oracle" / "_ref"
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "nestquant" / "runtime" / "inference_engine.py").exists(),
                                 reason="the reference is not installed under oracle/_ref")]


@pytest.fixture(scope="module")
def reference():
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import nestquant  # noqa: F401

    return nestquant


def _tiny(capacity=4, max_cache_len=96, layers=2):
    from nestquant_aiinfra_b200.engine import build_llama_w4a4kv4

    return build_llama_w4a4kv4(hidden_size=256, intermediate_size=512, num_layers=layers, num_heads=4, num_kv_heads=2,
                               head_dim=64, vocab_size=128, capacity=capacity, max_cache_len=max_cache_len, seed=3)


def _requests(reference, spec):
    from nestquant.runtime.continuous_batching import DecodeRequest

    gen = rng(11)
    return [DecodeRequest(f"r{i}", tuple(torch.randint(1, 128, (prompt,), generator=gen).tolist()), new)
            for i, (prompt, new) in enumerate(spec)]


def _run(engine, requests, limit=400):
    for request in requests:
        engine.submit(request)
    steps = 0
    while engine.has_work():
        engine.step()
        steps += 1
        assert steps < limit, "the engine did not drain"
    return steps


def test_reference_engine_drives_this_runner_through_a_continuous_batch(reference):
    """More requests than slots, different prompt and output lengths: requests finish, release their slot and new
    ones join while the others keep decoding (one captured graph; full pages packed inside it)."""
    from nestquant.runtime.continuous_batching import RequestStatus
    from nestquant.runtime.inference_engine import ContinuousBatchInferenceEngine

    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner

    model, cache = _tiny()
    runner = BatchedNQKVLlamaRunner(model, cache)
    engine = ContinuousBatchInferenceEngine(runner, pad_token_id=0)
    requests = _requests(reference, [(3, 20), (40, 4), (17, 33), (5, 2), (31, 18), (9, 9), (16, 17)])
    _run(engine, requests)
    for request in requests:
        assert request.status is RequestStatus.FINISHED
        assert len(request.generated_token_ids) == request.max_new_tokens
        assert all(0 <= t < 128 for t in request.generated_token_ids)
    assert runner.graph_captured and runner.graph_replay_count > 0 and runner.compact_prefill_calls > 0
    assert cache.manager.active_requests == 0
    for layer in cache.manager.layer_caches:
        assert layer.cold_cache.pool.allocated_pages == 0 and layer.hot_lengths.tolist() == [0] * 4
    from nestquant_aiinfra_b200.runtime import read_status

    assert read_status() == 0


def test_reference_engine_gets_the_same_tokens_with_the_weight_decode_ahead(reference):
    """Eight slots, so that the logits graph of the engine protocol decodes weights on the second stream: the
    reference's engine generates exactly the tokens it generates with every step on one stream."""
    from nestquant.runtime.inference_engine import ContinuousBatchInferenceEngine

    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner

    spec = [(3, 20), (40, 4), (17, 33), (5, 2), (31, 18), (9, 9), (16, 17), (22, 25), (7, 30), (12, 6), (28, 11)]
    generated = []
    for ahead in (False, True):
        model, cache = _tiny(capacity=8)
        runner = BatchedNQKVLlamaRunner(model, cache, weight_decode_ahead=ahead)
        engine = ContinuousBatchInferenceEngine(runner, pad_token_id=0)
        requests = _requests(reference, spec)
        _run(engine, requests)
        assert runner.graph_captured and (cache.decode_ahead is not None) == ahead
        if ahead:
            assert cache.decode_ahead.launches > 0
        generated.append([tuple(r.generated_token_ids) for r in requests])
    assert generated[0] == generated[1]
    from nestquant_aiinfra_b200.runtime import read_status

    assert read_status() == 0


def test_engine_protocol_prefill_equals_the_device_sampling_path(reference):
    """Same rows, same widths, same kernels: the protocol's logits give the tokens the device-side path samples,
    and both leave the same pages and hot tails behind."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner

    model, cache = _tiny()
    runner = BatchedNQKVLlamaRunner(model, cache, prefill_logits="last")
    lengths = [37, 37, 37, 37]
    prompts = [torch.randint(1, 128, (n,), generator=rng(50 + i)) for i, n in enumerate(lengths)]
    direct = runner.prefill_slots([0, 1, 2, 3], prompts).clone()
    state = [(l.page_counts.clone(), l.hot_lengths.clone(), l.pool.key_codes.clone(), l.hot_values.clone())
             for l in cache.layer_caches]
    cache.release_slots([0, 1, 2, 3])
    runner._prepared = True  # the engine's dummy warm-up is not needed for this comparison
    ids = torch.stack(prompts).cuda()
    positions = torch.arange(37, device="cuda").expand(4, -1).contiguous()
    mask = torch.ones(4, 37, dtype=torch.bool, device="cuda")
    logits = runner.prefill_slots(ids, positions=positions, write_mask=mask,
                                  valid_lengths=torch.full((4,), 37, device="cuda"))
    # "last" policy: one row of logits per request (the lm_head runs on the same [4, hidden] rows as in the
    # device-sampling path), aliased over the width
    assert tuple(logits.shape) == (4, 37, 128) and logits.stride(1) == 0
    assert torch.equal(logits[:, -1].argmax(dim=-1), direct)
    for layer, (counts, hot, codes, values) in zip(cache.layer_caches, state):
        assert torch.equal(layer.page_counts, counts) and torch.equal(layer.hot_lengths, hot)
        assert torch.equal(layer.pool.key_codes, codes) and torch.equal(layer.hot_values, values)
    # "all" policy: the logits of every position, as the reference returns them
    cache.release_slots([0, 1, 2, 3])
    runner.prefill_logits = "all"
    full = runner.prefill_slots(ids, positions=positions, write_mask=mask, valid_lengths=torch.full((4,), 37, device="cuda"))
    assert tuple(full.shape) == (4, 37, 128) and full.stride(1) == 128
    assert torch.allclose(full[:, 36].float(), logits[:, 36].float(), atol=2e-2, rtol=2e-2)


def test_forward_failure_after_kv_writes_releases_the_rows(reference):
    """Host-side failure injection: the decoder stack raises AFTER it has written K/V; the affected requests
    must be gone and their pages free (the reference's transactional prefill behaves the same way)."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner

    model, cache = _tiny(capacity=2)
    runner = BatchedNQKVLlamaRunner(model, cache)
    runner.prefill(torch.tensor([[1, 2, 3], [4, 5, 6]], device="cuda"))
    assert cache.manager.active_requests == 2
    inner = model.model
    original = inner.forward

    def failing(this, *args, **kwargs):
        original(*args, **kwargs)
        raise RuntimeError("injected post-KV failure")

    inner.forward = types.MethodType(failing, inner)
    try:
        mask = torch.ones((2, 20), device="cuda", dtype=torch.bool)
        with pytest.raises(RuntimeError, match="injected post-KV failure"):
            runner.prefill_slots(torch.randint(1, 128, (2, 20), generator=rng(1)).cuda(),
                                 positions=torch.arange(3, 23, device="cuda").expand(2, -1).contiguous(),
                                 write_mask=mask, valid_lengths=torch.full((2,), 23, device="cuda", dtype=torch.long))
    finally:
        inner.forward = original
    assert cache.manager.active_requests == 0
    for layer in cache.manager.layer_caches:
        assert layer.cold_cache.pool.allocated_pages == 0
        assert layer.cold_cache.page_counts.tolist() == [0, 0] and layer.sequence_lengths.tolist() == [0, 0]
    # the runner stays usable
    mask = torch.ones((2, 5), device="cuda", dtype=torch.bool)
    logits = runner.prefill_slots(torch.randint(1, 128, (2, 5), generator=rng(2)).cuda(),
                                  positions=torch.arange(5, device="cuda").expand(2, -1).contiguous(),
                                  write_mask=mask, valid_lengths=torch.full((2,), 5, device="cuda", dtype=torch.long))
    assert torch.isfinite(logits.float()).all() and cache.manager.active_requests == 2


def test_reference_runner_and_engine_on_this_cache_after_install(reference):
    """install() rebinds the reference's symbols: its BatchedNQKVLlamaRunner (graph pool, boundary graphs, host
    page reservations) then runs on this package's cache class and kernels, unchanged."""
    from nestquant_aiinfra_b200 import install as dropin

    dropin.install()
    try:
        from nestquant.runtime.continuous_batching import RequestStatus
        from nestquant.runtime.inference_engine import ContinuousBatchInferenceEngine
        from nestquant.runtime.nqkv_batched_runner import BatchedNQKVLlamaRunner as ReferenceRunner

        model, cache = _tiny(capacity=2, max_cache_len=64)
        runner = ReferenceRunner(model, cache)
        engine = ContinuousBatchInferenceEngine(runner, pad_token_id=0)
        requests = _requests(reference, [(5, 20), (19, 6), (14, 21)])
        _run(engine, requests)
        for request in requests:
            assert request.status is RequestStatus.FINISHED and len(request.generated_token_ids) == request.max_new_tokens
        assert runner.graph_captured and sum(runner.graph_replay_counts.values()) > 0
        assert runner.graph_boundary_replay_count > 0     # a 16-token page filled during decode
        assert cache.manager.active_requests == 0
        for layer in cache.manager.layer_caches:
            assert layer.cold_cache.pool.allocated_pages == 0
    finally:
        dropin.uninstall()


def test_checkpoint_written_by_the_reference_feeds_the_converter(reference, oracle, tmp_path):
    """NQMC container written and read by the reference's own code (CPU), converted by this package."""
    from nestquant.core.codec import generate_e8_dither_stateless
    from nestquant.core.model_checkpoint import PackedNestQuantModel
    from nestquant.core.model_checkpoint_file import NQMCFileReader
    from nestquant.core.quantizer import quantize_rows
    from nestquant.core.rotation import hadamard
    from nestquant.core.tensor_checkpoint import PackedNestQuantTensor
    from nestquant.models.rotated_linear import PAPER_HADAMARD_FORMAT
    from torch import nn

    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear, convert_linears_to_fused_nqrt_

    torch.manual_seed(0)
    model = nn.Module()
    model.block = nn.Module()
    model.block.q_proj, model.block.k_proj = nn.Linear(256, 128, bias=False), nn.Linear(256, 64, bias=False)
    model.block.down_proj = nn.Linear(512, 256, bias=False)
    names = ("block.q_proj", "block.k_proj", "block.down_proj")
    state, records, betas = dict(model.state_dict()), {}, (0.5, 0.75, 1.0, 1.25)
    for offset, name in enumerate(names):
        tensor_name = f"{name}.weight"
        stored = hadamard(state[tensor_name])
        seed = 20261101 + offset
        dither = generate_e8_dither_stateless(stored.numel() // 8, seed).to(stored.dtype).reshape(
            stored.shape[0], stored.shape[1] // 8, 8)
        records[tensor_name] = PackedNestQuantTensor.from_quantized_rows(
            tensor_name, quantize_rows(stored, q=14, betas=betas, dither=dither), dither_seed=seed)
        state[tensor_name] = stored
    path = tmp_path / "tiny.nqmc"
    PackedNestQuantModel.from_state_dict(state, records, model_metadata={"hadamard_rotation": {
        "format": PAPER_HADAMARD_FORMAT, "converted_linear_names": list(names), "skipped_tied_linear_names": [],
        "skipped_non_power_of_two_linear_names": [], "weight_storage": "source_model_dtype"}}).write_to_file(path)
    reader = NQMCFileReader(path)
    model.cuda()
    report = convert_linears_to_fused_nqrt_(model, reader, names, output_dtype=torch.float32,
                                            compute_backend="packed_w4a4_cuda_mma", activation_betas=ACT_BETAS)
    assert report.input_hadamard_names == tuple(sorted(names))
    assert report.shared_hadamard_groups == (("block.k_proj", "block.q_proj"),)
    for name, m in ((names[0], 9), (names[2], 40)):
        module = dict(model.named_modules())[name]
        assert isinstance(module, FusedNQRTLinear)
        k = module.in_features
        x = torch.randn(m, k, generator=rng(7 + m)).bfloat16()
        with torch.no_grad():
            actual = module(x.cuda()).cpu().numpy()
        assert actual.dtype == np.float32
        # expected from the reference's own dequantisation of the record it wrote
        w_deq = records[f"{name}.weight"].dequantize().float().numpy()
        x_rot = oracle.hadamard(x.float().numpy(), round_bf16=True)
        ac, ab, an = oracle.encode_packed(x_rot, ACT_BETAS)
        a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
        expected = oracle.gemm_bf16_operands(a_deq, w_deq)
        assert max_abs(actual, expected) <= MAX_ABS_TOL and rel_fro(actual, expected) <= REL_FRO_TOL, \
            (name, max_abs(actual, expected), rel_fro(actual, expected))
