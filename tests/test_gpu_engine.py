"""End-to-end W4A4KV4 Llama: HF plugin boundary, ragged prefill, CUDA-graph decode."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TINY = dict(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
            vocab_size=512)


def _build(capacity=4, max_cache_len=128, seed=3):
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4

    model, cache = build_llama_w4a4kv4(**TINY, capacity=capacity, max_cache_len=max_cache_len, seed=seed)
    return model, cache, BatchedNQKVLlamaRunner(model, cache)


def _prompts(lengths, seed=11):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, TINY["vocab_size"], (n,), generator=gen) for n in lengths]


def test_projections_are_converted_and_backend_installed():
    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear
    from nestquant_aiinfra_b200.hf_backend import BATCHED_NQKV_ATTENTION_NAME

    model, cache, _ = _build()
    fused = [m for m in model.modules() if isinstance(m, FusedNQRTLinear)]
    assert len(fused) == 7 * TINY["num_layers"]
    assert model.config._attn_implementation == BATCHED_NQKV_ATTENTION_NAME
    assert all(m.packed_device_bytes > 0 for m in fused)


def test_prefill_tracks_the_unquantised_model():
    """Last-token logits of the W4A4KV4 prefill stay close to the BF16 model they were quantised from."""
    from transformers import LlamaConfig, LlamaForCausalLM

    model, cache, runner = _build(seed=5)
    prompts = _prompts([5, 21, 40])
    runner.prefill_slots([0, 2, 3], prompts)
    lengths = cache.layer_caches[0].sequence_lengths.tolist()
    assert lengths == [5, 0, 21, 40]
    assert cache.layer_caches[1].page_counts.tolist() == [0, 0, 1, 2]
    assert cache.layer_caches[1].hot_lengths.tolist() == [5, 0, 5, 8]
    config = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=2048,
                         tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    torch.manual_seed(5)
    with torch.device("cuda"):
        reference = LlamaForCausalLM(config).to(torch.bfloat16).eval()
    with torch.no_grad():
        for slot, prompt in zip([0, 2, 3], prompts):
            ids = prompt.cuda().unsqueeze(0)
            expected = reference(input_ids=ids).logits[0, -1].float()
            runner.cache.release_slots([slot])
            model2_logits = None
            # re-run the quantised prefill for this prompt alone and read the logits
            runner.cache.register("probe", slot=slot)
            slot_ids = torch.tensor([slot], dtype=torch.int32, device="cuda")
            q_lens = torch.tensor([prompt.numel()], dtype=torch.int32, device="cuda")
            cache.set_prefill_state(slot_ids=slot_ids, query_lengths=q_lens)
            pos = torch.arange(prompt.numel(), device="cuda").unsqueeze(0)
            model2_logits = model(input_ids=ids, position_ids=pos, past_key_values=cache, use_cache=True).logits[0, -1].float()
            cache.set_decode_state()
            cosine = torch.nn.functional.cosine_similarity(model2_logits, expected, dim=0).item()
            assert cosine > 0.9, cosine


def test_prefill_from_empty_slots_uses_the_chunks_own_kv_and_agrees_with_the_paged_path():
    """Whole-prompt prefill (BF16 K/V of the chunk, as the reference) vs the same prompts through the quantised pages."""
    model, cache, runner = _build(seed=7)
    prompts = _prompts([37, 9, 64], seed=19)
    width = max(p.numel() for p in prompts)
    ids = torch.zeros((3, width), dtype=torch.long, device="cuda")
    for row, prompt in enumerate(prompts):
        ids[row, :prompt.numel()] = prompt.cuda()
    slot_ids = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    q_lens = torch.tensor([p.numel() for p in prompts], dtype=torch.int32, device="cuda")
    pos = torch.arange(width, device="cuda").unsqueeze(0).expand(3, width).contiguous()
    logits, pages = [], []
    for from_empty in (True, False):
        for slot in range(3):
            cache.register(f"probe-{from_empty}-{slot}", slot=slot)
        cache.set_prefill_state(slot_ids=slot_ids, query_lengths=q_lens, from_empty=from_empty)
        with torch.no_grad():
            out = model(input_ids=ids, position_ids=pos, past_key_values=cache, use_cache=True).logits.float()
        cache.set_decode_state()
        logits.append(torch.stack([out[row, int(q_lens[row]) - 1] for row in range(3)]))
        pages.append(cache.layer_caches[0].pool.key_codes[:8].clone())   # layer 0 sees identical inputs either way
        cache.release_slots([0, 1, 2])
    assert torch.equal(pages[0], pages[1])
    cosine = torch.nn.functional.cosine_similarity(logits[0], logits[1], dim=-1)
    assert float(cosine.min()) > 0.97, cosine


def test_bulk_page_writer_of_a_whole_prompt_equals_the_page_by_page_writer():
    """One encoder launch per tensor for all full pages of a chunk vs the append / pack loop: same pool, same metadata."""
    model, cache, runner = _build(capacity=4, max_cache_len=160, seed=13)
    prompts = _prompts([47, 16, 3, 130], seed=29)
    slots = [2, 0, 3, 1]
    width = max(p.numel() for p in prompts)
    ids = torch.zeros((4, width), dtype=torch.long, device="cuda")
    for row, prompt in enumerate(prompts):
        ids[row, :prompt.numel()] = prompt.cuda()
    slot_ids = torch.tensor(slots, dtype=torch.int32, device="cuda")
    lengths = [p.numel() for p in prompts]
    q_lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    pos = torch.arange(width, device="cuda").unsqueeze(0).expand(4, width).contiguous()
    snapshots = []
    for bulk in (True, False):
        for slot in slots:
            cache.register(f"probe-{bulk}-{slot}", slot=slot)
        extra = dict(host_slots=slots, host_lengths=lengths) if bulk else {}
        cache.set_prefill_state(slot_ids=slot_ids, query_lengths=q_lens, from_empty=True, **extra)
        with torch.no_grad():
            model(input_ids=ids, position_ids=pos, past_key_values=cache, use_cache=True)
        cache.set_decode_state()
        state = []
        for layer in cache.layer_caches:
            pool = layer.pool
            hot = [layer.hot_keys[s, :n % 16].clone() for s, n in zip(slots, lengths)]
            hot += [layer.hot_values[s, :n % 16].clone() for s, n in zip(slots, lengths)]
            used = torch.cat([torch.arange(n // 16) + s * cache.max_pages for s, n in zip(slots, lengths)]).cuda()
            state.append([t[used].clone() for t in (pool.key_codes, pool.key_betas, pool.key_norms, pool.value_codes,
                                                    pool.value_betas, pool.value_norms)] + hot +
                         [layer.page_indices.clone(), layer.page_counts.clone(), layer.last_page_len.clone(),
                          layer.hot_lengths.clone(), layer.sequence_lengths.clone()])
        snapshots.append(state)
        cache.release_slots(slots)
    for a, b in zip(*snapshots):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    assert snapshots[0][0][-4].tolist() == [1, 8, 2, 0]   # page counts by slot: 16, 130, 47 and 3 tokens


def test_fused_rope_scope_changes_no_bit(monkeypatch):
    """Rope + Q/K rotation from one launch per tensor vs the stock tensor ops: same tokens, same pages."""
    import contextlib

    import nestquant_aiinfra_b200.engine as engine

    results = []
    for fused in (True, False):
        if not fused:
            monkeypatch.setattr(engine, "fused_rope_scope", lambda: contextlib.nullcontext())
        model, cache, runner = _build(seed=9)
        first = runner.prefill_slots([0, 1, 3], _prompts([33, 4, 50], seed=23))
        tokens = [first.clone()] + [runner.decode_eager().clone() for _ in range(3)]
        results.append((tokens, cache.layer_caches[1].pool.key_codes.clone(), cache.layer_caches[1].hot_keys.clone()))
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.equal(a, b)
    assert torch.equal(results[0][1], results[1][1]) and torch.equal(results[0][2], results[1][2])


def test_graph_decode_equals_eager_decode():
    prompts = _prompts([7, 16, 33, 50])
    outputs = []
    for use_graph in (False, True):
        model, cache, runner = _build(seed=9)
        first = runner.prefill_slots([0, 1, 2, 3], prompts)
        if use_graph:
            runner.capture_decode_graph()
        tokens = [first.clone()]
        for _ in range(20):  # crosses page boundaries for every slot
            tokens.append(runner.decode().clone())
        torch.cuda.synchronize()
        state = [(c.sequence_lengths.clone(), c.page_counts.clone(), c.hot_lengths.clone(), c.hot_keys.clone())
                 for c in cache.layer_caches]
        outputs.append((torch.stack(tokens), state))
    (eager_tokens, eager_state), (graph_tokens, graph_state) = outputs
    assert torch.equal(eager_tokens, graph_tokens)
    for (a, b, c, d), (e, f, g, h) in zip(eager_state, graph_state):
        assert torch.equal(a, e) and torch.equal(b, f) and torch.equal(c, g) and torch.equal(d, h)
    assert eager_state[0][0].tolist() == [27, 36, 53, 70]


def test_weight_decode_ahead_changes_no_bit_of_a_step():
    """Captured decode steps of eight rows or more decode the weights of o / gate-up / down on a second stream
    during the layer's attention: same kernels on the same operands, so tokens, pages and hot tails are equal."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4

    prompts = _prompts([7, 16, 33, 50, 12, 3, 28, 41])
    runs = []
    for ahead in (False, True, True):
        model, cache = build_llama_w4a4kv4(**TINY, capacity=8, max_cache_len=128, seed=9)
        runner = BatchedNQKVLlamaRunner(model, cache, weight_decode_ahead=ahead)
        first = runner.prefill_slots(list(range(8)), prompts)
        runner.capture_decode_graph()
        assert (cache.decode_ahead is not None) == ahead
        tokens = [first.clone()]
        for step in range(24):
            if step == 8 and ahead and len(runs) == 2:   # switched off and on again in the middle of a run
                runner.disable_weight_decode_ahead()
                assert cache.decode_ahead is None
            if step == 16 and ahead and len(runs) == 2:
                assert runner.enable_weight_decode_ahead() > 0
            tokens.append(runner.decode().clone())
        torch.cuda.synchronize()
        if ahead and cache.decode_ahead is not None:
            assert cache.decode_ahead.launches >= 2 * TINY["num_layers"]
            assert len(cache.decode_ahead.layers[0]) == 3       # o_proj, gate/up (stacked), down_proj
        pools = [(c.pool.key_codes.clone(), c.pool.value_codes.clone(), c.hot_keys.clone()) for c in cache.layer_caches]
        runs.append((torch.stack(tokens), pools))
    for tokens, pools in runs[1:]:
        assert torch.equal(tokens, runs[0][0])
        for a, b in zip(runs[0][1], pools):
            assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_opt_in_decoded_copies_keep_the_generated_tokens():
    """Lattice pages change no bit of a step; resident weights only the order of FP32 sums in the projections.

    Both are switched on in the middle of a graph decode (the runner captures its graph again), across page
    boundaries, and compared with an untouched run of the same model.
    """
    prompts = _prompts([7, 16, 33, 50])
    runs = []
    for mode in ("packed", "lattice", "resident"):
        model, cache, runner = _build(seed=9)
        first = runner.prefill_slots([0, 1, 2, 3], prompts)
        runner.capture_decode_graph()
        tokens = [first.clone()]
        for step in range(24):
            if step == 6 and mode == "lattice":
                assert runner.enable_lattice_shadow() > 0
            if step == 6 and mode == "resident":
                assert runner.keep_decoded_weights() > 0
            tokens.append(runner.decode().clone())
        torch.cuda.synchronize()
        pools = [(c.pool.key_codes.clone(), c.pool.value_codes.clone(), c.hot_keys.clone()) for c in cache.layer_caches]
        runs.append((torch.stack(tokens), pools, cache))
    (packed_tokens, packed_pools, _), (lattice_tokens, lattice_pools, lattice_cache), (resident_tokens, _, _) = runs
    assert torch.equal(lattice_tokens, packed_tokens)
    for a, b in zip(packed_pools, lattice_pools):
        assert all(torch.equal(x, y) for x, y in zip(a, b))
    # the shadow of every page written before and after the switch is the decode of its codes
    for layer in lattice_cache.layer_caches:
        pool = layer.pool
        fresh = torch.zeros_like(pool.key_lattice)
        saved, pool.key_lattice = pool.key_lattice, fresh
        pool.expand_pages(torch.arange(pool.capacity, dtype=torch.int32))
        assert torch.equal(fresh, saved)
        pool.key_lattice = saved
    # resident weights: same operands, sums in another order; greedy tokens of a random-init model may flip on
    # near-ties, so compare the first steps after the switch only through agreement of most rows
    agree = (resident_tokens == packed_tokens).float().mean().item()
    assert agree > 0.9, agree


def test_released_slot_is_reused_and_inactive_rows_do_not_move():
    model, cache, runner = _build(seed=1)
    runner.prefill_slots([1], _prompts([9]))
    runner.capture_decode_graph()
    for _ in range(3):
        runner.decode()
    assert cache.layer_caches[0].sequence_lengths.tolist() == [0, 12, 0, 0]
    cache.release_slots([1])
    runner.prefill_slots([1, 3], _prompts([4, 18], seed=2))
    runner.decode()
    torch.cuda.synchronize()
    assert cache.layer_caches[0].sequence_lengths.tolist() == [0, 5, 0, 19]
    with pytest.raises(RuntimeError):
        cache.register("again", slot=3)


def test_tp_shard_runs_single_rank():
    """world = 1 shard of a tiny architecture: row-parallel modules, synthetic KV fill, graph decode."""
    from nestquant_aiinfra_b200.tensor_parallel import RowParallelNQRTLinear
    from nestquant_aiinfra_b200.tp_engine import TensorParallelRunner, build_llama_tp_shard, fill_cache_synthetic

    model, cache = build_llama_tp_shard(hidden_size=256, intermediate_size=7 * 64, num_layers=2, num_heads=4,
                                        num_kv_heads=2, head_dim=64, vocab_size=512, rank=0, world=1, capacity=3,
                                        max_cache_len=96, device="cuda")
    rows = [m for m in model.modules() if isinstance(m, RowParallelNQRTLinear)]
    assert len(rows) == 4 and {m.hadamard_block for m in rows} == {256, 64}   # 448 = 7 * 64
    fill_cache_synthetic(cache, 37)
    assert cache.layer_caches[1].page_counts.tolist() == [2, 2, 2] and cache.layer_caches[1].hot_lengths.tolist() == [5, 5, 5]
    runner = TensorParallelRunner(model, cache)
    runner.start_decode(37)
    eager = [runner.decode_eager().clone() for _ in range(3)]
    fill_cache_synthetic(cache, 37)
    runner.start_decode(37)
    runner.capture_decode_graph()
    graph = [runner.decode().clone() for _ in range(3)]
    assert all(torch.equal(a, b) for a, b in zip(eager, graph))
    assert cache.layer_caches[0].sequence_lengths.tolist() == [40, 40, 40]



def test_a_slot_at_its_cache_limit_cannot_touch_its_neighbour():
    """Static page ids are ``slot * max_pages + page``: a slot whose page table is full must stop packing, or its next
    id would be the first page of the following slot.  Slot 0 decodes far past the cache length; slot 1's pages, hot
    tail and attention output must not change."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4

    model, cache = build_llama_w4a4kv4(hidden_size=256, intermediate_size=512, num_layers=1, num_heads=4, num_kv_heads=2,
                                       head_dim=64, vocab_size=128, capacity=2, max_cache_len=32, seed=5)
    assert cache.max_pages == 2
    runner = BatchedNQKVLlamaRunner(model, cache)
    gen = torch.Generator().manual_seed(9)
    runner.prefill_slots([0, 1], [torch.randint(0, 128, (n,), generator=gen) for n in (30, 20)])  # ids inside this model's vocabulary
    layer = cache.layer_caches[0]
    pool = layer.pool
    before = [t.clone() for t in (pool.key_codes[2:4], pool.value_codes[2:4], pool.key_norms[2:4],
                                  layer.hot_keys[1], layer.hot_values[1], layer.page_indices[1])]
    cache.active_mask[1] = False          # only slot 0 decodes
    for _ in range(40):                   # 30 + 40 tokens: well past 2 pages + a full hot tail
        runner.decode_eager()
    torch.cuda.synchronize()
    assert int(layer.page_counts[0]) == 2 and int(layer.hot_lengths[0]) == 16   # saturated, nothing published beyond the table
    assert int(layer.sequence_lengths[0]) == 48 and int(layer.sequence_lengths[1]) == 20
    after = (pool.key_codes[2:4], pool.value_codes[2:4], pool.key_norms[2:4], layer.hot_keys[1], layer.hot_values[1],
             layer.page_indices[1])
    for a, b in zip(after, before):
        assert torch.equal(a, b)


def test_device_side_page_allocation_matches_static_ids_with_a_smaller_pool():
    """Pages popped from the device-side free stack instead of ``slot * max_pages + page``: same tokens and page
    contents as the static partition from a pool a third of its size; a released slot gives its pages back; the
    admission budget refuses what the pool could not hold.  Eager steps and replays of a captured graph."""
    import pytest

    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4

    common = dict(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                  vocab_size=128, capacity=4, max_cache_len=256, seed=7)        # static pool: 4 x 16 = 64 pages
    gen = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, 128, (n,), generator=gen) for n in (45, 9, 70)]
    slots = [0, 2, 3]
    tokens, caches = {}, {}
    for mode, extra in (("static", {}), ("device", dict(page_allocation="device", pool_pages=24))):
        model, cache = build_llama_w4a4kv4(**common, **extra)
        runner = BatchedNQKVLlamaRunner(model, cache)
        seen = [runner.prefill_slots(slots, prompts, max_tokens=112).clone()]   # budget: 7 pages each, 21 of the 24
        seen += [runner.decode_eager().clone() for _ in range(12)]              # eager steps across page boundaries
        runner.capture_decode_graph()
        seen += [runner.decode().clone() for _ in range(14)]                    # graph replays across more of them
        tokens[mode], caches[mode] = seen, cache
        if mode == "static":
            continue
    for a, b in zip(tokens["static"], tokens["device"]):
        assert torch.equal(a, b)
    static, device = caches["static"], caches["device"]
    for ls, ld in zip(static.layer_caches, device.layer_caches):
        assert torch.equal(ls.page_counts, ld.page_counts) and torch.equal(ls.hot_lengths, ld.hot_lengths)
        in_use = int(ld.page_counts.sum())
        assert ld.pool.allocated_pages == in_use and int(ld.pool.free_count) == 24 - in_use
        for slot in slots:
            for position in range(int(ld.page_counts[slot])):
                sid, did = int(ls.page_indices[slot, position]), int(ld.page_indices[slot, position])
                assert sid == slot * 16 + position and 0 <= did < 24
                assert torch.equal(ls.pool.key_codes[sid], ld.pool.key_codes[did])
                assert torch.equal(ls.pool.value_norms[sid], ld.pool.value_norms[did])
        ids = ld.page_indices[ld.page_indices >= 0].tolist()
        assert len(set(ids)) == len(ids) == in_use                                # no page handed out twice
    held = int(device.layer_caches[0].page_counts[3])
    device.release_slots([3])
    for layer in device.layer_caches:
        assert layer.page_indices[3].tolist() == [-1] * 16 and int(layer.sequence_lengths[3]) == 0
        assert layer.pool.allocated_pages == int(layer.page_counts.sum())
        free = layer.pool.free_ids[:int(layer.pool.free_count)].tolist()
        assert len(set(free)) == len(free) and not set(free) & set(layer.page_indices[layer.page_indices >= 0].tolist())
    assert held > 0
    device.register("late", slot=3, max_tokens=96)          # 7 + 7 + 6 = 20 pages of budget: fits the 24
    with pytest.raises(RuntimeError, match="exhausted"):
        device.register("too much", slot=1, max_tokens=80)   # 5 more pages do not


def test_producers_fused_into_the_projections_change_no_token():
    """Norms deferred into the q/k/v and gate/up encoder launch, SiLU * up inside down_proj's: same greedy tokens
    through a ragged prefill and eager + graph decode as with the separate launches, and fewer launches per step."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4
    from nestquant_aiinfra_b200.norm import FusedRMSNorm, FusedSiluMLP
    from nestquant_aiinfra_b200.runtime import launch_count

    common = dict(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                  vocab_size=128, capacity=4, max_cache_len=128, seed=11)
    gen = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, 128, (n,), generator=gen) for n in (17, 40, 5)]
    tokens, launches = {}, {}
    for fused in (False, True):
        model, cache = build_llama_w4a4kv4(**common, fuse_producers=fused)
        layer = model.model.layers[0]
        assert isinstance(layer.mlp, FusedSiluMLP) == fused
        assert isinstance(layer.input_layernorm, FusedRMSNorm) and layer.input_layernorm.defer == fused
        assert not model.model.norm.defer                       # the final norm feeds the dense lm_head
        runner = BatchedNQKVLlamaRunner(model, cache)
        seen = [runner.prefill_slots([0, 1, 3], prompts).clone()]
        before = launch_count()
        seen.append(runner.decode_eager().clone())
        launches[fused] = launch_count() - before
        seen += [runner.decode_eager().clone() for _ in range(3)]
        runner.capture_decode_graph()
        seen += [runner.decode().clone() for _ in range(4)]
        tokens[fused] = seen
    for a, b in zip(tokens[False], tokens[True]):
        assert torch.equal(a, b)
    assert launches[True] < launches[False]
