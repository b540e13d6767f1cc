"""GPU parity of the NQKV4 writers and the paged attention (through the C ABI).

Bit-exact gates: page payloads against the CPU checker and the committed reference vectors.
Tolerance gates: attention outputs, max abs <= 1e-2 and relative Frobenius <= 1e-3 against the
float64 softmax over the float32-dequantised pages.
"""

import numpy as np
import pytest
import torch

from helpers import KEY_BETAS, MAX_ABS_TOL, REL_FRO_TOL, VALUE_BETAS, max_abs, rel_fro, rng

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    assert torch.cuda.is_available()
    import nestquant_aiinfra_b200.runtime as runtime

    return runtime


def make_cache(rt, *, slots, max_pages, heads=8, dim=64, capacity=None, page=16):
    pool = rt.NQKVPagePool(capacity=capacity or slots * max_pages, page_size=page, num_kv_heads=heads, head_dim=dim,
                           key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    return rt.NQKVHotColdCache(pool, max_sequences=slots, max_pages_per_sequence=max_pages)


def fill_cache(rt, cache, lengths, seed, *, permute=True):
    """Write `lengths[s]` tokens per slot: full pages through the eager page writer, the rest hot."""
    pool = cache.pool
    page, heads, dim = pool.page_size, pool.num_kv_heads, pool.head_dim
    ids = torch.randperm(pool.capacity, generator=rng(seed)).tolist() if permute else list(range(pool.capacity))
    kv = {}
    for slot, length in enumerate(lengths):
        if length is None:
            continue
        cache.register(slot)
        k = torch.randn(length, heads, dim, generator=rng(seed + 10 * slot + 1))
        v = torch.randn(length, heads, dim, generator=rng(seed + 10 * slot + 2))
        k[:, 1 % heads, 5] *= 8.0
        v[:, 0, 17] *= 8.0
        k, v = k.bfloat16().cuda(), v.bfloat16().cuda()
        kv[slot] = (k, v)
        full = length // page
        for p in range(full):
            pid = ids.pop()
            prepared = rt.quantize_nqkv_page_cuda(k[p * page:(p + 1) * page], v[p * page:(p + 1) * page], page_size=page,
                                                   key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
            pool.key_codes[pid], pool.key_betas[pid], pool.key_norms[pid] = prepared.key_code_payload, prepared.key_beta_payload, prepared.key_norms
            pool.value_codes[pid], pool.value_betas[pid], pool.value_norms[pid] = prepared.value_code_payload, prepared.value_beta_payload, prepared.value_norms
            cache.page_indices[slot, p] = pid
        rest = length - full * page
        cache.page_counts[slot] = full
        cache.last_page_len[slot] = page if full else 0
        cache.hot_lengths[slot] = rest
        cache.sequence_lengths[slot] = length
        if rest:
            cache.hot_keys[slot, :rest] = k[full * page:]
            cache.hot_values[slot, :rest] = v[full * page:]
    torch.cuda.synchronize()
    return kv


@pytest.mark.parametrize("tag", ["page_11x8x64", "page_16x2x128"])
def test_page_writer_matches_reference_vectors(rt, golden, tag):
    k = torch.from_numpy(golden[f"{tag}_key"]).bfloat16().cuda()
    v = torch.from_numpy(golden[f"{tag}_value"]).bfloat16().cuda()
    page = rt.quantize_nqkv_page_cuda(k, v, page_size=16, q=14, key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    for tensor, suffix in ((page.key_code_payload, "_k_codes"), (page.key_beta_payload, "_k_beta"),
                           (page.key_norms, "_k_norms"), (page.value_code_payload, "_v_codes"),
                           (page.value_beta_payload, "_v_beta"), (page.value_norms, "_v_norms")):
        assert np.array_equal(tensor.cpu().numpy(), golden[tag + suffix]), suffix
    assert page.payload_bytes == int(golden[f"{tag}_payload_bytes"][0])


@pytest.mark.parametrize("valid", [1, 15, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_page_writer_fill_levels(rt, oracle, valid, dtype):
    k = (torch.randn(valid, 8, 64, generator=rng(valid)) * 2).to(dtype)
    v = torch.randn(valid, 8, 64, generator=rng(valid + 100)).to(dtype)
    page = rt.quantize_nqkv_page_cuda(k.cuda(), v.cuda(), page_size=16, key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    expected = oracle.kv_pack_page(k.float().numpy(), v.float().numpy(), page_size=16, key_betas=KEY_BETAS,
                                   value_betas=VALUE_BETAS)
    got = (page.key_code_payload, page.key_beta_payload, page.key_norms, page.value_code_payload,
           page.value_beta_payload, page.value_norms)
    for g, e in zip(got, expected):
        assert np.array_equal(g.cpu().numpy(), e)
    assert page.payload_bytes == 9728


def test_page_writer_errors(rt):
    k = torch.zeros(17, 8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        rt.quantize_nqkv_page_cuda(k, k, page_size=16, key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    with pytest.raises(ValueError):
        rt.quantize_nqkv_page_cuda(k[:4], k[:4], page_size=16, key_betas=KEY_BETAS)
    with pytest.raises(ValueError):
        rt.quantize_nqkv_page_cuda(k[:4].cpu(), k[:4].cpu(), page_size=16, key_betas=KEY_BETAS, value_betas=VALUE_BETAS)


def test_append_k1_and_masks(rt):
    cache = make_cache(rt, slots=4, max_pages=4, heads=2)
    for s in (0, 1, 3):
        cache.register(s)
    cache.hot_lengths[3] = 16  # full tail: the append must be refused
    slot_ids = torch.tensor([1, 0, 3, 2], dtype=torch.int32, device="cuda")
    active = torch.tensor([True, False, True, True], device="cuda")  # slot 2 is not registered
    k = torch.randn(4, 2, 64, generator=rng(1)).bfloat16().cuda()
    v = torch.randn(4, 2, 64, generator=rng(2)).bfloat16().cuda()
    rt.append_hot_k1_graph_safe(k, v, cache, slot_ids=slot_ids, active_mask=active)
    rt.append_hot_k1_graph_safe(v, k, cache, slot_ids=slot_ids, active_mask=active)
    assert cache.hot_lengths.tolist() == [0, 2, 0, 16] and cache.sequence_lengths.tolist() == [0, 2, 0, 0]
    assert torch.equal(cache.hot_keys[1, 0], k[0]) and torch.equal(cache.hot_values[1, 0], v[0])
    assert torch.equal(cache.hot_keys[1, 1], v[0]) and torch.equal(cache.hot_values[1, 1], k[0])
    assert int(cache.hot_keys[0].count_nonzero()) == 0 and int(cache.hot_keys[2].count_nonzero()) == 0
    assert int(cache.hot_keys[3].count_nonzero()) == 0


def test_append_ragged_mask_and_segment(rt):
    cache = make_cache(rt, slots=3, max_pages=4, heads=2)
    for s in range(3):
        cache.register(s)
    cache.hot_lengths[1] = 14
    cache.sequence_lengths[1] = 30
    slot_ids = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    k = torch.randn(3, 5, 2, 64, generator=rng(3)).bfloat16().cuda()
    v = torch.randn(3, 5, 2, 64, generator=rng(4)).bfloat16().cuda()
    mask = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 0, 0], [0, 0, 0, 0, 0]], dtype=torch.bool, device="cuda")
    rt._launch_append_hot_ragged_subpage_graph_safe(k, v, cache, slot_ids=slot_ids, write_mask=mask)
    # row 1 would overflow the page (14 + 3 > 16): data up to the page end is written, metadata is not bumped
    assert cache.hot_lengths.tolist() == [3, 14, 0] and cache.sequence_lengths.tolist() == [3, 30, 0]
    assert torch.equal(cache.hot_keys[0, :3], k[0, :3]) and torch.equal(cache.hot_values[0, :3], v[0, :3])
    assert torch.equal(cache.hot_keys[1, 14:16], k[1, :2])
    starts = torch.tensor([3, 0, 1], dtype=torch.int32, device="cuda")
    counts = torch.tensor([2, 0, 4], dtype=torch.int32, device="cuda")
    rt._launch_append_hot_ragged_segment_graph_safe(k, v, cache, slot_ids=slot_ids, source_starts=starts,
                                                    segment_counts=counts)
    assert cache.hot_lengths.tolist() == [5, 14, 4] and cache.sequence_lengths.tolist() == [5, 30, 4]
    assert torch.equal(cache.hot_keys[0, 3:5], k[0, 3:5]) and torch.equal(cache.hot_values[2, :4], v[2, 1:5])


def test_pack_publish_payload_byte_for_byte(rt, oracle):
    cache = make_cache(rt, slots=4, max_pages=3, capacity=16)
    pool = cache.pool
    for s in range(4):
        cache.register(s)
    k = torch.randn(4, 16, 8, 64, generator=rng(5)).bfloat16().cuda()
    v = torch.randn(4, 16, 8, 64, generator=rng(6)).bfloat16().cuda()
    cache.hot_keys.copy_(k)
    cache.hot_values.copy_(v)
    cache.hot_lengths.copy_(torch.tensor([16, 16, 9, 16], dtype=torch.int32))
    cache.page_counts[3] = 3  # table already full: the slot is left alone (nothing written to the pool, nothing published)
    targets = [5, 11, 2, 7]
    cache.graph_target_page_ids.copy_(torch.tensor(targets, dtype=torch.int32))
    boundary = torch.tensor([True, False, True, True], device="cuda")
    rt.launch_pack_full_hot_pages_graph_safe(cache, boundary_mask=boundary)
    torch.cuda.synchronize()
    assert cache.page_counts.tolist() == [1, 0, 0, 3] and cache.hot_lengths.tolist() == [0, 16, 9, 16]
    assert cache.page_indices[0].tolist() == [5, -1, -1] and cache.last_page_len.tolist() == [16, 0, 0, 0]
    for slot in (0,):
        expected = oracle.kv_pack_page(k[slot].float().cpu().numpy(), v[slot].float().cpu().numpy(), page_size=16,
                                       key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
        pid = targets[slot]
        got = (pool.key_codes[pid], pool.key_betas[pid], pool.key_norms[pid], pool.value_codes[pid],
               pool.value_betas[pid], pool.value_norms[pid])
        for g, e in zip(got, expected):
            assert np.array_equal(g.cpu().numpy(), e)
    untouched = [i for i in range(16) if i != 5]  # page 7, the full-table slot's target, included
    assert int(pool.key_codes[untouched].count_nonzero()) == 0 and int(pool.value_norms[untouched].count_nonzero()) == 0


def _check_attention(actual, expected):
    assert max_abs(actual, expected) <= MAX_ABS_TOL, (max_abs(actual, expected), rel_fro(actual, expected))
    assert rel_fro(actual, expected) <= REL_FRO_TOL, rel_fro(actual, expected)


@pytest.mark.parametrize("heads,dim,q_heads", [(8, 64, 32), (2, 128, 16), (2, 64, 2), (4, 32, 8), (1, 256, 2)])
def test_decode_attention_matches_checker(rt, oracle, heads, dim, q_heads):
    lengths = [1, 16, 17, 250, None, 0, 96]
    cache = make_cache(rt, slots=len(lengths), max_pages=16, heads=heads, dim=dim)
    fill_cache(rt, cache, lengths, seed=40)
    slot_ids = torch.tensor([3, 0, 6, 2, 1, 4, 5], dtype=torch.int32, device="cuda")
    active = torch.tensor([True, True, True, True, False, True, True], device="cuda")
    q = torch.randn(7, q_heads, dim, generator=rng(41)).bfloat16()
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=7, query_heads=q_heads, output_dtype=torch.float32)
    out = rt.nqkv_decode_attention_batched_k1(q.cuda(), cache, slot_ids=slot_ids, active_mask=active, workspace=ws)
    actual = out.cpu().numpy()
    expected = oracle.attn_decode(q.float().numpy(), slot_ids.cpu().numpy(), [1, 1, 1, 1, 0, 0, 0],
                                  rt.cache_arrays(cache), scale=1.0 / np.sqrt(dim))
    # rows: slot 1 masked off, slot 4 never registered, slot 5 registered but empty -> all zero
    assert not actual[4:].any()
    _check_attention(actual, expected)
    bf16 = rt.nqkv_decode_attention_batched_k1(q.cuda(), cache, slot_ids=slot_ids, active_mask=active)
    assert bf16.dtype == torch.bfloat16 and torch.equal(bf16.cpu(), torch.from_numpy(actual).bfloat16())


def test_decode_attention_long_context_over_127_pages(rt, oracle):
    # 131 cold pages + hot tail: beyond the reference kernel's 127-page limit
    cache = make_cache(rt, slots=2, max_pages=136)
    fill_cache(rt, cache, [2101, 2048], seed=50)
    slot_ids = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    active = torch.tensor([True, True], device="cuda")
    q = torch.randn(2, 32, 64, generator=rng(51)).bfloat16()
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=2, query_heads=32, output_dtype=torch.float32)
    out = rt.nqkv_decode_attention_batched_k1(q.cuda(), cache, slot_ids=slot_ids, active_mask=active, workspace=ws)
    expected = oracle.attn_decode(q.float().numpy(), [0, 1], [1, 1], rt.cache_arrays(cache), scale=0.125)
    _check_attention(out.cpu().numpy(), expected)


def test_decode_attention_argument_errors(rt):
    cache = make_cache(rt, slots=2, max_pages=4)
    q = torch.zeros(2, 32, 64, dtype=torch.bfloat16, device="cuda")
    ids = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
    on = torch.tensor([True, True], device="cuda")
    with pytest.raises(ValueError):
        rt.nqkv_decode_attention_batched_k1(q, cache, slot_ids=ids, active_mask=on)  # duplicate active slot
    with pytest.raises(ValueError):
        rt.nqkv_decode_attention_batched_k1(q[:, :12], cache, slot_ids=ids, active_mask=on)  # 12 % 8 != 0
    with pytest.raises(ValueError):
        rt.nqkv_decode_attention_batched_k1(q, cache, slot_ids=ids.long(), active_mask=on)


def test_append_reads_rows_of_a_stacked_projection_in_place(rt):
    """K1 append with K and V as column ranges of one [B, q + k + v] result (row stride, no copy) writes the
    same hot tails as with dense tensors."""
    tails = []
    for strided in (False, True):
        cache = make_cache(rt, slots=4, max_pages=2, heads=2)
        for s in range(4):
            cache.register(s)
        slot_ids = torch.tensor([2, 0, 3, 1], dtype=torch.int32, device="cuda")
        active = torch.tensor([True, True, False, True], device="cuda")
        for step in range(3):
            stacked = torch.randn(4, 256 + 128 + 128, generator=rng(300 + step)).bfloat16().cuda()
            k = stacked[:, 256:384].view(4, 2, 64)
            v = stacked[:, 384:].view(4, 2, 64)
            assert not v.is_contiguous()
            if not strided:
                k, v = k.contiguous(), v.contiguous()
            rt.append_hot_k1_graph_safe(k, v, cache, slot_ids=slot_ids, active_mask=active)
        tails.append((cache.hot_keys.clone(), cache.hot_values.clone(), cache.hot_lengths.clone()))
    assert tails[0][2].tolist() == [3, 3, 3, 0]
    assert all(torch.equal(a, b) for a, b in zip(*tails))


def test_prefill_attention_ragged_chunks_cross_pages(rt, oracle):
    lengths = [40, 16, 75, 5]
    cache = make_cache(rt, slots=4, max_pages=8)
    fill_cache(rt, cache, lengths, seed=60)
    q_lens = torch.tensor([9, 16, 64, 5], dtype=torch.int32, device="cuda")  # sub-page, exact page, multi-page, all-hot
    slot_ids = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device="cuda")
    q = torch.randn(4, 64, 32, 64, generator=rng(61)).bfloat16()
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=4, query_heads=32, output_dtype=torch.float32,
                                                 query_tokens=64)
    out = rt.nqkv_prefill_attention(q.cuda(), cache, slot_ids=slot_ids, query_lengths=q_lens, workspace=ws)
    expected = oracle.attn_prefill(q.float().numpy(), [0, 1, 2, 3], q_lens.cpu().numpy(), rt.cache_arrays(cache),
                                   scale=0.125)
    actual = out.cpu().numpy()
    assert not actual[0, 9:].any() and not actual[3, 5:].any()
    _check_attention(actual, expected)


@pytest.mark.parametrize("heads,dim,q_heads,q_tokens", [(2, 64, 8, 13), (2, 64, 4, 13), (2, 64, 2, 21),
                                                        (2, 128, 8, 13), (1, 128, 2, 10), (1, 128, 1, 19)])
def test_prefill_attention_query_tiles(rt, oracle, heads, dim, q_heads, q_tokens):
    """Chunk prefill with several query tokens per CTA (2, 4 or 8 by GQA group, both tiled head sizes): chunks
    that end inside a tile, a chunk of one token, an inactive row, query counts that are no multiple of the tile."""
    lengths = [40, 16, 75, 5, 300]
    cache = make_cache(rt, slots=5, max_pages=20, heads=heads, dim=dim)
    fill_cache(rt, cache, lengths, seed=90 + dim + q_heads)
    q_lens = torch.tensor([9, 1, q_tokens, 5, 0], dtype=torch.int32, device="cuda")
    slot_ids = torch.arange(5, dtype=torch.int32, device="cuda")
    q = torch.randn(5, q_tokens, q_heads, dim, generator=rng(91)).bfloat16()
    scale = dim ** -0.5
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=5, query_heads=q_heads, output_dtype=torch.float32,
                                                 query_tokens=q_tokens)
    out = rt.nqkv_prefill_attention(q.cuda(), cache, slot_ids=slot_ids, query_lengths=q_lens, scale=scale, workspace=ws)
    expected = oracle.attn_prefill(q.float().numpy(), [0, 1, 2, 3, 4], q_lens.cpu().numpy(), rt.cache_arrays(cache),
                                   scale=scale)
    actual = out.cpu().numpy()
    assert not actual[0, 9:].any() and not actual[1, 1:].any() and not actual[4].any()
    _check_attention(actual, expected)


def test_written_pages_round_trip_through_attention(rt, oracle):
    """append -> pack/publish -> attention: the whole write path feeds the read path."""
    cache = make_cache(rt, slots=2, max_pages=4, heads=2)
    cache.register(0)
    cache.register(1)
    slot_ids = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    active = torch.tensor([True, True], device="cuda")
    for step in range(37):
        k = torch.randn(2, 2, 64, generator=rng(700 + step)).bfloat16().cuda()
        v = torch.randn(2, 2, 64, generator=rng(800 + step)).bfloat16().cuda()
        rt.append_hot_k1_graph_safe(k, v, cache, slot_ids=slot_ids, active_mask=active)
        if (step + 1) % 16 == 0:
            cache.reserve_targets([0, 1])
            rt.launch_pack_full_hot_pages_graph_safe(cache, boundary_mask=active.clone())
    assert cache.page_counts.tolist() == [2, 2] and cache.hot_lengths.tolist() == [5, 5]
    assert cache.sequence_lengths.tolist() == [37, 37]
    q = torch.randn(2, 8, 64, generator=rng(9)).bfloat16()
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=2, query_heads=8, output_dtype=torch.float32)
    out = rt.nqkv_decode_attention_batched_k1(q.cuda(), cache, slot_ids=slot_ids, active_mask=active, workspace=ws)
    expected = oracle.attn_decode(q.float().numpy(), [0, 1], [1, 1], rt.cache_arrays(cache), scale=0.125)
    _check_attention(out.cpu().numpy(), expected)


def test_lattice_shadow_attention_is_bit_identical(oracle):
    """Opt-in decoded shadow of the pool: attention reads coordinates instead of searching, same bits out.

    Covers the three ways the shadow is written: conversion of a filled pool, the graph page writer
    (pack + publish), and an explicit page list.
    """
    import nestquant_aiinfra_b200.runtime as rt

    torch.manual_seed(11)
    page, heads, dim, q_heads, seqs, max_pages = 16, 2, 64, 8, 3, 6
    pool = rt.NQKVPagePool(capacity=seqs * max_pages, page_size=page, num_kv_heads=heads, head_dim=dim,
                           key_betas=KEY_BETAS, value_betas=VALUE_BETAS)
    cache = rt.NQKVHotColdCache(pool, max_sequences=seqs, max_pages_per_sequence=max_pages)
    for slot in range(seqs):
        cache.register(slot)
    slot_ids = torch.arange(seqs, dtype=torch.int32, device="cuda")
    everyone = torch.ones(seqs, dtype=torch.bool, device="cuda")

    def grow(tokens: int) -> None:
        for _ in range(tokens):
            key = (torch.randn(seqs, heads, dim, device="cuda") * 1.3).bfloat16()
            value = torch.randn(seqs, heads, dim, device="cuda").bfloat16()
            rt._launch_append_hot_k1_graph_safe(key, value, cache, slot_ids=slot_ids, active_mask=everyone)
            cache.graph_target_page_ids.copy_(slot_ids * max_pages + cache.page_counts)
            rt.launch_pack_full_hot_pages_graph_safe(cache, boundary_mask=everyone)

    def attend() -> torch.Tensor:
        query = torch.randn(seqs, q_heads, dim, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
        ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=seqs, query_heads=q_heads,
                                                     output_dtype=torch.float32)
        return rt._launch_nqkv_decode_attention_batched_k1(query, cache, slot_ids=slot_ids, active_mask=everyone,
                                                           attention_scale=0.125, workspace=ws).clone()

    grow(2 * page + 5)                      # two published pages + a hot tail, no shadow yet
    packed = attend()
    added = pool.enable_lattice_shadow()    # converts the pages already in the pool
    assert added == 2 * pool.capacity * page * heads * dim and pool.enable_lattice_shadow() == 0
    assert torch.equal(attend(), packed)
    grow(page + 3)                          # one more page through the graph writer, shadow written with it
    with_shadow = attend()
    key_lattice, value_lattice = pool.key_lattice, pool.value_lattice
    pool.key_lattice = pool.value_lattice = None
    assert torch.equal(attend(), with_shadow)   # the packed kernel on the same pool
    pool.key_lattice, pool.value_lattice = key_lattice, value_lattice
    # the shadow holds the doubled coordinates of the reference's decode
    codes = pool.key_codes[0].cpu().numpy().view(np.uint32)
    unpacked = np.stack([(codes >> (4 * j)) & 15 for j in range(8)], axis=1).astype(np.int64)
    expect = (2.0 * oracle.decode_nested(unpacked)).astype(np.int8)
    assert np.array_equal(pool.key_lattice[0].cpu().numpy().reshape(-1, 8), expect)
    # explicit page list: wipe one page's shadow and restore it
    pool.key_lattice[1].zero_()
    pool.expand_pages(torch.tensor([1, -1], dtype=torch.int32))
    assert torch.equal(attend(), with_shadow)


@pytest.mark.parametrize("heads,dim,q_heads", [(8, 64, 32), (2, 128, 16), (4, 32, 4), (1, 256, 2)])
def test_lattice_shadow_prefill_and_decode_shapes(rt, heads, dim, q_heads):
    """Every head_dim / GQA instantiation of the lattice-page kernel, causal chunk prefill and long decode:
    bit-identical to the packed kernel on a pool filled by the eager page writer (random physical page ids)."""
    lengths = [40, 16, 75, 5, 300]
    cache = make_cache(rt, slots=5, max_pages=20, heads=heads, dim=dim)
    fill_cache(rt, cache, lengths, seed=70 + dim)
    slot_ids = torch.arange(5, dtype=torch.int32, device="cuda")
    active = torch.ones(5, dtype=torch.bool, device="cuda")
    q_lens = torch.tensor([9, 16, 64, 5, 33], dtype=torch.int32, device="cuda")
    q_dec = torch.randn(5, q_heads, dim, generator=rng(71)).bfloat16().cuda()
    q_pre = torch.randn(5, 64, q_heads, dim, generator=rng(72)).bfloat16().cuda()
    scale = dim ** -0.5

    def run():
        ws1 = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=5, query_heads=q_heads,
                                                      output_dtype=torch.float32)
        dec = rt.nqkv_decode_attention_batched_k1(q_dec, cache, slot_ids=slot_ids, active_mask=active,
                                                  scale=scale, workspace=ws1).clone()
        ws2 = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=5, query_heads=q_heads,
                                                      output_dtype=torch.float32, query_tokens=64)
        pre = rt.nqkv_prefill_attention(q_pre, cache, slot_ids=slot_ids, query_lengths=q_lens,
                                        scale=scale, workspace=ws2).clone()
        return dec, pre

    packed_dec, packed_pre = run()
    assert cache.pool.enable_lattice_shadow() > 0
    shadow_dec, shadow_pre = run()
    assert torch.equal(shadow_dec, packed_dec) and torch.equal(shadow_pre, packed_pre)
    assert bool(packed_dec.abs().sum() > 0) and bool(packed_pre.abs().sum() > 0)
