"""Parity at the benchmark's full sizes through size-independent properties.

The CPU checker would need minutes at these sizes, so the tests use properties that pin the result
without it: two independent kernels must agree bit for bit (encoder reconstruction vs decode of the
emitted streams; weight encode -> decode -> encode idempotence), the tensor-core GEMM must match a
float32 product of the same BF16 operands, and sampled rows are still checked against the checker.
"""

import numpy as np
import pytest
import torch

from helpers import ACT_BETAS, MAX_ABS_TOL, REL_FRO_TOL, W_BETAS, max_abs, rel_fro, rng

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import nestquant_aiinfra_b200.runtime as runtime

    return runtime


@pytest.mark.parametrize("m,k", [(8192, 2048), (8192, 8192)])
def test_full_size_encode_streams(rt, oracle, m, k):
    from nestquant_aiinfra_b200.rotation import hadamard

    x = hadamard(torch.randn(m, k, generator=rng(2000 + m)).bfloat16().cuda())
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, keep_decoded=True)
    # (1) the BF16 reconstruction written by the encoder == decode kernel applied to the emitted streams
    assert torch.equal(act.decoded, rt.decode_packed_a4(act, dtype=torch.bfloat16))
    # (2) every code is a valid residue (< 14) and norms are finite and positive
    codes = act.code_payload
    assert int(((codes & 15) >= 14).sum()) == 0 and int(((codes >> 4) >= 14).sum()) == 0
    assert bool(torch.isfinite(act.row_norms).all()) and float(act.row_norms.min()) > 0
    # (3) deterministic: a second launch reproduces the streams bit for bit
    again = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
    assert torch.equal(again.code_payload, act.code_payload) and torch.equal(again.beta_payload, act.beta_payload)
    # (4) sampled rows against the CPU checker (first, last, a few in between)
    rows = [0, 1, m // 3, m // 2 + 1, m - 2, m - 1]
    sample = x[rows].float().cpu().numpy()
    ec, eb, en = oracle.encode_packed(sample, ACT_BETAS)
    got_codes = act.code_payload.view(m, k // 2)[rows].cpu().numpy().reshape(-1)
    got_betas = act.beta_payload.view(m, k // 32)[rows].cpu().numpy().reshape(-1)
    assert np.array_equal(got_codes, ec) and np.array_equal(got_betas, eb)
    assert np.array_equal(act.row_norms[rows].cpu().numpy(), en)


def test_full_size_weight_encode_is_idempotent(rt, oracle):
    """encode(decode(encode(W))) == encode(W) up to the fixed point: the float32 reconstruction of a
    dithered encode re-encodes to the same codes; sampled rows match the checker."""
    n, k, seed = 8192, 2048, 20261031
    from nestquant_aiinfra_b200.rotation import hadamard

    w = hadamard((0.02 * torch.randn(n, k, generator=rng(1002))).cuda())
    first = rt.quantize_weight_cuda(w, betas=W_BETAS, dither_seed=seed)
    rows = [0, 17, n // 2, n - 1]
    for r in rows:  # the dither counter is global: row r starts at block r * k / 8
        ec, eb, en = oracle.encode_packed(w[r:r + 1].cpu().numpy(), W_BETAS, seed=seed, block_offset=r * (k // 8))
        assert np.array_equal(first.code_payload.view(n, k // 2)[r].cpu().numpy(), ec)
        assert np.array_equal(first.beta_payload.view(n, k // 32)[r].cpu().numpy(), eb)
        assert np.array_equal(first.row_norms[r:r + 1].cpu().numpy(), en)
    decoded = rt.decode_packed_weight(first)
    assert bool(torch.isfinite(decoded.float()).all())
    rel = float((decoded.float() - w).norm() / w.norm())
    assert 0.01 < rel < 0.2, rel  # 4.25-bit reconstruction error of a Gaussian matrix


@pytest.mark.parametrize("m,n,k", [(8192, 8192, 2048), (8192, 2048, 8192), (5000, 2048, 4096), (2048, 512, 2048)])
def test_full_size_tensor_core_gemm_matches_float32_product(rt, m, n, k):
    a = (torch.randn(m, k, generator=rng(m + 1)) * 0.7).bfloat16().cuda()
    w = (torch.randn(n, k, generator=rng(n + 2)) * 0.02).bfloat16().cuda()
    out = rt.gemm_bf16_tc(a, w, out_dtype=torch.float32)
    assert rt.read_status() == 0
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        expected = a.float() @ w.float().T  # plain float32 reference of the same BF16 operands
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous
    err = float((out - expected).abs().max())
    fro = float((out - expected).norm() / expected.norm())
    assert err <= MAX_ABS_TOL and fro <= REL_FRO_TOL, (err, fro)
    # the BF16 output (paired tiles store it through shared memory) is the rounded accumulator, element for element
    rounded = rt.gemm_bf16_tc(a, w, out_dtype=torch.bfloat16)
    assert rt.read_status() == 0
    assert torch.equal(rounded, out.bfloat16())


def test_full_size_projection_tails_and_paths_agree(rt, oracle):
    """The same packed operands through the tensor path (M = 520, ragged tail) and row by row through
    the CUDA-core path (M = 1 calls) give the same projection within the accumulation tolerance."""
    from dataclasses import replace

    from helpers import make_weight_record

    n, k, m = 2048, 2048, 520
    record, _ = make_weight_record(oracle, n, k, seed=31, dither_seed=32)
    weight = rt.prepare_fused_linear(record)
    x = torch.randn(m, k, generator=rng(33)).bfloat16().cuda()
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, keep_decoded=True)
    full = rt.linear_packed_w4a4_fp32(act, weight).cpu().numpy()
    rows = [0, 255, 256, 511, 512, 519]
    for r in rows:
        one = replace(act, code_payload=act.code_payload.view(m, -1)[r].contiguous(),
                      beta_payload=act.beta_payload.view(m, -1)[r].contiguous(),
                      row_norms=act.row_norms[r:r + 1].contiguous(), original_shape=(1, k),
                      decoded=act.decoded[r:r + 1].contiguous())
        single = rt.linear_packed_w4a4_fp32(one, weight).cpu().numpy()[0]
        assert max_abs(single, full[r]) <= MAX_ABS_TOL and rel_fro(single, full[r]) <= REL_FRO_TOL


@pytest.mark.parametrize("m", [1, 4, 64, 8192])
def test_full_size_resident_weight_agrees_with_the_packed_call(rt, m):
    """gate/up shape: the opt-in resident decoded weight is the per-call decode kept in memory, so the two
    projections may differ only by the order of the FP32 sums."""
    from nestquant_aiinfra_b200.rotation import hadamard

    n, k = 8192, 2048
    w = hadamard((0.02 * torch.randn(n, k, generator=rng(1000))).cuda())
    packed = rt.quantize_weight_cuda(w, betas=W_BETAS, dither_seed=20261031, tensor_name="gate_up")
    resident = rt.keep_decoded_weight(packed)
    assert torch.equal(resident.decoded, rt.decode_packed_weight(packed))
    x = hadamard(torch.randn(m, k, generator=rng(2000 + m)).bfloat16().cuda())
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, keep_decoded=True)
    a = rt.linear_packed_w4a4_fp32(act, packed).cpu().numpy()
    b = rt.linear_packed_w4a4_fp32(act, resident).cpu().numpy()
    assert rt.read_status() == 0
    assert rel_fro(b, a) <= 1e-5 and max_abs(b, a) <= 1e-3, (rel_fro(b, a), max_abs(b, a))
    # against a float32 product of the same BF16 operands
    expected = (act.decoded.float() @ resident.decoded.float().T).cpu().numpy()
    assert rel_fro(b, expected) <= REL_FRO_TOL and max_abs(b, expected) <= MAX_ABS_TOL



# ---------------------------------------------------------------------------------------------------------
# Config 2 at its own size: 32 sequences x 256 cold pages (context 4096) + hot tail, 8 KV heads, head_dim 64,
# 1 % outlier channels (x8), keys Hadamard-rotated per head, random physical page permutation.
def _config2_cache(rt, *, totals, seed=4096):
    from helpers import KEY_BETAS, VALUE_BETAS
    from nestquant_aiinfra_b200.rotation import hadamard

    batch, heads, dim, page, ctx = 32, 8, 64, 16, 4096
    pages_per_seq = ctx // page
    capacity = batch * pages_per_seq
    pool = rt.NQKVPagePool(capacity=capacity, page_size=page, num_kv_heads=heads, head_dim=dim, key_betas=KEY_BETAS,
                           value_betas=VALUE_BETAS)
    cache = rt.NQKVHotColdCache(pool, max_sequences=batch, max_pages_per_sequence=pages_per_seq + 1)
    gen = rng(seed)
    perm = torch.randperm(capacity, generator=gen).cuda()
    rows = capacity * page * heads
    for which, (codes, betas, norms, table, values) in enumerate((
            (pool.key_codes, pool.key_betas, pool.key_norms, pool.beta_table, KEY_BETAS),
            (pool.value_codes, pool.value_betas, pool.value_norms, pool.value_beta_table, VALUE_BETAS))):
        x = torch.randn(batch, ctx, heads, dim, generator=gen)
        outliers = torch.randperm(heads * dim, generator=gen)[:6]     # ceil(0.01 * 8 * 64) (head, channel) pairs
        x.view(batch, ctx, heads * dim)[:, :, outliers] *= 8.0
        x = x.cuda()
        x = hadamard(x) if which == 0 else x
        act = rt.quantize_activation_cuda(x.bfloat16().reshape(rows, dim), q=14, betas=values, beta_table=table)
        codes[perm] = act.code_payload.view(capacity, -1)
        betas[perm] = act.beta_payload.view(capacity, -1)
        norms[perm] = act.row_norms.view(capacity, -1)
        del x, act
    for slot in range(batch):
        cache.register(slot)
    totals = torch.as_tensor(totals)
    cache.page_indices[:, :pages_per_seq] = perm.view(batch, pages_per_seq).to(torch.int32)
    cache.page_counts.copy_((totals // page).to(torch.int32))
    cache.last_page_len.copy_(torch.where(totals >= page, page, 0).to(torch.int32))
    cache.hot_lengths.copy_((totals % page).to(torch.int32))
    cache.sequence_lengths.copy_(totals.to(torch.int32))
    cache.hot_keys.copy_(torch.randn(cache.hot_keys.shape, generator=gen).bfloat16())
    cache.hot_values.copy_(torch.randn(cache.hot_values.shape, generator=gen).bfloat16())
    return cache, gen


def test_config2_decode_attention_at_full_size(rt, oracle):
    """Batch 32 x (256 pages + 1 hot token), 32 query heads: the FP32 output against the CPU checker."""
    from nestquant_aiinfra_b200.rotation import hadamard

    batch, q_heads, dim = 32, 32, 64
    cache, gen = _config2_cache(rt, totals=[4097] * batch)
    q = hadamard(torch.randn(batch, q_heads, dim, generator=gen).cuda()).bfloat16()
    slot_ids = torch.arange(batch, dtype=torch.int32, device="cuda")
    active = torch.ones(batch, dtype=torch.bool, device="cuda")
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=batch, query_heads=q_heads, output_dtype=torch.float32)
    out = rt.nqkv_decode_attention_batched_k1(q, cache, slot_ids=slot_ids, active_mask=active, workspace=ws)
    actual = out.cpu().numpy()
    expected = oracle.attn_decode(q.float().cpu().numpy(), list(range(batch)), [1] * batch, rt.cache_arrays(cache),
                                  scale=0.125)
    assert np.isfinite(actual).all()
    assert max_abs(actual, expected) <= MAX_ABS_TOL and rel_fro(actual, expected) <= REL_FRO_TOL, \
        (max_abs(actual, expected), rel_fro(actual, expected))


def test_config2_ragged_prefill_at_full_size(rt, oracle):
    """Start contexts U[0, 4032], chunk lengths U[1, 64] whose K/V are appended already: sub-page, exact-fill,
    one-boundary and multi-page chunks over cold pages plus hot tail, against the CPU checker."""
    from nestquant_aiinfra_b200.rotation import hadamard

    batch, q_heads, dim = 32, 32, 64
    draw = rng(77)
    starts = torch.randint(0, 4033, (batch,), generator=draw)
    chunks = torch.randint(1, 65, (batch,), generator=draw)
    starts[0], chunks[0] = 0, 5          # everything still hot
    starts[1], chunks[1] = 16, 16        # exact page fill
    starts[2], chunks[2] = 4032, 64      # the longest context, a multi-page chunk
    starts[3], chunks[3] = 30, 3         # one boundary crossed
    cache, gen = _config2_cache(rt, totals=(starts + chunks).tolist())
    t_max = int(chunks.max())
    q = hadamard(torch.randn(batch, t_max, q_heads, dim, generator=gen).cuda()).bfloat16()
    slot_ids = torch.arange(batch, dtype=torch.int32, device="cuda")
    q_lens = chunks.to(torch.int32).cuda()
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=batch, query_heads=q_heads, output_dtype=torch.float32,
                                                 query_tokens=t_max)
    out = rt.nqkv_prefill_attention(q, cache, slot_ids=slot_ids, query_lengths=q_lens, scale=0.125, workspace=ws)
    actual = out.cpu().numpy()
    expected = oracle.attn_prefill(q.float().cpu().numpy(), list(range(batch)), chunks.tolist(), rt.cache_arrays(cache),
                                   scale=0.125)
    for b in range(batch):
        assert not actual[b, int(chunks[b]):].any()      # rows beyond the chunk stay zero
    assert max_abs(actual, expected) <= MAX_ABS_TOL and rel_fro(actual, expected) <= REL_FRO_TOL, \
        (max_abs(actual, expected), rel_fro(actual, expected))
