"""GPU parity of the Hadamard kernel and of the FusedNQRTLinear plugin boundary."""

import numpy as np
import pytest
import torch

from helpers import ACT_BETAS, MAX_ABS_TOL, REL_FRO_TOL, W_BETAS as W_BETAS_LOCAL, make_weight_record, max_abs, rel_fro, rng

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n,dtype", [(3, 2048, torch.float32), (3, 2048, torch.bfloat16), (5, 64, torch.float32),
                                          (257, 64, torch.bfloat16), (4, 8192, torch.bfloat16), (7, 128, torch.float16),
                                          (2, 16384, torch.float32), (9, 8, torch.float32), (5, 8, torch.bfloat16),
                                          (131, 16, torch.bfloat16), (33, 32, torch.float16), (3, 512, torch.bfloat16),
                                          (2, 1024, torch.float16), (3, 4096, torch.bfloat16), (2, 32768, torch.bfloat16)])
def test_hadamard_bit_exact(oracle, golden, rows, n, dtype):
    from nestquant_aiinfra_b200.rotation import hadamard, hadamard_butterflies

    if (rows, n) == (3, 2048):
        key = "had_f32" if dtype == torch.float32 else "had_bf16"
        x = torch.from_numpy(golden[key + "_in"]).to(dtype)
        expected = torch.from_numpy(golden[key + "_out"]).to(dtype)
    elif (rows, n) == (5, 64):
        x, expected = torch.from_numpy(golden["had_64_in"]), torch.from_numpy(golden["had_64_out"])
    else:
        x = torch.randn(rows, n, generator=rng(n + rows)).to(dtype)
        expected = hadamard_butterflies(x)  # the reference's own op sequence, on the CPU
    got = hadamard(x.cuda()).cpu()
    assert got.dtype == dtype and torch.equal(got, expected)


@pytest.mark.parametrize("rows,n,dtype", [(64, 8192, torch.bfloat16), (5, 8192, torch.float16), (3, 2048, torch.float32),
                                          (130, 16, torch.bfloat16), (7, 8, torch.bfloat16), (1, 32768, torch.bfloat16)])
def test_hadamard_of_the_silu_product_in_one_launch(rows, n, dtype):
    """hadamard(silu(gate) * up) as one launch == the two tensor ops followed by the rotation kernel, bit for bit."""
    from nestquant_aiinfra_b200.rotation import hadamard, hadamard_silu_mul

    gate = (3.0 * torch.randn(rows, n, generator=rng(5 * n + rows))).to(dtype).cuda()
    up = torch.randn(rows, n, generator=rng(7 * n + rows)).to(dtype).cuda()
    expected = hadamard(torch.nn.functional.silu(gate) * up)
    got = hadamard_silu_mul(gate, up)
    assert got.dtype == dtype and torch.equal(got, expected)
    stacked = torch.cat([gate, up], dim=-1).unsqueeze(1)                           # column ranges of one result: read in place
    assert torch.equal(hadamard_silu_mul(stacked[..., :n], stacked[..., n:]), expected.unsqueeze(1))
    blocked = hadamard_silu_mul(gate.view(rows, -1, 8), up.view(rows, -1, 8))   # block-diagonal: rows of 8
    assert torch.equal(blocked, hadamard((torch.nn.functional.silu(gate) * up).view(rows, -1, 8)))


def test_hadamard_rejects_non_power_of_two():
    from nestquant_aiinfra_b200.rotation import hadamard

    with pytest.raises(ValueError):
        hadamard(torch.zeros(2, 24, device="cuda"))


def _linear_oracle(oracle, x_bf16: torch.Tensor, w_deq: np.ndarray) -> np.ndarray:
    m, k = x_bf16.shape
    rotated = oracle.hadamard(x_bf16.float().numpy(), round_bf16=True)
    ac, ab, an = oracle.encode_packed(rotated, ACT_BETAS)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
    return oracle.gemm_bf16_operands(a_deq, w_deq)


@pytest.mark.parametrize("m", [1, 5, 48, 300])
def test_fused_linear_forward_matches_checker(oracle, m):
    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear

    n, k = 256, 1024
    record, w_deq = make_weight_record(oracle, n, k, seed=11, dither_seed=123)
    layer = FusedNQRTLinear(record, input_hadamard=True, activation_betas=ACT_BETAS).cuda()
    x = torch.randn(2, m, k, generator=rng(m)).bfloat16()
    with torch.no_grad():
        y = layer(x.cuda())
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (2, m, n)
    expected = _linear_oracle(oracle, x.reshape(-1, k), w_deq)
    actual = y.float().cpu().numpy().reshape(-1, n)
    # output is BF16-rounded: allow one BF16 ulp of the largest output on top of the accumulator bar
    bar = MAX_ABS_TOL + float(np.abs(expected).max()) * 2 ** -8
    assert max_abs(actual, expected) <= bar
    assert rel_fro(actual, expected) <= 4e-3  # BF16 output rounding alone costs ~1.7e-3
    assert layer.a4_encode_count == 1 and layer.w4a4_cuda_mma_dispatch_count == 1


def test_shared_caches_encode_once(oracle):
    from nestquant_aiinfra_b200.fused_linear import (FusedNQRTLinear, SharedHadamardCache,
                                                       SharedPackedActivationCache)

    k = 512
    rec_a, _ = make_weight_record(oracle, 64, k, seed=1, dither_seed=1)
    rec_b, _ = make_weight_record(oracle, 128, k, seed=2, dither_seed=2)
    hcache, acache = SharedHadamardCache(2), SharedPackedActivationCache(2)
    kwargs = dict(input_hadamard=True, input_transform_cache=hcache, packed_activation_cache=acache,
                  activation_betas=ACT_BETAS)
    a, b = FusedNQRTLinear(rec_a, **kwargs).cuda(), FusedNQRTLinear(rec_b, **kwargs).cuda()
    solo = FusedNQRTLinear(rec_b, input_hadamard=True, activation_betas=ACT_BETAS).cuda()
    x = torch.randn(3, k, generator=rng(9)).bfloat16().cuda()
    with torch.no_grad():
        ya, yb, ys = a(x), b(x), solo(x)
    assert (hcache.misses, hcache.hits, acache.misses, acache.hits) == (1, 1, 1, 1)
    assert a.a4_encode_count == 1 and b.a4_encode_count == 0
    assert torch.equal(yb, ys) and ya.shape == (3, 64)


def test_fused_linear_errors(oracle):
    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear

    record, _ = make_weight_record(oracle, 64, 256, seed=1, dither_seed=1)
    with pytest.raises(ValueError):
        FusedNQRTLinear(record, activation_betas=None)
    with pytest.raises(ValueError):
        FusedNQRTLinear(record, compute_backend="tensor_core_dot", activation_betas=ACT_BETAS)
    layer = FusedNQRTLinear(record, activation_betas=ACT_BETAS).cuda()
    with pytest.raises(ValueError):
        layer(torch.zeros(1, 128, device="cuda"))
    with pytest.raises(ValueError):
        layer(torch.zeros(1, 256))


@pytest.mark.parametrize("rows,n,dtype", [(64, 2048, torch.bfloat16), (1, 8192, torch.bfloat16), (37, 448, torch.float16),
                                          (5, 2048, torch.float32)])
def test_rms_norm_follows_the_llama_formula(rows, n, dtype):
    """One-launch RMS norm vs the tensor-op formula of LlamaRMSNorm; only the order of the sum of squares differs."""
    from nestquant_aiinfra_b200.norm import rms_norm

    x = (torch.randn(rows, n, generator=rng(900 + n)) * 3).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(n, generator=rng(901))).to(dtype).cuda()
    eps = 1e-5
    xf = x.float()
    expected = w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)
    got = rms_norm(x, w, eps)
    assert got.dtype == dtype and got.shape == x.shape and torch.equal(got, rms_norm(x, w, eps))
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -22}[dtype]
    diff = (got.float() - expected.float()).abs()
    assert float((diff / expected.float().abs().clamp_min(1e-3)).max()) <= 2.5 * ulp   # at most one rounding step apart
    assert float((diff > 0).float().mean()) < 0.02


def test_fuse_rmsnorm_replaces_llama_norms():
    from transformers import LlamaConfig, LlamaForCausalLM

    from nestquant_aiinfra_b200.norm import FusedRMSNorm, fuse_rmsnorm_

    config = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=64, vocab_size=512)
    torch.manual_seed(0)
    model = LlamaForCausalLM(config).bfloat16().cuda().eval()
    ids = torch.randint(0, 512, (2, 9), generator=rng(77)).cuda()
    with torch.no_grad():
        before = model(ids).logits.float()
        assert fuse_rmsnorm_(model) == 5 and fuse_rmsnorm_(model) == 0   # 2 per layer + the final norm
        assert isinstance(model.model.norm, FusedRMSNorm)
        after = model(ids).logits.float()
    assert rel_fro(after.cpu().numpy(), before.cpu().numpy()) < 2e-2


@pytest.mark.parametrize("batch,heads,tokens,dim,dtype", [(5, 8, 1, 64, torch.bfloat16), (2, 4, 19, 128, torch.bfloat16),
                                                          (3, 2, 7, 64, torch.float16), (1, 3, 5, 32, torch.float32)])
def test_rope_and_rotation_in_one_launch_equal_the_tensor_ops(batch, heads, tokens, dim, dtype):
    """nq_rope_hadamard == apply_rotary_pos_emb, and == hadamard(rope.float()).to(dtype) with the rotation, bit for bit."""
    from transformers.models.llama.modeling_llama import rotate_half

    from nestquant_aiinfra_b200.rope import rope_hadamard
    from nestquant_aiinfra_b200.rotation import hadamard

    # the layout of Llama's attention module: [B, T, H*D] viewed as [B, T, H, D] and transposed
    x = torch.randn(batch, tokens, heads * dim, generator=rng(300 + dim)).to(dtype).cuda()
    x = x.view(batch, tokens, heads, dim).transpose(1, 2)
    angles = torch.rand(batch, tokens, dim, generator=rng(301)) * 6.28
    cos, sin = angles.cos().to(dtype).cuda(), angles.sin().to(dtype).cuda()
    stock = (x * cos.unsqueeze(1)) + (rotate_half(x) * sin.unsqueeze(1))
    assert torch.equal(rope_hadamard(x, cos, sin, rotate=False), stock)
    assert torch.equal(rope_hadamard(x, cos, sin), hadamard(stock.float()).to(dtype))
    assert torch.equal(rope_hadamard(x[:1], cos[:1], sin[:1]), rope_hadamard(x, cos, sin)[:1])
    # query and key heads of a layer in one launch: column ranges of one stacked [B, T, (Hq + Hk) * D] result
    from nestquant_aiinfra_b200.rope import rope_hadamard_pair

    both = torch.randn(batch, tokens, 3 * heads * dim, generator=rng(302 + dim)).to(dtype).cuda()
    q = both[..., :2 * heads * dim].view(batch, tokens, 2 * heads, dim).transpose(1, 2)
    k = both[..., 2 * heads * dim:].view(batch, tokens, heads, dim).transpose(1, 2)
    for rotate in (False, True):
        q_out, k_out = rope_hadamard_pair(q, k, cos, sin, rotate=rotate)
        assert torch.equal(q_out, rope_hadamard(q, cos, sin, rotate=rotate))
        assert torch.equal(k_out, rope_hadamard(k, cos, sin, rotate=rotate))


def test_stacked_projection_group_equals_the_members_own_projections(oracle):
    """q/k/v-style group: one launch sequence over the stacked weight, column ranges equal to the members' own results."""
    from nestquant_aiinfra_b200.fused_linear import (FusedNQRTLinear, SharedPackedActivationCache,
                                                     SharedProjectionGroup)
    from nestquant_aiinfra_b200.runtime import quantize_weight_cuda

    k, sizes = 512, (256, 128, 128)
    weights = [quantize_weight_cuda((0.02 * torch.randn(n, k, generator=rng(700 + n))).cuda(), betas=W_BETAS_LOCAL,
                                    dither_seed=1000 + n) for n in sizes]
    for m in (1, 5, 16, 40, 200):
        x = torch.randn(m, k, generator=rng(710 + m)).bfloat16().cuda()
        cache = SharedPackedActivationCache(len(sizes))
        members = [FusedNQRTLinear(w, activation_betas=ACT_BETAS, packed_activation_cache=cache) for w in weights]
        with torch.no_grad():
            alone = [FusedNQRTLinear(w, activation_betas=ACT_BETAS)(x) for w in weights]
            group = SharedProjectionGroup(members)
            together = [member(x) for member in members]
        assert group.launches == 1 and cache.misses == 1
        for a, b in zip(alone, together):
            assert b.shape == a.shape
            if m < 8:   # CUDA-core path: the K split does not depend on N, so not a bit moves
                assert torch.equal(a, b)
            else:       # tensor-core path: the split-K layout follows the tile count; same operands, other summation order
                assert rel_fro(b.float().cpu().numpy(), a.float().cpu().numpy()) < 2e-3
        assert sum(member.packed_device_bytes for member in members) == \
            sum(t.numel() * t.element_size() for t in (group.stacked.code_payload, group.stacked.beta_payload,
                                                       group.stacked.row_norms)) + 3 * 16


def test_keep_decoded_weights_switches_modules_and_groups(oracle):
    """keep_decoded_weights_ turns every packed module (stand-alone or member of a stacked group) into the resident mode."""
    from torch import nn

    from nestquant_aiinfra_b200.fused_linear import (FusedNQRTLinear, SharedPackedActivationCache,
                                                     SharedProjectionGroup, keep_decoded_weights_)
    from nestquant_aiinfra_b200.runtime import quantize_weight_cuda

    k, sizes = 512, (256, 128)
    weights = [quantize_weight_cuda((0.02 * torch.randn(n, k, generator=rng(900 + n))).cuda(), betas=W_BETAS_LOCAL,
                                    dither_seed=2000 + n) for n in sizes]
    solo_weight = quantize_weight_cuda((0.02 * torch.randn(128, k, generator=rng(950))).cuda(), betas=W_BETAS_LOCAL,
                                       dither_seed=77)
    cache = SharedPackedActivationCache(len(sizes))
    members = [FusedNQRTLinear(w, activation_betas=ACT_BETAS, packed_activation_cache=cache) for w in weights]
    SharedProjectionGroup(members)
    solo = FusedNQRTLinear(solo_weight, activation_betas=ACT_BETAS)
    model = nn.ModuleList([*members, solo])
    for m in (1, 3, 40):
        x = torch.randn(m, k, generator=rng(960 + m)).bfloat16().cuda()
        with torch.no_grad():
            before = [module(x) for module in model]
    added = keep_decoded_weights_(model)
    assert added == 2 * k * (sum(sizes) + 128)
    assert keep_decoded_weights_(model) == 0
    assert members[0]._group.stacked.decoded is not None and solo._prepared.decoded is not None
    with torch.no_grad():
        after = [module(x) for module in model]
    for a, b in zip(before, after):
        assert a.shape == b.shape
        assert rel_fro(b.float().cpu().numpy(), a.float().cpu().numpy()) < 2e-3  # bf16 outputs, other summation order
