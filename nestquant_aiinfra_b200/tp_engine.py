"""Tensor-parallel W4A4KV4 Llama shard: one process per GPU, NCCL all-reduce after o_proj / down_proj.

Each rank builds only ITS shard of the architecture (heads / tp, kv heads / tp, FFN / tp around the
full hidden size) as a stock Hugging Face Llama whose column-parallel projections are packed NQRT4
modules and whose o_proj / down_proj are ``RowParallelNQRTLinear`` (self-contained K shard +
all-reduce).  The reference has no multi-GPU path; the shard definitions are those of
``tensor_parallel.py``.  The lm_head is replicated (vocab-parallel logits are not needed for a
greedy argmax on identical hidden states).
"""

from __future__ import annotations

import torch
from torch import nn

from .engine import BatchedNQKVLlamaRunner
from .formats import ACTIVATION_BETAS, KEY_BETAS, VALUE_BETAS, WEIGHT_BETAS, tensor_dither_seed
from .fused_linear import (FusedNQRTLinear, SharedHadamardCache, SharedPackedActivationCache,
                           SharedProjectionGroup)
from .hf_backend import BatchedNQKVLlamaCache, install_batched_nqkv_llama_backend
from .norm import fuse_rmsnorm_
from .rotation import hadamard
from .runtime.w4a4 import quantize_activation_cuda, quantize_weight_cuda
from .tensor_parallel import RowParallelNQRTLinear

COLUMN = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj")
ROW = ("self_attn.o_proj", "mlp.down_proj")
GROUPS = (("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("mlp.gate_proj", "mlp.up_proj"))


def full_projection_weight(layer: int, name: str, rows: int, cols: int, *, seed: int, device: torch.device,
                           std: float = 0.02) -> torch.Tensor:
    """The unsharded ``[rows, cols]`` float32 weight of one projection of the synthetic model.

    A pure function of (seed, layer, name): every rank regenerates the same full tensor and cuts its
    own slice out of it, so the ranks together hold ONE model (not ``world`` copies of a shard).
    """
    gen = torch.Generator(device=device).manual_seed(tensor_dither_seed(seed + 1000003, f"{layer}.{name}"))
    return torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32) * std


def build_llama_tp_shard(*, hidden_size: int, intermediate_size: int, num_layers: int, num_heads: int,
                         num_kv_heads: int, head_dim: int, vocab_size: int, rank: int, world: int, capacity: int,
                         max_cache_len: int, device: torch.device | str, seed: int = 0, process_group=None):
    """Shard ``rank`` of ``world`` of ONE random-init Llama architecture, converted to W4A4KV4.

    Column-parallel projections (q, k, v, gate, up) take the rank's output rows of the full
    weight and encode them with the full tensor's dither seed and ``block_offset = first_row * K / 8``:
    the streams are byte for byte the rank's row range of the unsharded record.  Row-parallel
    projections (o, down) take the rank's input features of the full weight as a self-contained
    shard (``RowParallelNQRTLinear``).  Embeddings, norms and lm_head are replicated.
    """
    from transformers import LlamaConfig, LlamaForCausalLM

    if num_heads % world or num_kv_heads % world or intermediate_size % world:
        raise ValueError("heads, kv heads and the FFN width must be divisible by the tensor-parallel degree")
    if (intermediate_size // world) % 32 or (num_heads // world * head_dim) % 32:
        raise ValueError("row-parallel K shards must be multiples of 32")
    device = torch.device(device)
    config = LlamaConfig(hidden_size=hidden_size, intermediate_size=intermediate_size // world,
                         num_hidden_layers=num_layers, num_attention_heads=num_heads // world,
                         num_key_value_heads=num_kv_heads // world, head_dim=head_dim, vocab_size=vocab_size,
                         max_position_embeddings=max(max_cache_len, 2048), tie_word_embeddings=False,
                         attention_bias=False, mlp_bias=False)
    torch.manual_seed(seed)  # replicated tensors (embeddings, norms, lm_head) must agree across ranks
    previous = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)  # create the parameters in BF16 (a 70B shard in FP32 would not fit)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(config).to(torch.bfloat16)
    finally:
        torch.set_default_dtype(previous)
    model.eval()
    full_shapes = {"self_attn.q_proj": (num_heads * head_dim, hidden_size),
                   "self_attn.k_proj": (num_kv_heads * head_dim, hidden_size),
                   "self_attn.v_proj": (num_kv_heads * head_dim, hidden_size),
                   "self_attn.o_proj": (hidden_size, num_heads * head_dim),
                   "mlp.gate_proj": (intermediate_size, hidden_size), "mlp.up_proj": (intermediate_size, hidden_size),
                   "mlp.down_proj": (hidden_size, intermediate_size)}
    for index, layer in enumerate(model.model.layers):
        caches = {}
        for group in GROUPS:
            pair = (SharedHadamardCache(len(group)), SharedPackedActivationCache(len(group)))
            for member in group:
                caches[member] = pair
        for name in COLUMN + ROW:
            parent_name, child_name = name.split(".")
            parent = getattr(layer, parent_name)
            linear = getattr(parent, child_name)
            full_name = f"model.layers.{index}.{name}.weight"
            rows, cols = full_shapes[name]
            full = full_projection_weight(index, name, rows, cols, seed=seed, device=device)
            if name in ROW:
                lo, hi = cols // world * rank, cols // world * (rank + 1)
                if tuple(linear.weight.shape) != (rows, hi - lo):
                    raise RuntimeError(f"{name}: shard shape {tuple(linear.weight.shape)} is not a K slice of {(rows, cols)}")
                fused = RowParallelNQRTLinear(full[:, lo:hi].contiguous(), rank, world,
                                              dither_seed=tensor_dither_seed(58, f"{full_name}.tp{rank}of{world}"),
                                              weight_betas=WEIGHT_BETAS, activation_betas=ACTIVATION_BETAS,
                                              process_group=process_group)
            else:
                lo, hi = rows // world * rank, rows // world * (rank + 1)
                if tuple(linear.weight.shape) != (hi - lo, cols):
                    raise RuntimeError(f"{name}: shard shape {tuple(linear.weight.shape)} is not a row range of {(rows, cols)}")
                prepared = quantize_weight_cuda(hadamard(full[lo:hi].contiguous()), betas=WEIGHT_BETAS,
                                                dither_seed=tensor_dither_seed(58, full_name), tensor_name=full_name,
                                                block_offset=lo * (cols // 8))
                hcache, acache = caches[name]
                fused = FusedNQRTLinear(prepared, full_name, input_hadamard=True, input_transform_cache=hcache,
                                        activation_betas=ACTIVATION_BETAS, packed_activation_cache=acache)
            setattr(parent, child_name, fused.to(device))
            del linear, full
        for group in GROUPS:  # q/k/v and gate/up shards: one decode + GEMM launch sequence per group
            SharedProjectionGroup([getattr(getattr(layer, name.split(".")[0]), name.split(".")[1]) for name in group])
        torch.cuda.empty_cache()
    cache = BatchedNQKVLlamaCache(capacity=capacity, num_layers=num_layers, num_query_heads=num_heads // world,
                                  num_kv_heads=num_kv_heads // world, head_dim=head_dim, max_cache_len=max_cache_len,
                                  key_betas=KEY_BETAS, value_betas=VALUE_BETAS, dtype=torch.bfloat16, device=device)
    install_batched_nqkv_llama_backend(model, cache)
    fuse_rmsnorm_(model)  # one launch per normalisation instead of six tensor kernels
    return model, cache


@torch.no_grad()
def attach_peer_all_reduce(model: torch.nn.Module, max_rows: int, device: torch.device | str, process_group=None):
    """Give every row-parallel projection of ``model`` the peer-memory sum (``tensor_parallel.PeerAllReduce``) in place
    of the NCCL all-reduce; ``max_rows`` is the largest number of token rows a call will carry.  Returns the reducer
    (its ``status()`` is non-zero when a bounded wait gave up); raises when symmetric memory cannot be set up, in
    which case the modules keep NCCL."""
    from .tensor_parallel import PeerAllReduce

    rows = [m for m in model.modules() if isinstance(m, RowParallelNQRTLinear)]
    if not rows:
        raise ValueError("model has no row-parallel projections")
    width = max(m.out_features for m in rows)
    reducer = PeerAllReduce(int(max_rows) * width, torch.device(device), process_group)
    for module in rows:
        module.peer_all_reduce = reducer
    return reducer


def fill_cache_synthetic(cache: BatchedNQKVLlamaCache, context: int, *, seed: int = 4096) -> None:
    """Fill every slot with ``context`` tokens of seeded synthetic K/V through the page encoder.

    Stands in for a prefill (the page writer is the same kernel): full pages go to the static page
    ids ``slot * max_pages + page``, the remainder to the hot tail.
    """
    page, heads, dim, capacity = cache.page_size, cache.num_kv_heads, cache.head_dim, cache.capacity
    full, rest = context // page, context % page
    if full > cache.max_pages:
        raise ValueError("context exceeds the cache length")
    gen = torch.Generator(device=cache.device).manual_seed(seed)
    slots = torch.arange(capacity, device=cache.device)
    ids = (slots[:, None] * cache.max_pages + torch.arange(full, device=cache.device)[None, :]).reshape(-1)
    for slot in range(capacity):
        if slot not in cache._sequence_of_slot:
            cache.register(f"synthetic-{slot}", slot=slot)
    for layer in cache.layer_caches:
        pool = layer.pool
        for codes, betas, norms, table, values, rotate in (
                (pool.key_codes, pool.key_betas, pool.key_norms, pool.beta_table, pool.betas, True),
                (pool.value_codes, pool.value_betas, pool.value_norms, pool.value_beta_table, pool.value_beta_values, False)):
            if full:
                x = torch.randn(capacity * full * page * heads, dim, generator=gen, device=cache.device)
                x = (hadamard(x) if rotate else x).bfloat16()
                act = quantize_activation_cuda(x, q=14, betas=values, beta_table=table, keep_decoded=False)
                codes[ids] = act.code_payload.view(capacity * full, -1)
                betas[ids] = act.beta_payload.view(capacity * full, -1)
                norms[ids] = act.row_norms.view(capacity * full, -1)
                del x, act
        if full:
            pool.expand_pages(ids)  # keeps the opt-in decoded shadow current (no-op without one)
            layer.page_indices[:, :full] = ids.view(capacity, full).to(torch.int32)
        layer.page_counts.fill_(full)
        layer.last_page_len.fill_(page if full else 0)
        layer.hot_lengths.fill_(rest)
        layer.sequence_lengths.fill_(context)
        if rest:
            layer.hot_keys[:, :rest] = torch.randn(capacity, rest, heads, dim, generator=gen, device=cache.device).bfloat16()
            layer.hot_values[:, :rest] = torch.randn(capacity, rest, heads, dim, generator=gen, device=cache.device).bfloat16()


class TensorParallelRunner(BatchedNQKVLlamaRunner):
    """Decode runner of one shard: same step, collectives happen inside the row-parallel modules."""

    def __init__(self, model, cache, *, weight_decode_ahead: bool = False, **options) -> None:
        # one stream per shard unless asked: the second stream's decodes would share the SMs with the collective
        super().__init__(model, cache, weight_decode_ahead=weight_decode_ahead, **options)

    def start_decode(self, context: int, *, seed: int = 1) -> None:
        gen = torch.Generator().manual_seed(seed)  # identical tokens on every rank
        vocab = self.model.config.vocab_size
        self.tokens.copy_(torch.randint(0, vocab, self.tokens.shape, generator=gen).to(self.device))
        self.positions.fill_(context)
