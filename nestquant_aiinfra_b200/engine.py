"""W4A4KV4 Llama runner: GPU weight conversion, ragged prefill and CUDA-graph decode.

Counterpart of the reference's ``BatchedNQKVLlamaRunner`` (runtime/nqkv_batched_runner.py:
eager prefill :190-225, graph decode :302-361) reduced to what drives the hot path: the
model is a stock Hugging Face ``LlamaForCausalLM`` whose 7 projections per layer are
``FusedNQRTLinear`` modules and whose attention goes through ``BatchedNQKVLlamaCache``.
Because page ids are assigned on the device, one captured graph serves every decode step
(the reference needs a second "boundary" graph and a host read of the hot lengths).
"""

from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from .formats import ACTIVATION_BETAS, KEY_BETAS, VALUE_BETAS, WEIGHT_BETAS, tensor_dither_seed
from .fused_linear import (FusedNQRTLinear, SharedHadamardCache, SharedPackedActivationCache,
                           SharedProjectionGroup, keep_decoded_weights_)
from .hf_backend import BatchedNQKVLlamaCache, install_batched_nqkv_llama_backend
from .norm import fuse_rmsnorm_
from .rope import fused_rope_scope
from .rotation import hadamard
from .runtime.w4a4 import quantize_weight_cuda

PROJECTIONS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
               "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")
SHARE_GROUPS = (("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("mlp.gate_proj", "mlp.up_proj"))


def quantize_llama_projections_(model: nn.Module, *, weight_betas: Sequence[float] = WEIGHT_BETAS,
                                activation_betas: Sequence[float] = ACTIVATION_BETAS, project_seed: int = 58,
                                group_shared_inputs: bool = True) -> int:
    """Replace every decoder projection by a packed NQRT4 module, encoding W*H on the GPU.

    The input of each module is Hadamard-rotated, so the stored weight is ``hadamard(W)``
    (``(xH)(WH)^T = xW^T``); the dither seed is the reference's per-tensor seed
    (models/quantization.py:382-384).  Returns the number of converted projections.
    """
    converted = 0
    for layer_index, layer in enumerate(model.model.layers):
        caches = {}
        for group in SHARE_GROUPS:
            pair = (SharedHadamardCache(len(group)), SharedPackedActivationCache(len(group)))
            for member in group:
                caches[member] = pair
        for name in PROJECTIONS:
            parent_name, child_name = name.split(".")
            parent = getattr(layer, parent_name)
            linear = getattr(parent, child_name)
            if not isinstance(linear, nn.Linear) or linear.bias is not None:
                raise ValueError(f"layer {layer_index} {name} is not a bias-free nn.Linear")
            full_name = f"model.layers.{layer_index}.{name}.weight"
            rotated = hadamard(linear.weight.detach().float())
            prepared = quantize_weight_cuda(rotated, betas=weight_betas,
                                            dither_seed=tensor_dither_seed(project_seed, full_name),
                                            tensor_name=full_name)
            hcache, acache = caches.get(name, (None, None))
            fused = FusedNQRTLinear(prepared, full_name, input_hadamard=True, input_transform_cache=hcache,
                                    activation_betas=tuple(activation_betas), packed_activation_cache=acache)
            setattr(parent, child_name, fused.to(linear.weight.device))
            del linear, rotated
            converted += 1
        if group_shared_inputs:  # q/k/v and gate/up: one decode + GEMM launch sequence per group
            for group in SHARE_GROUPS:
                members = [getattr(getattr(layer, name.split(".")[0]), name.split(".")[1]) for name in group]
                SharedProjectionGroup(members)
    torch.cuda.empty_cache()
    return converted


def build_llama_w4a4kv4(*, hidden_size: int, intermediate_size: int, num_layers: int, num_heads: int,
                        num_kv_heads: int, head_dim: int, vocab_size: int, capacity: int, max_cache_len: int,
                        device: torch.device | str = "cuda", seed: int = 0, page_size: int = 16):
    """Random-init Llama architecture converted to W4A4KV4: returns ``(model, cache)``."""
    from transformers import LlamaConfig, LlamaForCausalLM

    config = LlamaConfig(hidden_size=hidden_size, intermediate_size=intermediate_size, num_hidden_layers=num_layers,
                         num_attention_heads=num_heads, num_key_value_heads=num_kv_heads, head_dim=head_dim,
                         vocab_size=vocab_size, max_position_embeddings=max(max_cache_len, 2048),
                         tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    torch.manual_seed(seed)
    device = torch.device(device)
    previous = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)  # create the parameters in BF16 (a 70B shard in FP32 would not fit)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(config).to(torch.bfloat16)
    finally:
        torch.set_default_dtype(previous)
    model.eval()
    quantize_llama_projections_(model)
    cache = BatchedNQKVLlamaCache(capacity=capacity, num_layers=num_layers, num_query_heads=num_heads,
                                  num_kv_heads=num_kv_heads, head_dim=head_dim, max_cache_len=max_cache_len,
                                  page_size=page_size, key_betas=KEY_BETAS, value_betas=VALUE_BETAS,
                                  dtype=torch.bfloat16, device=device)
    install_batched_nqkv_llama_backend(model, cache)
    fuse_rmsnorm_(model)  # one launch per normalisation instead of six tensor kernels
    return model, cache


class BatchedNQKVLlamaRunner:
    """Greedy ragged prefill + fixed-width graph decode over a ``BatchedNQKVLlamaCache``."""

    def __init__(self, model: nn.Module, cache: BatchedNQKVLlamaCache) -> None:
        self.model, self.cache = model, cache
        self.device = cache.device
        c = cache.capacity
        self.tokens = torch.zeros((c, 1), dtype=torch.long, device=self.device)
        self.positions = torch.zeros((c, 1), dtype=torch.long, device=self.device)
        self.next_tokens = torch.zeros(c, dtype=torch.long, device=self.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._generation = [0] * c

    @torch.no_grad()
    def prefill_slots(self, slots: Sequence[int], prompts: Sequence[torch.Tensor]) -> torch.Tensor:
        """Whole-prompt prefill of ``prompts[i]`` into ``slots[i]``; returns the greedy next token per row."""
        if len(slots) != len(prompts) or not slots:
            raise ValueError("slots and prompts must be non-empty and of equal length")
        width = max(int(p.numel()) for p in prompts)
        ids = torch.zeros((len(slots), width), dtype=torch.long, device=self.device)
        lengths = []
        assignments = []
        for row, (slot, prompt) in enumerate(zip(slots, prompts)):
            self._generation[slot] += 1
            assignments.append((f"slot-{slot}-generation-{self._generation[slot]}", slot))
            ids[row, :prompt.numel()] = prompt.to(self.device)
            lengths.append(int(prompt.numel()))
        self.cache.register_batch(assignments)
        slot_ids = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        q_lens = torch.tensor(lengths, dtype=torch.int32, device=self.device)
        positions = torch.arange(width, device=self.device).unsqueeze(0).expand(len(slots), width).contiguous()
        self.cache.set_prefill_state(slot_ids=slot_ids, query_lengths=q_lens, from_empty=True,  # slots were just registered
                                     host_slots=list(slots), host_lengths=lengths)
        try:
            with fused_rope_scope():
                hidden = self.model.model(input_ids=ids, position_ids=positions, past_key_values=self.cache,
                                          use_cache=True).last_hidden_state
        finally:
            self.cache.set_decode_state()
        last = hidden[torch.arange(len(slots), device=self.device), q_lens.long() - 1]
        next_tokens = self.model.lm_head(last).argmax(dim=-1)
        index = slot_ids.long()
        self.tokens[index, 0] = next_tokens
        self.positions[index, 0] = q_lens.long()
        return next_tokens

    @torch.no_grad()
    def _step(self) -> None:
        with fused_rope_scope():  # rope + Q/K Hadamard rotation in one launch per tensor
            logits = self.model(input_ids=self.tokens, position_ids=self.positions, past_key_values=self.cache,
                                use_cache=True).logits
        self.next_tokens.copy_(logits[:, -1].argmax(dim=-1))
        active = self.cache.active_mask
        self.tokens[:, 0] = torch.where(active, self.next_tokens, self.tokens[:, 0])
        self.positions[:, 0] += active.long()

    def decode_eager(self) -> torch.Tensor:
        """One decode step for every active slot without a graph; returns the new tokens ``[capacity]``."""
        self.cache.set_decode_state()
        self._step()
        return self.next_tokens

    def capture_decode_graph(self) -> None:
        """Capture one fixed-width decode step (all ``capacity`` rows, inactive rows masked on the device)."""
        self.cache.set_decode_state()
        state = self._snapshot()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._step()  # warm-up: loads kernels, sizes workspaces
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self._restore(state)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step()
        torch.cuda.synchronize(self.device)
        self._restore(state)
        self.graph = graph

    def decode(self) -> torch.Tensor:
        if self.graph is None:
            return self.decode_eager()
        self.graph.replay()
        return self.next_tokens

    # Opt-in modes that spend spare HBM on decoded copies (off by default; the packed data stay the record).
    # Both change which kernels a step launches, so a captured graph is captured again.
    def keep_decoded_weights(self) -> int:
        """Keep the decoded BF16 weights of every packed projection resident; returns the bytes added."""
        added = keep_decoded_weights_(self.model)
        if self.graph is not None:
            self.capture_decode_graph()
        return added

    def enable_lattice_shadow(self) -> int:
        """Keep the decoded lattice coordinates of the KV pages beside their codes; returns the bytes added."""
        added = self.cache.enable_lattice_shadow()
        if self.graph is not None:
            self.capture_decode_graph()
        return added

    # the warm-up and the capture run a real step; put the cache back afterwards
    def _snapshot(self):
        per_layer = []
        for cache in self.cache.layer_caches:
            per_layer.append(tuple(t.clone() for t in (cache.page_indices, cache.page_counts, cache.last_page_len,
                                                       cache.hot_lengths, cache.sequence_lengths, cache.hot_keys,
                                                       cache.hot_values)))
        return per_layer, self.tokens.clone(), self.positions.clone()

    def _restore(self, state) -> None:
        per_layer, tokens, positions = state
        for cache, saved in zip(self.cache.layer_caches, per_layer):
            for dst, src in zip((cache.page_indices, cache.page_counts, cache.last_page_len, cache.hot_lengths,
                                 cache.sequence_lengths, cache.hot_keys, cache.hot_values), saved):
                dst.copy_(src)
        self.tokens.copy_(tokens)
        self.positions.copy_(positions)
