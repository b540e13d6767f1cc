"""W4A4KV4 Llama runner: GPU weight conversion, ragged prefill and CUDA-graph decode.

Counterpart of the reference's ``BatchedNQKVLlamaRunner`` (runtime/nqkv_batched_runner.py:
eager prefill :190-225, graph decode :302-361): the model is a stock Hugging Face
``LlamaForCausalLM`` whose 7 projections per layer are ``FusedNQRTLinear`` modules and whose
attention goes through ``BatchedNQKVLlamaCache``.  Because page ids are assigned on the device,
one captured graph serves every decode step (the reference needs a second "boundary" graph and a
host read of the hot lengths).

The runner can be driven in two ways:

* as the ``RaggedDecodeBackend`` of the reference's continuous-batching engine
  (runtime/inference_engine.py:14-32): ``prefill(input_ids)``, ``prefill_slots(input_ids,
  positions=, write_mask=, valid_lengths=)``, ``capture(...)``, ``decode(token, positions=,
  active_mask=, valid_lengths=)`` returning logits, ``clear_slots(slot_mask)``;
* with sampling kept on the device: ``prefill_slots(slots, prompts)`` and ``decode()`` returning
  the greedy tokens of all rows (what the throughput benchmark uses).
"""

from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from .formats import ACTIVATION_BETAS, KEY_BETAS, VALUE_BETAS, WEIGHT_BETAS, tensor_dither_seed
from .fused_linear import (FusedNQRTLinear, SharedHadamardCache, SharedPackedActivationCache,
                           SharedProjectionGroup, WeightDecodeAhead, keep_decoded_weights_)
from .hf_backend import BatchedNQKVLlamaCache, install_batched_nqkv_llama_backend
from .norm import fuse_rmsnorm_, fuse_silu_mlp_
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
                        device: torch.device | str = "cuda", seed: int = 0, page_size: int = 16,
                        page_allocation: str = "static", pool_pages: int | None = None,
                        fuse_producers: bool = True):
    """Random-init Llama architecture converted to W4A4KV4: returns ``(model, cache)``.

    ``fuse_producers`` moves the decoder layers' RMS norms and the MLP's SiLU * up into the encoder launch of the
    projections they feed (same bits, fewer launches per step).
    """
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
                                  dtype=torch.bfloat16, device=device, page_allocation=page_allocation,
                                  pool_pages=pool_pages)
    install_batched_nqkv_llama_backend(model, cache)
    fuse_rmsnorm_(model, defer_into_projections=fuse_producers)  # one launch per normalisation, or none at all
    if fuse_producers:
        fuse_silu_mlp_(model)
    return model, cache


class BatchedNQKVLlamaRunner:
    """Greedy ragged prefill + fixed-width graph decode over a ``BatchedNQKVLlamaCache``."""

    def __init__(self, model: nn.Module, cache: BatchedNQKVLlamaCache, *, execution_policy: str = "full",
                 prefill_logits: str = "last", weight_decode_ahead: bool = True) -> None:
        if not isinstance(model, nn.Module):
            raise TypeError("model must be a torch module")
        if not isinstance(cache, BatchedNQKVLlamaCache):
            raise TypeError("cache must be a BatchedNQKVLlamaCache")
        if execution_policy not in {"fixed", "decode", "full"}:
            raise ValueError("execution_policy must be fixed, decode, or full")
        if prefill_logits not in {"last", "all"}:
            raise ValueError("prefill_logits must be last or all")
        self.model, self.cache = model, cache
        self.device = cache.device
        self.execution_policy = execution_policy
        # Captured decode steps of at least eight rows decode the weights a layer needs after its attention on a
        # second stream while the attention runs (``enable_weight_decode_ahead``; bit-identical results, one
        # layer's decoded weights of scratch).  False keeps every step on one stream.
        self.weight_decode_ahead = bool(weight_decode_ahead)
        # scratch of a switched-off decode-ahead: a graph captured earlier may still write to it when replayed
        self._retired_decode_ahead: list = []
        self._idle_decode_ahead = None  # switched off by the user: attached again when switched back on
        # "last": prefill_slots evaluates the lm_head at the last prompt token of every row only and returns a
        # [capacity, width, vocab] VIEW whose columns all alias that row's logits (no memory), which is what a
        # sampler reads; "all" materialises the logits of every position as the reference does.
        self.prefill_logits = prefill_logits
        c = cache.capacity
        self.batch_size = c
        self.max_cache_len = cache.max_cache_len
        self.tokens = torch.zeros((c, 1), dtype=torch.long, device=self.device)
        self.positions = torch.zeros((c, 1), dtype=torch.long, device=self.device)
        self.next_tokens = torch.zeros(c, dtype=torch.long, device=self.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._generation = [0] * c
        # state of the engine protocol
        self.logits: torch.Tensor | None = None            # [capacity, 1, vocab], written by the captured step
        self.logits_graph: torch.cuda.CUDAGraph | None = None
        self._prepared = False
        self.compact_prefill_calls = 0
        self.compact_prefill_rows = 0
        self.graph_replay_count = 0

    # ------------------------------------------------------------------ reference engine protocol
    @property
    def graph_captured(self) -> bool:
        return self.logits_graph is not None

    def _validate_common(self, input_ids, positions, write_mask, valid_lengths) -> None:
        if input_ids.dtype != torch.long or input_ids.ndim != 2:
            raise ValueError("input_ids must be rank-2 torch.long")
        if input_ids.shape[0] != self.batch_size:
            raise ValueError("input batch must equal fixed runner capacity")
        if positions.dtype != torch.long or positions.shape != input_ids.shape:
            raise ValueError("positions must be torch.long and match input_ids")
        if write_mask.dtype != torch.bool or write_mask.shape != input_ids.shape:
            raise ValueError("write_mask must be bool and match input_ids")
        if valid_lengths.dtype != torch.long or tuple(valid_lengths.shape) != (self.batch_size,):
            raise ValueError("valid_lengths must have shape [batch_size]")
        if any(t.device != self.device for t in (input_ids, positions, write_mask, valid_lengths)):
            raise ValueError("runner inputs must be on the model CUDA device")
        if bool(write_mask.any().item()):
            written = positions[write_mask]
            if int(written.min().item()) < 0:
                raise ValueError("written positions must be non-negative")
            if int(written.max().item()) >= self.max_cache_len:
                raise ValueError("written positions exceed the NQKV cache")

    def _register_new_rows(self, row_mask: torch.Tensor) -> None:
        assignments = []
        for slot in row_mask.nonzero(as_tuple=False).flatten().cpu().tolist():
            try:
                self.cache.manager.sequence_id(slot)
            except KeyError:
                self._generation[slot] += 1
                assignments.append((f"slot-{slot}-generation-{self._generation[slot]}", slot))
        if assignments:
            self.cache.register_batch(assignments)

    def _hidden(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Decoder stack only; ends the cache's prefill transaction (releasing the rows after a failure)."""
        try:
            with fused_rope_scope():
                hidden = self.model.model(input_ids=input_ids, position_ids=positions, past_key_values=self.cache,
                                          use_cache=True).last_hidden_state
        except Exception:
            self.cache.finish_prefill_page_transaction(success=False)
            raise
        self.cache.finish_prefill_page_transaction(success=True)
        return hidden

    def _prefill_logits(self, hidden: torch.Tensor, write_mask: torch.Tensor) -> torch.Tensor:
        """``[rows, width, vocab]`` logits of a prefill, per the ``prefill_logits`` policy."""
        if self.prefill_logits == "all" or hidden.shape[1] == 1:
            return self.model.lm_head(hidden)
        rows, width = write_mask.shape
        last = (write_mask.sum(dim=1) - 1).clamp_min(0)
        picked = self.model.lm_head(hidden[torch.arange(rows, device=self.device), last])
        return picked[:, None, :].expand(rows, width, picked.shape[-1])

    def _engine_prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Warm all fixed rows with ``input_ids [capacity, width]``; the engine clears them right afterwards."""
        if input_ids.dtype != torch.long or input_ids.ndim != 2:
            raise ValueError("input_ids must be rank-2 torch.long")
        if input_ids.shape[0] != self.batch_size or input_ids.device != self.device:
            raise ValueError("input_ids batch or device does not match the runner")
        width = input_ids.shape[1]
        if width < 1 or width > self.max_cache_len:
            raise ValueError("prefill width is outside the NQKV cache")
        positions = torch.arange(width, device=self.device).expand(self.batch_size, -1).contiguous()
        write_mask = torch.ones_like(input_ids, dtype=torch.bool)
        self._register_new_rows(write_mask.any(dim=1))
        self.cache.disable_graph_decode()
        self.cache.set_batch_state(active_mask=write_mask.any(dim=1), write_mask=write_mask)
        logits = self._prefill_logits(self._hidden(input_ids, positions), write_mask)
        self._prepared = True
        return logits

    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self._engine_prefill(input_ids)

    def _engine_prefill_slots(self, input_ids, positions, write_mask, valid_lengths) -> torch.Tensor:
        if not self._prepared:
            raise RuntimeError("initial prefill must prepare the runner")
        self._validate_common(input_ids, positions, write_mask, valid_lengths)
        row_active = write_mask.any(dim=1)
        self._register_new_rows(row_active)
        self.cache.disable_graph_decode()
        active_count = int(row_active.sum().item())
        if self.execution_policy != "full" or active_count in (0, self.batch_size):
            self.cache.set_batch_state(active_mask=row_active, write_mask=write_mask)
            return self._prefill_logits(self._hidden(input_ids, positions), write_mask)
        # only the rows that write take part in the forward
        self.compact_prefill_calls += 1
        self.compact_prefill_rows += active_count
        compact_mask = write_mask[row_active]
        self.cache.set_prefill_execution_state(slot_ids=self.cache.slot_ids[row_active], write_mask=compact_mask)
        compact = self._prefill_logits(self._hidden(input_ids[row_active], positions[row_active]), compact_mask)
        if self.prefill_logits == "last" and compact.shape[1] > 1:
            picked = torch.zeros((self.batch_size, compact.shape[-1]), device=self.device, dtype=compact.dtype)
            picked[row_active] = compact[:, 0]
            return picked[:, None, :].expand(self.batch_size, input_ids.shape[1], picked.shape[-1])
        logits = torch.zeros((self.batch_size, compact.shape[1], compact.shape[2]), device=self.device, dtype=compact.dtype)
        logits[row_active] = compact
        return logits

    def _logits_step(self) -> None:
        with fused_rope_scope():
            out = self.model(input_ids=self.tokens, position_ids=self.positions, past_key_values=self.cache,
                             use_cache=True).logits
        self.logits.copy_(out)

    @torch.inference_mode()
    def capture(self, sample_token: torch.Tensor, *, positions: torch.Tensor, active_mask: torch.Tensor,
                valid_lengths: torch.Tensor) -> None:
        """Capture ONE fixed-width decode step that returns logits (inactive rows are masked on the device;
        full hot pages are detected and packed inside the same graph, so no boundary graph is needed)."""
        if not self._prepared:
            raise RuntimeError("prefill must prepare the runner before warmup")
        if self.logits_graph is not None:
            return
        self._validate_common(sample_token, positions, active_mask, valid_lengths)
        if sample_token.shape[1] != 1:
            raise ValueError("decode capture takes one token per row")
        self.tokens.copy_(sample_token)
        self.positions.copy_(positions)
        self.cache.active_mask.copy_(active_mask[:, 0])
        self.cache.set_decode_state()
        self._ensure_decode_ahead()
        vocab = self.model.config.vocab_size
        dtype = next(self.model.parameters()).dtype
        self.logits = torch.zeros((self.batch_size, 1, vocab), device=self.device, dtype=dtype)
        state = self._snapshot()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._logits_step()  # warm-up: loads kernels, sizes workspaces
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self._restore(state)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self._capture_stream()):
            self._logits_step()
        torch.cuda.synchronize(self.device)
        self._restore(state)
        self.logits_graph = graph

    def _engine_decode(self, token, positions, active_mask, valid_lengths) -> torch.Tensor:
        if self.logits_graph is None or self.logits is None:
            raise RuntimeError("capture must warm the runner before decode")
        self._validate_common(token, positions, active_mask, valid_lengths)
        if token.shape[1] != 1:
            raise ValueError("decode takes one token per row")
        self.tokens.copy_(token)
        self.positions.copy_(positions)
        self.cache.active_mask.copy_(active_mask[:, 0])
        self.cache.set_decode_state()
        self.logits_graph.replay()
        self.graph_replay_count += 1
        return torch.where(active_mask[:, :, None], self.logits, torch.zeros((), device=self.device, dtype=self.logits.dtype))

    def clear_slots(self, slot_mask: torch.Tensor) -> None:
        if slot_mask.dtype != torch.bool or tuple(slot_mask.shape) != (self.batch_size,):
            raise ValueError("slot_mask must be bool with shape [batch_size]")
        if slot_mask.device != self.device:
            raise ValueError("slot_mask must be on the model device")
        self.cache.release_slots(slot_mask.nonzero(as_tuple=False).flatten().cpu().tolist())

    # ------------------------------------------------------------------ device-side sampling
    @torch.no_grad()
    def prefill_slots(self, slots, prompts=None, *, positions: torch.Tensor | None = None,
                      write_mask: torch.Tensor | None = None, valid_lengths: torch.Tensor | None = None,
                      max_tokens: int | None = None) -> torch.Tensor:
        """Two call forms.

        ``prefill_slots(input_ids, positions=, write_mask=, valid_lengths=)`` is the engine protocol
        (runtime/nqkv_batched_runner.py:190-225): ``input_ids [capacity, width]``, rows that write are
        new requests; returns logits ``[capacity, width, vocab]`` (see ``prefill_logits``).

        ``prefill_slots(slots, prompts)`` is whole-prompt prefill of ``prompts[i]`` into ``slots[i]``
        with the sampling on the device; returns the greedy next token per row.  ``max_tokens`` (prompt plus
        the tokens the request may still generate) is the admission budget of a cache with device-side page
        allocation; it defaults to the cache length.
        """
        if positions is not None or write_mask is not None or valid_lengths is not None:
            if prompts is not None or positions is None or write_mask is None or valid_lengths is None:
                raise TypeError("the engine form takes input_ids, positions=, write_mask= and valid_lengths=")
            with torch.inference_mode():
                return self._engine_prefill_slots(slots, positions, write_mask, valid_lengths)
        if prompts is None:
            raise TypeError("prefill_slots(slots, prompts) needs the prompts")
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
        self.cache.register_batch(assignments, max_tokens=max_tokens)
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
        self._ensure_decode_ahead()
        state = self._snapshot()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._step()  # warm-up: loads kernels, sizes workspaces
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self._restore(state)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self._capture_stream()):
            self._step()
        torch.cuda.synchronize(self.device)
        self._restore(state)
        self.graph = graph

    def _capture_stream(self) -> torch.cuda.Stream:
        """The step is captured on a stream of the highest priority, so that its kernels keep their priority as
        graph nodes over the weight decodes that run beside them on the lowest one."""
        if getattr(self, "_step_stream", None) is None:
            self._step_stream = torch.cuda.Stream(self.device, priority=-5)
        return self._step_stream

    def decode(self, token: torch.Tensor | None = None, *, positions: torch.Tensor | None = None,
               active_mask: torch.Tensor | None = None, valid_lengths: torch.Tensor | None = None) -> torch.Tensor:
        """``decode()``: one step for every active slot, greedy tokens ``[capacity]`` sampled on the device.

        ``decode(token, positions=, active_mask=, valid_lengths=)``: the engine protocol
        (runtime/nqkv_batched_runner.py:302-361), one graph replay, returns logits ``[capacity, 1, vocab]``
        with the rows that are not active zeroed.
        """
        if token is not None:
            if positions is None or active_mask is None or valid_lengths is None:
                raise TypeError("the engine form takes token, positions=, active_mask= and valid_lengths=")
            with torch.inference_mode():
                return self._engine_decode(token, positions, active_mask, valid_lengths)
        if self.graph is None:
            return self.decode_eager()
        self.graph.replay()
        return self.next_tokens

    def enable_weight_decode_ahead(self) -> int:
        """Decode the weights of ``o_proj``, gate / up and ``down_proj`` of a layer on a second stream while the
        layer's paged attention runs (``fused_linear.WeightDecodeAhead``): same kernels, same results, the idle
        tail of the attention filled.  Costs one layer's decoded weights of scratch (returned, in bytes) and takes
        effect for decode steps of at least eight rows; a captured decode graph is captured again."""
        self.weight_decode_ahead = True
        if self.cache.decode_ahead is not None:
            return 0
        self._ensure_decode_ahead()
        self._recapture()
        return 0 if self.cache.decode_ahead is None else self.cache.decode_ahead.scratch_bytes

    def disable_weight_decode_ahead(self) -> None:
        self.weight_decode_ahead = False
        self._retire_decode_ahead(reusable=True)
        self._recapture()

    def _retire_decode_ahead(self, reusable: bool = False) -> None:
        ahead = self.cache.decode_ahead or (None if reusable else self._idle_decode_ahead)
        if ahead is None:
            return
        ahead.detach()
        self.cache.decode_ahead = None
        if reusable:
            self._idle_decode_ahead = ahead
        else:
            self._idle_decode_ahead = None
            self._retired_decode_ahead.append(ahead)

    def _ensure_decode_ahead(self) -> None:
        if not self.weight_decode_ahead or self.cache.decode_ahead is not None:
            return
        if self.batch_size < WeightDecodeAhead.MIN_ROWS:
            return
        if self._idle_decode_ahead is not None:
            ahead, self._idle_decode_ahead = self._idle_decode_ahead, None
            ahead.attach()
        else:
            layers = getattr(getattr(self.model, "model", None), "layers", None)
            if layers is None:  # not a decoder stack this runner knows how to walk: every step stays on one stream
                return
            ahead = WeightDecodeAhead(layers, self.device)
        if any(ahead.layers):
            self.cache.decode_ahead = ahead

    def _recapture(self) -> None:
        # (a logits graph of the engine protocol keeps replaying the mode it was captured in)
        if self.graph is not None:
            self.capture_decode_graph()

    # Opt-in modes that spend spare HBM on decoded copies (off by default; the packed data stay the record).
    # Both change which kernels a step launches, so a captured graph is captured again.
    def keep_decoded_weights(self) -> int:
        """Keep the decoded BF16 weights of every packed projection resident; returns the bytes added."""
        self._retire_decode_ahead()  # nothing is left to decode ahead, and the units point at weights replaced now
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
            per_layer.append(tuple(t.clone() for t in self._state_tensors(cache)))
        return per_layer, self.tokens.clone(), self.positions.clone()

    @staticmethod
    def _state_tensors(cache):
        tensors = [cache.page_indices, cache.page_counts, cache.last_page_len, cache.hot_lengths,
                   cache.sequence_lengths, cache.hot_keys, cache.hot_values]
        if cache.pool.free_ids is not None:  # device-side allocator: a warm-up step may pop pages
            tensors += [cache.pool.free_ids, cache.pool.free_count]
        return tensors

    def _restore(self, state) -> None:
        per_layer, tokens, positions = state
        for cache, saved in zip(self.cache.layer_caches, per_layer):
            for dst, src in zip(self._state_tensors(cache), saved):
                dst.copy_(src)
        self.tokens.copy_(tokens)
        self.positions.copy_(positions)
