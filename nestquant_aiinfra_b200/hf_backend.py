"""Hugging Face plugin boundary of the NQKV4 cache: ``Cache`` subclass + attention interface.

Mirror of ``nestquant.runtime.nqkv_batched_hf_backend`` (BatchedNQKVLlamaCache :26-631,
_batched_nqkv_attention_interface :633-651, install_batched_nqkv_llama_backend :654-680):
``update`` rotates K with the Hadamard transform (V is not rotated), appends the new tokens to
the BF16 hot tail and packs full pages; the attention interface rotates Q and runs the paged
kernel for decode (one token) or for a whole-prompt chunk.

Differences from the reference, all on the host side: page ids are assigned statically
(``slot * max_pages + page``), so the page writer needs no host reservation and the same
captured graph serves boundary and non-boundary steps; a prefill chunk that continues a cached
sequence reads the pages it has just written plus the hot tail (the reference only prefills from
empty slots, with SDPA over the chunk's BF16 K/V -- which is what a prefill from empty slots does
here too).

Two ways to drive the cache:

* the reference's runner protocol (runtime/nqkv_batched_hf_backend.py:147-354, 493-531):
  ``set_batch_state`` / ``set_decode_execution_state`` / ``set_prefill_execution_state`` /
  ``enable_graph_decode`` / ``disable_graph_decode`` / ``finish_prefill_page_transaction`` and the
  ``manager`` object its runner reaches into.  The reference's ``BatchedNQKVLlamaRunner`` and
  ``ContinuousBatchInferenceEngine`` can drive this class unchanged;
* ``set_decode_state`` / ``set_prefill_state`` of this package's own runner, which additionally
  allows a chunk to continue a cached sequence and one graph for every decode step.
"""

from __future__ import annotations

import math
from typing import Hashable, Sequence

import torch
from transformers.cache_utils import Cache

from .rope import rotation_done
from .rotation import hadamard
from .runtime.w4a4 import quantize_activation_cuda
from .runtime.kv import (BatchedNQKVAttentionWorkspace, NQKVHotColdCache, NQKVPagePool,
                         _launch_append_hot_k1_graph_safe, _launch_append_hot_ragged_segment_graph_safe,
                         _launch_nqkv_decode_attention_batched_k1, launch_pack_full_hot_pages_graph_safe,
                         nqkv_prefill_attention)

BATCHED_NQKV_ATTENTION_NAME = "nestquant_batched_nqkv_k1"


class StaticPageManager:
    """What the reference's runner expects behind ``cache.manager`` (runtime/nqkv_batch_manager.py).

    The reference reserves the target page of every slot that is about to fill its hot tail on the
    host, commits the reservation after the forward and cancels it when the forward failed
    (runtime/nqkv_batched_runner.py:344-359).  Here the page a slot publishes next is a pure function
    of the device-side page table (``slot * max_pages + page_counts[slot]``, computed inside the same
    launch sequence as the pack), so there is nothing to reserve, commit or cancel: the three calls
    are kept for the runner and do nothing.
    """

    def __init__(self, owner: "BatchedNQKVLlamaCache") -> None:
        self._owner = owner

    @property
    def layer_caches(self) -> list[NQKVHotColdCache]:
        return self._owner.layer_caches

    @property
    def request_ids(self) -> tuple[Hashable, ...]:
        return tuple(self._owner._sequence_of_slot.values())

    @property
    def active_requests(self) -> int:
        return len(self._owner._sequence_of_slot)

    def sequence_id(self, slot: int) -> Hashable:
        return self._owner._sequence_of_slot[slot]  # KeyError for a free slot, as the runner expects

    def register(self, sequence_id: Hashable, *, slot: int) -> None:
        self._owner.register(sequence_id, slot=slot)

    def register_batch(self, assignments: Sequence[tuple[Hashable, int]]) -> None:
        self._owner.register_batch(assignments)

    def release_slots(self, slots: Sequence[int]) -> tuple[Hashable, ...]:
        return self._owner.release_slots(slots)

    def reserve_graph_transition_pages(self, slots: Sequence[int]) -> tuple[int, ...]:
        return ()

    def commit_graph_transition_pages(self, slots: Sequence[int]) -> None:
        return None

    def cancel_graph_transition_pages(self, slots: Sequence[int]) -> None:
        return None


class BatchedNQKVLlamaCache(Cache):
    """Multi-layer fixed-capacity NQKV cache driven by scheduler slot state."""

    def __init__(self, *, capacity: int, num_layers: int, num_query_heads: int, num_kv_heads: int, head_dim: int,
                 max_cache_len: int, page_size: int = 16, q: int = 14, key_betas: Sequence[float],
                 value_betas: Sequence[float], dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str = "cuda", page_allocation: str = "static",
                 pool_pages: int | None = None) -> None:
        super().__init__(layers=[])
        for name, value in (("capacity", capacity), ("num_layers", num_layers), ("num_query_heads", num_query_heads),
                            ("num_kv_heads", num_kv_heads), ("head_dim", head_dim), ("max_cache_len", max_cache_len),
                            ("page_size", page_size)):
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be a positive integer")
        if num_query_heads % num_kv_heads:
            raise ValueError("num_query_heads must be divisible by num_kv_heads")
        target = torch.device(device)
        if target.type == "cuda" and target.index is None:
            target = torch.device("cuda", torch.cuda.current_device())
        max_pages = math.ceil(max_cache_len / page_size)
        # "static": page ids are slot * max_pages + page (the pool is a fixed partition, as the reference sizes it);
        # "device": the pool is a device-side free stack of `pool_pages` pages shared by all slots, popped by the
        # page writers and pushed back on release; the host only keeps an admission budget (see `register`).
        if page_allocation not in {"static", "device"}:
            raise ValueError("page_allocation must be static or device")
        if pool_pages is None:
            pool_pages = capacity * max_pages
        if isinstance(pool_pages, bool) or not isinstance(pool_pages, int) or pool_pages < 1:
            raise ValueError("pool_pages must be a positive integer")
        if page_allocation == "static" and pool_pages != capacity * max_pages:
            raise ValueError("static page ids need a pool of capacity * ceil(max_cache_len / page_size) pages")
        self.page_allocation, self.pool_pages = page_allocation, pool_pages
        self._page_budget: dict[int, int] = {}   # slot -> pages its request may need at most (device allocation)
        self.layer_caches: list[NQKVHotColdCache] = []
        for _ in range(num_layers):
            pool = NQKVPagePool(capacity=pool_pages, page_size=page_size, num_kv_heads=num_kv_heads,
                                head_dim=head_dim, q=q, key_betas=key_betas, value_betas=value_betas,
                                output_dtype=dtype, device=target)
            layer = NQKVHotColdCache(pool, max_sequences=capacity, max_pages_per_sequence=max_pages)
            pool.page_accounting = (lambda c=layer: c.page_counts.sum().item())  # ids are assigned on the device
            if page_allocation == "device":
                pool.enable_device_allocator()
            self.layer_caches.append(layer)
        self.capacity, self.num_layers = capacity, num_layers
        self.num_query_heads, self.num_kv_heads, self.head_dim = num_query_heads, num_kv_heads, head_dim
        self._max_cache_len, self.page_size, self.max_pages = max_cache_len, page_size, max_pages
        self.dtype, self.device = dtype, target
        self.slot_ids = torch.arange(capacity, device=target, dtype=torch.int32)
        self.active_mask = torch.zeros(capacity, device=target, dtype=torch.bool)
        self.execution_slot_ids = self.slot_ids
        self.execution_active_mask = self.active_mask
        self._all_slots = torch.ones(capacity, device=target, dtype=torch.bool)
        self._page_base = torch.arange(capacity, device=target, dtype=torch.int32) * max_pages
        self._decode_workspace = BatchedNQKVAttentionWorkspace.create(
            self.layer_caches[0], batch_size=capacity, query_heads=num_query_heads, output_dtype=dtype)
        # optional fused_linear.WeightDecodeAhead of the model this cache serves (the runner installs it)
        self.decode_ahead = None
        self._prefill: tuple[torch.Tensor, torch.Tensor] | None = None  # (slot_ids, query_lengths)
        self._prefill_from_empty = False
        self._bulk_host: tuple[list[int], list[int]] | None = None   # (slots, lengths) of a prefill from empty slots
        self._bulk_plan = None
        self._prefill_workspace: BatchedNQKVAttentionWorkspace | None = None
        self._sequence_of_slot: dict[int, Hashable] = {}
        # state of the reference's runner protocol
        self.manager = StaticPageManager(self)
        self.boundary_mask = torch.zeros(capacity, device=target, dtype=torch.bool)
        self._write_mask: torch.Tensor | None = None
        self._k1_mask: torch.Tensor | None = None          # active rows of an eager one-token forward
        self._graph_decode_enabled = False
        self._graph_boundary_pack_enabled = False
        self._fresh_slots: set[int] = set()                # registered, nothing written yet
        self._transaction_slots: tuple[int, ...] = ()      # slots the running prefill writes to
        # switches the reference's runner sets; every ragged layout goes through the same writer here
        self.ragged_subpage_enabled = True
        self.ragged_full_page_pack_enabled = True
        self.ragged_cross_page_enabled = True
        self.ragged_multi_page_enabled = True
        self.multi_page_batched_pack_enabled = True

    # ------------------------------------------------------------------ host control plane

    def enable_lattice_shadow(self) -> int:
        """Keep the decoded lattice coordinates of every layer's pages beside their codes (opt-in).

        Trades HBM (8 bits per cached entry beside the page's 4.25) for attention time: the paged
        attention then reads the coordinates instead of searching E8 for every block, with
        bit-identical outputs.  Call it outside a graph capture and re-capture afterwards.  Returns
        the bytes added.
        """
        return sum(cache.pool.enable_lattice_shadow() for cache in self.layer_caches)

    def _admit(self, slots: Sequence[int], max_tokens: int | None) -> None:
        """Admission budget of the device-side allocator: the pages every admitted request may need at its longest
        must fit the pool, so that a pop on the device always finds a page."""
        if self.page_allocation != "device":
            return
        tokens = self._max_cache_len if max_tokens is None else int(max_tokens)
        if not 1 <= tokens <= self._max_cache_len:
            raise ValueError("max_tokens must be in [1, max_cache_len]")
        pages = math.ceil(tokens / self.page_size)
        if sum(self._page_budget.values()) + pages * len(slots) > self.pool_pages:
            raise RuntimeError("NQKV page pool exhausted")
        for slot in slots:
            self._page_budget[int(slot)] = pages

    def register(self, sequence_id: Hashable, *, slot: int, max_tokens: int | None = None) -> None:
        if slot in self._sequence_of_slot:
            raise RuntimeError(f"slot {slot} is already registered")
        self._admit([slot], max_tokens)
        for cache in self.layer_caches:
            cache.register(slot, sequence_id)
        self.active_mask[slot] = True
        self._sequence_of_slot[slot] = sequence_id
        self._fresh_slots.add(int(slot))

    def register_batch(self, assignments: Sequence[tuple[Hashable, int]], *, max_tokens: int | None = None) -> None:
        """Register several sequences at once (one index upload instead of scalar writes per slot and layer)."""
        slots = [int(slot) for _, slot in assignments]
        if len(set(slots)) != len(slots) or any(slot in self._sequence_of_slot for slot in slots):
            raise RuntimeError("a slot of the batch is already registered")
        if any(not 0 <= slot < self.capacity for slot in slots):
            raise ValueError("slot outside cache capacity")
        if not slots:
            return
        self._admit(slots, max_tokens)
        index = torch.tensor(slots, dtype=torch.long, device=self.device)
        for cache in self.layer_caches:
            cache.register_many(index)
        self.active_mask.index_fill_(0, index, True)
        for sequence_id, slot in assignments:
            self._sequence_of_slot[slot] = sequence_id
            self._fresh_slots.add(int(slot))
            for cache in self.layer_caches:
                cache._slot_of_sequence[sequence_id] = slot

    def release_slots(self, slots: Sequence[int]) -> tuple[Hashable, ...]:
        released, freed = [], []
        for slot in slots:
            if slot not in self._sequence_of_slot:
                continue
            released.append(self._sequence_of_slot.pop(slot))
            for cache in self.layer_caches:
                cache._slot_of_sequence.pop(released[-1], None)
            freed.append(int(slot))
            self._fresh_slots.discard(int(slot))
        if freed:
            index = torch.tensor(freed, dtype=torch.long, device=self.device)
            if self.page_allocation == "device":
                mask = torch.zeros(self.capacity, dtype=torch.bool, device=self.device).index_fill_(0, index, True)
                for slot in freed:
                    self._page_budget.pop(slot, None)
            for cache in self.layer_caches:
                cache.active.index_fill_(0, index, False)
                if self.page_allocation == "device":
                    cache.device_release_slots(mask)  # pages back to the stack, tables and lengths cleared
                    continue
                cache.sequence_lengths.index_fill_(0, index, 0)
                cache.hot_lengths.index_fill_(0, index, 0)
                cache.page_counts.index_fill_(0, index, 0)
            self.active_mask.index_fill_(0, index, False)
        return tuple(released)

    def set_decode_state(self, *, slot_ids: torch.Tensor | None = None, active_mask: torch.Tensor | None = None) -> None:
        """Rows of the next one-token forwards: row i serves slot ``slot_ids[i]`` when ``active_mask[i]``."""
        self.execution_slot_ids = self.slot_ids if slot_ids is None else slot_ids
        self.execution_active_mask = self.active_mask if active_mask is None else active_mask
        self._prefill = None
        self._k1_mask = None
        self._write_mask = None
        self._graph_decode_enabled = False
        self._fresh_slots.clear()  # rows of a decode step are written to on the device; none counts as empty any more

    def set_prefill_state(self, *, slot_ids: torch.Tensor, query_lengths: torch.Tensor, from_empty: bool = False,
                          host_slots: Sequence[int] | None = None, host_lengths: Sequence[int] | None = None) -> None:
        """Rows of the next multi-token forward: row i appends ``query_lengths[i]`` tokens to ``slot_ids[i]``.

        ``from_empty`` states that every one of these slots holds no tokens yet (a whole-prompt
        prefill).  Attention then runs over the chunk's own BF16 keys and values, as the reference's
        ``prefill`` does (runtime/nqkv_batched_hf_backend.py:569-589); otherwise (a chunk that
        continues a cached sequence) over the quantised pages plus the hot tail.  When the caller
        also passes the slots and lengths as host integers, the page writer encodes all full pages
        of the chunk in one launch per tensor instead of walking the chunk page by page (same pages,
        same metadata).
        """
        if slot_ids.dtype != torch.int32 or query_lengths.dtype != torch.int32 or slot_ids.shape != query_lengths.shape:
            raise ValueError("slot_ids and query_lengths must be int32 tensors of the same shape")
        self._prefill = (slot_ids, query_lengths)
        self._prefill_from_empty = bool(from_empty)
        self._bulk_plan = None
        self._bulk_host = None
        self._k1_mask = None
        self._graph_decode_enabled = False
        if from_empty and host_slots is not None and host_lengths is not None:
            if len(host_slots) != slot_ids.numel() or len(host_lengths) != slot_ids.numel():
                raise ValueError("host_slots / host_lengths must match slot_ids")
            self._bulk_host = ([int(v) for v in host_slots], [int(v) for v in host_lengths])
            self._fresh_slots.difference_update(self._bulk_host[0])

    # ------------------------------------------------------------------ the reference's runner protocol
    @property
    def max_cache_len(self) -> int:
        return self._max_cache_len

    @property
    def graph_decode_enabled(self) -> bool:
        return self._graph_decode_enabled

    def _enter_rows(self, slot_ids: torch.Tensor, write_mask: torch.Tensor) -> None:
        """Common part of the two prefill-capable states: row ``i`` writes ``write_mask[i].sum()`` tokens to ``slot_ids[i]``."""
        host_mask = write_mask.detach().cpu()
        counts = host_mask.sum(dim=1).tolist()
        width = write_mask.shape[1]
        for row, count in enumerate(counts):  # the writers take prefix masks (right-padded prompts)
            if count and not bool(host_mask[row, :count].all()):
                raise ValueError("write_mask rows must be prefixes (valid tokens first, padding after)")
        slots = slot_ids.tolist()
        written = [(slot, count) for slot, count in zip(slots, counts) if count]
        self._write_mask = write_mask
        self._transaction_slots = tuple(slot for slot, _ in written)
        self._graph_decode_enabled = False
        self._bulk_plan = None
        self._bulk_host = None
        if width == 1:
            # one token per row: the decode writer and the paged decode kernel, as the reference does for T = 1
            self._prefill = None
            self._k1_mask = write_mask[:, 0].contiguous()
        else:
            self._k1_mask = None
            self._prefill = (slot_ids, write_mask.sum(dim=1).to(torch.int32))
            self._prefill_from_empty = True  # the reference's prefill semantic: SDPA over the chunk's own K/V
            if written and all(slot in self._fresh_slots for slot, _ in written):
                self._bulk_host = (slots, [int(c) for c in counts])  # rows with 0 tokens are skipped by the plan
        self._fresh_slots.difference_update(slot for slot, _ in written)

    def set_batch_state(self, *, active_mask: torch.Tensor, write_mask: torch.Tensor) -> None:
        """Rows of the next forward are the ``capacity`` logical slots (runtime/nqkv_batched_hf_backend.py:147-280)."""
        if active_mask.dtype != torch.bool or tuple(active_mask.shape) != (self.capacity,):
            raise ValueError("active_mask must be bool with shape [capacity]")
        if write_mask.dtype != torch.bool or write_mask.ndim != 2:
            raise ValueError("write_mask must be bool with shape [capacity, tokens]")
        if write_mask.shape[0] != self.capacity:
            raise ValueError("write_mask batch must equal cache capacity")
        if active_mask.device != self.device or write_mask.device != self.device:
            raise ValueError("batch state tensors must be on the cache device")
        if bool((write_mask.any(dim=1) & ~active_mask).any().item()):
            raise ValueError("inactive rows cannot request KV writes")
        self.active_mask.copy_(active_mask)
        self.execution_slot_ids = self.slot_ids
        self.execution_active_mask = self.active_mask
        self._enter_rows(self.slot_ids, write_mask)

    def set_decode_execution_state(self, *, slot_ids: torch.Tensor, active_mask: torch.Tensor) -> None:
        """Map compact one-token rows to logical slots (runtime/nqkv_batched_hf_backend.py:282-317)."""
        if slot_ids.dtype != torch.int32 or slot_ids.ndim != 1:
            raise ValueError("execution slot_ids must be rank-1 torch.int32")
        if active_mask.dtype != torch.bool or active_mask.shape != slot_ids.shape:
            raise ValueError("execution active_mask must be bool and match slot_ids")
        if slot_ids.device != self.device or active_mask.device != self.device:
            raise ValueError("execution state tensors must be on the cache device")
        if not 1 <= slot_ids.numel() <= self.capacity:
            raise ValueError("execution row count must be within cache capacity")
        if bool(((slot_ids < 0) | (slot_ids >= self.capacity)).any().item()):
            raise ValueError("execution slot_ids are outside logical capacity")
        selected = slot_ids[active_mask]
        if selected.numel() != torch.unique(selected).numel():
            raise ValueError("active execution rows must map to unique logical slots")
        self.execution_slot_ids = slot_ids
        self.execution_active_mask = active_mask
        self._write_mask = active_mask[:, None]
        self._prefill = None
        self._k1_mask = None
        self._bulk_host = None
        self._transaction_slots = ()

    def set_prefill_execution_state(self, *, slot_ids: torch.Tensor, write_mask: torch.Tensor) -> None:
        """Compact prefill rows: row ``i`` writes to logical slot ``slot_ids[i]`` (:319-333)."""
        if write_mask.dtype != torch.bool or write_mask.ndim != 2:
            raise ValueError("execution write_mask must be rank-2 bool")
        self.set_decode_execution_state(slot_ids=slot_ids, active_mask=write_mask.any(dim=1))
        self._enter_rows(slot_ids, write_mask)

    def enable_graph_decode(self, *, boundary_pack: bool = False) -> None:
        """One-token updates go through the host-free writer; full hot pages are packed only when
        ``boundary_pack`` is set, for the rows of ``boundary_mask`` (:335-349)."""
        self._graph_decode_enabled = True
        self._graph_boundary_pack_enabled = bool(boundary_pack)
        self._write_mask = self.execution_active_mask[:, None]
        self._prefill = None
        self._k1_mask = None
        self._bulk_host = None
        self._transaction_slots = ()
        self._fresh_slots.clear()

    def disable_graph_decode(self) -> None:
        self._graph_decode_enabled = False
        self._graph_boundary_pack_enabled = False

    def finish_prefill_page_transaction(self, *, success: bool) -> None:
        """End of one eager prefill forward (:493-531).  Pages have static ids, so there is nothing to
        commit; after a failed forward the slots it wrote to are released, as the reference does,
        so that no half-written sequence stays registered."""
        slots = self._transaction_slots
        self._transaction_slots = ()
        self._bulk_host = None
        self._bulk_plan = None
        self.boundary_mask.zero_()
        if not success and slots:
            self.release_slots(slots)

    # ------------------------------------------------------------------ Cache interface
    def _pack_full_pages(self, cache: NQKVHotColdCache, mask: torch.Tensor | None = None) -> None:
        mask = self._all_slots if mask is None else mask
        if self.page_allocation == "device":
            cache.device_alloc_targets(mask)   # pops a page for every slot that is about to pack
        # static ids (slot * max_pages + page_counts) are formed inside the pack kernels: no id tensor to refresh
        launch_pack_full_hot_pages_graph_safe(cache, boundary_mask=mask,
                                              static_page_ids=self.page_allocation != "device")

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int, cache_kwargs=None):
        self._validate_layer(layer_idx)
        cache = self.layer_caches[layer_idx]
        rows, heads, tokens, dim = key_states.shape
        if heads != self.num_kv_heads or dim != self.head_dim:
            raise ValueError("key/value states do not match the cache geometry")
        # keys that come out of the fused rope launch are rotated already
        rotated_key = (key_states if rotation_done(key_states) and key_states.dtype == self.dtype
                       else hadamard(key_states.float()).to(self.dtype))
        if tokens == 1 and self._prefill is None:
            if rows != self.execution_slot_ids.numel():
                raise ValueError("decode rows do not match the execution slot ids")
            mask = self.execution_active_mask if self._k1_mask is None else self._k1_mask
            _launch_append_hot_k1_graph_safe(rotated_key[:, :, 0], value_states[:, :, 0].to(self.dtype), cache,
                                             slot_ids=self.execution_slot_ids, active_mask=mask)
            if not self._graph_decode_enabled:
                self._pack_full_pages(cache)
            elif self._graph_boundary_pack_enabled:  # the reference's boundary graph: only the rows the runner marked
                self._pack_full_pages(cache, self.boundary_mask)
            return rotated_key, value_states
        if self._prefill is None:
            raise RuntimeError("multi-token update needs set_prefill_state(slot_ids, query_lengths)")
        slot_ids, query_lengths = self._prefill
        if rows != slot_ids.numel():
            raise ValueError("prefill rows do not match the prefill slot ids")
        key_nhd = rotated_key.permute(0, 2, 1, 3).contiguous()
        value_nhd = value_states.to(self.dtype).permute(0, 2, 1, 3).contiguous()
        if self._bulk_host is not None:
            self._write_chunk_from_empty(cache, key_nhd, value_nhd)
            return rotated_key, value_states
        consumed = torch.zeros_like(query_lengths)
        index = slot_ids.long()
        for _ in range(math.ceil(tokens / self.page_size) + 1):
            room = self.page_size - cache.hot_lengths[index]
            counts = torch.clamp(torch.minimum(room, query_lengths - consumed), min=0).to(torch.int32)
            _launch_append_hot_ragged_segment_graph_safe(key_nhd, value_nhd, cache, slot_ids=slot_ids,
                                                         source_starts=consumed, segment_counts=counts)
            self._pack_full_pages(cache)
            consumed = consumed + counts
        return rotated_key, value_states

    def _plan_chunk_from_empty(self, tokens: int):
        """Index tensors of a whole-prompt chunk ``[rows, tokens]``: which tokens fill whole pages, which stay hot."""
        slots, lengths = self._bulk_host
        page, device = self.page_size, self.device
        full_idx, page_ids, tail_src, tail_slot, tail_pos, table_rows, table_cols = [], [], [], [], [], [], []
        rows = [(row, slot, length) for row, (slot, length) in enumerate(zip(slots, lengths)) if length > 0]
        slots, lengths = [slot for _, slot, _ in rows], [length for _, _, length in rows]
        table = torch.full((len(rows), self.max_pages), -1, dtype=torch.int32)
        for index, (row, slot, length) in enumerate(rows):
            if length > tokens or length // page > self.max_pages:
                raise ValueError("prefill length exceeds the chunk or the cache length")
            full, rest = length // page, length % page
            full_idx.append(torch.arange(full * page) + row * tokens)
            ids = torch.arange(full) + slot * self.max_pages
            page_ids.append(ids)
            table[index, :full] = ids.to(torch.int32)
            table_rows.append(torch.full((full,), index))
            table_cols.append(torch.arange(full))
            tail_src.append(torch.arange(rest) + row * tokens + full * page)
            tail_slot.append(torch.full((rest,), slot))
            tail_pos.append(torch.arange(rest))
        cat = lambda parts: torch.cat(parts).to(device) if parts else torch.zeros(0, dtype=torch.long, device=device)  # noqa: E731
        lengths_t = torch.tensor(lengths, dtype=torch.int32)
        return {"tokens": tokens, "full_idx": cat(full_idx), "page_ids": cat(page_ids), "tail_src": cat(tail_src),
                "tail_slot": cat(tail_slot), "tail_pos": cat(tail_pos), "table": table.to(device),
                "table_rows": cat(table_rows), "table_cols": cat(table_cols),
                "slots": torch.tensor(slots, dtype=torch.long, device=device),
                "full": (lengths_t // page).to(device), "rest": (lengths_t % page).to(device),
                "lengths": lengths_t.to(device)}

    def _write_chunk_from_empty(self, cache: NQKVHotColdCache, key_nhd: torch.Tensor, value_nhd: torch.Tensor) -> None:
        """All full pages of the chunk through one encoder launch per tensor, the remainder into the hot tail.

        Leaves pool and metadata exactly as the page-by-page writer does (static page ids
        ``slot * max_pages + page``).
        """
        rows, tokens = key_nhd.shape[0], key_nhd.shape[1]
        plan = self._bulk_plan
        if plan is None or plan["tokens"] != tokens:
            plan = self._bulk_plan = self._plan_chunk_from_empty(tokens)
        pool, dim = cache.pool, self.head_dim
        page_ids, page_table = plan["page_ids"], plan["table"]
        if self.page_allocation == "device" and page_ids.numel():
            # the pages come off this layer's device-side stack instead of the static partition
            popped = pool.device_alloc_pages(page_ids.numel())
            page_ids = popped.long()
            page_table = torch.full_like(plan["table"], -1)
            page_table[plan["table_rows"], plan["table_cols"]] = popped
        for flat, codes, betas, norms, table, values, hot in (
                (key_nhd.view(rows * tokens, -1), pool.key_codes, pool.key_betas, pool.key_norms, pool.beta_table,
                 pool.betas, cache.hot_keys),
                (value_nhd.view(rows * tokens, -1), pool.value_codes, pool.value_betas, pool.value_norms,
                 pool.value_beta_table, pool.value_beta_values, cache.hot_values)):
            pages = page_ids.numel()
            if pages:
                packed = quantize_activation_cuda(flat[plan["full_idx"]].view(-1, dim), q=14, betas=values,
                                                  beta_table=table, keep_decoded=False)
                codes[page_ids] = packed.code_payload.view(pages, -1)
                betas[page_ids] = packed.beta_payload.view(pages, -1)
                norms[page_ids] = packed.row_norms.view(pages, -1)
            if plan["tail_src"].numel():
                hot[plan["tail_slot"], plan["tail_pos"]] = flat[plan["tail_src"]].view(-1, self.num_kv_heads, dim)
        pool.expand_pages(page_ids)  # keeps the opt-in decoded shadow current (no-op without one)
        slots = plan["slots"]
        cache.page_indices[slots] = page_table
        cache.page_counts[slots] = plan["full"]
        cache.last_page_len[slots] = torch.where(plan["full"] > 0, self.page_size, 0).to(torch.int32)
        cache.hot_lengths[slots] = plan["rest"]
        cache.sequence_lengths[slots] = plan["lengths"]

    def attend(self, layer_idx: int, query_states: torch.Tensor, *, scale: float) -> torch.Tensor:
        """Decode: ``query_states [rows, Hq, 1, D]`` -> ``[rows, 1, Hq, D]``."""
        self._validate_layer(layer_idx)
        expected = (self.execution_slot_ids.numel(), self.num_query_heads, 1, self.head_dim)
        if tuple(query_states.shape) != expected:
            raise ValueError("batched NQKV decode requires [rows, heads, 1, dim]")
        query = (query_states if rotation_done(query_states) and query_states.dtype == self.dtype
                 else hadamard(query_states.float()).to(self.dtype))[:, :, 0].contiguous()
        if self.decode_ahead is not None:
            # the weights the layer needs after its attention are decoded on a second stream meanwhile
            self.decode_ahead.launch(layer_idx, query.shape[0], at_attention=True)
        workspace = self._decode_workspace
        if query.shape[0] != workspace.batch_size:
            workspace = BatchedNQKVAttentionWorkspace.create(self.layer_caches[layer_idx], batch_size=query.shape[0],
                                                             query_heads=self.num_query_heads, output_dtype=self.dtype)
        output = _launch_nqkv_decode_attention_batched_k1(
            query, self.layer_caches[layer_idx], slot_ids=self.execution_slot_ids,
            active_mask=self.execution_active_mask, attention_scale=scale, workspace=workspace)
        return output.unsqueeze(1)

    def prefill(self, *args, scale: float, key_states: torch.Tensor | None = None,
                value_states: torch.Tensor | None = None) -> torch.Tensor:
        """Causal attention of a whole chunk: ``[rows, Hq, T, D]`` -> ``[rows, T, Hq, D]``.

        Called as ``prefill(layer_idx, query_states, scale=..., key_states=..., value_states=...)`` by this
        package's attention interface, or in the reference's form ``prefill(query, key, value,
        attention_mask, scale=...)`` (runtime/nqkv_batched_hf_backend.py:569-589), which has no layer index
        and always means the chunk's own K/V.

        A prefill from empty slots uses the chunk's BF16 keys (already rotated by ``update``) and values,
        right-padded rows included (causality keeps valid queries away from the padding); any other
        chunk reads the pages just written and the hot tail.
        """
        if args and isinstance(args[0], torch.Tensor):  # the reference's call form
            if len(args) != 4:
                raise TypeError("prefill(query, key, value, attention_mask, *, scale) takes four tensors")
            query_states, key_states, value_states, attention_mask = args
            rotated_query = (query_states if rotation_done(query_states) and query_states.dtype == self.dtype
                             else hadamard(query_states.float()).to(self.dtype))
            out = _dense_attention(rotated_query, key_states.to(self.dtype), value_states.to(self.dtype),
                                   attention_mask, scale, self.num_query_heads != self.num_kv_heads)
            return out.transpose(1, 2)
        if len(args) != 2:
            raise TypeError("prefill(layer_idx, query_states, *, scale, key_states, value_states)")
        layer_idx, query_states = args
        self._validate_layer(layer_idx)
        if self._prefill is None:
            raise RuntimeError("prefill attention needs set_prefill_state(slot_ids, query_lengths)")
        slot_ids, query_lengths = self._prefill
        if self._prefill_from_empty and key_states is not None and value_states is not None:
            rotated_query = (query_states if rotation_done(query_states) and query_states.dtype == self.dtype
                             else hadamard(query_states.float()).to(self.dtype))
            out = _dense_attention(rotated_query, key_states.to(self.dtype), value_states.to(self.dtype), None, scale,
                                   self.num_query_heads != self.num_kv_heads)
            return out.transpose(1, 2)
        query = (query_states if rotation_done(query_states) and query_states.dtype == self.dtype
                 else hadamard(query_states.float()).to(self.dtype)).permute(0, 2, 1, 3).contiguous()
        rows, tokens = query.shape[0], query.shape[1]
        ws = self._prefill_workspace
        if ws is None or (ws.batch_size, ws.query_tokens) != (rows, tokens):
            ws = self._prefill_workspace = BatchedNQKVAttentionWorkspace.create(
                self.layer_caches[layer_idx], batch_size=rows, query_heads=self.num_query_heads,
                output_dtype=self.dtype, query_tokens=tokens)
        out = nqkv_prefill_attention(query, self.layer_caches[layer_idx], slot_ids=slot_ids,
                                     query_lengths=query_lengths, scale=scale, workspace=ws)
        return out.view(rows, tokens, self.num_query_heads, self.head_dim)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        self._validate_layer(layer_idx)
        lengths = self.layer_caches[layer_idx].sequence_lengths
        return int(lengths.max().item()) if self._sequence_of_slot else 0

    def get_max_length(self, layer_idx: int | None = None) -> int:
        return self._max_cache_len

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return self._max_cache_len

    def get_mask_sizes(self, query_length, layer_idx: int = 0) -> tuple[int, int]:
        return self._max_cache_len, 0

    @property
    def batch_size(self) -> int:
        return self.capacity

    @property
    def is_compileable(self) -> bool:
        return False

    def reorder_cache(self, beam_idx) -> None:
        raise NotImplementedError("batched NQKV backend does not support beam search")

    def _validate_layer(self, layer_idx: int) -> None:
        if isinstance(layer_idx, bool) or not isinstance(layer_idx, int):
            raise TypeError("layer_idx must be an integer")
        if not 0 <= layer_idx < self.num_layers:
            raise ValueError("layer_idx is outside the batched NQKV layer range")


def _dense_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, attention_mask, scale: float,
                     grouped: bool) -> torch.Tensor:
    """Attention of a fresh prompt over its own unquantised K/V (the reference's prefill semantic,
    runtime/nqkv_hf_backend.py:127-150): the library's scaled-dot-product attention.

    The flash backend is asked for first: torch's default choice on this GPU builds an execution plan for every
    new (batch, length) it meets, which on ragged prompts costs more than the attention itself (64 prompts of
    128..2048 tokens in eight groups: 3.1 s, against 0.6 s once every plan exists; flash: 0.6 s from the first call).
    """
    from torch.nn.attention import SDPBackend, sdpa_kernel

    order = [SDPBackend.FLASH_ATTENTION, SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]
    with sdpa_kernel(order, set_priority=True):
        return torch.nn.functional.scaled_dot_product_attention(
            query, key, value, attn_mask=attention_mask, dropout_p=0.0, is_causal=attention_mask is None, scale=scale,
            enable_gqa=grouped)


def _batched_nqkv_attention_interface(module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                      attention_mask: torch.Tensor | None, **kwargs):
    cache = getattr(module, "_nestquant_batched_nqkv_cache", None)
    if not isinstance(cache, BatchedNQKVLlamaCache):
        raise RuntimeError("Llama attention module has no batched NQKV cache")
    if kwargs.get("dropout", 0.0) != 0.0:
        raise ValueError("batched NQKV backend supports inference dropout=0 only")
    scale = float(kwargs.get("scaling", module.scaling))
    if query.shape[2] == 1 and cache._prefill is None:
        return cache.attend(module.layer_idx, query, scale=scale), None
    return cache.prefill(module.layer_idx, query, scale=scale, key_states=key, value_states=value), None


def install_batched_nqkv_llama_backend(model: torch.nn.Module, cache: BatchedNQKVLlamaCache) -> str:
    """Attach fixed-capacity batched NQKV attention to every Llama layer."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    if not isinstance(model, torch.nn.Module):
        raise TypeError("model must be a torch module")
    if not isinstance(cache, BatchedNQKVLlamaCache):
        raise TypeError("cache must be a BatchedNQKVLlamaCache")
    ALL_ATTENTION_FUNCTIONS.register(BATCHED_NQKV_ATTENTION_NAME, _batched_nqkv_attention_interface)
    attached = 0
    for module in model.modules():
        if module.__class__.__name__ == "LlamaAttention":
            if not 0 <= module.layer_idx < cache.num_layers:
                raise ValueError("Llama layer index disagrees with batched NQKV cache")
            module._nestquant_batched_nqkv_cache = cache
            module.config._attn_implementation = BATCHED_NQKV_ATTENTION_NAME
            attached += 1
    if attached != cache.num_layers:
        raise ValueError(f"expected {cache.num_layers} LlamaAttention modules, found {attached}")
    if hasattr(model, "config"):
        model.config._attn_implementation = BATCHED_NQKV_ATTENTION_NAME
    return BATCHED_NQKV_ATTENTION_NAME
