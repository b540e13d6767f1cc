"""NQKV4 paged KV cache: device data model and the operators that read and write it.

Host mirror of the reference's KV runtime, same names and argument meaning:
``NQKVPagePool`` (runtime/nqkv_pool.py:22-267), page-table metadata of
``PagedNQKVCache`` (runtime/paged_nqkv_cache.py:26-137), ``NQKVHotColdCache``
(runtime/nqkv_hot_cache.py:14-37), ``quantize_nqkv_page_cuda`` /
``PreparedNQKVPage`` (runtime/nqkv_page.py:192-329), the graph-safe writers
(runtime/nqkv_graph_writer.py:291-473, runtime/nqkv_graph_pack.py:76-135) and
``nqkv_decode_attention_batched_k1`` (runtime/nqkv_attention_k1.py:763-942).

The tensors keep the reference's SoA layout, fixed addresses and dtypes, so the
reference's control plane (page allocation, reservations, scheduling) can drive
them unchanged; only the kernels are new.  The small host-side allocator below
exists so the operators can be used and tested stand-alone.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Sequence

import torch

from .. import _lib
from .w4a4 import _DTYPE_TAG, _ptr, _stream

_INT = ctypes.c_int
_I64 = ctypes.c_int64


def _betas(values: Sequence[float]) -> tuple[float, ...]:
    out = tuple(float(v) for v in values)
    if len(out) != 4 or any(not math.isfinite(v) or v <= 0 for v in out):
        raise ValueError("the NQKV4 kernels need four positive finite betas")
    return out


# --------------------------------------------------------------------------- data model
class NQKVPagePool:
    """Preallocated SoA page storage; tensors never move (graph-stable addresses)."""

    def __init__(self, *, capacity: int, page_size: int, num_kv_heads: int, head_dim: int, q: int = 14,
                 betas: Sequence[float] | None = None, key_betas: Sequence[float] | None = None,
                 value_betas: Sequence[float] | None = None, output_dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str = "cuda") -> None:
        for name, value in (("capacity", capacity), ("page_size", page_size),
                            ("num_kv_heads", num_kv_heads), ("head_dim", head_dim)):
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be a positive integer")
        if head_dim % 32:
            raise ValueError("head_dim must be divisible by 32 for the sm_100a kernels")
        if q != 14:
            raise ValueError("the sm_100a kernels implement q=14")
        if betas is not None:
            if key_betas is not None or value_betas is not None:
                raise ValueError("pass legacy betas or key_betas/value_betas, not both")
            key_betas = value_betas = betas
            self.format_version = 1
        else:
            if key_betas is None or value_betas is None:
                raise ValueError("v2 requires both key_betas and value_betas")
            self.format_version = 2
        target = torch.device(device)
        if target.type != "cuda" or not torch.cuda.is_available():
            raise ValueError("NQKVPagePool requires an available CUDA device")
        if target.index is None:
            target = torch.device("cuda", torch.cuda.current_device())
        self.capacity, self.page_size, self.num_kv_heads, self.head_dim, self.q = capacity, page_size, num_kv_heads, head_dim, q
        self.betas, self.value_beta_values = _betas(key_betas), _betas(value_betas)
        self.output_dtype, self.device = output_dtype, target
        self.code_width, self.beta_width = 4, 2
        rows = page_size * num_kv_heads
        self._row_count = rows
        self._code_bytes, self._beta_bytes = rows * head_dim // 2, rows * head_dim // 32
        self.key_codes = torch.zeros((capacity, self._code_bytes), device=target, dtype=torch.uint8)
        self.key_betas = torch.zeros((capacity, self._beta_bytes), device=target, dtype=torch.uint8)
        self.key_norms = torch.zeros((capacity, rows), device=target, dtype=torch.float32)
        self.value_codes = torch.zeros_like(self.key_codes)
        self.value_betas = torch.zeros_like(self.key_betas)
        self.value_norms = torch.zeros_like(self.key_norms)
        self.beta_table = torch.tensor(self.betas, device=target, dtype=torch.float32)
        self.value_beta_table = torch.tensor(self.value_beta_values, device=target, dtype=torch.float32)
        self._free = list(range(capacity - 1, -1, -1))
        self.page_accounting = None  # optional callable returning the pages in use (see ``allocated_pages``)
        # device-side free stack (``enable_device_allocator``)
        self.free_ids: torch.Tensor | None = None
        self.free_count: torch.Tensor | None = None
        # opt-in decoded shadow of the code streams (``enable_lattice_shadow``): int8 [capacity, P*H*D]
        self.key_lattice: torch.Tensor | None = None
        self.value_lattice: torch.Tensor | None = None

    def enable_device_allocator(self) -> None:
        """Hand the pool's free pages to a device-side stack (``free_ids[0 .. free_count)``).

        Afterwards the page writers pop their target pages on the device (``device_alloc_targets``,
        ``device_alloc_pages``) and ``device_release_slots`` pushes them back; ``allocate`` / ``release``
        of the host list must not be used any more.
        """
        if self.free_ids is not None:
            return
        self.free_ids = torch.tensor(self._free, dtype=torch.int32, device=self.device)
        if self.free_ids.numel() < self.capacity:  # pages the host list had already handed out stay out
            self.free_ids = torch.cat([self.free_ids, torch.zeros(self.capacity - self.free_ids.numel(),
                                                                  dtype=torch.int32, device=self.device)])
        self.free_count = torch.tensor([len(self._free)], dtype=torch.int32, device=self.device)
        self._free = []

    def device_alloc_pages(self, count: int) -> torch.Tensor:
        """Pop ``count`` page ids on the device (no host sync): int32 ``[count]``."""
        if self.free_ids is None:
            raise RuntimeError("the pool has no device-side allocator")
        out = torch.empty(count, dtype=torch.int32, device=self.device)
        status = _lib.lib().nq_kv_alloc_pages(_INT(count), _ptr(self.free_ids), _ptr(self.free_count), _ptr(out),
                                              _stream(self.device))
        _lib.check(status, "device_alloc_pages")
        return out

    def enable_lattice_shadow(self) -> int:
        """Keep the decoded lattice coordinates of every page beside its codes (opt-in; returns the bytes added).

        Decoding a block is a pure function of its codeword and is what bounds the paged attention;
        with the shadow (8 bits per entry beside the page's 4.25) attention reads the coordinates
        instead of searching for them and returns bit-identical outputs.  Pages already in the pool
        are converted now; the page writers of this package keep the shadow current afterwards.
        The NQKV4 streams stay the record and are unchanged.
        """
        if self.key_lattice is not None:
            return 0
        entries = self._row_count * self.head_dim
        self.key_lattice = torch.zeros((self.capacity, entries), device=self.device, dtype=torch.int8)
        self.value_lattice = torch.zeros_like(self.key_lattice)
        self.expand_pages(torch.arange(self.capacity, dtype=torch.int32, device=self.device))
        return 2 * self.capacity * entries

    def expand_pages(self, page_ids: torch.Tensor) -> None:
        """Refresh the decoded shadow of the listed pages (no-op without a shadow)."""
        if self.key_lattice is None or page_ids.numel() == 0:
            return
        ids = page_ids.to(device=self.device, dtype=torch.int32).contiguous()
        for codes, lattice in ((self.key_codes, self.key_lattice), (self.value_codes, self.value_lattice)):
            status = _lib.lib().nq_kv_expand_pages(
                _ptr(codes), _ptr(lattice), _ptr(ids), ctypes.c_int64(ids.numel()), _INT(self.capacity),
                _INT(self.page_size), _INT(self.num_kv_heads), _INT(self.head_dim), _stream(self.device))
            _lib.check(status, "expand_pages")

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def allocated_pages(self) -> int:
        """Pages in use: handed out by ``allocate``, or -- for an owner that assigns page ids on the device --
        the pages its page tables hold (``page_accounting``; reads the device)."""
        if self.free_count is not None:
            return self.capacity - int(self.free_count.item())
        if self.page_accounting is not None:
            return int(self.page_accounting())
        return self.capacity - len(self._free)

    @property
    def page_payload_bytes(self) -> int:
        return 2 * (self._code_bytes + self._beta_bytes + 4 * self._row_count)

    def allocate(self) -> int:
        if not self._free:
            raise RuntimeError("NQKV page pool exhausted")
        return self._free.pop()

    def release(self, page_id: int) -> None:
        self._free.append(int(page_id))


class NQKVHotColdCache:
    """Per-slot BF16 hot tail over packed cold pages, plus the fixed-address page tables."""

    def __init__(self, pool: NQKVPagePool, *, max_sequences: int, max_pages_per_sequence: int) -> None:
        if not isinstance(pool, NQKVPagePool):
            raise TypeError("pool must be an NQKVPagePool")
        self.pool = pool
        self.max_sequences, self.max_pages_per_sequence = int(max_sequences), int(max_pages_per_sequence)
        dev = pool.device
        s, p = self.max_sequences, self.max_pages_per_sequence
        self.page_indices = torch.full((s, p), -1, dtype=torch.int32, device=dev)
        self.page_counts = torch.zeros(s, dtype=torch.int32, device=dev)
        self.last_page_len = torch.zeros(s, dtype=torch.int32, device=dev)
        self.hot_lengths = torch.zeros(s, dtype=torch.int32, device=dev)
        self.sequence_lengths = torch.zeros(s, dtype=torch.int32, device=dev)
        self.active = torch.zeros(s, dtype=torch.bool, device=dev)
        shape = (s, pool.page_size, pool.num_kv_heads, pool.head_dim)
        self.hot_keys = torch.zeros(shape, device=dev, dtype=pool.output_dtype)
        self.hot_values = torch.zeros_like(self.hot_keys)
        self.graph_target_page_ids = torch.zeros(s, dtype=torch.int32, device=dev)
        self._slot_of_sequence: dict = {}

    # the reference reaches these through ``cache.cold_cache``; keep both spellings
    @property
    def cold_cache(self) -> "NQKVHotColdCache":
        return self

    @property
    def last_page_lens(self) -> torch.Tensor:
        return self.last_page_len

    def total_tokens(self, sequence_id) -> int:
        """Tokens held for a sequence registered under ``sequence_id`` (reads the device)."""
        return int(self.sequence_lengths[self._slot_of_sequence[sequence_id]].item())

    def register(self, slot: int, sequence_id=None) -> int:
        if not 0 <= slot < self.max_sequences:
            raise ValueError("slot outside cache capacity")
        if sequence_id is not None:
            self._slot_of_sequence[sequence_id] = slot
        self.active[slot] = True
        self.page_counts[slot] = 0
        self.last_page_len[slot] = 0
        self.hot_lengths[slot] = 0
        self.sequence_lengths[slot] = 0
        self.page_indices[slot].fill_(-1)
        return slot

    def register_many(self, index: torch.Tensor) -> None:
        """``register`` for all slots of a device index tensor: six launches, no host-to-device scalar copies."""
        self.active.index_fill_(0, index, True)
        self.page_counts.index_fill_(0, index, 0)
        self.last_page_len.index_fill_(0, index, 0)
        self.hot_lengths.index_fill_(0, index, 0)
        self.sequence_lengths.index_fill_(0, index, 0)
        self.page_indices.index_fill_(0, index, -1)

    def device_alloc_targets(self, boundary_mask: torch.Tensor) -> None:
        """Pop one target page on the device for every slot that is about to pack (graph safe, no host reads)."""
        pool = self.pool
        if pool.free_ids is None:
            raise RuntimeError("the pool has no device-side allocator")
        status = _lib.lib().nq_kv_alloc_targets(
            _ptr(self.hot_lengths), _ptr(boundary_mask), _ptr(self.page_counts), _ptr(pool.free_ids),
            _ptr(pool.free_count), _ptr(self.graph_target_page_ids), _INT(self.max_sequences),
            _INT(self.max_pages_per_sequence), _INT(pool.page_size), _stream(pool.device))
        _lib.check(status, "device_alloc_targets")

    def device_release_slots(self, slot_mask: torch.Tensor) -> None:
        """Push the pages of the selected slots back to the device-side stack and empty those slots."""
        pool = self.pool
        if pool.free_ids is None:
            raise RuntimeError("the pool has no device-side allocator")
        if slot_mask.dtype != torch.bool or tuple(slot_mask.shape) != (self.max_sequences,):
            raise ValueError("slot_mask must be bool with cache capacity shape")
        status = _lib.lib().nq_kv_release_pages(
            _ptr(slot_mask), _ptr(self.page_indices), _ptr(self.page_counts), _ptr(self.last_page_len),
            _ptr(self.hot_lengths), _ptr(self.sequence_lengths), _ptr(pool.free_ids), _ptr(pool.free_count),
            _INT(self.max_sequences), _INT(self.max_pages_per_sequence), _INT(pool.capacity), _stream(pool.device))
        _lib.check(status, "device_release_slots")

    def reserve_targets(self, slots: Sequence[int]) -> list[int]:
        """Allocate one target page per slot for the next boundary pack (host control plane)."""
        ids = [self.pool.allocate() for _ in slots]
        if ids:
            index = torch.tensor(list(slots), dtype=torch.long, device=self.pool.device)
            self.graph_target_page_ids[index] = torch.tensor(ids, dtype=torch.int32, device=self.pool.device)
        return ids


@dataclass(frozen=True)
class PreparedNQKVPage:
    """Six payload tensors of one packed page (runtime/nqkv_page.py:192-238)."""

    key_code_payload: torch.Tensor
    key_beta_payload: torch.Tensor
    key_norms: torch.Tensor
    value_code_payload: torch.Tensor
    value_beta_payload: torch.Tensor
    value_norms: torch.Tensor
    key_beta_table: torch.Tensor
    value_beta_table: torch.Tensor
    page_size: int
    valid_tokens: int
    num_kv_heads: int
    head_dim: int
    q: int
    code_width: int
    beta_width: int
    output_dtype: torch.dtype

    @property
    def payload_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (
            self.key_code_payload, self.key_beta_payload, self.key_norms,
            self.value_code_payload, self.value_beta_payload, self.value_norms))


def quantize_nqkv_page_cuda(key: torch.Tensor, value: torch.Tensor, *, page_size: int, q: int = 14,
                            betas: Sequence[float] | None = None, key_betas: Sequence[float] | None = None,
                            value_betas: Sequence[float] | None = None,
                            key_beta_table: torch.Tensor | None = None,
                            value_beta_table: torch.Tensor | None = None) -> PreparedNQKVPage:
    """Quantise and bit-pack one NHD page prefix in one launch (bit-exact with the CPU page format)."""
    if not isinstance(key, torch.Tensor) or not isinstance(value, torch.Tensor):
        raise TypeError("key and value must be torch tensors")
    if key.shape != value.shape or key.ndim != 3:
        raise ValueError("key and value must share NHD shape [tokens, kv_heads, head_dim]")
    if key.device != value.device or key.dtype != value.dtype or key.device.type != "cuda":
        raise ValueError("key and value must share CUDA device and dtype")
    if not key.is_floating_point() or key.dtype not in _DTYPE_TAG:
        raise TypeError("key and value must be float16, bfloat16 or float32")
    if not 1 <= key.shape[0] <= page_size:
        raise ValueError("token count must be in [1, page_size]")
    if key.shape[2] % 8:
        raise ValueError("head_dim must be divisible by 8")
    if betas is not None:
        if key_betas is not None or value_betas is not None:
            raise ValueError("pass legacy betas or key_betas/value_betas, not both")
        key_betas = value_betas = betas
    elif key_betas is None or value_betas is None:
        raise ValueError("v2 requires both key_betas and value_betas")
    kb, vb = _betas(key_betas), _betas(value_betas)
    if q != 14:
        raise ValueError("the sm_100a kernels implement q=14")
    valid, heads, dim = key.shape
    dev = key.device
    if key_beta_table is None:
        key_beta_table = torch.tensor(kb, device=dev, dtype=torch.float32)
    if value_beta_table is None:
        value_beta_table = torch.tensor(vb, device=dev, dtype=torch.float32)
    rows = page_size * heads
    out = [torch.empty(rows * dim // 2, dtype=torch.uint8, device=dev),
           torch.empty(rows * dim // 32, dtype=torch.uint8, device=dev),
           torch.empty(rows, dtype=torch.float32, device=dev)]
    out += [torch.empty_like(t) for t in out]
    key, value = key.contiguous(), value.contiguous()
    status = _lib.lib().nq_kv_quantize_page(
        _ptr(key), _ptr(value), _DTYPE_TAG[key.dtype], _INT(valid), _INT(page_size), _INT(heads), _INT(dim),
        _ptr(key_beta_table), _ptr(value_beta_table), *[_ptr(t) for t in out], _stream(dev))
    _lib.check(status, "quantize_nqkv_page_cuda")
    return PreparedNQKVPage(out[0], out[1], out[2], out[3], out[4], out[5], key_beta_table, value_beta_table,
                            page_size, valid, heads, dim, q, 4, 2, key.dtype)


# --------------------------------------------------------------------------- writers
def _rows_in_place(tensor: torch.Tensor) -> tuple[torch.Tensor, int]:
    """``(tensor, row_stride)`` for the append kernel: rows (the first axis) that are contiguous inside but lie a
    fixed distance apart -- the K or V columns of a stacked projection result -- are read where they are
    (stride in elements); anything else is made dense first (stride 0)."""
    if tensor.is_contiguous():
        return tensor, 0
    inner = 1
    for size, stride in zip(reversed(tensor.shape[1:]), reversed(tensor.stride()[1:])):
        if size != 1 and stride != inner:
            return tensor.contiguous(), 0
        inner *= size
    row = tensor.stride(0)
    if tensor.shape[0] > 1 and (row < inner or (row * tensor.element_size()) % 16 or tensor.data_ptr() % 16):
        return tensor.contiguous(), 0
    return tensor, int(row) if tensor.shape[0] > 1 else 0


def _append(cache: NQKVHotColdCache, key: torch.Tensor, value: torch.Tensor, mode: int, slot_ids: torch.Tensor,
            mask: torch.Tensor | None, source_starts: torch.Tensor | None, segment_counts: torch.Tensor | None,
            what: str) -> None:
    pool = cache.pool
    if key.shape != value.shape or key.dtype != pool.output_dtype or value.dtype != pool.output_dtype:
        raise ValueError("key and value must share shape and the cache dtype")
    if key.device != pool.device:
        raise ValueError("key and value must be on the cache device")
    if slot_ids.dtype != torch.int32 or slot_ids.ndim != 1:
        raise ValueError("slot_ids must be int32 with shape [batch]")
    batch = slot_ids.shape[0]
    tokens = 1 if mode == 0 else key.shape[1]
    expected = (batch, pool.num_kv_heads, pool.head_dim) if mode == 0 else \
        (batch, tokens, pool.num_kv_heads, pool.head_dim)
    if tuple(key.shape) != expected:
        raise ValueError(f"key and value must have shape {expected}")
    key, key_stride = _rows_in_place(key)
    value, value_stride = _rows_in_place(value)
    status = _lib.lib().nq_kv_append(
        _ptr(key), _ptr(value), _DTYPE_TAG[key.dtype], _INT(batch), _INT(tokens), _INT(mode), _ptr(slot_ids),
        _ptr(mask), _ptr(source_starts), _ptr(segment_counts), _ptr(cache.active), _ptr(cache.hot_keys),
        _ptr(cache.hot_values), _ptr(cache.hot_lengths), _ptr(cache.sequence_lengths), _INT(cache.max_sequences),
        _INT(pool.page_size), _INT(pool.num_kv_heads), _INT(pool.head_dim), _I64(key_stride), _I64(value_stride),
        _stream(pool.device))
    _lib.check(status, what)


def _launch_append_hot_k1_graph_safe(key: torch.Tensor, value: torch.Tensor, cache: NQKVHotColdCache, *,
                                     slot_ids: torch.Tensor, active_mask: torch.Tensor) -> None:
    """One new token per active row: key/value ``[B, H, D]`` (nqkv_graph_writer.py:291-332)."""
    if active_mask.dtype != torch.bool or active_mask.shape != slot_ids.shape:
        raise ValueError("active_mask must be bool with shape [batch]")
    _append(cache, key, value, 0, slot_ids, active_mask, None, None, "append_hot_k1")


def _launch_append_hot_ragged_subpage_graph_safe(key: torch.Tensor, value: torch.Tensor, cache: NQKVHotColdCache, *,
                                                 slot_ids: torch.Tensor, write_mask: torch.Tensor) -> None:
    """Prefix-masked multi-token append: key/value ``[B, T, H, D]`` (nqkv_graph_writer.py:373-419)."""
    if write_mask.dtype != torch.bool or tuple(write_mask.shape) != tuple(key.shape[:2]):
        raise ValueError("write_mask must be bool with shape [batch, tokens]")
    _append(cache, key, value, 1, slot_ids, write_mask.contiguous(), None, None, "append_hot_ragged_subpage")


def _launch_append_hot_ragged_segment_graph_safe(key: torch.Tensor, value: torch.Tensor, cache: NQKVHotColdCache, *,
                                                 slot_ids: torch.Tensor, source_starts: torch.Tensor,
                                                 segment_counts: torch.Tensor) -> None:
    """Per-row ``(source_start, count)`` segment append (nqkv_graph_writer.py:422-473)."""
    for name, t in (("source_starts", source_starts), ("segment_counts", segment_counts)):
        if t.dtype != torch.int32 or t.shape != slot_ids.shape:
            raise ValueError(f"{name} must be int32 with shape [batch]")
    _append(cache, key, value, 2, slot_ids, None, source_starts, segment_counts, "append_hot_ragged_segment")


append_hot_k1_graph_safe = _launch_append_hot_k1_graph_safe


def launch_pack_full_hot_pages_graph_safe(cache: NQKVHotColdCache, *, boundary_mask: torch.Tensor,
                                          batched_encode: bool = True, static_page_ids: bool = False) -> None:
    """Encode and publish the full hot pages of the boundary-selected slots (nqkv_graph_pack.py:76-135).

    ``static_page_ids=True``: the pool is a fixed partition of ``max_pages_per_sequence`` pages per slot and slot
    ``s`` packs into page ``s * max_pages + page_counts[s]``; ``cache.graph_target_page_ids`` is not read."""
    pool = cache.pool
    if boundary_mask.dtype != torch.bool or tuple(boundary_mask.shape) != (cache.max_sequences,):
        raise ValueError("boundary_mask must be bool with cache capacity shape")
    if boundary_mask.device != pool.device:
        raise ValueError("boundary_mask must be on the cache device")
    args = [
        _ptr(cache.hot_keys), _ptr(cache.hot_values), _DTYPE_TAG[pool.output_dtype], _ptr(cache.hot_lengths),
        _ptr(boundary_mask), _ptr(None if static_page_ids else cache.graph_target_page_ids), _ptr(pool.key_codes),
        _ptr(pool.key_betas),
        _ptr(pool.key_norms), _ptr(pool.value_codes), _ptr(pool.value_betas), _ptr(pool.value_norms),
        _ptr(pool.beta_table), _ptr(pool.value_beta_table), _ptr(cache.page_indices), _ptr(cache.page_counts),
        _ptr(cache.last_page_len), _INT(cache.max_sequences), _INT(cache.max_pages_per_sequence),
        _INT(pool.capacity), _INT(pool.page_size), _INT(pool.num_kv_heads), _INT(pool.head_dim)]
    if pool.key_lattice is not None:  # the decoded shadow of the published pages is written with them
        status = _lib.lib().nq_kv_pack_publish_lattice(*args, _ptr(pool.key_lattice), _ptr(pool.value_lattice),
                                                       _stream(pool.device))
    else:
        status = _lib.lib().nq_kv_pack_publish(*args, _stream(pool.device))
    _lib.check(status, "launch_pack_full_hot_pages_graph_safe")


# --------------------------------------------------------------------------- attention
@dataclass
class BatchedNQKVAttentionWorkspace:
    """Fixed-address output and split partials (nqkv_attention_k1.py:531-594)."""

    output: torch.Tensor
    partials: torch.Tensor
    batch_size: int
    query_tokens: int
    query_heads: int
    head_dim: int
    max_pages: int

    @classmethod
    def create(cls, cache: NQKVHotColdCache, *, batch_size: int, query_heads: int,
               output_dtype: torch.dtype = torch.bfloat16, query_tokens: int = 1) -> "BatchedNQKVAttentionWorkspace":
        pool = cache.pool
        if output_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("output_dtype must be bfloat16 or float32")
        nbytes = _lib.lib().nq_kv_attention_workspace_bytes(
            _INT(batch_size), _INT(query_tokens), _INT(query_heads), _INT(pool.num_kv_heads), _INT(pool.head_dim),
            _INT(cache.max_pages_per_sequence))
        shape = (batch_size, query_heads, pool.head_dim) if query_tokens == 1 else \
            (batch_size, query_tokens, query_heads, pool.head_dim)
        return cls(output=torch.zeros(shape, dtype=output_dtype, device=pool.device),
                   partials=torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=pool.device),
                   batch_size=batch_size, query_tokens=query_tokens, query_heads=query_heads,
                   head_dim=pool.head_dim, max_pages=cache.max_pages_per_sequence)


def _attention(query4: torch.Tensor, cache: NQKVHotColdCache, slot_ids: torch.Tensor,
               active_mask: torch.Tensor | None, q_lens: torch.Tensor | None, scale: float,
               workspace: BatchedNQKVAttentionWorkspace, what: str) -> None:
    pool = cache.pool
    batch, tokens, heads, dim = query4.shape
    if workspace.output.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("the attention output buffer must be bfloat16 or float32")
    if (workspace.batch_size, workspace.query_tokens, workspace.query_heads, workspace.head_dim,
            workspace.max_pages) != (batch, tokens, heads, dim, cache.max_pages_per_sequence):
        raise ValueError("attention workspace configuration does not match query and cache")
    if workspace.output.numel() != batch * tokens * heads * dim or workspace.output.device != pool.device:
        raise ValueError("attention output buffer does not match the query")
    out_tag = _lib.NQ_BF16 if workspace.output.dtype == torch.bfloat16 else _lib.NQ_F32
    args = [
        _ptr(query4), _DTYPE_TAG[query4.dtype], _INT(batch), _INT(tokens), _INT(heads), _ptr(slot_ids),
        _ptr(active_mask), _ptr(q_lens), _ptr(cache.active), _ptr(cache.sequence_lengths), _ptr(cache.page_indices),
        _ptr(cache.page_counts), _ptr(cache.last_page_len), _ptr(cache.hot_lengths),
        _ptr(pool.key_codes), _ptr(pool.key_betas), _ptr(pool.key_norms), _ptr(pool.value_codes),
        _ptr(pool.value_betas), _ptr(pool.value_norms), _ptr(pool.beta_table), _ptr(pool.value_beta_table),
        _ptr(cache.hot_keys), _ptr(cache.hot_values), _INT(cache.max_sequences), _INT(cache.max_pages_per_sequence),
        _INT(pool.capacity), _INT(pool.page_size), _INT(pool.num_kv_heads), _INT(dim), ctypes.c_float(scale),
        _ptr(workspace.partials), ctypes.c_size_t(workspace.partials.numel()), _ptr(workspace.output), _INT(out_tag)]
    if pool.key_lattice is not None:  # read the decoded shadow instead of searching E8 per block
        status = _lib.lib().nq_kv_attention_lattice(*args, _ptr(pool.key_lattice), _ptr(pool.value_lattice),
                                                    _stream(pool.device))
    else:
        status = _lib.lib().nq_kv_attention(*args, _stream(pool.device))
    _lib.check(status, what)


def _default_output_dtype(query: torch.Tensor) -> torch.dtype:
    """Output dtype of a workspace created on the fly: the kernel writes bfloat16 or float32 only."""
    return torch.bfloat16 if query.dtype == torch.bfloat16 else torch.float32


def _validate_query(query: torch.Tensor, cache: NQKVHotColdCache, slot_ids: torch.Tensor, ndim: int) -> None:
    pool = cache.pool
    if not isinstance(query, torch.Tensor) or query.ndim != ndim:
        raise ValueError("query must have shape [batch, query_heads, head_dim]" if ndim == 3 else
                         "query must have shape [batch, tokens, query_heads, head_dim]")
    if query.dtype not in _DTYPE_TAG:
        raise ValueError("query must be float16, bfloat16 or float32")
    if query.device != pool.device or query.shape[-1] != pool.head_dim:
        raise ValueError("query must match the cache CUDA device and head_dim")
    if query.shape[-2] < 1 or query.shape[-2] % pool.num_kv_heads:
        raise ValueError("query_heads must be a positive multiple of num_kv_heads")
    if slot_ids.dtype != torch.int32 or tuple(slot_ids.shape) != (query.shape[0],):
        raise ValueError("slot_ids must be int32 with shape [batch]")
    if pool.output_dtype != torch.bfloat16:
        raise ValueError("the attention kernel reads a BF16 hot tail")


def _launch_nqkv_decode_attention_batched_k1(query: torch.Tensor, cache: NQKVHotColdCache, *, slot_ids: torch.Tensor,
                                             active_mask: torch.Tensor, attention_scale: float,
                                             workspace: BatchedNQKVAttentionWorkspace) -> torch.Tensor:
    """Graph-safe launch (no host reads): packed-cold plus BF16-hot decode attention."""
    batch, heads, dim = query.shape
    _attention(query.contiguous().view(batch, 1, heads, dim), cache, slot_ids, active_mask, None,
               attention_scale, workspace, "nqkv_decode_attention_batched_k1")
    return workspace.output


def nqkv_decode_attention_batched_k1(query: torch.Tensor, cache: NQKVHotColdCache, *, slot_ids: torch.Tensor,
                                     active_mask: torch.Tensor, scale: float | None = None,
                                     workspace: BatchedNQKVAttentionWorkspace | None = None) -> torch.Tensor:
    """Fused packed-cold plus BF16-hot GQA attention for a ragged decode batch; no page-count cap."""
    _validate_query(query, cache, slot_ids, 3)
    if active_mask.dtype != torch.bool or active_mask.shape != slot_ids.shape:
        raise ValueError("active_mask must be bool with shape [batch]")
    if slot_ids.device != cache.pool.device or active_mask.device != cache.pool.device:
        raise ValueError("slot_ids and active_mask must be on the cache device")
    slots = slot_ids.tolist()
    enabled = active_mask.tolist()
    if any(s < 0 or s >= cache.max_sequences for s in slots):
        raise ValueError("slot_ids contain a slot outside cache capacity")
    live = [s for s, e in zip(slots, enabled) if e]
    if len(set(live)) != len(live):
        raise ValueError("active slot_ids must be unique")
    batch, heads, _ = query.shape
    if workspace is None:
        workspace = BatchedNQKVAttentionWorkspace.create(cache, batch_size=batch, query_heads=heads,
                                                         output_dtype=_default_output_dtype(query))
    if (workspace.batch_size, workspace.query_tokens, workspace.query_heads, workspace.max_pages) != \
            (batch, 1, heads, cache.max_pages_per_sequence):
        raise ValueError("batched workspace configuration does not match query and cache")
    attention_scale = 1.0 / math.sqrt(cache.pool.head_dim) if scale is None else float(scale)
    return _launch_nqkv_decode_attention_batched_k1(query, cache, slot_ids=slot_ids, active_mask=active_mask,
                                                    attention_scale=attention_scale, workspace=workspace)


def nqkv_prefill_attention(query: torch.Tensor, cache: NQKVHotColdCache, *, slot_ids: torch.Tensor,
                           query_lengths: torch.Tensor, scale: float | None = None,
                           workspace: BatchedNQKVAttentionWorkspace | None = None) -> torch.Tensor:
    """Causal chunk attention that reads the pages: ``query [B, T, Hq, D]``.

    The chunk's own K/V must already be appended; query ``i`` of row ``b`` attends to the
    first ``total_b - query_lengths[b] + i + 1`` tokens.  Rows beyond ``query_lengths[b]`` are zero.
    """
    _validate_query(query, cache, slot_ids, 4)
    if query_lengths.dtype != torch.int32 or query_lengths.shape != slot_ids.shape:
        raise ValueError("query_lengths must be int32 with shape [batch]")
    batch, tokens, heads, _ = query.shape
    if workspace is None:
        workspace = BatchedNQKVAttentionWorkspace.create(cache, batch_size=batch, query_heads=heads,
                                                         output_dtype=_default_output_dtype(query),
                                                         query_tokens=tokens)
    attention_scale = 1.0 / math.sqrt(cache.pool.head_dim) if scale is None else float(scale)
    _attention(query.contiguous(), cache, slot_ids, None, query_lengths, attention_scale, workspace,
               "nqkv_prefill_attention")
    return workspace.output


def cache_arrays(cache: NQKVHotColdCache) -> dict:
    """Host copies of every cache tensor under the reference's names (for checkers and debugging)."""
    pool = cache.pool
    return {
        "page_indices": cache.page_indices.cpu().numpy(), "page_counts": cache.page_counts.cpu().numpy(),
        "last_page_lens": cache.last_page_len.cpu().numpy(), "hot_lengths": cache.hot_lengths.cpu().numpy(),
        "key_codes": pool.key_codes.cpu().numpy(), "key_betas": pool.key_betas.cpu().numpy(),
        "key_norms": pool.key_norms.cpu().numpy(), "value_codes": pool.value_codes.cpu().numpy(),
        "value_betas": pool.value_betas.cpu().numpy(), "value_norms": pool.value_norms.cpu().numpy(),
        "key_beta_table": pool.beta_table.cpu().numpy(), "value_beta_table": pool.value_beta_table.cpu().numpy(),
        "hot_keys": cache.hot_keys.float().cpu().numpy(), "hot_values": cache.hot_values.float().cpu().numpy(),
    }
