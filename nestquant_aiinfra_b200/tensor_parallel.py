"""Tensor-parallel sharding of the packed W4A4 projections (Megatron layout, one process per GPU).

The reference is single-GPU; this module defines how its formats shard:

* column-parallel (q, k, v, gate, up): shard the OUTPUT rows.  Row norms, beta ids, codes and the
  dither counter are per output row, so a rank's shard is the contiguous row range of the
  unsharded record: bit-identical sub-streams, with ``block_offset = first_row * K / 8`` keeping
  the global dither counter.  The input is replicated; every rank encodes the same A4.
* row-parallel (o_proj, down_proj): shard the INPUT features.  The reference's row norm, sqrt(K)
  scale and Hadamard are defined over the full K (and K = 28672 of the 70B FFN is not a power of
  two), so each rank's slice is a self-contained projection ``[N, K/tp]``: its weight slice is
  encoded after slicing (own norms, own dither seed), its input slice is rotated with a
  block-diagonal Hadamard whose block is the largest power of two dividing K/tp, and A4-encoded
  with its own norm.  Partial outputs are summed with one all-reduce (NCCL over NVLink on GPUs).
"""

from __future__ import annotations

from dataclasses import replace
from typing import Callable, Sequence

import torch
from torch import nn

from .formats import ACTIVATION_BETAS, WEIGHT_BETAS


def shard_range(total: int, world: int, rank: int, *, multiple: int = 1) -> tuple[int, int]:
    """Contiguous ``[begin, end)`` of ``total`` units owned by ``rank``; shards are multiples of ``multiple``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if total % (world * multiple):
        raise ValueError(f"{total} is not divisible into {world} shards of a multiple of {multiple}")
    size = total // world
    return rank * size, (rank + 1) * size


def largest_power_of_two_divisor(n: int) -> int:
    if n < 1:
        raise ValueError("n must be positive")
    return n & (-n)


def block_hadamard(x: torch.Tensor, block: int) -> torch.Tensor:
    """Block-diagonal normalised Hadamard along the last axis (blocks of ``block`` features)."""
    from .rotation import hadamard

    k = x.shape[-1]
    if block < 1 or block & (block - 1) or k % block:
        raise ValueError("block must be a power of two dividing the feature dimension")
    if block == k:
        return hadamard(x)
    return hadamard(x.reshape(*x.shape[:-1], k // block, block)).reshape(x.shape)


def shard_column_parallel(prepared, rank: int, world: int):
    """Row-range view of a prepared weight (no re-encode): the rank's output channels."""
    n, k = prepared.rows, int(prepared.record.feature_count)
    begin, end = shard_range(n, world, rank, multiple=8)
    bpr = k // 8
    return replace(
        prepared,
        code_payload=prepared.code_payload[begin * k // 2:end * k // 2],
        beta_payload=prepared.beta_payload[begin * bpr // 4:end * bpr // 4],
        row_norms=prepared.row_norms[begin:end],
        block_offset=int(prepared.block_offset) + begin * bpr,
        out_features=end - begin,
    )


class ColumnParallelNQRTLinear(nn.Module):
    """``y[:, shard] = Q(xH) . W[shard]^T``; output stays sharded (feeds the row-parallel partner)."""

    def __init__(self, prepared, rank: int, world: int, *, activation_betas: Sequence[float] = ACTIVATION_BETAS,
                 input_hadamard: bool = True) -> None:
        super().__init__()
        from .fused_linear import FusedNQRTLinear

        self.rank, self.world = rank, world
        self.inner = FusedNQRTLinear(shard_column_parallel(prepared, rank, world), input_hadamard=input_hadamard,
                                     activation_betas=tuple(activation_betas))
        self.out_features, self.in_features = self.inner.out_features, self.inner.in_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(x)


class PeerAllReduce:
    """Sum of the ranks' BF16 partial outputs read straight out of peer memory (``nq_tp_allreduce_bf16``).

    One instance serves every row-parallel projection of a rank: it owns a buffer in symmetric memory
    (``torch.distributed._symmetric_memory``: the same allocation mapped into every process of the group) that
    holds this rank's partial and its flag pad, and the peers' addresses of both.  ``reduce(partial)`` copies the
    partial into the buffer and launches the kernel; the result is a fresh local tensor.  All ranks must call it
    in the same order with the same shapes (they do: the model code is the same on every rank).  Works under
    CUDA-graph capture (the call number lives in device memory).  One node only; NCCL remains the fallback.
    """

    PAD_BYTES = 128

    def __init__(self, max_elements: int, device: torch.device, process_group=None) -> None:
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        group = process_group if process_group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerAllReduce serves at most 8 ranks")
        if max_elements < 8 or max_elements % 8:
            raise ValueError("max_elements must be a positive multiple of 8")
        self.max_elements = int(max_elements)
        self.device = torch.device(device)
        nbytes = self.PAD_BYTES + 2 * self.max_elements
        self._buffer = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._buffer.zero_()
        self._handle = symm.rendezvous(self._buffer, group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # every pad is zero before anybody's first call
        bases = [int(ptr) for ptr in self._handle.buffer_ptrs]
        pointer_array = ctypes.c_void_p * self.world
        self._pads = pointer_array(*bases)
        self._partials = pointer_array(*[base + self.PAD_BYTES for base in bases])
        self._local_partial = self._buffer[self.PAD_BYTES:].view(torch.bfloat16)
        self._lib = _lib
        self.calls = 0

    def status(self) -> int:
        """Non-zero when a bounded wait of an earlier call gave up (1: partials, 2: end of reading)."""
        torch.cuda.synchronize(self.device)
        return int(self._buffer[:self.PAD_BYTES].view(torch.int32)[18].item())

    def reduce(self, partial: torch.Tensor) -> torch.Tensor:
        import ctypes

        if partial.dtype != torch.bfloat16 or partial.device != self.device:
            raise ValueError("PeerAllReduce sums bfloat16 tensors of its own device")
        count = partial.numel()
        if count > self.max_elements or count % 8:
            raise ValueError("partial must have a multiple of 8 elements, at most max_elements")
        self._local_partial[:count].copy_(partial.reshape(-1))
        out = torch.empty_like(partial, memory_format=torch.contiguous_format)
        status = self._lib.lib().nq_tp_allreduce_bf16(
            self._partials, self._pads, self.rank, self.world, ctypes.c_void_p(out.data_ptr()),
            ctypes.c_int64(count), ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        self._lib.check(status, "nq_tp_allreduce_bf16")
        self.calls += 1
        return out


class RowParallelNQRTLinear(nn.Module):
    """``y = all_reduce_sum( Q(x[:, shard] H_blk) . W[:, shard]^T )`` with a self-contained shard.

    ``weight_slice`` is this rank's ``[N, K/tp]`` float weight; it is rotated with the same
    block-diagonal Hadamard as the input and encoded here (``encode`` is injectable so the
    host logic can be exercised without a GPU).
    """

    def __init__(self, weight_slice: torch.Tensor, rank: int, world: int, *, dither_seed: int,
                 weight_betas: Sequence[float] = WEIGHT_BETAS, activation_betas: Sequence[float] = ACTIVATION_BETAS,
                 process_group=None, project: Callable[[torch.Tensor], torch.Tensor] | None = None,
                 reduce_dtype: torch.dtype | None = None) -> None:
        super().__init__()
        self.rank, self.world, self.process_group = rank, world, process_group
        self.out_features, self.in_features = int(weight_slice.shape[0]), int(weight_slice.shape[1])
        self.hadamard_block = largest_power_of_two_divisor(self.in_features)
        if self.hadamard_block < 32:
            raise ValueError("the K shard must be divisible by 32")
        self._project = project
        self.inner = None
        # measurement hook: a list here receives one (start, end) CUDA-event pair per all-reduce
        self.collective_events: list | None = None
        # a PeerAllReduce here replaces the NCCL all-reduce (BF16 partials, one node)
        self.peer_all_reduce: PeerAllReduce | None = None
        if project is None:
            from .fused_linear import FusedNQRTLinear
            from .runtime.w4a4 import quantize_weight_cuda

            rotated = block_hadamard(weight_slice.float(), self.hadamard_block)
            prepared = quantize_weight_cuda(rotated, betas=weight_betas, dither_seed=dither_seed)
            # reduce_dtype = float32 sums the ranks' FP32 accumulators (parity checks); None sums in the input dtype
            self.inner = FusedNQRTLinear(prepared, input_hadamard=False, activation_betas=tuple(activation_betas),
                                         output_dtype=reduce_dtype)
            self.inner.input_rotation_block = self.hadamard_block  # rotated inside the encoder launch when it fits

    @property
    def packed_device_bytes(self) -> int:
        return 0 if self.inner is None else self.inner.packed_device_bytes

    def forward(self, x_slice: torch.Tensor) -> torch.Tensor:
        if x_slice.shape[-1] != self.in_features:
            raise ValueError(f"input feature dimension {x_slice.shape[-1]} does not match the shard {self.in_features}")
        if self._project is not None:
            partial = self._project(x_slice)
        else:
            partial = self.inner(x_slice)
        if self.world > 1:
            import torch.distributed as dist

            peer = self.peer_all_reduce if partial.dtype == torch.bfloat16 and partial.is_cuda else None

            def collective(tensor: torch.Tensor) -> torch.Tensor:
                if peer is not None:
                    return peer.reduce(tensor)
                dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.process_group)
                return tensor

            events = self.collective_events
            if events is not None and partial.is_cuda:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                partial = collective(partial)
                end.record()
                events.append((start, end))
            else:
                partial = collective(partial)
        return partial
