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

            events = self.collective_events
            if events is not None and partial.is_cuda:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.process_group)
                end.record()
                events.append((start, end))
            else:
                dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.process_group)
        return partial
