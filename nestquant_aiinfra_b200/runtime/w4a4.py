"""Packed W4A4 projection: host mirror of the reference's operator interface.

Same names, argument meaning and error behaviour as
``nestquant.runtime.triton_w4a4_linear`` (``PreparedNQA4Activation``,
``quantize_activation_cuda``; triton_w4a4_linear.py:489-617),
``nestquant.runtime.triton_fused_linear`` (``PreparedNQRTLinear``,
``prepare_fused_linear``; triton_fused_linear.py:136-165) and
``nestquant.runtime.cuda_w4a4_mma`` (``can_use_*`` / ``linear_packed_w4a4_*``;
cuda_w4a4_mma.py:44-704).  Every function launches hand-written sm_100a kernels
through the C ABI on the current torch stream; there is no Triton, no backend
dispatch and no CPU fallback.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math
from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np
import torch

from .. import _lib
from ..formats import (STATELESS_DITHER_ALGORITHM, UPSTREAM_CODEC_SEMANTICS)

_DTYPE_TAG = {torch.float32: _lib.NQ_F32, torch.bfloat16: _lib.NQ_BF16, torch.float16: _lib.NQ_F16}


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_I64 = ctypes.c_int64

# ---------------------------------------------------------------------------
# workspaces: one zero-initialised buffer per (device, stream), grown on demand.
# The first WS_COUNTER_BYTES hold the split-K arrival counters; kernels leave
# them zero, so the buffer can be reused by every later call.
# ---------------------------------------------------------------------------
_WORKSPACES: dict[tuple[int, int, bool], torch.Tensor] = {}


def workspace_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for the projection kernels, one per (device, stream, eager | capture).

    Only the counter words at the front have to start at zero, and every kernel leaves them at
    zero, so one buffer serves all calls of a stream.  Buffers requested while a CUDA graph is being
    captured come from the graph's private pool and are kept apart from the eager one; they are
    reused by later calls of the same and of later captures on that stream (graphs captured on
    one stream replay one after the other, like eager calls).
    """
    capturing = torch.cuda.is_current_stream_capturing()
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream, capturing)
    buffer = _WORKSPACES.get(key)
    if buffer is None or buffer.numel() < nbytes:
        size = max(nbytes, (64 << 20) if capturing else (1 << 20))  # a capture rarely has to grow it: each growth is a fill node
        buffer = torch.zeros(size, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buffer
    return buffer


# ---------------------------------------------------------------------------
# prepared (device-resident) operands
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class PreparedNQA4Activation:
    """GPU-resident packed activation rows (triton_w4a4_linear.py:489-519).

    ``decoded`` is an optional extra of this implementation: the BF16
    reconstruction the encoder produced in the same launch.  The projection
    kernels use it when present and decode the packed streams otherwise.
    """

    code_payload: torch.Tensor
    beta_payload: torch.Tensor
    row_norms: torch.Tensor
    beta_table: torch.Tensor
    original_shape: tuple[int, ...]
    q: int
    code_width: int
    beta_width: int
    output_dtype: torch.dtype
    decoded: torch.Tensor | None = None

    @property
    def token_count(self) -> int:
        return math.prod(self.original_shape[:-1])

    @property
    def feature_count(self) -> int:
        return self.original_shape[-1]

    @property
    def resident_bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.code_payload, self.beta_payload, self.row_norms, self.beta_table))


@dataclass(frozen=True)
class PreparedNQRTLinear:
    """GPU-resident packed NQRT4 weight streams (triton_fused_linear.py:136-144)."""

    record: Any
    code_payload: torch.Tensor
    beta_payload: torch.Tensor
    row_norms: torch.Tensor
    beta_table: torch.Tensor
    # Global index of this view's first E8 block inside its record: a row-range shard keeps the
    # dither counter of the unsharded weight (the reference always passes 0, cuda_w4a4_mma.py:243).
    block_offset: int = 0
    out_features: int | None = None
    # A weight that stacks the rows of several tensors sharing one input (q/k/v, gate/up):
    # (first_row, block_offset, dither_seed) per tensor, see ``group_prepared_linears``.
    segments: tuple[tuple[int, int, int], ...] | None = None
    # Opt-in: the BF16 ``[rows, K]`` reconstruction kept in device memory (``keep_decoded_weight``).
    # With it the projection skips the per-call weight decode and reads 4x the packed bytes instead.
    decoded: torch.Tensor | None = None

    @property
    def rows(self) -> int:
        return int(self.record.indices.shape[0]) if self.out_features is None else int(self.out_features)


def _payload_tensor(payload, device: torch.device) -> torch.Tensor:
    if isinstance(payload, torch.Tensor):
        return payload.to(device=device, dtype=torch.uint8).contiguous()
    array = np.frombuffer(payload, dtype=np.uint8) if isinstance(payload, (bytes, bytearray, memoryview)) \
        else np.ascontiguousarray(payload, dtype=np.uint8)
    return torch.from_numpy(array.copy()).to(device)


def prepare_fused_linear(record, *, device: torch.device | str = "cuda") -> PreparedNQRTLinear:
    """Copy only the packed streams and compact metadata to the GPU.

    ``record`` is a ``PackedNestQuantTensor`` of this package or of the
    reference (same attribute names).
    """
    for name in ("indices", "row_norms", "betas", "feature_count"):
        if not hasattr(record, name):
            raise TypeError("record must be a PackedNestQuantTensor")
    target = torch.device(device)
    if target.type != "cuda" or not torch.cuda.is_available():
        raise ValueError("packed Linear preparation requires CUDA")
    if record.dither_seed is None or record.dither_algorithm != STATELESS_DITHER_ALGORITHM:
        raise ValueError("packed Linear requires NQRT v4 stateless dither")
    if record.codec_semantics != UPSTREAM_CODEC_SEMANTICS:
        raise ValueError("packed Linear requires upstream E8 semantics")
    return PreparedNQRTLinear(
        record=record,
        code_payload=_payload_tensor(record.indices.code_payload, target),
        beta_payload=_payload_tensor(record.indices.beta_payload, target),
        row_norms=record.row_norms.to(device=target, dtype=torch.float32).contiguous(),
        beta_table=torch.tensor(tuple(record.betas), device=target, dtype=torch.float32),
    )


ROTATED_MAX_K = 16384  # NQ_ROTATED_MAX_K of the library header


def can_rotate_in_encoder(feature_count: int, hadamard_block: int) -> bool:
    """Whether ``quantize_activation_cuda(..., hadamard_block=...)`` can fuse the rotation for these sizes."""
    return (isinstance(hadamard_block, int) and hadamard_block >= 8 and hadamard_block & (hadamard_block - 1) == 0
            and feature_count % 32 == 0 and 32 <= feature_count <= ROTATED_MAX_K
            and feature_count % hadamard_block == 0)


def prefer_rotation_in_encoder(rows: int, feature_count: int) -> bool:
    """Whether the fused launch beats ``hadamard`` + encoder for this shape.

    Up to 4096 features the fused launch is the faster one at every row count; longer rows need so
    much shared memory for the transform next to the encoder's own that occupancy drops, and a
    launch with few rows would repeat the long transform in every CTA a row is split over: there
    the two launches win (measured on 8192 features: 1.5 ms fused against 0.85 ms for 8644 rows).
    """
    return feature_count <= 4096


def prefer_producer_in_encoder(rows: int, feature_count: int) -> bool:
    """Whether the elementwise producer of a projection input (RMS norm; SiLU(gate) * up), the rotation and the
    encode should run as ONE launch for this shape.

    Up to 4096 features the rotation is done inside the encoder anyway and the producer rides along (measured:
    9.6 against 11.9 us for one row of 2048, 16.8 against 19.4 us for 256 rows).  Longer rows (the 8192-wide input
    of down_proj) are split over several CTAs that each repeat producer and transform; there the separate
    transform kernel in front of the plain encoder is the faster path at every row count (64 rows of 8192:
    27.5 us for transform + encode against 39 us for the single launch), so the producer stays a launch of its own.
    """
    del rows
    return feature_count <= 4096


def quantize_activation_cuda(
    inputs: torch.Tensor, *, q: int, betas: Sequence[float],
    beta_table: torch.Tensor | None = None, keep_decoded: bool = False, hadamard_block: int | None = None,
    rmsnorm: tuple[torch.Tensor, float] | None = None, silu_mul_with: torch.Tensor | None = None,
) -> PreparedNQA4Activation:
    """Encode floating activations into packed NQA4 payloads in one launch.

    Bit-exact with ``pack_nestquant_indices(quantize_rows(inputs.float(), q, betas))``
    of the reference CPU path.  With ``hadamard_block`` the rows are first rotated by the
    normalised Hadamard transform of that block size (the whole row when it equals the feature
    count) inside the same launch; the result equals ``quantize_activation_cuda(hadamard(inputs))``
    bit for bit (see ``can_rotate_in_encoder``).

    ``rmsnorm=(weight, eps)`` encodes ``rms_norm(inputs, weight, eps)`` and ``silu_mul_with=up`` encodes
    ``silu(inputs) * up`` instead of ``inputs`` -- the producer, the rotation (``hadamard_block`` is required) and
    the encode in one launch, bit-identical to the separate launches.

    ``keep_decoded=True`` also writes the BF16 reconstruction of the rows (``2 * M * K`` bytes) that a
    projection called next would otherwise decode for itself; callers that only want the packed
    streams (the KV page writers, a caller that stores the encoding) leave it off.
    """
    if not isinstance(inputs, torch.Tensor) or not inputs.is_floating_point():
        raise TypeError("inputs must be a floating-point tensor")
    if inputs.device.type != "cuda" or inputs.ndim < 1 or inputs.numel() == 0:
        raise ValueError("inputs must be a nonempty CUDA tensor")
    if inputs.shape[-1] % 8:
        raise ValueError("activation feature dimension must be divisible by 8")
    beta_values = tuple(float(value) for value in betas)
    if not beta_values or any(not math.isfinite(value) or value <= 0 for value in beta_values):
        raise ValueError("betas must be positive finite values")
    code_width = max(1, math.ceil(math.log2(q)))
    beta_width = max(1, math.ceil(math.log2(len(beta_values))))
    if code_width not in {1, 2, 4, 8} or beta_width not in {1, 2, 4, 8}:
        raise ValueError("packed activation fields require 1, 2, 4, or 8 bits")
    if q != 14 or len(beta_values) != 4:
        raise ValueError("the sm_100a encoder implements q=14 with four betas")
    if inputs.dtype not in _DTYPE_TAG:
        raise ValueError("inputs must use float16, bfloat16, or float32")
    k = inputs.shape[-1]
    producer = None
    if rmsnorm is not None or silu_mul_with is not None:
        if rmsnorm is not None and silu_mul_with is not None:
            raise ValueError("pass rmsnorm or silu_mul_with, not both")
        if hadamard_block is None:
            raise ValueError("a producer is fused into the rotate-and-encode launch: hadamard_block is required")
        if rmsnorm is not None:
            weight, eps = rmsnorm
            if (not isinstance(weight, torch.Tensor) or tuple(weight.shape) != (k,) or weight.dtype != inputs.dtype
                    or weight.device != inputs.device):
                raise ValueError("the norm weight must be a vector of the feature size with the input's dtype and device")
            producer = ("rmsnorm", weight.contiguous(), float(eps))
        else:
            up = silu_mul_with
            if (not isinstance(up, torch.Tensor) or up.shape != inputs.shape or up.dtype != inputs.dtype
                    or up.device != inputs.device):
                raise ValueError("silu_mul_with must match the input's shape, dtype and device")
            producer = ("silu_mul", up, 0.0)
    rows = inputs.reshape(-1, k)
    if hadamard_block is not None:
        if not can_rotate_in_encoder(k, hadamard_block):
            raise ValueError("hadamard_block must be a power of two >= 8 dividing a feature count <= 16384")
        if producer is None:
            rows = rows.contiguous()
    if rows.stride(-1) != 1 or (rows.stride(0) * rows.element_size()) % 16 or rows.data_ptr() % 16:
        rows = rows.contiguous()
    second = None
    if producer is not None and producer[0] == "silu_mul":
        second = producer[1].reshape(-1, k)
        if (second.stride(-1) != 1 or second.stride(0) != rows.stride(0) or second.data_ptr() % 16):
            rows, second = rows.contiguous(), second.contiguous()   # the kernel takes one row stride for both
    device = inputs.device
    if beta_table is None:
        beta_table = torch.tensor(beta_values, device=device, dtype=torch.float32)
    elif (beta_table.device != device or beta_table.dtype != torch.float32 or beta_table.ndim != 1
          or beta_table.numel() != len(beta_values) or not beta_table.is_contiguous()):
        raise ValueError("beta_table must be contiguous float32 on the input device")
    m = rows.shape[0]
    codes = torch.empty(m * k // 2, dtype=torch.uint8, device=device)
    beta_ids = torch.empty(m * k // 32, dtype=torch.uint8, device=device)
    norms = torch.empty(m, dtype=torch.float32, device=device)
    decoded = torch.empty((m, k), dtype=torch.bfloat16, device=device) if keep_decoded else None
    if producer is not None and producer[0] == "rmsnorm":
        status = _lib.lib().nq_a4_encode_rmsnorm_rotated(
            _ptr(rows), _ptr(producer[1]), ctypes.c_float(producer[2]), _DTYPE_TAG[inputs.dtype], _I64(m), _I64(k),
            _I64(rows.stride(0)), _I64(hadamard_block), _ptr(beta_table), _ptr(codes), _ptr(beta_ids), _ptr(norms),
            _ptr(decoded), _stream(device))
    elif producer is not None:
        status = _lib.lib().nq_a4_encode_silu_mul_rotated(
            _ptr(rows), _ptr(second), _DTYPE_TAG[inputs.dtype], _I64(m), _I64(k), _I64(rows.stride(0)),
            _I64(hadamard_block), _ptr(beta_table), _ptr(codes), _ptr(beta_ids), _ptr(norms), _ptr(decoded),
            _stream(device))
    elif hadamard_block is None:
        status = _lib.lib().nq_a4_encode(
            _ptr(rows), _DTYPE_TAG[inputs.dtype], _I64(m), _I64(k), _I64(rows.stride(0)), _ptr(beta_table),
            _ptr(codes), _ptr(beta_ids), _ptr(norms), _ptr(decoded), _stream(device))
    else:
        status = _lib.lib().nq_a4_encode_rotated(
            _ptr(rows), _DTYPE_TAG[inputs.dtype], _I64(m), _I64(k), _I64(hadamard_block), _ptr(beta_table),
            _ptr(codes), _ptr(beta_ids), _ptr(norms), _ptr(decoded), _stream(device))
    _lib.check(status, "quantize_activation_cuda")
    return PreparedNQA4Activation(
        code_payload=codes, beta_payload=beta_ids, row_norms=norms, beta_table=beta_table,
        original_shape=tuple(inputs.shape), q=q, code_width=code_width, beta_width=beta_width,
        output_dtype=inputs.dtype, decoded=decoded)


def quantize_weight_cuda(weight: torch.Tensor, *, betas: Sequence[float], dither_seed: int,
                         tensor_name: str = "weight", q: int = 14, block_offset: int = 0) -> PreparedNQRTLinear:
    """Encode a ``[N, K]`` weight on the GPU into NQRT4 streams (stateless dither).

    ``block_offset`` is the global index of the weight's first E8 block inside its record: a row
    range ``[lo, hi)`` of a larger tensor encoded with ``block_offset = lo * K / 8`` and the tensor's
    seed yields exactly the bytes of that row range of the whole tensor's streams, so
    tensor-parallel ranks can encode their own output rows.

    Bit-exact with the reference's CPU encode
    (``quantize_rows(W, 14, betas, dither=generate_e8_dither_stateless(N*K/8, seed))``
    followed by ``PackedNestQuantTensor.from_quantized_rows``).  Returns the prepared
    (device-resident) weight; ``.record`` carries the metadata and host copies are made
    lazily by ``record.indices`` consumers only.
    """
    from ..formats import PackedNestQuantIndices, PackedNestQuantTensor

    if not isinstance(weight, torch.Tensor) or not weight.is_floating_point() or weight.ndim != 2:
        raise TypeError("weight must be a floating-point [N, K] tensor")
    if weight.device.type != "cuda":
        raise ValueError("weight must be a CUDA tensor")
    if q != 14 or len(tuple(betas)) != 4:
        raise ValueError("the sm_100a encoder implements q=14 with four betas")
    if weight.dtype not in _DTYPE_TAG:
        raise ValueError("weight must use float16, bfloat16, or float32")
    w = weight.contiguous()
    n, k = w.shape
    device = w.device
    beta_table = torch.tensor(tuple(float(b) for b in betas), device=device, dtype=torch.float32)
    codes = torch.empty(n * k // 2, dtype=torch.uint8, device=device)
    beta_ids = torch.empty(n * k // 32, dtype=torch.uint8, device=device)
    norms = torch.empty(n, dtype=torch.float32, device=device)
    status = _lib.lib().nq_w4_encode(_ptr(w), _DTYPE_TAG[w.dtype], _I64(n), _I64(k), _I64(k), _ptr(beta_table),
                                     _I64(int(dither_seed)), _I64(int(block_offset)), _ptr(codes), _ptr(beta_ids),
                                     _ptr(norms), _stream(device))
    _lib.check(status, "quantize_weight_cuda")
    record = PackedNestQuantTensor(
        tensor_name=tensor_name,
        indices=PackedNestQuantIndices((n, k // 8, 8), 14, 4, b"", b""),
        row_norms=norms, betas=tuple(float(b) for b in betas), feature_count=k, dither_seed=int(dither_seed))
    return PreparedNQRTLinear(record=record, code_payload=codes, beta_payload=beta_ids, row_norms=norms,
                              beta_table=beta_table, block_offset=int(block_offset),
                              out_features=n if block_offset else None)


# ---------------------------------------------------------------------------
# predicates (host only; return False instead of raising, as the reference does)
# ---------------------------------------------------------------------------
def _tensors(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear):
    return (activation.code_payload, activation.beta_payload, activation.row_norms, activation.beta_table,
            weight.code_payload, weight.beta_payload, weight.row_norms, weight.beta_table)


def can_use_w4a4(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear) -> bool:
    """Formats and device invariants shared by every M regime."""
    record = weight.record
    tensors = _tensors(activation, weight)
    return bool(
        activation.token_count >= 1
        and activation.feature_count == record.feature_count
        and activation.q == 14 and activation.code_width == 4 and activation.beta_width == 2
        and activation.beta_table.numel() == 4
        and record.feature_count % 32 == 0
        and weight.rows % 8 == 0
        and record.indices.q == 14 and record.indices.code_bit_width == 4
        and record.indices.beta_count == 4 and record.indices.beta_index_bit_width == 2
        and record.dither_seed is not None
        and record.dither_algorithm == STATELESS_DITHER_ALGORITHM
        and record.codec_semantics == UPSTREAM_CODEC_SEMANTICS
        and all(t.is_contiguous() for t in tensors)
        and all(t.device == activation.code_payload.device for t in tensors)
        and activation.code_payload.device.type == "cuda"
    )


def can_use_w4a4_gemv_m1(activation, weight) -> bool:
    return activation.token_count == 1 and can_use_w4a4(activation, weight)


def can_use_w4a4_mma_small_m(activation, weight) -> bool:
    return activation.token_count in (2, 4, 8) and can_use_w4a4(activation, weight)


def can_use_w4a4_mma_m16(activation, weight) -> bool:
    return activation.token_count == 16 and can_use_w4a4(activation, weight)


def can_use_w4a4_mma_large_m_staged(activation, weight) -> bool:
    return activation.token_count in (32, 64, 128) and can_use_w4a4(activation, weight)


def can_use_w4a4_mma_chunked_staged(activation, weight) -> bool:
    return can_use_w4a4(activation, weight)


# ---------------------------------------------------------------------------
# the projection
# ---------------------------------------------------------------------------
def _run(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear, out_dtype: torch.dtype,
         *, use_decoded: bool = True, fused: bool = False) -> torch.Tensor:
    record = weight.record
    m, k, n = activation.token_count, activation.feature_count, weight.rows
    device = activation.code_payload.device
    library = _lib.lib()
    decoded = activation.decoded if use_decoded else None
    if weight.decoded is not None:
        nbytes = library.nq_w4a4_resident_workspace_bytes(_I64(m), _I64(n), _I64(k))
        workspace = workspace_for(device, nbytes)
        out = torch.empty((m, n), dtype=out_dtype, device=device)
        status = library.nq_w4a4_gemm_resident(
            _ptr(activation.code_payload), _ptr(activation.beta_payload), _ptr(activation.row_norms),
            _ptr(activation.beta_table), _ptr(decoded), _ptr(weight.decoded), _I64(m), _I64(n), _I64(k),
            _ptr(out), _DTYPE_TAG[out_dtype], _ptr(workspace), ctypes.c_size_t(workspace.numel()), _stream(device))
        _lib.check(status, "linear_packed_w4a4(resident)")
        return out
    nbytes = library.nq_w4a4_workspace_bytes(_I64(m), _I64(n), _I64(k))
    workspace = workspace_for(device, nbytes)
    out = torch.empty((m, n), dtype=out_dtype, device=device)
    if weight.segments:
        count = len(weight.segments)
        table = lambda column: (ctypes.c_int64 * count)(*[int(entry[column]) for entry in weight.segments])  # noqa: E731
        status = library.nq_w4a4_gemm_grouped(
            _ptr(activation.code_payload), _ptr(activation.beta_payload), _ptr(activation.row_norms),
            _ptr(activation.beta_table), _ptr(decoded),
            _ptr(weight.code_payload), _ptr(weight.beta_payload), _ptr(weight.row_norms), _ptr(weight.beta_table),
            _I64(m), _I64(n), _I64(k), ctypes.c_int(count), table(0), table(1), table(2),
            _ptr(out), _DTYPE_TAG[out_dtype], _ptr(workspace), ctypes.c_size_t(workspace.numel()), _stream(device))
        _lib.check(status, "linear_packed_w4a4")
        return out
    entry = library.nq_w4a4_gemm_fused if fused else library.nq_w4a4_gemm
    status = entry(
        _ptr(activation.code_payload), _ptr(activation.beta_payload), _ptr(activation.row_norms),
        _ptr(activation.beta_table), _ptr(decoded),
        _ptr(weight.code_payload), _ptr(weight.beta_payload), _ptr(weight.row_norms), _ptr(weight.beta_table),
        _I64(m), _I64(n), _I64(k), _I64(int(weight.block_offset)), _I64(int(record.dither_seed)),
        _ptr(out), _DTYPE_TAG[out_dtype], _ptr(workspace), ctypes.c_size_t(workspace.numel()), _stream(device))
    _lib.check(status, "linear_packed_w4a4")
    return out


MAX_GROUP = 4  # NQ_MAX_SEGMENTS of the library


def group_prepared_linears(weights: Sequence[PreparedNQRTLinear]) -> tuple[PreparedNQRTLinear, list[PreparedNQRTLinear]]:
    """Stack packed weights that share an input into one launchable weight.

    Returns the stacked weight (its streams are the members' streams one after the other, every
    member keeping its own dither counters) and the members again as views into the stacked
    buffers, so the originals can be dropped and no byte is held twice.  Each output column of a
    projection with the stacked weight has the member's own operands (bit-equal result on the
    CUDA-core path; same sums in possibly another order on the tensor-core path).
    """
    if not 2 <= len(weights) <= MAX_GROUP:
        raise ValueError(f"a group holds 2..{MAX_GROUP} weights")
    first = weights[0]
    k = int(first.record.feature_count)
    for w in weights:
        if not isinstance(w, PreparedNQRTLinear) or w.segments:
            raise TypeError("members must be plain PreparedNQRTLinear weights")
        if int(w.record.feature_count) != k or w.code_payload.device != first.code_payload.device:
            raise ValueError("members must share the feature count and the device")
        if not torch.equal(w.beta_table, first.beta_table):
            raise ValueError("members must share the beta table")
    codes = torch.cat([w.code_payload[:w.rows * k // 2] for w in weights])
    betas = torch.cat([w.beta_payload[:w.rows * k // 32] for w in weights])
    norms = torch.cat([w.row_norms[:w.rows] for w in weights])
    segments, views, row = [], [], 0
    for w in weights:
        segments.append((row, int(w.block_offset), int(w.record.dither_seed)))
        views.append(PreparedNQRTLinear(
            record=w.record, code_payload=codes[row * k // 2:(row + w.rows) * k // 2],
            beta_payload=betas[row * k // 32:(row + w.rows) * k // 32], row_norms=norms[row:row + w.rows],
            beta_table=first.beta_table, block_offset=w.block_offset, out_features=w.rows))
        row += w.rows
    stacked = PreparedNQRTLinear(record=first.record, code_payload=codes, beta_payload=betas, row_norms=norms,
                                 beta_table=first.beta_table, block_offset=0, out_features=row,
                                 segments=tuple(segments))
    return stacked, views


def read_status(device: torch.device | str = "cuda", *, clear: bool = False) -> int:
    """Device status of every projection workspace of ``device`` (synchronises the device); 0 = ok.

    A bounded wait that gave up inside the tcgen05 kernel leaves its code in the status word of the
    workspace that call used.  Eager calls and calls captured into CUDA graphs use different
    workspaces (one per stream and mode), so the words of all of them are combined here: the first
    non-zero code found is returned.  The words are sticky; ``clear=True`` zeroes them after reading.
    """
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.synchronize(device)
    found = 0
    for (index, _stream_id, _capturing), workspace in list(_WORKSPACES.items()):
        if index != device.index:
            continue
        value = ctypes.c_uint32(0)
        _lib.check(_lib.lib().nq_w4a4_status(_ptr(workspace), ctypes.byref(value), _stream(device)), "read_status")
        if value.value and not found:
            found = int(value.value)
        if clear and value.value:
            workspace[_lib.WS_STATUS_OFFSET:_lib.WS_STATUS_OFFSET + 4].zero_()
    return found


def _check_types(activation, weight) -> None:
    if not isinstance(activation, PreparedNQA4Activation):
        raise TypeError("activation must be PreparedNQA4Activation")
    if not isinstance(weight, PreparedNQRTLinear):
        raise TypeError("weight must be PreparedNQRTLinear")


def _output_dtype(activation: PreparedNQA4Activation) -> torch.dtype:
    return torch.bfloat16 if activation.output_dtype == torch.bfloat16 else torch.float32


def linear_packed_w4a4(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear) -> torch.Tensor:
    """Packed W4A4 projection for any token count (one entry, native tails)."""
    _check_types(activation, weight)
    if not can_use_w4a4(activation, weight):
        raise ValueError("activation or packed weight is unsupported by the W4A4 kernels")
    out = _run(activation, weight, _output_dtype(activation))
    n = weight.rows
    return out.to(activation.output_dtype).reshape(*activation.original_shape[:-1], n)


def linear_packed_w4a4_fp32(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear) -> torch.Tensor:
    """The FP32 accumulator before output rounding (reference: ``*_fp32_probe``)."""
    _check_types(activation, weight)
    if not can_use_w4a4(activation, weight):
        raise ValueError("activation or packed weight is unsupported by the W4A4 kernels")
    n = weight.rows
    return _run(activation, weight, torch.float32).reshape(*activation.original_shape[:-1], n)


def linear_packed_w4a4_fused_fp32(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear) -> torch.Tensor:
    """The projection as ONE launch (the kernel decodes the weight beside its own MMAs) instead of the default
    decode launch followed by the GEMM launch; identical result.  Not the default: it is not faster yet."""
    _check_types(activation, weight)
    if not can_use_w4a4(activation, weight) or weight.segments or weight.decoded is not None:
        raise ValueError("the fused entry takes a plain packed weight")
    n = weight.rows
    return _run(activation, weight, torch.float32, fused=True).reshape(*activation.original_shape[:-1], n)


def _regime(name: str, predicate):
    def run(activation: PreparedNQA4Activation, weight: PreparedNQRTLinear) -> torch.Tensor:
        _check_types(activation, weight)
        if not predicate(activation, weight):
            raise ValueError(f"activation or packed weight is unsupported by {name}")
        return linear_packed_w4a4(activation, weight)

    run.__name__ = name
    run.__doc__ = f"Reference entry ``{name}`` (runtime/cuda_w4a4_mma.py); same kernels for every M."
    return run


linear_packed_w4a4_gemv_m1 = _regime("linear_packed_w4a4_gemv_m1", can_use_w4a4_gemv_m1)
linear_packed_w4a4_mma_small_m = _regime("linear_packed_w4a4_mma_small_m", can_use_w4a4_mma_small_m)
linear_packed_w4a4_mma_m16 = _regime("linear_packed_w4a4_mma_m16", can_use_w4a4_mma_m16)
linear_packed_w4a4_mma_large_m_staged = _regime("linear_packed_w4a4_mma_large_m_staged",
                                                can_use_w4a4_mma_large_m_staged)
linear_packed_w4a4_mma_chunked_staged = _regime("linear_packed_w4a4_mma_chunked_staged",
                                                can_use_w4a4_mma_chunked_staged)


def linear_packed_w4a4_gemv_m1_fp32_probe(activation, weight) -> torch.Tensor:
    _check_types(activation, weight)
    if not can_use_w4a4_gemv_m1(activation, weight):
        raise ValueError("activation or packed weight is unsupported by W4A4 M1")
    return linear_packed_w4a4_fp32(activation, weight)


def decode_packed_a4(activation: PreparedNQA4Activation, *, dtype: torch.dtype | None = None) -> torch.Tensor:
    """Decode packed A4 rows with the production arithmetic (diagnostic).

    Bit-identical to ``QuantizedRows.dequantize`` of the reference in float32;
    ``dtype`` defaults to the activation's output dtype (reference:
    ``decode_packed_a4_m16``, cuda_w4a4_mma.py:688-696).
    """
    if not isinstance(activation, PreparedNQA4Activation):
        raise TypeError("activation must be PreparedNQA4Activation")
    dtype = activation.output_dtype if dtype is None else dtype
    kernel_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    m, k = activation.token_count, activation.feature_count
    device = activation.code_payload.device
    out = torch.empty((m, k), dtype=kernel_dtype, device=device)
    status = _lib.lib().nq_a4_decode(
        _ptr(activation.code_payload), _ptr(activation.beta_payload), _ptr(activation.row_norms),
        _ptr(activation.beta_table), _I64(m), _I64(k), _ptr(out), _DTYPE_TAG[kernel_dtype], _stream(device))
    _lib.check(status, "decode_packed_a4")
    return out.to(dtype).reshape(*activation.original_shape)


decode_packed_a4_m16 = decode_packed_a4


def decode_packed_weight(weight: PreparedNQRTLinear, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """BF16 ``[N, K]`` reconstruction of a packed weight (dither regenerated); ``out`` may receive it."""
    if not isinstance(weight, PreparedNQRTLinear):
        raise TypeError("weight must be PreparedNQRTLinear")
    if weight.segments:
        raise ValueError("decode the members of a stacked weight one by one")
    record = weight.record
    n, k = weight.rows, int(record.feature_count)
    device = weight.code_payload.device
    if out is None:
        out = torch.empty((n, k), dtype=torch.bfloat16, device=device)
    elif (out.dtype != torch.bfloat16 or tuple(out.shape) != (n, k) or not out.is_contiguous()
          or out.device != device):
        raise ValueError("out must be a contiguous bfloat16 [N, K] tensor on the weight's device")
    status = _lib.lib().nq_w4_decode(
        _ptr(weight.code_payload), _ptr(weight.beta_payload), _ptr(weight.row_norms), _ptr(weight.beta_table),
        _I64(n), _I64(k), _I64(int(weight.block_offset)), _I64(int(record.dither_seed)), _ptr(out), _stream(device))
    _lib.check(status, "decode_packed_weight")
    return out


def keep_decoded_weight(weight: PreparedNQRTLinear,
                        members: Sequence[PreparedNQRTLinear] | None = None) -> PreparedNQRTLinear:
    """Return ``weight`` with its BF16 reconstruction kept in device memory (opt-in).

    The packed streams stay as they are (they remain the record of truth); the decoded matrix
    costs ``2 * N * K`` bytes more and lets every later projection skip the weight decode: the
    small-token GEMV becomes a stream over BF16 bound by HBM, the tensor-core path loses its
    decode launch.  The values are those the packed kernels regenerate per call, so results
    agree with the packed path up to the order of the FP32 sums.  For a stacked weight pass the
    member views of ``group_prepared_linears`` as ``members``.
    """
    if not isinstance(weight, PreparedNQRTLinear):
        raise TypeError("weight must be PreparedNQRTLinear")
    if weight.decoded is not None:
        return weight
    k = int(weight.record.feature_count)
    if weight.segments:
        if members is None or sum(member.rows for member in members) != weight.rows:
            raise ValueError("a stacked weight needs its member views to be decoded")
        decoded = torch.empty((weight.rows, k), dtype=torch.bfloat16, device=weight.code_payload.device)
        row = 0
        for member in members:
            decode_packed_weight(member, out=decoded[row:row + member.rows])
            row += member.rows
    else:
        decoded = decode_packed_weight(weight)
    return dataclasses.replace(weight, decoded=decoded)


def gemm_bf16_tc(a_dec: torch.Tensor, w_dec: torch.Tensor, *, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """tcgen05 GEMM on decoded BF16 operands ``A[m,k]``, ``W[n,k]`` (measurement / test building block)."""
    if a_dec.dtype != torch.bfloat16 or w_dec.dtype != torch.bfloat16:
        raise TypeError("operands must be bfloat16")
    if a_dec.ndim != 2 or w_dec.ndim != 2 or a_dec.shape[1] != w_dec.shape[1]:
        raise ValueError("operands must be [m,k] and [n,k]")
    a_dec, w_dec = a_dec.contiguous(), w_dec.contiguous()
    (m, k), n = a_dec.shape, w_dec.shape[0]
    device = a_dec.device
    workspace = workspace_for(device, _lib.WS_COUNTER_BYTES)
    out = torch.empty((m, n), dtype=out_dtype, device=device)
    status = _lib.lib().nq_bf16_gemm_tc(_ptr(a_dec), _ptr(w_dec), _I64(m), _I64(n), _I64(k), _ptr(out),
                                        _DTYPE_TAG[out_dtype], _ptr(workspace), ctypes.c_size_t(workspace.numel()),
                                        _stream(device))
    _lib.check(status, "gemm_bf16_tc")
    return out


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_lib.lib().nq_launch_count())
