"""``FusedNQRTLinear``: the module-level plugin boundary of the packed W4A4 projection.

Mirror of ``nestquant.models.fused_linear`` (FusedNQRTLinear :130-421,
SharedHadamardCache :49-84, SharedPackedActivationCache :87-127,
convert_linears_to_fused_nqrt_ :543-695) restricted to the served backend
``compute_backend="packed_w4a4_cuda_mma"``: Hadamard on the input when asked,
one on-the-fly A4 encode (shared between projections that receive the same
input tensor object), one packed projection call, cast to the output dtype.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from .rotation import hadamard, hadamard_silu_mul
from .runtime.w4a4 import (PreparedNQA4Activation, PreparedNQRTLinear, linear_packed_w4a4, linear_packed_w4a4_fp32,
                           prepare_fused_linear, prefer_producer_in_encoder,
                           quantize_activation_cuda, can_rotate_in_encoder, prefer_rotation_in_encoder,
                           group_prepared_linears, keep_decoded_weight, decode_packed_weight)

_BACKENDS = {"packed_w4a4_cuda_mma", "packed_w4a4_cuda_gemv_m1", "packed_w4a4"}


class _SharedByIdentity:
    """One value computed from an input tensor, handed to ``uses_per_input`` consumers of that same object.

    Projections that read the same hidden state (q/k/v, gate/up) are called one after the other with
    the very same tensor object; the first call computes, the following ones fetch, and the entry is
    dropped when the last consumer has been served.  Inference only: a cached value carries no graph.
    """

    _what = "shared input"

    def __init__(self, uses_per_input: int) -> None:
        if isinstance(uses_per_input, bool) or not isinstance(uses_per_input, int):
            raise TypeError("uses_per_input must be an integer")
        if uses_per_input < 2:
            raise ValueError("uses_per_input must be at least two")
        self.uses_per_input = uses_per_input
        self.hits = self.misses = 0
        self._key: torch.Tensor | None = None
        self._value: Any = None
        self._left = 0

    def _require_inference(self) -> None:
        if torch.is_grad_enabled():
            raise RuntimeError(f"{self._what} caching requires inference or no-grad mode")

    def _fetch(self, inputs: torch.Tensor):
        """The stored value if ``inputs`` is the object it was computed from (and counts the use), else None."""
        if self._key is not inputs or self._left <= 0:
            return None
        value = self._value
        self.hits += 1
        self._left -= 1
        if self._left == 0:
            self.clear()
        return value

    def _store(self, inputs: torch.Tensor, value) -> None:
        self._key, self._value, self._left = inputs, value, self.uses_per_input - 1
        self.misses += 1

    def clear(self) -> None:
        self._key = self._value = None
        self._left = 0


class SharedHadamardCache(_SharedByIdentity):
    """Reuse one Hadamard result for modules sharing an input (models/fused_linear.py:49-84)."""

    _what = "shared Hadamard"
    _IN_ENCODER = object()  # marker: the rotation runs inside the encoder launch, there is no tensor to hand out

    def transform(self, inputs: torch.Tensor) -> torch.Tensor:
        self._require_inference()
        cached = self._fetch(inputs)
        if cached is not None and cached is not self._IN_ENCODER:
            return cached
        output = hadamard(inputs)
        if cached is None:
            self._store(inputs, output)
        return output

    def note_rotation_in_encoder(self, inputs: torch.Tensor) -> None:
        """Same hit / miss accounting as ``transform`` when the encoder launch does the rotation itself."""
        self._require_inference()
        if self._fetch(inputs) is None:
            self._store(inputs, self._IN_ENCODER)


class SharedPackedActivationCache(_SharedByIdentity):
    """Reuse one packed A4 encoding for projections sharing an input tensor (models/fused_linear.py:87-127)."""

    _what = "shared A4"

    def encode(self, inputs: torch.Tensor, *, q: int, betas: tuple[float, ...],
               beta_table: torch.Tensor | None = None, hadamard_block: int | None = None,
               rmsnorm: tuple[torch.Tensor, float] | None = None) -> tuple[PreparedNQA4Activation, bool]:
        """``(packed, encoded_now)``: the second item tells the caller whether this call ran the encoder."""
        self._require_inference()
        packed = self._fetch(inputs)
        if packed is not None:
            return packed, False
        packed = quantize_activation_cuda(inputs, q=q, betas=betas, beta_table=beta_table,
                                          hadamard_block=hadamard_block, keep_decoded=True, rmsnorm=rmsnorm)
        self._store(inputs, packed)
        return packed, True


class SharedProjectionGroup:
    """One launch sequence for projections that share an input (q/k/v, gate/up).

    The members' packed weights are stacked (``group_prepared_linears``); the first member called
    with a packed activation runs the projection over all stacked rows, every member returns its
    own column range of that result.  Members must receive the same packed activation object
    (a shared ``SharedPackedActivationCache``); a member called with another one just triggers a
    new projection.  The operands of every output column are the member's own (same decoded
    weights, same activation); on the tensor-core path the split of K follows the tile count, so
    sums may be taken in another order than in the member's own launch.
    """

    SEPARATE_FROM = 512  # rows from which every member runs its own projection

    def __init__(self, members: "list[FusedNQRTLinear]", device: torch.device | str | None = None) -> None:
        if any(member._prepared is None for member in members) and device is None:
            raise ValueError("members without a prepared weight need the target device")
        prepared = [member._prepared if device is None else member._prepared_for(torch.device(device))
                    for member in members]
        self.stacked, views = group_prepared_linears(prepared)
        self.views = views
        self.bounds = []
        start = 0
        for index, (member, view) in enumerate(zip(members, views)):
            member._prepared = view          # the member keeps a view: no stream is held twice
            member._group, member._group_index = self, index
            self.bounds.append((start, start + view.rows))
            start += view.rows
        self._packed = None
        self._output: torch.Tensor | None = None
        self._remaining = 0
        self.launches = 0
        self._ahead: "_AheadUnit | None" = None  # set by WeightDecodeAhead

    def keep_decoded_weight(self) -> int:
        """Keep the BF16 reconstruction of the stacked weight in device memory (opt-in, see
        ``runtime.keep_decoded_weight``); returns the bytes this adds."""
        self.stacked = keep_decoded_weight(self.stacked, self.views)
        return self.stacked.decoded.numel() * 2

    def project(self, packed: PreparedNQA4Activation, index: int) -> torch.Tensor:
        if packed.token_count >= self.SEPARATE_FROM and not (self._ahead is not None and self._ahead.armed):
            # many rows: the launches saved by stacking no longer matter, while every member would have to copy
            # its column range out of the stacked result (tensor ops on a column slice fall off their vectorised
            # kernels): the member's own projection writes a contiguous result at the same decode + GEMM work
            view = self.views[index]
            if self.stacked.decoded is not None:  # resident decoded weights: the member's rows of the stacked matrix
                start, end = self.bounds[index]
                view = dataclasses.replace(view, decoded=self.stacked.decoded[start:end])
            return linear_packed_w4a4(packed, view)
        if self._packed is not packed or self._output is None:
            stacked = self.stacked
            if self._ahead is not None and self._ahead.armed:
                stacked = self._ahead.take(packed.token_count)
            self._output = linear_packed_w4a4(packed, stacked)
            self._packed = packed
            self._remaining = len(self.bounds)
            self.launches += 1
        start, end = self.bounds[index]
        output = self._output[..., start:end]
        self._remaining -= 1
        if self._remaining <= 0:
            self._packed = self._output = None
        return output


class FusedNQRTLinear(nn.Module):
    """Apply one packed NQRT v4 weight without materialising a BF16 matrix in the module.

    ``source`` is a checkpoint reader exposing ``get_entry(name).shape`` and
    ``read_named_record(name) -> (name, record)`` (the reference's ``NQMCFileReader``),
    a packed record, or an already prepared weight.  Bias is not supported by the CUDA
    path (the reference routes biased projections to its Triton kernel).
    """

    def __init__(self, source: Any, weight_name: str = "weight", bias: torch.Tensor | None = None, *,
                 input_hadamard: bool = False, input_transform_cache: SharedHadamardCache | None = None,
                 output_dtype: torch.dtype | None = None, compute_backend: str = "packed_w4a4_cuda_mma",
                 activation_q: int = 14, activation_betas: tuple[float, ...] | None = None,
                 packed_activation_cache: SharedPackedActivationCache | None = None,
                 force_w4a4_tiled_fallback: bool = False, enable_m1_down_splitk: bool = False) -> None:
        super().__init__()
        if compute_backend not in _BACKENDS:
            raise ValueError("unsupported fused NQRT compute_backend (this build serves packed_w4a4_cuda_mma)")
        if not activation_betas:
            raise ValueError("packed_w4a4 requires activation_betas")
        if bias is not None:
            raise ValueError("the packed W4A4 CUDA path requires bias=None")
        if force_w4a4_tiled_fallback:
            raise ValueError("there is no Triton fallback in this build")
        if not isinstance(enable_m1_down_splitk, bool):
            raise TypeError("enable_m1_down_splitk must be a bool")
        self._prepared: PreparedNQRTLinear | None = None
        self._record = None
        self.reader = None
        if isinstance(source, PreparedNQRTLinear):
            self._prepared = source
            shape = (source.rows, int(source.record.feature_count))
        elif hasattr(source, "read_named_record"):
            self.reader = source
            entry = source.get_entry(weight_name)
            if getattr(entry, "kind", "nestquant") != "nestquant":
                raise ValueError("FusedNQRTLinear requires a packed NestQuant record")
            shape = tuple(entry.shape)
        elif hasattr(source, "indices") and hasattr(source, "feature_count"):
            self._record = source
            shape = (int(source.indices.shape[0]), int(source.feature_count))
        else:
            raise TypeError("source must be a checkpoint reader, a packed record or a prepared weight")
        if len(shape) != 2 or not all(shape):
            raise ValueError("weight record must have nonempty [out, in] shape")
        self.out_features, self.in_features = int(shape[0]), int(shape[1])
        if input_hadamard and self.in_features & (self.in_features - 1):
            raise ValueError("Hadamard input transform requires power-of-two in_features")
        if input_transform_cache is not None and not isinstance(input_transform_cache, SharedHadamardCache):
            raise TypeError("input_transform_cache must be a SharedHadamardCache or None")
        if input_transform_cache is not None and not input_hadamard:
            raise ValueError("input_transform_cache requires input_hadamard=True")
        if output_dtype is not None and output_dtype not in {torch.float16, torch.bfloat16, torch.float32}:
            raise ValueError("output_dtype must be float16, bfloat16, float32, or None")
        self.weight_name = weight_name
        self.input_hadamard = input_hadamard
        # block-diagonal rotation of the input (tensor-parallel K shards); set by the owner, None = off
        self.input_rotation_block: int | None = None
        # set by SharedProjectionGroup: this projection runs as a column range of a stacked weight
        self._group: "SharedProjectionGroup | None" = None
        self._group_index = 0
        self._ahead: "_AheadUnit | None" = None  # set by WeightDecodeAhead
        self._ahead_trigger = None  # (scheduler, layer) on a layer's first projection, see WeightDecodeAhead.EARLY_START
        self.input_transform_cache = input_transform_cache
        self.output_dtype = output_dtype
        self.compute_backend = compute_backend
        self.activation_q = activation_q
        self.activation_betas = tuple(float(b) for b in activation_betas)
        self.packed_activation_cache = packed_activation_cache
        self.enable_m1_down_splitk = enable_m1_down_splitk
        self.register_buffer("activation_beta_table",
                             torch.tensor(self.activation_betas, dtype=torch.float32), persistent=False)
        self.bias = None
        self.a4_call_count = 0
        self.a4_encode_count = 0
        self.w4a4_cuda_mma_dispatch_count = 0
        self.w4a4_tiled_fallback_count = 0

    @property
    def prepared(self) -> bool:
        return self._prepared is not None

    @property
    def packed_device_bytes(self) -> int:
        p = self._prepared
        if p is None:
            return 0
        return sum(t.numel() * t.element_size() for t in (p.code_payload, p.beta_payload, p.row_norms, p.beta_table))

    def keep_decoded_weight(self, device: torch.device | str | None = None) -> int:
        """Opt out of the module's default of never holding a BF16 matrix: keep the decoded weight
        in device memory (``2 * out * in`` bytes more) so that later calls skip the weight decode.
        A member of a ``SharedProjectionGroup`` converts the group's stacked weight.  Returns the
        bytes added."""
        if self._group is not None:
            return 0 if self._group.stacked.decoded is not None else self._group.keep_decoded_weight()
        prepared = self._prepared if device is None else self._prepared_for(torch.device(device))
        if prepared is None:
            raise ValueError("no prepared weight yet: pass the target device")
        if prepared.decoded is not None:
            return 0
        self._prepared = keep_decoded_weight(prepared)
        return self._prepared.decoded.numel() * 2

    def clear_prepared(self) -> None:
        if self.reader is not None or self._record is not None:
            self._prepared = None

    def _prepared_for(self, device: torch.device) -> PreparedNQRTLinear:
        prepared = self._prepared
        if prepared is not None and prepared.code_payload.device == device:
            return prepared
        if self.reader is not None:
            _, record = self.reader.read_named_record(self.weight_name)
        elif self._record is not None:
            record = self._record
        else:
            raise RuntimeError("prepared weight lives on another device and no record is attached")
        prepared = prepare_fused_linear(record, device=device)
        self._prepared = prepared
        return prepared

    def _check_inputs(self, inputs: torch.Tensor) -> None:
        if not isinstance(inputs, torch.Tensor) or not inputs.is_floating_point():
            raise TypeError("inputs must be a floating-point tensor")
        if inputs.ndim == 0 or inputs.shape[-1] != self.in_features:
            actual = None if inputs.ndim == 0 else inputs.shape[-1]
            raise ValueError(f"input feature dimension {actual} does not match {self.in_features}")
        if inputs.device.type != "cuda":
            raise ValueError("FusedNQRTLinear requires CUDA inputs")

    def _finish(self, packed: PreparedNQA4Activation, encoded: bool, prepared: PreparedNQRTLinear,
                original_dtype: torch.dtype) -> torch.Tensor:
        self.a4_call_count += 1
        self.a4_encode_count += int(encoded)
        if self._group is None and self._ahead is not None and self._ahead.armed:
            prepared = self._ahead.take(packed.token_count)
        if self._group is not None:
            outputs = self._group.project(packed, self._group_index)
        elif self.output_dtype == torch.float32:
            outputs = linear_packed_w4a4_fp32(packed, prepared)  # the accumulator itself, not rounded to the input dtype first
        else:
            outputs = linear_packed_w4a4(packed, prepared)
        self.w4a4_cuda_mma_dispatch_count += 1
        return outputs.to(self.output_dtype or original_dtype)

    def forward_silu_mul(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """``self(silu(gate) * up)`` -- the Llama MLP's input of ``down_proj``.  When the shape allows it, SiLU, the
        product, the rotation and the A4 encode run as ONE launch (same bits as the tensor ops followed by the
        rotate-and-encode); otherwise this is literally ``self(silu(gate) * up)``."""
        self._check_inputs(gate)
        if up.shape != gate.shape or up.dtype != gate.dtype or up.device != gate.device:
            raise ValueError("gate and up must share shape, dtype and device")
        block = self.in_features if self.input_hadamard else self.input_rotation_block
        rows = gate.numel() // self.in_features
        if block is None or torch.is_grad_enabled() or gate.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            return self.forward(torch.nn.functional.silu(gate) * up)
        if not can_rotate_in_encoder(self.in_features, block) or not prefer_producer_in_encoder(rows, self.in_features):
            # long rows: product and rotation as one launch in front of the plain encoder
            if self.input_transform_cache is not None:
                return self.forward(torch.nn.functional.silu(gate) * up)
            shape = gate.shape
            if block != self.in_features:
                blocked = (*shape[:-1], self.in_features // block, block)
                gate, up = gate.reshape(blocked), up.reshape(blocked)
            return self._encode_and_project(hadamard_silu_mul(gate, up).reshape(shape), None, None, gate.dtype)
        prepared = self._prepared_for(gate.device)
        beta_table = self.activation_beta_table
        if beta_table.device != gate.device:
            beta_table = beta_table.to(gate.device)
        packed = quantize_activation_cuda(gate, q=self.activation_q, betas=self.activation_betas, beta_table=beta_table,
                                          hadamard_block=block, keep_decoded=True, silu_mul_with=up)
        return self._finish(packed, True, prepared, gate.dtype)

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        self._check_inputs(inputs)
        if self._ahead_trigger is not None and inputs.ndim >= 2 and inputs.shape[-2] == 1:
            # first projection of a decoder layer in a decode step: the weights the layer needs after its attention
            # start decoding on the second stream now
            self._ahead_trigger[0].launch(self._ahead_trigger[1], inputs.numel() // self.in_features)
        original_dtype = inputs.dtype
        # The rotation of the input runs inside the encoder launch when the sizes allow it
        # (bit-identical to hadamard() followed by the encoder); otherwise as its own launch.
        wanted_block = self.in_features if self.input_hadamard else self.input_rotation_block
        rotate_in_encoder = (wanted_block is not None
                             and inputs.dtype in (torch.bfloat16, torch.float16, torch.float32)
                             and can_rotate_in_encoder(self.in_features, wanted_block)
                             and prefer_rotation_in_encoder(inputs.numel() // self.in_features, self.in_features))
        # A normalisation that its module left pending (norm.FusedRMSNorm(defer=True)) is done inside the same
        # launch when the rotation is; otherwise it is materialised once for all consumers of this input.
        pending_norm = getattr(inputs, "_nq_pending_norm", None)
        if pending_norm is not None and not rotate_in_encoder:
            materialised = getattr(inputs, "_nq_materialised", None)
            if materialised is None:
                from .norm import rms_norm

                materialised = rms_norm(inputs, *pending_norm)
                inputs._nq_materialised = materialised
            inputs, pending_norm = materialised, None
        if rotate_in_encoder:
            if self.input_transform_cache is not None:
                self.input_transform_cache.note_rotation_in_encoder(inputs)
            compute_inputs, block = inputs, wanted_block
        else:
            block = None
            if self.input_transform_cache is not None:
                compute_inputs = self.input_transform_cache.transform(inputs)
            elif self.input_hadamard:
                compute_inputs = hadamard(inputs)
            elif self.input_rotation_block is not None:
                b = self.input_rotation_block
                compute_inputs = hadamard(inputs.reshape(*inputs.shape[:-1], self.in_features // b, b)).reshape(inputs.shape)
            else:
                compute_inputs = inputs
        return self._encode_and_project(compute_inputs, block, pending_norm, original_dtype)

    def _encode_and_project(self, compute_inputs: torch.Tensor, block: int | None, pending_norm,
                            original_dtype: torch.dtype) -> torch.Tensor:
        """A4 encode (rotating by ``block`` and applying ``pending_norm`` inside the launch when given) + projection."""
        prepared = self._prepared_for(compute_inputs.device)
        beta_table = self.activation_beta_table
        if beta_table.device != compute_inputs.device:
            beta_table = beta_table.to(compute_inputs.device)
        if self.packed_activation_cache is None:
            packed = quantize_activation_cuda(compute_inputs, q=self.activation_q, betas=self.activation_betas,
                                              beta_table=beta_table, hadamard_block=block, keep_decoded=True,
                                              rmsnorm=pending_norm)
            encoded = True
        else:
            packed, encoded = self.packed_activation_cache.encode(
                compute_inputs, q=self.activation_q, betas=self.activation_betas, beta_table=beta_table,
                hadamard_block=block, rmsnorm=pending_norm)
        return self._finish(packed, encoded, prepared, original_dtype)


class _AheadUnit:
    """One packed weight (a module's own or a group's stacked one) whose BF16 form another stream prepares."""

    def __init__(self, owner, packed: PreparedNQRTLinear, members: "list[PreparedNQRTLinear] | None") -> None:
        self.owner = owner
        self.packed = packed
        self.members = members                      # member views of a stacked weight, else None
        self.resident: PreparedNQRTLinear | None = None  # `packed` with the scratch as its decoded matrix
        self.event: torch.cuda.Event | None = None
        self.armed = False

    def bind(self, scratch: torch.Tensor) -> None:
        rows, k = self.packed.rows, int(self.packed.record.feature_count)
        self.resident = dataclasses.replace(self.packed, decoded=scratch[:rows * k].view(rows, k))

    def decode(self) -> None:
        """Queue the decode on the current stream and remember where it ends."""
        out = self.resident.decoded
        if self.members is None:
            decode_packed_weight(self.packed, out=out)
        else:
            row = 0
            for member in self.members:
                decode_packed_weight(member, out=out[row:row + member.rows])
                row += member.rows
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(out.device))
        self.armed = True

    def take(self, token_count: int) -> PreparedNQRTLinear:
        """The weight to project with; the caller's stream waits for the decode (which joins the two streams)."""
        self.armed = False
        torch.cuda.current_stream(self.resident.decoded.device).wait_event(self.event)
        # below eight rows the packed path runs the CUDA-core kernel, not decode + tcgen05: keep its sums
        return self.resident if token_count >= WeightDecodeAhead.MIN_ROWS else self.packed


class WeightDecodeAhead:
    """Decode the packed weights a decoder layer needs AFTER its attention WHILE the attention runs.

    The paged attention of a decode step leaves SMs idle towards its end (sequences of different lengths);
    the weight decodes of ``o_proj``, gate / up and ``down_proj`` of the same layer do not depend on it.
    ``launch(layer)`` -- called at the layer's first projection of a decode step (``EARLY_START``), or right
    before the layer's attention is queued -- forks a second stream of the lowest priority
    from the current one, queues those decodes there into scratch matrices shared by all layers, and
    the projections then wait for "their" decode and run the tensor-core GEMM on the scratch (the
    resident entry of the library).  Same kernels on the same operands as the plain sequence, so the
    results are bit-identical; inside a CUDA graph capture the second stream becomes a parallel branch
    of the graph.  Every armed unit must be consumed before the step ends (the projections of the layer
    do that), otherwise a capture would end with an unjoined stream.
    """

    MIN_ROWS = 8
    # Fork at the layer's FIRST projection (a decode step's q_proj call) instead of right before its attention: the
    # decodes then also fill the SMs that the short launches leading up to the attention leave idle.  This only pays
    # because the second stream has the lowest priority and the runner captures its step on a stream of the highest
    # one: with equal priorities the full-grid decode kernels take the SMs from exactly those launches.
    EARLY_START = True
    _BEFORE_ATTENTION = ("q_proj", "k_proj", "v_proj")

    def __init__(self, layers, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device, priority=0)  # lowest: the decodes only fill what the step leaves idle
        self.layers: list[list[_AheadUnit]] = []
        sizes: list[int] = []
        self.triggers: list[tuple[FusedNQRTLinear, int]] = []
        for layer_index, layer in enumerate(layers):
            units: list[_AheadUnit] = []
            seen: set[int] = set()
            first = True
            for name, module in layer.named_modules():
                if not isinstance(module, FusedNQRTLinear):
                    continue
                if any(part in self._BEFORE_ATTENTION for part in name.split(".")):
                    if first and self.EARLY_START:
                        module._ahead_trigger = (self, layer_index)
                        self.triggers.append((module, layer_index))
                    first = False
                    continue
                group = module._group
                if group is not None:
                    if id(group) in seen or group.stacked.decoded is not None:
                        continue
                    seen.add(id(group))
                    units.append(_AheadUnit(group, group.stacked, list(group.views)))
                else:
                    prepared = module._prepared_for(self.device)
                    if prepared.decoded is None:
                        units.append(_AheadUnit(module, prepared, None))
            for index, unit in enumerate(units):
                elements = unit.packed.rows * int(unit.packed.record.feature_count)
                if index == len(sizes):
                    sizes.append(elements)
                sizes[index] = max(sizes[index], elements)
            self.layers.append(units)
        self.scratch = [torch.empty(n, dtype=torch.bfloat16, device=self.device) for n in sizes]
        for units in self.layers:
            for index, unit in enumerate(units):
                unit.bind(self.scratch[index])
                unit.owner._ahead = unit
        self.launches = 0

    @property
    def scratch_bytes(self) -> int:
        return sum(t.numel() * 2 for t in self.scratch)

    def launch(self, layer_index: int, rows: int, *, at_attention: bool = False) -> None:
        if rows < self.MIN_ROWS or not 0 <= layer_index < len(self.layers) or not self.layers[layer_index]:
            return
        if at_attention and self.triggers and any(unit.armed for unit in self.layers[layer_index]):
            return  # queued at the layer's first projection already
        # (the first caller of a layer always queues: units a failed step left armed are decoded afresh)
        main = torch.cuda.current_stream(self.device)
        fork = torch.cuda.Event()
        fork.record(main)
        self.stream.wait_event(fork)
        with torch.cuda.stream(self.stream):
            for unit in self.layers[layer_index]:
                unit.decode()
        self.launches += 1

    def detach(self) -> None:
        for units in self.layers:
            for unit in units:
                unit.owner._ahead = None
                unit.armed = False
        for module, _ in self.triggers:
            module._ahead_trigger = None

    def attach(self) -> None:
        for units in self.layers:
            for unit in units:
                unit.owner._ahead = unit
        for module, layer_index in self.triggers:
            module._ahead_trigger = (self, layer_index)


def keep_decoded_weights_(model: nn.Module, device: torch.device | str | None = None) -> int:
    """Switch every ``FusedNQRTLinear`` of ``model`` to resident decoded weights; returns the bytes added.

    An explicit trade for machines with HBM to spare: 4x the packed weight bytes stay resident and
    no projection regenerates dither or searches E8 for its weight again.  The reference has no
    such mode (its modules never hold a BF16 matrix).
    """
    return sum(module.keep_decoded_weight(device) for module in model.modules()
               if isinstance(module, FusedNQRTLinear))


HADAMARD_METADATA_FORMAT = "local_hadamard_linear_v1"  # models/rotated_linear.py:18
_SERVED_BACKENDS = ("packed_w4a4", "packed_w4a4_cuda_mma", "packed_w4a4_cuda_gemv_m1")


@dataclass(frozen=True)
class FusedNQRTConversionReport:
    """What a conversion replaced (same fields as the reference's report, models/fused_linear.py:533-540)."""

    replaced_linear_names: tuple[str, ...]
    input_hadamard_names: tuple[str, ...]
    shared_hadamard_groups: tuple[tuple[str, ...], ...]
    grouped_qkv_groups: tuple[tuple[str, str, str], ...]
    w4a4_tiled_fallback_names: tuple[str, ...] = ()
    m1_down_splitk_fallback_names: tuple[str, ...] = ()


def _rotated_module_names(metadata) -> set[str]:
    """Modules whose stored weight is Hadamard-rotated, from the checkpoint metadata (models/fused_linear.py:720-732)."""
    entry = (metadata or {}).get("hadamard_rotation")
    if entry is None:
        return set()
    if not isinstance(entry, dict) or entry.get("format") != HADAMARD_METADATA_FORMAT:
        raise ValueError("unsupported or malformed Hadamard checkpoint metadata")
    names = entry.get("converted_linear_names")
    if not isinstance(names, list) or any(not isinstance(n, str) or not n for n in names):
        raise ValueError("Hadamard converted module names must be nonempty strings")
    return set(names)


def _input_sharing_groups(names: set[str]) -> tuple[tuple[str, ...], ...]:
    """q/k/v of one attention block and gate/up of one MLP receive the same input tensor."""
    buckets: dict[tuple[str, str], list[str]] = {}
    for name in sorted(names):
        parent, _, leaf = name.rpartition(".")
        kind = "qkv" if leaf in ("q_proj", "k_proj", "v_proj") else "gate_up" if leaf in ("gate_proj", "up_proj") else None
        if kind is not None:
            buckets.setdefault((parent, kind), []).append(name)
    return tuple(tuple(group) for group in buckets.values() if len(group) > 1)


def _name_collection(value, what: str) -> tuple[str, ...]:
    if isinstance(value, (str, bytes)):
        raise TypeError(f"{what} must be a collection of module names")
    names = tuple(value)
    if any(not isinstance(name, str) or not name for name in names):
        raise ValueError(f"{what} must contain nonempty module names")
    return names


def convert_linears_to_fused_nqrt_(model: nn.Module, reader: Any, include_names, *,
                                   output_dtype: torch.dtype | None = None, group_qkv: bool = False,
                                   compute_backend: str = "packed_w4a4_cuda_mma", activation_q: int = 14,
                                   activation_betas: tuple[float, ...] | None = None,
                                   w4a4_tiled_fallback_names=(), enable_m1_down_splitk: bool = False,
                                   m1_down_splitk_fallback_names=()) -> FusedNQRTConversionReport:
    """Replace the selected ``nn.Linear`` modules of ``model`` by packed NQRT modules, all or nothing.

    Signature and behaviour of the reference's converter (models/fused_linear.py:543-695):
    ``include_names`` are MODULE names; ``reader`` is the checkpoint reader (``get_entry(name)`` with
    ``.kind`` / ``.shape``, ``read_named_record(name)``, ``model_metadata``), e.g. the reference's
    ``NQMCFileReader``.  Which modules rotate their input comes from the checkpoint metadata;
    q/k/v and gate/up of one block are found by name and share one rotation and one A4 encode per
    forward.  Everything is validated before the first module is replaced.

    Differences, all forced by there being one backend here: ``compute_backend`` must be one of the
    packed W4A4 CUDA names; ``group_qkv`` stacks q/k/v into one weight decoded and multiplied by one
    launch sequence (the reference runs one grouped Triton kernel) and needs the modules on a CUDA
    device at conversion time; modules listed in ``w4a4_tiled_fallback_names`` /
    ``m1_down_splitk_fallback_names`` are accepted, reported, and run on the same kernels as the rest.
    """
    if not isinstance(model, nn.Module):
        raise TypeError("model must be a torch.nn.Module")
    for attribute in ("get_entry", "read_named_record"):
        if not callable(getattr(reader, attribute, None)):
            raise TypeError("reader must be a checkpoint reader (get_entry, read_named_record, model_metadata)")
    requested = _name_collection(include_names, "include_names")
    if not requested:
        raise ValueError("include_names must contain nonempty module names")
    if len(set(requested)) != len(requested):
        raise ValueError("include_names must be unique")
    if not isinstance(group_qkv, bool):
        raise TypeError("group_qkv must be a bool")
    if not isinstance(enable_m1_down_splitk, bool):
        raise TypeError("enable_m1_down_splitk must be a bool")
    tiled_names = frozenset(_name_collection(w4a4_tiled_fallback_names, "w4a4_tiled_fallback_names"))
    splitk_names = frozenset(_name_collection(m1_down_splitk_fallback_names, "m1_down_splitk_fallback_names"))
    wanted = set(requested)
    if not tiled_names <= wanted:
        raise ValueError("w4a4_tiled_fallback_names must be included in include_names")
    if not splitk_names <= wanted:
        raise ValueError("m1_down_splitk_fallback_names must be included in include_names")
    if splitk_names and not enable_m1_down_splitk:
        raise ValueError("m1_down_splitk_fallback_names requires enable_m1_down_splitk=True")
    if compute_backend not in _SERVED_BACKENDS:
        raise ValueError(f"unsupported fused NQRT compute_backend (this build serves {', '.join(_SERVED_BACKENDS)})")
    if not activation_betas:
        raise ValueError("packed_w4a4 requires activation_betas")

    modules = dict(model.named_modules())
    rotated = _rotated_module_names(getattr(reader, "model_metadata", None)) & wanted
    share_groups = _input_sharing_groups(rotated)
    qkv_groups: tuple[tuple[str, str, str], ...] = ()
    if group_qkv:
        parents = sorted({name.rpartition(".")[0] for name in rotated})
        complete = [tuple(f"{parent}.{leaf}_proj" for leaf in ("q", "k", "v")) for parent in parents]
        qkv_groups = tuple(group for group in complete if all(name in rotated for name in group))
        if tiled_names & {name for group in qkv_groups for name in group}:
            raise ValueError("w4a4_tiled_fallback_names cannot use grouped QKV replacement")

    staged = []
    for name in requested:  # validate everything first: a failure must leave the model untouched
        module = modules.get(name)
        if not isinstance(module, nn.Linear):
            raise ValueError(f"module is not a Linear: {name}")
        if module.bias is not None:
            raise ValueError(f"the packed W4A4 CUDA path requires bias=None: {name}")
        entry = reader.get_entry(f"{name}.weight")
        if getattr(entry, "kind", "nestquant") != "nestquant":
            raise ValueError(f"module weight is not packed: {name}")
        if tuple(module.weight.shape) != tuple(entry.shape):
            raise ValueError(f"quantized weight shape mismatch: {name}.weight")
        staged.append((name, module))

    caches = {}
    for group in share_groups:
        pair = (SharedHadamardCache(len(group)), SharedPackedActivationCache(len(group)))
        for name in group:
            caches[name] = pair
    built: dict[str, FusedNQRTLinear] = {}
    for name, module in staged:
        hcache, acache = caches.get(name, (None, None))
        fused = FusedNQRTLinear(
            reader, f"{name}.weight", None, input_hadamard=name in rotated, input_transform_cache=hcache,
            output_dtype=module.weight.dtype if output_dtype is None else output_dtype,
            compute_backend=compute_backend, activation_q=activation_q, activation_betas=tuple(activation_betas),
            packed_activation_cache=acache,
            enable_m1_down_splitk=enable_m1_down_splitk and name not in splitk_names)
        fused.to(device=module.weight.device)
        fused.train(module.training)
        built[name] = fused
    for group in qkv_groups:
        device = modules[group[0]].weight.device
        if device.type != "cuda":
            raise ValueError("group_qkv stacks the packed weights on the device: move the model to CUDA first")
        SharedProjectionGroup([built[name] for name in group], device=device)
    for name, _ in staged:
        parent_name, _, child_name = name.rpartition(".")
        setattr(model if not parent_name else modules[parent_name], child_name, built[name])
    return FusedNQRTConversionReport(
        replaced_linear_names=tuple(sorted(requested)), input_hadamard_names=tuple(sorted(rotated)),
        shared_hadamard_groups=share_groups, grouped_qkv_groups=qkv_groups,
        w4a4_tiled_fallback_names=tuple(sorted(tiled_names)),
        m1_down_splitk_fallback_names=tuple(sorted(splitk_names)))
