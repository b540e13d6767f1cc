"""``FusedNQRTLinear``: the module-level plugin boundary of the packed W4A4 projection.

Mirror of ``nestquant.models.fused_linear`` (FusedNQRTLinear :130-421,
SharedHadamardCache :49-84, SharedPackedActivationCache :87-127,
convert_linears_to_fused_nqrt_ :543-695) restricted to the served backend
``compute_backend="packed_w4a4_cuda_mma"``: Hadamard on the input when asked,
one on-the-fly A4 encode (shared between projections that receive the same
input tensor object), one packed projection call, cast to the output dtype.
"""

from __future__ import annotations

from typing import Any, Iterable

import torch
from torch import nn

from .rotation import hadamard
from .runtime.w4a4 import (PreparedNQA4Activation, PreparedNQRTLinear, linear_packed_w4a4, linear_packed_w4a4_fp32,
                           prepare_fused_linear,
                           quantize_activation_cuda, can_rotate_in_encoder, prefer_rotation_in_encoder,
                           group_prepared_linears, keep_decoded_weight)

_BACKENDS = {"packed_w4a4_cuda_mma", "packed_w4a4_cuda_gemv_m1", "packed_w4a4"}


class SharedHadamardCache:
    """Reuse one inference-only Hadamard result for modules sharing an input."""

    def __init__(self, uses_per_input: int) -> None:
        if isinstance(uses_per_input, bool) or not isinstance(uses_per_input, int):
            raise TypeError("uses_per_input must be an integer")
        if uses_per_input < 2:
            raise ValueError("uses_per_input must be at least two")
        self.uses_per_input = uses_per_input
        self._input = None
        self._output = None
        self._remaining = 0
        self.hits = 0
        self.misses = 0

    def transform(self, inputs: torch.Tensor) -> torch.Tensor:
        if torch.is_grad_enabled():
            raise RuntimeError("shared Hadamard caching requires inference or no-grad mode")
        if self._input is inputs and self._output is not None:
            self.hits += 1
            output = self._output
            self._remaining -= 1
            if self._remaining == 0:
                self.clear()
            return output
        output = hadamard(inputs)
        self._input, self._output = inputs, output
        self._remaining = self.uses_per_input - 1
        self.misses += 1
        return output

    def note_rotation_in_encoder(self, inputs: torch.Tensor) -> None:
        """Same hit / miss accounting as ``transform`` when the encoder launch does the rotation itself."""
        if torch.is_grad_enabled():
            raise RuntimeError("shared Hadamard caching requires inference or no-grad mode")
        if self._input is inputs and self._remaining > 0:
            self.hits += 1
            self._remaining -= 1
            if self._remaining == 0:
                self.clear()
            return
        self._input, self._output = inputs, None
        self._remaining = self.uses_per_input - 1
        self.misses += 1

    def clear(self) -> None:
        self._input = self._output = None
        self._remaining = 0


class SharedPackedActivationCache:
    """Reuse one packed A4 encoding for projections sharing an input tensor (by identity)."""

    def __init__(self, uses_per_input: int) -> None:
        if isinstance(uses_per_input, bool) or not isinstance(uses_per_input, int):
            raise TypeError("uses_per_input must be an integer")
        if uses_per_input < 2:
            raise ValueError("uses_per_input must be at least two")
        self.uses_per_input = uses_per_input
        self._input = None
        self._packed: PreparedNQA4Activation | None = None
        self._remaining = 0
        self.hits = 0
        self.misses = 0

    def encode(self, inputs: torch.Tensor, *, q: int, betas: tuple[float, ...],
               beta_table: torch.Tensor | None = None,
               hadamard_block: int | None = None) -> tuple[PreparedNQA4Activation, bool]:
        if torch.is_grad_enabled():
            raise RuntimeError("shared A4 caching requires inference or no-grad mode")
        if self._input is inputs and self._packed is not None:
            self.hits += 1
            packed = self._packed
            self._remaining -= 1
            if self._remaining == 0:
                self.clear()
            return packed, False
        packed = quantize_activation_cuda(inputs, q=q, betas=betas, beta_table=beta_table,
                                          hadamard_block=hadamard_block, keep_decoded=True)
        self._input, self._packed = inputs, packed
        self._remaining = self.uses_per_input - 1
        self.misses += 1
        return packed, True

    def clear(self) -> None:
        self._input = self._packed = None
        self._remaining = 0


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

    def keep_decoded_weight(self) -> int:
        """Keep the BF16 reconstruction of the stacked weight in device memory (opt-in, see
        ``runtime.keep_decoded_weight``); returns the bytes this adds."""
        self.stacked = keep_decoded_weight(self.stacked, self.views)
        return self.stacked.decoded.numel() * 2

    def project(self, packed: PreparedNQA4Activation, index: int) -> torch.Tensor:
        if self._packed is not packed or self._output is None:
            self._output = linear_packed_w4a4(packed, self.stacked)
            self._packed = packed
            self._remaining = len(self.bounds)
            self.launches += 1
        start, end = self.bounds[index]
        output = self._output[..., start:end]
        if packed.token_count >= 512:
            # many rows: tensor ops on a column slice fall off their vectorised kernels, a copy is cheaper
            output = output.contiguous()
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

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if not isinstance(inputs, torch.Tensor) or not inputs.is_floating_point():
            raise TypeError("inputs must be a floating-point tensor")
        if inputs.ndim == 0 or inputs.shape[-1] != self.in_features:
            actual = None if inputs.ndim == 0 else inputs.shape[-1]
            raise ValueError(f"input feature dimension {actual} does not match {self.in_features}")
        if inputs.device.type != "cuda":
            raise ValueError("FusedNQRTLinear requires CUDA inputs")
        original_dtype = inputs.dtype
        # The rotation of the input runs inside the encoder launch when the sizes allow it
        # (bit-identical to hadamard() followed by the encoder); otherwise as its own launch.
        wanted_block = self.in_features if self.input_hadamard else self.input_rotation_block
        rotate_in_encoder = (wanted_block is not None
                             and inputs.dtype in (torch.bfloat16, torch.float16, torch.float32)
                             and can_rotate_in_encoder(self.in_features, wanted_block)
                             and prefer_rotation_in_encoder(inputs.numel() // self.in_features, self.in_features))
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
        prepared = self._prepared_for(inputs.device)
        beta_table = self.activation_beta_table
        if beta_table.device != inputs.device:
            beta_table = beta_table.to(inputs.device)
        if self.packed_activation_cache is None:
            packed = quantize_activation_cuda(compute_inputs, q=self.activation_q, betas=self.activation_betas,
                                              beta_table=beta_table, hadamard_block=block, keep_decoded=True)
            encoded = True
        else:
            packed, encoded = self.packed_activation_cache.encode(
                compute_inputs, q=self.activation_q, betas=self.activation_betas, beta_table=beta_table,
                hadamard_block=block)
        self.a4_call_count += 1
        self.a4_encode_count += int(encoded)
        if self._group is not None:
            outputs = self._group.project(packed, self._group_index)
        elif self.output_dtype == torch.float32:
            outputs = linear_packed_w4a4_fp32(packed, prepared)  # the accumulator itself, not rounded to the input dtype first
        else:
            outputs = linear_packed_w4a4(packed, prepared)
        self.w4a4_cuda_mma_dispatch_count += 1
        return outputs.to(self.output_dtype or original_dtype)


def keep_decoded_weights_(model: nn.Module, device: torch.device | str | None = None) -> int:
    """Switch every ``FusedNQRTLinear`` of ``model`` to resident decoded weights; returns the bytes added.

    An explicit trade for machines with HBM to spare: 4x the packed weight bytes stay resident and
    no projection regenerates dither or searches E8 for its weight again.  The reference has no
    such mode (its modules never hold a BF16 matrix).
    """
    return sum(module.keep_decoded_weight(device) for module in model.modules()
               if isinstance(module, FusedNQRTLinear))


def convert_linears_to_fused_nqrt_(model: nn.Module, reader: Any, names: Iterable[str], *,
                                   compute_backend: str = "packed_w4a4_cuda_mma", activation_q: int = 14,
                                   activation_betas: tuple[float, ...] | None = None,
                                   input_hadamard_names: Iterable[str] | None = None,
                                   share_groups: Iterable[Iterable[str]] = (),
                                   enable_m1_down_splitk: bool = False, **_ignored) -> dict[str, int]:
    """Replace ``nn.Linear`` children named in ``names`` (``...proj.weight``) by packed modules.

    ``share_groups`` lists module names that receive the same input tensor (q/k/v, gate/up):
    they share one Hadamard and one A4 encode per forward, as the reference does
    (models/fused_linear.py:616-627).
    """
    wanted = {name[:-len(".weight")] if name.endswith(".weight") else name for name in names}
    hadamard_names = wanted if input_hadamard_names is None else {
        n[:-len(".weight")] if n.endswith(".weight") else n for n in input_hadamard_names}
    caches: dict[str, tuple[SharedHadamardCache, SharedPackedActivationCache]] = {}
    for group in share_groups:
        members = [m for m in group if m in wanted]
        if len(members) >= 2:
            pair = (SharedHadamardCache(len(members)), SharedPackedActivationCache(len(members)))
            for member in members:
                caches[member] = pair
    converted = 0
    for module_name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{module_name}.{child_name}" if module_name else child_name
            if full not in wanted or not isinstance(child, nn.Linear):
                continue
            had = full in hadamard_names
            hcache, acache = caches.get(full, (None, None))
            fused = FusedNQRTLinear(reader, full + ".weight", None, input_hadamard=had,
                                    input_transform_cache=hcache if had else None,
                                    compute_backend=compute_backend, activation_q=activation_q,
                                    activation_betas=activation_betas, packed_activation_cache=acache,
                                    enable_m1_down_splitk=enable_m1_down_splitk)
            setattr(module, child_name, fused)
            converted += 1
    return {"converted": converted, "requested": len(wanted)}
