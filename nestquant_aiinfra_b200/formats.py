"""Wire-format records of the packed W4A4KV4 path (host side, no arithmetic).

Field names follow the reference so its objects can be passed in unchanged
(duck typing): ``PackedNestQuantIndices`` is NQPK v1 (core/packing.py:24-134),
``PackedNestQuantTensor`` is the NQRT v4 weight record
(core/tensor_checkpoint.py:41-118).  Only the fields the hot path reads exist.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass

import torch

UPSTREAM_CODEC_SEMANTICS = "e8_upstream_half_coset_tie_v1"
STATELESS_DITHER_ALGORITHM = "lcg31_mix_v1"

ACTIVATION_BETAS = tuple(v / 14 for v in (3.47, 4.74, 6.90, 18.11))
WEIGHT_BETAS = tuple(v / 14 for v in (4.0, 5.5, 7.0, 18.0))
KEY_BETAS = (0.25, 0.3271428571428571, 0.46214285714285713, 1.2185714285714284)
VALUE_BETAS = (0.2521428571428571, 0.3992857142857143, 0.687142857142857, 2.073571428571429)


def _bits(cardinality: int) -> int:
    return max(1, (cardinality - 1).bit_length())


@dataclass(frozen=True)
class PackedNestQuantIndices:
    """Packed residue and beta-index byte streams of one tensor."""

    shape: tuple[int, ...]
    q: int
    beta_count: int
    code_payload: bytes
    beta_payload: bytes

    @property
    def code_bit_width(self) -> int:
        return _bits(self.q)

    @property
    def beta_index_bit_width(self) -> int:
        return _bits(self.beta_count)


@dataclass(frozen=True)
class PackedNestQuantTensor:
    """One NQRT v4 weight: packed indices, row norms, beta table, dither seed."""

    tensor_name: str
    indices: PackedNestQuantIndices
    row_norms: torch.Tensor
    betas: tuple[float, ...]
    feature_count: int
    output_dtype: torch.dtype = torch.float32
    dither_seed: int | None = None
    dither_algorithm: str | None = STATELESS_DITHER_ALGORITHM
    codec_semantics: str = UPSTREAM_CODEC_SEMANTICS

    @property
    def packed_bytes(self) -> int:
        return (len(self.indices.code_payload) + len(self.indices.beta_payload)
                + 4 * self.row_norms.numel() + 4 * len(self.betas))


def tensor_dither_seed(project_seed: int, tensor_name: str) -> int:
    """Per-tensor stateless dither seed (models/quantization.py:382-384)."""
    payload = f"nqrt-v4\0{project_seed}\0{tensor_name}".encode("utf-8")
    return int.from_bytes(hashlib.sha256(payload).digest()[:4], "little") % (2 ** 31)
