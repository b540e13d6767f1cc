"""Seeded synthetic inputs and error metrics shared by the CPU and GPU tests."""

from __future__ import annotations

import numpy as np
import torch

KEY_BETAS = (0.25, 0.3271428571428571, 0.46214285714285713, 1.2185714285714284)
VALUE_BETAS = (0.2521428571428571, 0.3992857142857143, 0.687142857142857, 2.073571428571429)
ACT_BETAS = tuple(v / 14 for v in (3.47, 4.74, 6.90, 18.11))
W_BETAS = tuple(v / 14 for v in (4.0, 5.5, 7.0, 18.0))
UNIT_BETAS = (0.25, 0.5, 0.75, 1.0)

# Projection / attention parity bar: max abs <= 1e-2 and relative Frobenius <= 1e-3
# against the BF16-operand product accumulated in float64.
MAX_ABS_TOL = 1e-2
REL_FRO_TOL = 1e-3


def rng(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def rel_fro(actual: np.ndarray, expected: np.ndarray) -> float:
    denom = float(np.linalg.norm(expected.astype(np.float64)))
    return float(np.linalg.norm(actual.astype(np.float64) - expected.astype(np.float64))) / max(denom, 1e-30)


def max_abs(actual: np.ndarray, expected: np.ndarray) -> float:
    return float(np.abs(actual.astype(np.float64) - expected.astype(np.float64)).max())


def make_weight_record(oracle, n: int, k: int, *, seed: int, dither_seed: int, betas=W_BETAS, std: float = 0.02,
                       rotate: bool = True):
    """Encode a seeded synthetic weight with the CPU checker -> (record, dequantized f32 [n,k])."""
    from nestquant_aiinfra_b200.formats import PackedNestQuantIndices, PackedNestQuantTensor

    w = (std * torch.randn(n, k, generator=rng(seed))).numpy()
    if rotate:
        w = oracle.hadamard(w)
    codes, beta_ids, norms = oracle.encode_packed(w, betas, seed=dither_seed)
    deq = oracle.dequantize_rows(codes, beta_ids, norms, betas, n, k, seed=dither_seed)
    record = PackedNestQuantTensor(
        tensor_name=f"w{seed}",
        indices=PackedNestQuantIndices((n, k // 8, 8), 14, 4, codes.tobytes(), beta_ids.tobytes()),
        row_norms=torch.from_numpy(norms.copy()), betas=tuple(betas), feature_count=k,
        dither_seed=dither_seed)
    return record, deq
