"""Generate the golden fixtures in this folder from the reference implementation.

Run where the reference project is importable::

    PYTHONPATH=/path/to/NestQuant-AIInfra python tests/golden/make_golden.py

Every array written here is an output of the reference's own CPU code
(``nestquant.core``) on seeded inputs; the inputs are stored next to the outputs
so the tests never need the reference at run time.  The fixtures pin the CPU
checker in ``oracle/`` and, through it, the CUDA kernels.
"""

from __future__ import annotations

import hashlib
import math
import sys
from pathlib import Path

import numpy as np
import torch

from nestquant.core.codec import decode_nested, generate_e8_dither_stateless
from nestquant.core.kv_format import PackedNQKVPage
from nestquant.core.lattice import nearest_e8
from nestquant.core.packing import pack_nestquant_indices
from nestquant.core.quantizer import quantize_rows
from nestquant.core.rotation import hadamard

HERE = Path(__file__).resolve().parent
ACT_BETAS = tuple(v / 14 for v in (3.47, 4.74, 6.90, 18.11))
W_BETAS = tuple(v / 14 for v in (4.0, 5.5, 7.0, 18.0))
KEY_BETAS = (0.25, 0.3271428571428571, 0.46214285714285713, 1.2185714285714284)
VALUE_BETAS = (0.2521428571428571, 0.3992857142857143, 0.687142857142857, 2.073571428571429)
UNIT_BETAS = (0.25, 0.5, 0.75, 1.0)


def rng(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def u8(payload: bytes) -> np.ndarray:
    return np.frombuffer(payload, dtype=np.uint8).copy()


def pack(q) -> tuple[np.ndarray, np.ndarray]:
    packed = pack_nestquant_indices(q.codes, q.beta_indices, q=14, beta_count=len(q.betas))
    return u8(packed.code_payload), u8(packed.beta_payload)


def main() -> None:
    torch.set_num_threads(max(1, torch.get_num_threads()))
    out: dict[str, np.ndarray] = {}

    # --- E8 nearest point: random points plus hand-made ties ------------------------
    x = torch.randn(2048, 8, generator=rng(11)) * 3.0
    half_grid = torch.randint(-6, 7, (1024, 8), generator=rng(12)).float() * 0.5
    quarter = torch.randint(-8, 9, (1024, 8), generator=rng(13)).float() * 0.25
    pts = torch.cat([x, half_grid, quarter, half_grid / 14.0 * 7.0])
    out["e8_in"] = pts.numpy()
    out["e8_out"] = nearest_e8(pts)[0].numpy()

    # --- stateless dither ----------------------------------------------------------
    seed = 20261029
    out["dither_seed"] = np.array([seed], dtype=np.int64)
    out["dither_blocks_0_64"] = generate_e8_dither_stateless(64, seed).numpy()
    out["dither_blocks_off"] = generate_e8_dither_stateless(32, 12345, block_offset=1_000_003).numpy()

    # --- decode_nested: the three boundary codewords + random codes -----------------
    boundary = torch.tensor([[5, 12, 3, 0, 7, 3, 9, 2], [5, 5, 2, 7, 2, 4, 10, 2],
                             [3, 0, 2, 12, 4, 9, 7, 2]])
    codes = torch.cat([boundary, torch.randint(0, 14, (4093, 8), generator=rng(21))])
    out["decode_codes"] = codes.numpy().astype(np.uint8)
    out["decode_out"] = decode_nested(codes, 14).numpy()

    # --- activation / KV style encodes (no dither) ------------------------------------
    cases = {
        "a4_2048": (hadamard(torch.randn(8, 2048, generator=rng(2000))), ACT_BETAS),
        "a4_8192_bf16": (hadamard(torch.randn(4, 8192, generator=rng(2001)).bfloat16()).float(), ACT_BETAS),
        "kv_64_bf16": (torch.randn(64, 64, generator=rng(2002)).bfloat16().float(), KEY_BETAS),
        "kv_128_bf16": (torch.randn(32, 128, generator=rng(2003)).bfloat16().float() * 3.0, VALUE_BETAS),
        "unit_betas_256": (torch.randn(16, 256, generator=rng(2004)), UNIT_BETAS),
    }
    zero_row = torch.randn(4, 64, generator=rng(2005))
    zero_row[2] = 0.0
    cases["zero_row_64"] = (zero_row, KEY_BETAS)
    # Half-integer multiples of beta on a normalised row: dense E8 / beta ties.
    for name, (matrix, betas) in cases.items():
        q = quantize_rows(matrix, 14, betas)
        cp, bp = pack(q)
        out[f"{name}_x"] = matrix.numpy()
        out[f"{name}_betas"] = np.array(betas, dtype=np.float64)
        out[f"{name}_codes"] = cp
        out[f"{name}_beta_ids"] = bp
        out[f"{name}_norms"] = q.row_norms.numpy()
        out[f"{name}_dequant"] = q.dequantize().numpy()

    # --- weight encode with stateless dither -------------------------------------------
    w = hadamard(0.02 * torch.randn(96, 512, generator=rng(1000)))
    d = generate_e8_dither_stateless(96 * 64, seed).reshape(96, 64, 8)
    qw = quantize_rows(w, 14, W_BETAS, dither=d)
    cp, bp = pack(qw)
    out["w_x"] = w.numpy()
    out["w_codes"], out["w_beta_ids"] = cp, bp
    out["w_norms"] = qw.row_norms.numpy()
    out["w_dequant"] = qw.dequantize().numpy()
    out["w_overloaded_fraction"] = np.array([qw.overloaded.float().mean().item()])

    # --- config-0 style product on a small shape -------------------------------------------
    a = hadamard(torch.randn(6, 512, generator=rng(2000)))
    qa = quantize_rows(a, 14, ACT_BETAS)
    out["y_a_x"] = a.numpy()
    out["y"] = (qa.dequantize() @ qw.dequantize().T).numpy()

    # --- NQKV v2 page ----------------------------------------------------------------
    for tag, (valid, heads, dim) in {"page_11x8x64": (11, 8, 64), "page_16x2x128": (16, 2, 128)}.items():
        k = torch.randn(valid, heads, dim, generator=rng(3000 + valid)).bfloat16()
        v = torch.randn(valid, heads, dim, generator=rng(3100 + valid)).bfloat16()
        k[:, 1, 5] *= 8.0
        page = PackedNQKVPage.from_tensors(k, v, page_size=16, q=14, key_betas=KEY_BETAS,
                                           value_betas=VALUE_BETAS)
        dk, dv = page.dequantize(output_dtype=torch.float32)
        out[f"{tag}_key"] = k.float().numpy()
        out[f"{tag}_value"] = v.float().numpy()
        out[f"{tag}_k_codes"] = u8(page.key_indices.code_payload)
        out[f"{tag}_k_beta"] = u8(page.key_indices.beta_payload)
        out[f"{tag}_k_norms"] = page.key_norms.numpy()
        out[f"{tag}_v_codes"] = u8(page.value_indices.code_payload)
        out[f"{tag}_v_beta"] = u8(page.value_indices.beta_payload)
        out[f"{tag}_v_norms"] = page.value_norms.numpy()
        out[f"{tag}_dk"] = dk.numpy()
        out[f"{tag}_dv"] = dv.numpy()
        out[f"{tag}_payload_bytes"] = np.array([page.payload_bytes])

    # --- Hadamard ----------------------------------------------------------------------
    h32 = torch.randn(3, 2048, generator=rng(4000))
    hb = torch.randn(3, 2048, generator=rng(4001)).bfloat16()
    h64 = torch.randn(5, 64, generator=rng(4002))
    out["had_f32_in"], out["had_f32_out"] = h32.numpy(), hadamard(h32).numpy()
    out["had_bf16_in"], out["had_bf16_out"] = hb.float().numpy(), hadamard(hb).float().numpy()
    out["had_64_in"], out["had_64_out"] = h64.numpy(), hadamard(h64).numpy()

    # --- full-size config-0 digests (inputs are regenerated from the seed by the tests) ----
    a0 = hadamard(torch.randn(16, 2048, generator=rng(2000)))
    qa0 = quantize_rows(a0, 14, ACT_BETAS)
    cp0, bp0 = pack(qa0)
    out["cfg0_a_code_sha256"] = u8(hashlib.sha256(cp0.tobytes()).digest())
    out["cfg0_a_beta_sha256"] = u8(hashlib.sha256(bp0.tobytes()).digest())
    out["cfg0_a_norms"] = qa0.row_norms.numpy()
    out["cfg0_a_x"] = a0.numpy()

    np.savez_compressed(HERE / "reference_vectors.npz", **out)
    total = sum(v.nbytes for v in out.values())
    print(f"wrote {len(out)} arrays, {total/1e6:.2f} MB raw -> {HERE / 'reference_vectors.npz'}")
    print("torch", torch.__version__, "threads", torch.get_num_threads(), "python", sys.version.split()[0])
    print("sqrt(2048) check", math.sqrt(2048))


if __name__ == "__main__":
    main()
