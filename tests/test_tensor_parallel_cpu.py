"""Host logic of the tensor-parallel sharding, exercised with two gloo ranks on the CPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nestquant_aiinfra_b200.tensor_parallel import (RowParallelNQRTLinear, block_hadamard,
                                                      largest_power_of_two_divisor, shard_range)


def test_shard_ranges_and_errors():
    assert shard_range(8192, 8, 3) == (3072, 4096)
    assert [shard_range(64, 4, r, multiple=8) for r in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        shard_range(100, 8, 0)
    with pytest.raises(ValueError):
        shard_range(64, 4, 4)
    assert [largest_power_of_two_divisor(28672 // tp) for tp in (1, 2, 4, 8)] == [4096, 2048, 1024, 512]
    assert [largest_power_of_two_divisor(8192 // tp) for tp in (2, 4, 8)] == [4096, 2048, 1024]


def test_block_hadamard_is_block_diagonal_and_orthogonal():
    x = torch.randn(3, 3584)  # 7 * 512: the 70B down_proj shard at tp = 8
    y = block_hadamard(x, 512)
    assert torch.allclose(block_hadamard(y, 512), x, atol=1e-5)      # H is its own inverse
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    z = x.clone()
    z[:, 512:] = 0
    assert torch.count_nonzero(block_hadamard(z, 512)[:, 512:]) == 0  # blocks do not mix
    with pytest.raises(ValueError):
        block_hadamard(x, 1024)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _row_parallel_worker(rank: int, world: int, port: int, result_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import nq_oracle as oracle

        gen = torch.Generator().manual_seed(0)  # same stream on every rank
        n, k, m = 64, 1024, 5
        weight = 0.02 * torch.randn(n, k, generator=gen)
        x = torch.randn(m, k, generator=gen)
        lo, hi = shard_range(k, world, rank, multiple=32)
        w_slice, x_slice = weight[:, lo:hi].contiguous(), x[:, lo:hi].contiguous()
        block = largest_power_of_two_divisor(hi - lo)
        w_rot = block_hadamard(w_slice, block).numpy()
        wc, wb, wn = oracle.encode_packed(w_rot, oracle.WEIGHT_BETAS, seed=100 + rank)
        w_deq = oracle.dequantize_rows(wc, wb, wn, oracle.WEIGHT_BETAS, n, hi - lo, seed=100 + rank)

        def project(x_shard: torch.Tensor) -> torch.Tensor:  # CPU stand-in of the packed projection of this shard
            rotated = block_hadamard(x_shard, block).numpy()
            ac, ab, an = oracle.encode_packed(rotated, oracle.ACTIVATION_BETAS)
            a_deq = oracle.dequantize_rows(ac, ab, an, oracle.ACTIVATION_BETAS, m, hi - lo)
            return torch.from_numpy(oracle.gemm_f32(a_deq, w_deq))

        layer = RowParallelNQRTLinear(w_slice, rank, world, dither_seed=100 + rank, project=project)
        assert layer.hadamard_block == block
        out = layer(x_slice)
        np.save(os.path.join(result_dir, f"rank{rank}.npy"), out.numpy())
        # end to end: the reduced output is the sum over ALL ranks of the products of their dequantised shards,
        # recomputed here from scratch for every shard (max abs <= 1e-2, relative Frobenius <= 1e-3)
        expected = np.zeros((m, n), dtype=np.float64)
        for r in range(world):
            r_lo, r_hi = shard_range(k, world, r, multiple=32)
            r_block = largest_power_of_two_divisor(r_hi - r_lo)
            rw = block_hadamard(weight[:, r_lo:r_hi].contiguous(), r_block).numpy()
            c, b, nrm = oracle.encode_packed(rw, oracle.WEIGHT_BETAS, seed=100 + r)
            rw_deq = oracle.dequantize_rows(c, b, nrm, oracle.WEIGHT_BETAS, n, r_hi - r_lo, seed=100 + r)
            rx = block_hadamard(x[:, r_lo:r_hi].contiguous(), r_block).numpy()
            c, b, nrm = oracle.encode_packed(rx, oracle.ACTIVATION_BETAS)
            rx_deq = oracle.dequantize_rows(c, b, nrm, oracle.ACTIVATION_BETAS, m, r_hi - r_lo)
            expected += oracle.gemm_f32(rx_deq, rw_deq).astype(np.float64)
        actual = out.numpy().astype(np.float64)
        assert float(np.abs(actual - expected).max()) <= 1e-2
        assert float(np.linalg.norm(actual - expected) / np.linalg.norm(expected)) <= 1e-3
        exact = x @ weight.T
        rel = float((out - exact).norm() / exact.norm())
        assert rel < 0.2, rel  # W4A4 quantisation noise of two independent shards (information, not the parity bar)
    finally:
        dist.destroy_process_group()


def test_row_parallel_all_reduce_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_row_parallel_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "rank0.npy"), np.load(tmp_path / "rank1.npy")
    assert np.array_equal(a, b)  # every rank holds the same reduced output
