"""Tensor-parallel shards of the packed projection on the GPU.

Single-GPU tests run both shards on one device; the two-rank NCCL test needs two GPUs and
is skipped otherwise (NVLS off, plain peer paths)."""

import os
import socket

import numpy as np
import pytest
import torch

from helpers import ACT_BETAS, MAX_ABS_TOL, REL_FRO_TOL, W_BETAS, make_weight_record, max_abs, rel_fro, rng

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 7, 64])
def test_column_shards_equal_slices_of_the_unsharded_projection(oracle, m):
    import nestquant_aiinfra_b200.runtime as rt
    from nestquant_aiinfra_b200.tensor_parallel import shard_column_parallel

    n, k = 512, 1024
    record, _ = make_weight_record(oracle, n, k, seed=21, dither_seed=99)
    full = rt.prepare_fused_linear(record)
    x = torch.randn(m, k, generator=rng(m)).bfloat16().cuda()
    act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
    expected = rt.linear_packed_w4a4_fp32(act, full)
    for world in (2, 4):
        parts = [rt.linear_packed_w4a4_fp32(act, shard_column_parallel(full, r, world)) for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=1), expected)  # same dither counters, same bits
    shard = shard_column_parallel(full, 1, 2)
    assert shard.block_offset == 256 * (k // 8) and shard.rows == 256
    assert torch.equal(rt.decode_packed_weight(shard), rt.decode_packed_weight(full)[256:])


def test_row_parallel_shard_matches_checker_on_one_gpu(oracle):
    from nestquant_aiinfra_b200.tensor_parallel import RowParallelNQRTLinear, block_hadamard, shard_range

    n, k, m, world = 256, 7 * 512, 9, 1   # K = 3584 = 7 * 2^9: block-diagonal Hadamard with 512-wide blocks
    weight = 0.02 * torch.randn(n, k, generator=rng(1))
    x = torch.randn(m, k, generator=rng(2)).bfloat16()
    layer = RowParallelNQRTLinear(weight.cuda(), 0, world, dither_seed=77).cuda()
    assert layer.hadamard_block == 512
    with torch.no_grad():
        out = layer(x.cuda()).float().cpu().numpy()
    w_rot = block_hadamard(weight, 512).numpy()
    wc, wb, wn = oracle.encode_packed(w_rot, W_BETAS, seed=77)
    w_deq = oracle.dequantize_rows(wc, wb, wn, W_BETAS, n, k, seed=77)
    x_rot = np.concatenate([oracle.hadamard(x.float().numpy()[:, i:i + 512], round_bf16=True) for i in range(0, k, 512)], axis=1)
    ac, ab, an = oracle.encode_packed(x_rot, ACT_BETAS)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
    expected = oracle.gemm_bf16_operands(a_deq, w_deq)
    bar = MAX_ABS_TOL + float(np.abs(expected).max()) * 2 ** -8   # output is BF16
    assert max_abs(out, expected) <= bar and rel_fro(out, expected) <= 4e-3


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nestquant_aiinfra_b200.tensor_parallel import RowParallelNQRTLinear, shard_range

        n, k, m = 256, 2048, 6
        weight = 0.02 * torch.randn(n, k, generator=rng(5))
        x = torch.randn(m, k, generator=rng(6)).bfloat16()
        lo, hi = shard_range(k, world, rank, multiple=32)
        layer = RowParallelNQRTLinear(weight[:, lo:hi].contiguous().cuda(), rank, world, dither_seed=300 + rank).cuda()
        with torch.no_grad():
            out = layer(x[:, lo:hi].contiguous().cuda())
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), out.float().cpu().numpy())
        exact = (x.float() @ weight.T).numpy()
        rel = rel_fro(out.float().cpu().numpy(), exact)
        assert rel < 0.2, rel
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_parallel_all_reduce_two_nccl_ranks(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_nccl_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "rank0.npy"), np.load(tmp_path / "rank1.npy")
    assert np.array_equal(a, b)
