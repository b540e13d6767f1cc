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
    layer = RowParallelNQRTLinear(weight.cuda(), 0, world, dither_seed=77, reduce_dtype=torch.float32).cuda()
    assert layer.hadamard_block == 512
    with torch.no_grad():
        out = layer(x.cuda())
    assert out.dtype == torch.float32   # the FP32 accumulator, as the other projection tests compare
    out = out.cpu().numpy()
    w_rot = block_hadamard(weight, 512).numpy()
    wc, wb, wn = oracle.encode_packed(w_rot, W_BETAS, seed=77)
    w_deq = oracle.dequantize_rows(wc, wb, wn, W_BETAS, n, k, seed=77)
    x_rot = np.concatenate([oracle.hadamard(x.float().numpy()[:, i:i + 512], round_bf16=True) for i in range(0, k, 512)], axis=1)
    ac, ab, an = oracle.encode_packed(x_rot, ACT_BETAS)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, k)
    expected = oracle.gemm_bf16_operands(a_deq, w_deq)
    assert max_abs(out, expected) <= MAX_ABS_TOL and rel_fro(out, expected) <= REL_FRO_TOL


def test_rank_encoded_rows_equal_the_row_range_of_the_unsharded_record():
    """A rank that encodes only its output rows (block_offset = first_row * K / 8) gets the bytes of the full encode."""
    import nestquant_aiinfra_b200.runtime as rt
    from nestquant_aiinfra_b200.tensor_parallel import shard_column_parallel

    n, k, world = 256, 1024, 4
    w = (0.02 * torch.randn(n, k, generator=rng(31))).cuda()
    full = rt.quantize_weight_cuda(w, betas=W_BETAS, dither_seed=4242)
    for rank in range(world):
        lo, hi = n // world * rank, n // world * (rank + 1)
        own = rt.quantize_weight_cuda(w[lo:hi].contiguous(), betas=W_BETAS, dither_seed=4242, block_offset=lo * (k // 8))
        view = shard_column_parallel(full, rank, world)
        assert own.block_offset == view.block_offset and own.rows == view.rows
        assert torch.equal(own.code_payload, view.code_payload) and torch.equal(own.beta_payload, view.beta_payload)
        assert torch.equal(own.row_norms, view.row_norms)
        assert torch.equal(rt.decode_packed_weight(own), rt.decode_packed_weight(full)[lo:hi])


def shard_product(oracle, weight, x, lo, hi, seed):
    """CPU checker's product of one self-contained K shard: block-rotated, encoded, dequantised, BF16 operands."""
    from nestquant_aiinfra_b200.tensor_parallel import block_hadamard, largest_power_of_two_divisor

    block = largest_power_of_two_divisor(hi - lo)
    n, m = weight.shape[0], x.shape[0]
    w_rot = block_hadamard(weight[:, lo:hi].contiguous(), block).numpy()
    wc, wb, wn = oracle.encode_packed(w_rot, W_BETAS, seed=seed)
    w_deq = oracle.dequantize_rows(wc, wb, wn, W_BETAS, n, hi - lo, seed=seed)
    xs = x[:, lo:hi].float().numpy()
    x_rot = np.concatenate([oracle.hadamard(xs[:, i:i + block], round_bf16=True) for i in range(0, hi - lo, block)], axis=1)
    ac, ab, an = oracle.encode_packed(x_rot, ACT_BETAS)
    a_deq = oracle.dequantize_rows(ac, ab, an, ACT_BETAS, m, hi - lo)
    return oracle.gemm_bf16_operands(a_deq, w_deq).astype(np.float64)


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
        layer = RowParallelNQRTLinear(weight[:, lo:hi].contiguous().cuda(), rank, world, dither_seed=300 + rank,
                                      reduce_dtype=torch.float32).cuda()
        with torch.no_grad():
            out = layer(x[:, lo:hi].contiguous().cuda())
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), out.cpu().numpy())
        # end to end: the reduced output against the sum of the checker's products of the dequantised shards
        from oracle import nq_oracle as oracle

        expected = sum(shard_product(oracle, weight, x, *shard_range(k, world, r, multiple=32), 300 + r)
                       for r in range(world))
        actual = out.cpu().numpy()
        assert max_abs(actual, expected) <= MAX_ABS_TOL and rel_fro(actual, expected) <= REL_FRO_TOL, \
            (max_abs(actual, expected), rel_fro(actual, expected))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_parallel_all_reduce_two_nccl_ranks(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_nccl_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "rank0.npy"), np.load(tmp_path / "rank1.npy")
    assert np.array_equal(a, b)


def _peer_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from nestquant_aiinfra_b200.tensor_parallel import PeerAllReduce, RowParallelNQRTLinear, shard_range

        reducer = PeerAllReduce(128 * 1024, device)
        # plain tensors, several calls in a row, sizes that change: every call sums what the ranks hold
        results = []
        for call, count in enumerate((64, 4096, 128 * 1024, 4096)):
            mine = torch.randn(count, generator=rng(100 * call + rank)).bfloat16().to(device)
            total = sum(torch.randn(count, generator=rng(100 * call + r)).bfloat16().float() for r in range(world))
            out = reducer.reduce(mine)
            assert torch.equal(out.cpu(), total.bfloat16())  # float32 sum in rank order, one rounding
            results.append(out)
        # the same calls replayed from a CUDA graph: the call number lives in device memory
        static = torch.randn(4096, generator=rng(900 + rank)).bfloat16().to(device)
        expected = sum(torch.randn(4096, generator=rng(900 + r)).bfloat16().float() for r in range(world)).bfloat16()
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            reducer.reduce(static)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                first = reducer.reduce(static)
                second = reducer.reduce(first)  # two dependent collectives inside one graph
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(device)
        assert torch.equal(first.cpu(), expected)
        assert torch.equal(second.cpu(), (expected.float() * world).bfloat16())
        assert reducer.status() == 0
        # the row-parallel projection with the peer collective: same gate as with NCCL
        n, k, m = 256, 2048, 8
        weight = 0.02 * torch.randn(n, k, generator=rng(5))
        x = torch.randn(m, k, generator=rng(6)).bfloat16()
        lo, hi = shard_range(k, world, rank, multiple=32)
        layer = RowParallelNQRTLinear(weight[:, lo:hi].contiguous().cuda(), rank, world, dither_seed=300 + rank).cuda()
        layer.peer_all_reduce = reducer
        with torch.no_grad():
            out = layer(x[:, lo:hi].contiguous().cuda())
        torch.cuda.synchronize()
        assert out.dtype == torch.bfloat16 and reducer.status() == 0
        np.save(os.path.join(out_dir, f"peer{rank}.npy"), out.float().cpu().numpy())
        from oracle import nq_oracle as oracle

        expected = sum(shard_product(oracle, weight, x, *shard_range(k, world, r, multiple=32), 300 + r)
                       for r in range(world))
        actual = out.float().cpu().numpy()
        # BF16 partials and a BF16 result: the stated gates plus the rounding of the output dtype
        assert max_abs(actual, expected) <= MAX_ABS_TOL + 2.0 ** -8 * np.abs(expected).max()
        assert rel_fro(actual, expected) <= 4e-3
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_peer_memory_all_reduce(tmp_path, world):
    """nq_tp_allreduce_bf16 over symmetric memory: exact sums, graph replay, and the projection end to end
    (two ranks: the one-shot kernel; four ranks: the two-shot kernel)."""
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outputs = [np.load(tmp_path / f"peer{r}.npy") for r in range(world)]
    assert all(np.array_equal(outputs[0], other) for other in outputs[1:])
