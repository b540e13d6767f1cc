"""The workspace-free small-M projection entry point, nq_w4a4_gemv_static.

Some hosts of this library may not allocate device memory at the point where they call a
projection: they own nothing but the input and output buffers they were handed, or they sit in a
decode loop where reaching cudaMalloc (which can stall the whole device) is not acceptable.  For
them the library carries its own fixed scratch array.  This test calls that entry point through
the C ABI twice in a row and checks both results against the regular entry point
(nq_w4a4_gemm with a caller-provided workspace) on the same packed operands -- bit for bit where
both entries run the same CUDA-core kernel (fewer than 8 rows), within the projection tolerance
where the regular entry takes its tensor-core path -- and against the CPU checker's product of the
BF16-rounded dequantised operands.  One more case runs the largest shape the built-in scratch
admits, where the split-K partial sums fill it to the last byte, with both output dtypes.

Collected last on purpose (file name), and valid both alone in a fresh process and after the
rest of the suite.
"""

import ctypes

import numpy as np
import pytest
import torch

from helpers import ACT_BETAS, MAX_ABS_TOL, REL_FRO_TOL, make_weight_record, max_abs, rel_fro, rng

pytestmark = pytest.mark.gpu

I64 = ctypes.c_int64


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _static(lib, act, weight, m, n, k, seed, out):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tag = 1 if out.dtype == torch.bfloat16 else 0  # NQ_BF16 / NQ_F32
    return lib.nq_w4a4_gemv_static(_p(act.code_payload), _p(act.beta_payload), _p(act.row_norms), _p(act.beta_table),
                                   _p(weight.code_payload), _p(weight.beta_payload), _p(weight.row_norms),
                                   _p(weight.beta_table), I64(m), I64(n), I64(k), I64(0), I64(seed), _p(out), tag, stream)


@pytest.mark.parametrize("m,n,k", [(1, 512, 2048), (3, 256, 8192), (16, 2048, 2048)])
def test_static_scratch_entry_matches_workspace_entry(oracle, m, n, k):
    import nestquant_aiinfra_b200 as nq
    import nestquant_aiinfra_b200.runtime as rt

    lib = nq.lib()
    seed = 4321 + m
    record, w_deq = make_weight_record(oracle, n, k, seed=77 + n, dither_seed=seed)
    weight = rt.prepare_fused_linear(record)
    results = []
    for call in range(2):  # two calls in a row share the built-in scratch
        x = torch.randn(m, k, generator=rng(100 * call + m)).bfloat16().cuda()
        act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
        expected = rt.linear_packed_w4a4_fp32(act, weight)
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        status = _static(lib, act, weight, m, n, k, seed, out)
        assert status == 0, lib.nq_last_error()
        torch.cuda.synchronize()
        a, e = out.cpu().numpy(), expected.cpu().numpy()
        assert np.isfinite(a).all()
        if m < 8:  # both entries ran the split-K CUDA-core kernel: same sums in the same order
            assert np.array_equal(a, e), (call, max_abs(a, e))
        else:      # the regular entry took the tcgen05 path: same operands, another order of the sums
            assert max_abs(a, e) <= MAX_ABS_TOL and rel_fro(a, e) <= REL_FRO_TOL, (call, max_abs(a, e), rel_fro(a, e))
        # and directly against the CPU checker
        codes, beta_ids, norms = (t.cpu().numpy() for t in (act.code_payload, act.beta_payload, act.row_norms))
        a_deq = oracle.dequantize_rows(codes, beta_ids, norms, ACT_BETAS, m, k)
        reference = oracle.gemm_bf16_operands(a_deq, w_deq)
        assert max_abs(a, reference) <= MAX_ABS_TOL and rel_fro(a, reference) <= REL_FRO_TOL, \
            (call, max_abs(a, reference), rel_fro(a, reference))
        results.append(a)
    assert not np.array_equal(results[0], results[1])  # different inputs really went through


def test_static_scratch_entry_at_its_largest_shape():
    """m = 16, n = k = 8192: the partial sums occupy the whole built-in scratch; float32 and bfloat16 outputs."""
    import nestquant_aiinfra_b200 as nq
    import nestquant_aiinfra_b200.runtime as rt
    from helpers import W_BETAS

    lib = nq.lib()
    m, n, k, seed = 16, 8192, 8192, 97531
    w = (0.02 * torch.randn(n, k, generator=rng(11))).cuda()
    weight = rt.quantize_weight_cuda(w, betas=W_BETAS, dither_seed=seed)  # bit-exact with the CPU encode (tested elsewhere)
    del w
    for call in range(2):
        x = torch.randn(m, k, generator=rng(500 + call)).bfloat16().cuda()
        act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS)
        expected = rt.linear_packed_w4a4_fp32(act, weight).cpu().numpy()
        out32 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        out16 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _static(lib, act, weight, m, n, k, seed, out32) == 0, lib.nq_last_error()
        assert _static(lib, act, weight, m, n, k, seed, out16) == 0, lib.nq_last_error()
        torch.cuda.synchronize()
        a = out32.cpu().numpy()
        assert np.isfinite(a).all()
        assert max_abs(a, expected) <= MAX_ABS_TOL and rel_fro(a, expected) <= REL_FRO_TOL, \
            (call, max_abs(a, expected), rel_fro(a, expected))
        # the bfloat16 output is the same sums rounded once at the store
        assert torch.equal(out16, out32.bfloat16())


def test_static_scratch_entry_rejects_oversized_shapes(oracle):
    import nestquant_aiinfra_b200 as nq
    import nestquant_aiinfra_b200.runtime as rt

    lib = nq.lib()
    record, _ = make_weight_record(oracle, 64, 256, seed=5, dither_seed=6)
    weight = rt.prepare_fused_linear(record)
    act = rt.quantize_activation_cuda(torch.randn(1, 256, generator=rng(1)).bfloat16().cuda(), q=14, betas=ACT_BETAS)
    out = torch.zeros(17, 64, dtype=torch.float32, device="cuda")
    assert _static(lib, act, weight, 17, 64, 256, 6, out) == -1          # m beyond the limit
    assert b"built-in scratch" in lib.nq_last_error()
    assert _static(lib, act, weight, 1, 16384, 256, 6, out) == -1        # n beyond the limit
    assert _static(lib, act, weight, 1, 64, 16384, 6, out) == -1         # k beyond the limit
