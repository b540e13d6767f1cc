"""The workspace-free small-M projection entry point, nq_w4a4_gemv_static.

Some hosts of this library may not allocate device memory at the point where they call a
projection: they own nothing but the input and output buffers they were handed, or they sit in a
decode loop where reaching cudaMalloc (which can stall the whole device) is not acceptable.  For
them the library carries its own fixed scratch array.  This test calls that entry point through
the C ABI twice in a row and checks both results against the regular entry point
(nq_w4a4_gemm with a caller-provided workspace) on the same packed operands.

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
    return lib.nq_w4a4_gemv_static(_p(act.code_payload), _p(act.beta_payload), _p(act.row_norms), _p(act.beta_table),
                                   _p(weight.code_payload), _p(weight.beta_payload), _p(weight.row_norms),
                                   _p(weight.beta_table), I64(m), I64(n), I64(k), I64(0), I64(seed), _p(out), 0, stream)


@pytest.mark.parametrize("m,n,k", [(1, 512, 2048), (3, 256, 8192), (16, 2048, 2048)])
def test_static_scratch_entry_matches_workspace_entry(oracle, m, n, k):
    import nestquant_aiinfra_b200 as nq
    import nestquant_aiinfra_b200.runtime as rt

    lib = nq.lib()
    seed = 4321 + m
    record, _ = make_weight_record(oracle, n, k, seed=77 + n, dither_seed=seed)
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
        assert max_abs(a, e) <= MAX_ABS_TOL and rel_fro(a, e) <= REL_FRO_TOL, (call, max_abs(a, e), rel_fro(a, e))
        results.append(a)
    assert not np.array_equal(results[0], results[1])  # different inputs really went through


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
