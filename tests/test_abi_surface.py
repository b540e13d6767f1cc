"""The C-ABI library builds, loads and exports every symbol the public header declares."""

import pytest


def test_library_builds_and_exports_declared_symbols():
    import nestquant_aiinfra_b200 as nq
    from nestquant_aiinfra_b200 import _lib

    nq.build_library()
    library = nq.lib()
    names = _lib.declared_symbols()
    assert "nq_a4_encode" in names and "nq_w4a4_gemm" in names
    missing = [name for name in names if not hasattr(library, name)]
    assert not missing, missing
    assert library.nq_abi_version() == 1


def test_argument_errors_do_not_need_a_gpu():
    import ctypes

    import nestquant_aiinfra_b200 as nq

    library = nq.lib()
    status = library.nq_a4_encode(None, 1, ctypes.c_int64(1), ctypes.c_int64(64), ctypes.c_int64(64),
                                  None, None, None, None, None, None)
    assert status == -1 and b"null" in library.nq_last_error()
    assert library.nq_w4a4_workspace_bytes(ctypes.c_int64(1), ctypes.c_int64(2048), ctypes.c_int64(2048)) >= 65536


def test_operators_reject_cpu_tensors():
    import torch

    from nestquant_aiinfra_b200.runtime import quantize_activation_cuda

    with pytest.raises(ValueError):
        quantize_activation_cuda(torch.zeros(1, 64), q=14, betas=(0.25, 0.5, 0.75, 1.0))
    with pytest.raises(TypeError):
        quantize_activation_cuda([1.0], q=14, betas=(0.25, 0.5, 0.75, 1.0))
