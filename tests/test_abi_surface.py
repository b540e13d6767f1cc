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


def test_workspace_queries_and_argument_errors_of_the_opt_in_entries():
    """Host-side logic of the sizing queries and argument checks (no kernel is launched)."""
    import ctypes

    import nestquant_aiinfra_b200 as nq

    library = nq.lib()
    i64, null = ctypes.c_int64, ctypes.c_void_p(0)
    library.nq_w4a4_resident_workspace_bytes.restype = ctypes.c_size_t
    library.nq_kv_attention_workspace_bytes.restype = ctypes.c_size_t
    counters = 65536
    # streaming GEMV (m < 5): counters + room for the decoded activation rows, no split-K partials
    assert library.nq_w4a4_resident_workspace_bytes(i64(1), i64(8192), i64(2048)) == counters + 4096
    assert library.nq_w4a4_resident_workspace_bytes(i64(4), i64(96), i64(4096)) == counters + 4 * 4096 * 2
    # tensor-core path (m >= 5): at least the decoded rows, never more than the packed entry asks for
    resident = library.nq_w4a4_resident_workspace_bytes(i64(64), i64(2048), i64(2048))
    packed = library.nq_w4a4_workspace_bytes(i64(64), i64(2048), i64(2048))
    assert counters + 64 * 2048 * 2 <= resident < packed and packed - resident >= 2048 * 2048 * 2
    assert library.nq_w4a4_resident_workspace_bytes(i64(0), i64(64), i64(64)) == 0
    # attention split partials: config 2 (32 rows x 8 KV heads, 257 page slots) runs as 9 splits = 3.9 waves of
    # the 4 CTAs resident per SM; a prefill-sized grid needs no split
    per_split = 32 * 32 * (64 + 2) * 4
    assert library.nq_kv_attention_workspace_bytes(32, 1, 32, 8, 64, 256) == 9 * per_split + 256
    assert library.nq_kv_attention_workspace_bytes(8, 1024, 32, 8, 64, 256) == 8 * 1024 * 32 * 66 * 4 + 256
    assert library.nq_kv_attention_workspace_bytes(0, 1, 32, 8, 64, 256) == 0
    # null pointers are rejected before anything touches the device
    assert library.nq_kv_expand_pages(null, null, null, i64(1), 4, 16, 8, 64, null) == -1
    assert b"nq_kv_expand_pages" in library.nq_last_error()
    args = [null] * 3 + [i64(1)] + [ctypes.c_int(v) for v in (4, 16, 8, 48)] + [null]
    args[0] = args[1] = args[2] = ctypes.c_void_p(16)
    assert library.nq_kv_expand_pages(*args) == -1     # head_dim must be a multiple of 32
    assert library.nq_w4a4_gemm_resident(null, null, null, null, null, null, i64(1), i64(64), i64(256), null,
                                         0, null, ctypes.c_size_t(0), null) == -1
