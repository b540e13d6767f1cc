"""Host-side helpers that decide how tensors are handed to the kernels (CPU, no launch)."""

import torch


def test_append_rows_are_read_in_place_only_when_they_are_rows_of_one_stride():
    from nestquant_aiinfra_b200.runtime.kv import _rows_in_place

    dense = torch.zeros(4, 2, 64, dtype=torch.bfloat16)
    tensor, stride = _rows_in_place(dense)
    assert tensor is dense and stride == 0
    stacked = torch.zeros(4, 512, dtype=torch.bfloat16)
    value = stacked[:, 384:].view(4, 2, 64)             # column range of a stacked q/k/v result
    tensor, stride = _rows_in_place(value)
    assert tensor is value and stride == 512
    one_row = stacked[:1, 384:].view(1, 2, 64)
    assert _rows_in_place(one_row)[1] == 0               # a single row needs no stride
    transposed = torch.zeros(4, 64, 2, dtype=torch.bfloat16).transpose(1, 2)   # rows are not contiguous inside
    tensor, stride = _rows_in_place(transposed)
    assert tensor.is_contiguous() and stride == 0 and tensor.shape == transposed.shape
    odd = torch.zeros(4, 520, dtype=torch.bfloat16)[:, 4:132].view(4, 2, 64)   # 8-byte offset: not 16-byte aligned
    tensor, stride = _rows_in_place(odd)
    assert tensor.is_contiguous() and stride == 0


def test_hadamard_of_the_silu_product_falls_back_to_the_tensor_ops_off_the_gpu():
    from nestquant_aiinfra_b200.rotation import hadamard, hadamard_silu_mul

    gate, up = torch.randn(3, 64), torch.randn(3, 64)
    assert torch.equal(hadamard_silu_mul(gate, up), hadamard(torch.nn.functional.silu(gate) * up))


def test_projection_group_threshold_and_decode_ahead_constants():
    from nestquant_aiinfra_b200.fused_linear import SharedProjectionGroup, WeightDecodeAhead

    # from this many rows on the packed path runs decode + tcgen05 (the library's kTcMinM): only then is the
    # resident entry on a decode-ahead scratch the same sequence of kernels
    assert WeightDecodeAhead.MIN_ROWS == 8
    assert SharedProjectionGroup.SEPARATE_FROM == 512
