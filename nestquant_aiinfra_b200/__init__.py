"""B200-native (sm_100a) implementation of NestQuant's packed W4A4KV4 hot path.

Host code is Python/PyTorch (device memory, streams, ``torch.distributed``);
all arithmetic runs in hand-written CUDA behind the C ABI declared in
``include/nq_b200.h``.
"""

from ._lib import build_library, lib, LIB_PATH  # noqa: F401
from . import formats  # noqa: F401

__all__ = ["build_library", "lib", "LIB_PATH", "formats"]
