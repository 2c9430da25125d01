"""plaquant_b200: the mixed NVFP4 / MXFP8 quantised-linear hot path for NVIDIA B200 (sm_100a).

Host side is Python/PyTorch (memory, streams); every kernel lives in libplq_b200.so, a C-ABI
CUDA library declared in include/plq.h.  There is no CPU or PyTorch fallback.
"""
from ._lib import PlqError, lib, LIB_PATH  # noqa: F401
from . import ops  # noqa: F401
from .ops import (PackedMatrix, pack, unpack, mixed_gemm, gemv, gemv_tc, alloc_packed, check_device_status,  # noqa: F401
                  silu_mul_pack, add_rmsnorm_pack,
                  SF_ROWMAJOR, SF_TILED)

__version__ = "0.1.0"
