"""ctypes binding of libplq_b200.so.  No fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libplq_b200.so")

_vp, _i64, _i32, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); mirrors include/plq.h
SIGNATURES = {
    "plq_version": (_i32, []),
    "plq_status_string": (ctypes.c_char_p, [_i32]),
    "plq_last_cuda_error": (_i32, []),
    "plq_device_check": (_i32, []),
    "plq_sf_tiled_bytes": (_i64, [_i64, _i64]),
    "plq_pack": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _i32, _vp]),
    "plq_rmsnorm_pack": (_i32, [_vp, _vp, _f32, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _i32, _vp]),
    "plq_unpack": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp]),
    "plq_mixed_gemm": (_i32, [_vp] * 8 + [_i64] * 4 + [_vp, _i64, _vp, _vp]),
    "plq_mixed_gemm_variant": (_i32, [_vp] * 8 + [_i64] * 4 + [_vp, _i64, _vp, _vp, _i32]),
    "plq_gemv_workspace_bytes": (_i64, [_i64]),
    "plq_gemv": (_i32, [_vp] * 8 + [_i64] * 4 + [_vp, _i64, _vp, _i64, _vp]),
    "plq_gemv_static_scratch": (_i32, [_vp] * 8 + [_i64] * 4 + [_vp, _i64, _vp]),
    "plq_silu_mul_pack": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _i32, _vp]),
    "plq_add_rmsnorm_pack": (_i32, [_vp, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _i32, _vp]),
    "plq_allreduce_add_rmsnorm_pack": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _i32,
                                              _vp, _vp, _vp, _vp, _i32, _vp, _vp]),
    "plq_reduce_scatter_add_rmsnorm_pack": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _i64, _i64, _vp, _vp, _vp, _f32, _i64,
                                                   _i64, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "plq_rope_kv_append": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp]),
    "plq_gptq_block_frozen": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _vp]),
    "plq_gemv_tc": (_i32, [_vp] * 8 + [_i64] * 4 + [_vp, _i64, _vp, _i32, _vp]),
}

_lib = None


class PlqError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"plq status {status}: {text}")
        self.status = status


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built (python -m plaquant_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m plaquant_b200.build` "
                "(nvcc, sm_100a).  plaquant_b200 has no CPU or PyTorch fallback path.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        text = lib().plq_status_string(status).decode()
        if status == -5:
            text += f" [cudaError {lib().plq_last_cuda_error()}]"
        raise PlqError(status, text)
