"""ctypes front end of oracle/plq_oracle.c (the multi-threaded C port of the reference's CPU
path).  Test infrastructure and timed CPU baseline only."""
from __future__ import annotations

import ctypes

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        h = ctypes.CDLL(_build.build_oracle())
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        h.plqo_prepare.argtypes = [vp, vp, f32, i64, i32, i32, i32, vp, vp, vp, vp]
        h.plqo_dequant.argtypes = [vp, vp, vp, vp, i64, i32, i32, vp]
        h.plqo_matmul_nt.argtypes = [vp, vp, i64, i64, i32, vp]
        h.plqo_num_threads.restype = i32
        h.plqo_set_num_threads.argtypes = [i32]
        h.plqo_set_num_threads.restype = None
        _lib = h
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None and a.size else None


def prepare(x_bits: np.ndarray, k_hi: int, gamma_bits=None, eps: float = 1e-6, hadamard: bool = True) -> dict:
    """x_bits: uint16 bf16 patterns [rows, K].  Same dict as oracle.formats.pack_mixed."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, k = x.shape
    k_lo = k - k_hi
    out = {"rows": rows, "k_lo": k_lo, "k_hi": k_hi,
           "lo_codes": np.zeros((rows, k_lo // 2), np.uint8), "lo_sf": np.zeros((rows, k_lo // 16), np.uint8),
           "hi_codes": np.zeros((rows, k_hi), np.uint8), "hi_sf": np.zeros((rows, k_hi // 32), np.uint8)}
    g = None if gamma_bits is None else np.ascontiguousarray(gamma_bits, dtype=np.uint16)
    lib().plqo_prepare(_p(x), _p(g), eps, rows, k, k_hi, int(hadamard), _p(out["lo_codes"]), _p(out["lo_sf"]),
                       _p(out["hi_codes"]), _p(out["hi_sf"]))
    return out


def dequant(p: dict) -> np.ndarray:
    out = np.empty((p["rows"], p["k_lo"] + p["k_hi"]), np.float32)
    lib().plqo_dequant(_p(p["lo_codes"]), _p(p["lo_sf"]), _p(p["hi_codes"]), _p(p["hi_sf"]), p["rows"], p["k_lo"],
                       p["k_hi"], _p(out))
    return out


def linear(px: dict, pw: dict) -> np.ndarray:
    a, b = dequant(px), dequant(pw)
    y = np.empty((a.shape[0], b.shape[0]), np.float32)
    lib().plqo_matmul_nt(_p(a), _p(b), a.shape[0], b.shape[0], a.shape[1], _p(y))
    return y


def set_num_threads(n: int) -> None:
    """OpenMP team size of the port (launchers such as torchrun export OMP_NUM_THREADS=1 to their workers)."""
    lib().plqo_set_num_threads(int(n))


def num_threads() -> int:
    return int(lib().plqo_num_threads())
