"""CPU-side checks of the boundary: the library builds, loads, exports every symbol that
include/plq.h declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from plaquant_b200 import build, _lib
    build.build_library()
    return _lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "plq.h")).read()
    return sorted(set(re.findall(r"PLQ_API[^;(]*?\b(plq_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from plaquant_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/plq.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(lib):
    assert lib.plq_version() >= 100
    for code in (0, -1, -2, -3, -4, -5, -6, -7, 1, 99):
        assert lib.plq_status_string(code)
    assert lib.plq_sf_tiled_bytes(300, 62) == 3 * 16 * 512
    assert lib.plq_sf_tiled_bytes(1, 1) == 512


def test_argument_checks_run_before_any_device_work(lib):
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    # shape errors
    assert lib.plq_pack(p16, 4, 256, 32, 0, p16, p16, p16, p16, 0, None) == -2
    assert lib.plq_pack(p16, 4, 192, 64, 1, p16, p16, p16, p16, 0, None) == -2
    assert lib.plq_pack(p16, 4, 65536, 0, 0, p16, p16, p16, p16, 0, None) == -7
    # null / alignment
    assert lib.plq_pack(None, 4, 256, 64, 0, p16, p16, p16, p16, 0, None) == -1
    assert lib.plq_pack(p16 + 2, 4, 256, 64, 0, p16, p16, p16, p16, 0, None) == -3
    assert lib.plq_rmsnorm_pack(p16, None, 1e-6, 4, 256, 64, 1, p16, p16, p16, p16, 0, None) == -1
    assert lib.plq_gemv(p16, p16, p16, p16, p16, p16, p16, p16, 9, 64, 192, 64, p16, 64, None, 0, None) == -2
    assert lib.plq_mixed_gemm(p16, p16, p16, p16, p16, p16, p16, p16, 16, 12, 192, 64, p16, 16, p16, None) == -2
    assert lib.plq_mixed_gemm(p16, p16, p16, p16, p16, p16, p16, p16, 16, 16, 192, 64, p16, 16, None, None) == -1


def test_no_gpu_means_arch_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    buf = (ctypes.c_uint8 * 8192)()
    p16 = (ctypes.addressof(buf) + 15) & ~15
    assert lib.plq_device_check() == -4
    assert lib.plq_pack(p16, 1, 256, 64, 0, p16, p16, p16, p16, 0, None) == -4
    import plaquant_b200 as plq
    with pytest.raises(RuntimeError):
        plq.pack(torch.zeros(1, 256, dtype=torch.bfloat16), 64)
