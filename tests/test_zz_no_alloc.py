"""The workspace-free decode GEMV entry point (plq_gemv_static_scratch), called through the C ABI.

It exists for hosts that cannot allocate device memory for the library (all of HBM already belongs
to the host's own pool, or the plugin interface carries inputs and outputs only).  Its results must
be those of plq_gemv, call after call, although every call reuses one scratch array that still
holds the previous call's partial sums.  Collected last so that a failure here cannot hide others.
"""
import pytest
import torch

from tests._util import synth_activation, synth_weight

pytestmark = pytest.mark.gpu
plq = pytest.importorskip("plaquant_b200")


def _static_gemv(pa, pb):
    from plaquant_b200 import _lib
    y = torch.empty(pa.rows, pb.rows, dtype=torch.bfloat16, device=pa.device)
    p = lambda t: None if t.numel() == 0 else t.data_ptr()
    st = _lib.lib().plq_gemv_static_scratch(p(pa.lo_codes), p(pa.lo_sf), p(pa.hi_codes), p(pa.hi_sf), p(pb.lo_codes),
                                            p(pb.lo_sf), p(pb.hi_codes), p(pb.hi_sf), pa.rows, pb.rows, pa.k_lo, pa.k_hi,
                                            y.data_ptr(), y.stride(0), torch.cuda.current_stream().cuda_stream)
    _lib.check(st)
    return y


def test_static_scratch_gemv_equals_workspace_gemv_twice_in_a_row():
    # K = 4096 with N = 4096 makes the kernel cut K into 8 slices, so the scratch really is used
    k, k_hi, n = 4096, 128, 4096
    w = plq.pack(synth_weight(n, k, seed=77).cuda(), k_hi, hadamard=True, sf_layout="rowmajor")
    x1 = plq.pack(synth_activation(8, k, seed=78).cuda(), k_hi, hadamard=True, sf_layout="rowmajor")
    x2 = plq.pack(synth_activation(3, k, seed=79).cuda(), k_hi, hadamard=True, sf_layout="rowmajor")
    want1, want2 = plq.gemv(x1, w), plq.gemv(x2, w)
    got1 = _static_gemv(x1, w)
    got2 = _static_gemv(x2, w)          # second call: scratch still holds the first call's partial sums
    got1_again = _static_gemv(x1, w)
    torch.cuda.synchronize()
    # same kernel, same fixed summation order: bit-identical, well inside the 1e-3 rel-L2 of the GEMV tests
    assert torch.equal(got1, want1) and torch.equal(got2, want2) and torch.equal(got1_again, want1)


def test_static_scratch_gemv_with_changing_widths_and_at_its_maximum():
    """Calls of different N share the one array: a wide call (N = 28672) followed by a narrow one (N = 4096) and
    the widest the entry point accepts (N = 32768), each against plq_gemv with a caller's workspace."""
    k, k_hi = 4096, 128
    x = plq.pack(synth_activation(4, k, seed=80).cuda(), k_hi, hadamard=True, sf_layout="rowmajor")
    ws = {n: plq.pack(synth_weight(n, k, seed=81 + n % 7).cuda(), k_hi, hadamard=True, sf_layout="rowmajor")
          for n in (28672, 4096, 32768)}
    want = {n: plq.gemv(x, w) for n, w in ws.items()}
    for n in (28672, 4096, 32768, 4096, 28672):
        got = _static_gemv(x, ws[n])
        torch.cuda.synchronize()
        assert torch.equal(got, want[n]), n


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    from plaquant_b200 import _lib
    x = plq.pack(synth_activation(1, 128, seed=1).cuda(), 64, sf_layout="rowmajor")
    p = x.lo_codes.data_ptr()
    st = _lib.lib().plq_gemv_static_scratch(p, p, p, p, p, p, p, p, 1, 32768 + 16, 64, 64, p, 32768 + 16, None)
    assert st == -7
    assert b"maximum" in _lib.lib().plq_status_string(st)
