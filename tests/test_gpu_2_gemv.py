"""Decode GEMV (m <= 8) against the CPU oracle and against the fused GEMM on the same operands."""
import numpy as np
import pytest
import torch

from oracle import formats as F
from tests._util import f32_of, packed_to_numpy, rel_l2, synth_activation, synth_weight

pytestmark = pytest.mark.gpu
plq = pytest.importorskip("plaquant_b200")

TOL = 1e-3   # rel-L2 in the output dtype


@pytest.mark.parametrize("m", [1, 2, 4, 8, 3])
@pytest.mark.parametrize("n,k,k_hi", [(256, 4096, 128), (200, 14336, 448), (136, 192, 64), (16, 64, 0),
                                       (128, 128, 128), (1024, 8192, 256)])
def test_gemv_against_oracle(m, n, k, k_hi):
    x = synth_activation(m, k, seed=10 * m + 1)
    w = synth_weight(n, k, seed=n + k)
    had = k % 128 == 0
    pa = plq.pack(x.cuda(), k_hi, hadamard=had, sf_layout="rowmajor")
    pb = plq.pack(w.cuda(), k_hi, hadamard=had, sf_layout="rowmajor")
    y = f32_of(plq.gemv(pa, pb))
    want = F.round_to_bf16(F.linear(packed_to_numpy(pa), packed_to_numpy(pb)))
    r = rel_l2(y, want)
    assert r <= TOL, r


@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
def test_llama8b_shapes_gemv_vs_gemm_and_oracle_rows(n, k):
    """Full decode shapes at m = 8: agreement with the tensor-memory GEMM on identical operands,
    a sample of output columns against the oracle, and run-to-run determinism."""
    k_hi = k // 32
    x = synth_activation(8, k, seed=42)
    w = synth_weight(n, k, seed=n // 7 + k)
    xc, wc = x.cuda(), w.cuda()
    pa_r = plq.pack(xc, k_hi, hadamard=True, sf_layout="rowmajor")
    pb_r = plq.pack(wc, k_hi, hadamard=True, sf_layout="rowmajor")
    y = plq.gemv(pa_r, pb_r)
    assert torch.equal(y, plq.gemv(pa_r, pb_r))
    pa_t = plq.pack(xc, k_hi, hadamard=True, sf_layout="tiled")
    pb_t = plq.pack(wc, k_hi, hadamard=True, sf_layout="tiled")
    yg = plq.mixed_gemm(pa_t, pb_t)
    plq.check_device_status()
    assert rel_l2(f32_of(y), f32_of(yg)) <= TOL
    sel = np.sort(np.random.default_rng(2).choice(n, 64, replace=False))
    nb = packed_to_numpy(pb_r)
    sub = {**nb, "rows": len(sel), **{key: nb[key][sel] for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf")}}
    want = F.round_to_bf16(F.linear(packed_to_numpy(pa_r), sub))
    assert rel_l2(f32_of(y)[:, sel], want) <= TOL


def test_gemv_argument_errors():
    x = synth_activation(9, 256, seed=1).cuda()
    pa = plq.pack(x, 64, sf_layout="rowmajor")
    with pytest.raises(plq.PlqError) as e:
        plq.gemv(pa, pa)          # m = 9 > 8
    assert e.value.status == -2


# ---- tensor-core GEMV (tiled scale layout, the operands of the fused GEMM) ----------------------
@pytest.mark.parametrize("m", [1, 2, 4, 8, 3, 9, 16])
@pytest.mark.parametrize("n,k,k_hi", [(256, 4096, 128), (200, 14336, 448), (136, 192, 64), (16, 64, 0),
                                       (128, 128, 128), (1024, 8192, 256), (8, 13952, 64)])
def test_gemv_tc_against_oracle(m, n, k, k_hi):
    x = synth_activation(m, k, seed=10 * m + 1)
    w = synth_weight(n, k, seed=n + k)
    had = k % 128 == 0
    pa = plq.pack(x.cuda(), k_hi, hadamard=had, sf_layout="tiled")
    pb = plq.pack(w.cuda(), k_hi, hadamard=had, sf_layout="tiled")
    y = f32_of(plq.gemv_tc(pa, pb))
    plq.check_device_status()
    want = F.round_to_bf16(F.linear(packed_to_numpy(pa), packed_to_numpy(pb)))
    r = rel_l2(y, want)
    assert r <= TOL, r


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
def test_llama8b_shapes_gemv_tc(n, k, m):
    """Full decode shapes at m = 1, 2, 4, 8 and 16: agreement with the fused GEMM on the identical operands, a sample of
    output columns against the oracle, and run-to-run determinism."""
    k_hi = k // 32
    xc, wc = synth_activation(m, k, seed=42).cuda(), synth_weight(n, k, seed=n // 7 + k).cuda()
    pa = plq.pack(xc, k_hi, hadamard=True, sf_layout="tiled")
    pb = plq.pack(wc, k_hi, hadamard=True, sf_layout="tiled")
    y = plq.gemv_tc(pa, pb)
    assert torch.equal(y, plq.gemv_tc(pa, pb))
    torch.cuda.synchronize()       # the weights are complete: the early-prefetch variant may be used
    assert torch.equal(y, plq.gemv_tc(pa, pb, static_weights=True))
    yg = plq.mixed_gemm(pa, pb)
    plq.check_device_status()
    assert rel_l2(f32_of(y), f32_of(yg)) <= TOL
    sel = np.sort(np.random.default_rng(2).choice(n, 64, replace=False))
    nb = packed_to_numpy(pb)
    sub = {**nb, "rows": len(sel), **{key: nb[key][sel] for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf")}}
    want = F.round_to_bf16(F.linear(packed_to_numpy(pa), sub))
    assert rel_l2(f32_of(y)[:, sel], want) <= TOL


def test_gemv_tc_argument_errors():
    x = synth_activation(17, 256, seed=1).cuda()
    pa = plq.pack(x, 64, sf_layout="tiled")
    with pytest.raises(plq.PlqError) as e:
        plq.gemv_tc(pa, pa)          # m = 17 > 16
    assert e.value.status == -2
