"""The C port of the oracle (oracle/plq_oracle.c) must agree bit for bit with the numpy oracle,
which is pinned against the reference-generated fixtures."""
import os

import numpy as np
import pytest

from oracle import cport, formats as F
from tests._util import bits_of, synth_activation, synth_gamma, synth_weight


@pytest.mark.parametrize("rows,k,k_hi,norm,had", [(9, 512, 64, False, False), (6, 4096, 128, True, True),
                                                 (4, 1024, 0, False, True), (3, 14336, 448, True, False),
                                                 (5, 128, 128, False, False)])
def test_c_port_equals_numpy_oracle(rows, k, k_hi, norm, had):
    x = synth_activation(rows, k, seed=rows * 31 + k)
    gamma = synth_gamma(k, seed=5) if norm else None
    want = F.prepare_activation(F.bf16_bits_to_f32(bits_of(x)), k_hi,
                                gamma=None if gamma is None else F.bf16_bits_to_f32(bits_of(gamma)), eps=1e-6,
                                hadamard=had)
    got = cport.prepare(bits_of(x), k_hi, None if gamma is None else bits_of(gamma), 1e-6, had)
    for key in ("lo_codes", "lo_sf", "hi_codes", "hi_sf"):
        assert np.array_equal(got[key], want[key]), key
    assert np.array_equal(cport.dequant(got), F.dequant_mixed(want))


def test_c_port_on_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "pack_small.npz"))
    got = cport.prepare(g["a_x"], int(g["a_khi"]), hadamard=False)
    assert np.array_equal(F.unpack_nibbles(got["lo_codes"]), g["a_lo_codes"])
    assert np.array_equal(got["lo_sf"], g["a_lo_sf"])
    assert np.array_equal(got["hi_codes"], g["a_hi_codes"]) and np.array_equal(got["hi_sf"], g["a_hi_sf"])
    assert np.array_equal(F.f32_to_bf16_bits(cport.dequant(got)), g["a_fq"])


def test_c_port_linear_close_to_numpy():
    x = synth_activation(8, 1024, seed=2); w = synth_weight(64, 1024, seed=3)
    px = cport.prepare(bits_of(x), 32); pw = cport.prepare(bits_of(w), 32)
    a, b = cport.linear(px, pw), F.linear(px, pw)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 1e-5
    assert cport.num_threads() >= 1
