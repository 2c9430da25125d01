"""The numpy oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py) and against the reference's known-answer tests
(reference tests/test_fake_quant_mxfp8_nvfp4.py:52-62, 110-140, 225-326, 422-449)."""
import os

import numpy as np
import pytest

from oracle import formats as F


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_pack_matches_reference_intermediates(golden_dir, case):
    g = _load(golden_dir, "pack_small.npz")
    x = F.bf16_bits_to_f32(g[f"{case}_x"])
    k_hi = int(g[f"{case}_khi"])
    p = F.pack_mixed(x, k_hi)
    if p["k_lo"]:
        assert np.array_equal(F.unpack_nibbles(p["lo_codes"]), g[f"{case}_lo_codes"])
        assert np.array_equal(p["lo_sf"], g[f"{case}_lo_sf"])
    if p["k_hi"]:
        assert np.array_equal(p["hi_codes"], g[f"{case}_hi_codes"])
        assert np.array_equal(p["hi_sf"], g[f"{case}_hi_sf"])
    # dequantised values == the routed fake quantiser's bf16 output, bit for bit
    assert np.array_equal(F.f32_to_bf16_bits(F.dequant_mixed(p)), g[f"{case}_fq"])


def test_scale_bytes_for_every_bf16_block_maximum(golden_dir):
    g = _load(golden_dir, "scales_exhaustive.npz")
    v = F.bf16_bits_to_f32(np.arange(0, 0x7F80, dtype=np.uint16))
    b16 = np.zeros((v.size, 16), np.float32); b16[:, 3] = v
    b32 = np.zeros((v.size, 32), np.float32); b32[:, 5] = v
    assert np.array_equal(F.nvfp4_scale_codes(b16).reshape(-1), g["nvfp4"])
    assert np.array_equal(F.mxfp8_scale_codes(b32).reshape(-1), g["mxfp8"])
    assert g["nvfp4"][0] == 0x01 and g["mxfp8"][0] == 1      # all-zero block quirks
    assert g["nvfp4"].max() == 0x7E                          # saturates at 448, never NaN


def test_known_answers(golden_dir):
    g = _load(golden_dir, "kats.npz")
    assert np.array_equal(F.E2M1_POS, g["e2m1_grid"]) and np.array_equal(F.E4M3_POS, g["e4m3_grid"])
    for x, y, grid in ((g["x4"], g["y4"], F.E2M1_POS), (g["x8"], g["y8"], F.E4M3_POS)):
        idx, neg = F.round_to_grid_rne(x, grid)
        mine = np.where(neg, -grid[idx], grid[idx])
        assert np.array_equal(mine.view(np.uint32), y.view(np.uint32))   # incl. sign of zero
    # the reference's tie KATs, spelled out
    idx, _ = F.round_to_grid_rne(np.float32([1.25, 1.75, 2.5, 5.0, 1.1, 1.4]), F.E2M1_POS)
    assert list(F.E2M1_POS[idx]) == [1.0, 2.0, 2.0, 4.0, 1.0, 1.5]
    a = 2.0 ** -6
    idx, neg = F.round_to_grid_rne(np.float32([0.5 * (a + 1.125 * a), -0.5 * (a + 1.125 * a)]), F.E4M3_POS)
    assert list(F.E4M3_POS[idx]) == [a, a] and list(neg) == [False, True]


def test_reference_properties():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    for fq in (F.fake_quantize_nvfp4, F.fake_quantize_mxfp8):
        once = fq(x)
        assert np.array_equal(once, fq(once))                # idempotent
    assert not F.fake_quantize_nvfp4(np.zeros((1, 16), np.float32)).any()
    assert not F.fake_quantize_mxfp8(np.zeros((1, 32), np.float32)).any()
    assert np.array_equal(F.fake_quantize_nvfp4(np.full((1, 16), 1.5, np.float32)), np.full((1, 16), 1.5, np.float32))
    # segment routing [main 224 NVFP4 | high 32 MXFP8]
    p = F.pack_mixed(F.round_to_bf16(x), 32)
    d = F.dequant_mixed(p)
    assert np.array_equal(d[:, :224], F.fake_quantize_nvfp4(F.round_to_bf16(x)[:, :224]))
    assert np.array_equal(d[:, 224:], F.fake_quantize_mxfp8(F.round_to_bf16(x)[:, 224:]))


def test_sf_tiling_roundtrip():
    rng = np.random.default_rng(1)
    for rows, n in ((128, 4), (300, 62), (5, 7), (256, 248)):
        sf = rng.integers(0, 255, (rows, n), dtype=np.uint8)
        t = F.tile_sf(sf)
        assert t.size == -(-rows // 128) * 128 * -(-n // 4) * 4
        assert np.array_equal(F.untile_sf(t, rows, n), sf)
        r, k = rows - 1, n - 1
        off = ((r // 128) * (-(-n // 4)) + k // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + k % 4
        assert t[off] == sf[r, k]


def test_norm_and_rotation_restatement_close_to_torch(golden_dir):
    g = _load(golden_dir, "norm_rot.npz")
    x = F.bf16_bits_to_f32(g["x"]); gamma = F.bf16_bits_to_f32(g["gamma"])
    # Sylvester order and normalisation
    assert np.allclose(g["h128_row1"], np.float32(1 / np.sqrt(128)) * np.where(np.arange(128) & 1, -1, 1))
    for mine, ref in ((F.rms_norm_det(x, gamma, 1e-6), g["norm"]),
                      (F.block_hadamard_det(x), g["rot_only"]),
                      (F.block_hadamard_det(F.rms_norm_det(x, gamma, 1e-6)), g["norm_rot"])):
        a, b = F.f32_to_bf16_bits(mine).astype(np.int32), ref.astype(np.int32)
        mism = (a != b).mean()
        # a different float32 summation order moves a value across a bf16 rounding boundary
        # only rarely, and then by one bf16 ulp
        assert mism < 5e-3, mism
        assert np.abs(a - b).max() <= 1


def test_linear_config0_against_reference(golden_dir):
    """Single quantised linear: X [16,4096] x W [4096,4096], K split 3968 + 128."""
    torch = pytest.importorskip("torch")
    g = _load(golden_dir, "linear_cfg0.npz")
    gen = torch.Generator().manual_seed(1)
    W = (torch.randn(4096, 4096, generator=gen) * 0.02).to(torch.bfloat16)
    wbits = W.view(torch.int16).numpy().view(np.uint16)
    assert int(wbits.astype(np.uint64).sum()) == int(g["w_checksum"])
    # feed the oracle the reference's own rotated tensors: pack tier, no summation-order slack
    xr = F.bf16_bits_to_f32(g["xr"])
    px = F.pack_mixed(xr, 128)
    wr4 = F.bf16_bits_to_f32(g["wr_rows"])
    pw4 = F.pack_mixed(wr4, 128)
    assert np.array_equal(F.f32_to_bf16_bits(F.dequant_mixed(pw4)), g["wq_rows"])
    # whole product: rotate W with the restatement, compare with the reference's product
    wr = F.block_hadamard_det(F.bf16_bits_to_f32(wbits))
    y = F.linear(px, F.pack_mixed(wr, 128))
    ref = g["y_f32"]
    rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
    assert rel < 1e-3, rel
    yb = F.bf16_bits_to_f32(F.f32_to_bf16_bits(y)); refb = F.bf16_bits_to_f32(g["y_bf16"])
    rel_b = np.linalg.norm(yb - refb) / np.linalg.norm(refb)
    assert rel_b < 3e-3, rel_b


def test_gptq_frozen_scale_loop_against_reference(golden_dir):
    """oracle/gptq.py against the output of the reference's own GPTQ class (FP path, scales frozen on the original
    weight) on a seeded single-block problem: every rounded weight identical."""
    from oracle import gptq as G
    g = _load(golden_dir, "gptq_frozen.npz")
    w = F.bf16_bits_to_f32(g["w"])
    k_hi = int(g["k_hi"])
    frozen = F.pack_mixed(w, k_hi)                       # the scales round-to-nearest packing gives the original weight
    q, err, codes = G.gptq_block_frozen(w, g["hinv"], frozen["lo_sf"], frozen["hi_sf"], k_hi, 0, w.shape[1])
    assert np.array_equal(q, g["q"])
    # the rounding differs from plain round-to-nearest on a fair share of the elements (otherwise the test says little)
    rtn = F.dequant_mixed(frozen)
    assert 0.02 < np.mean(q != rtn) < 0.6
    # codes and values are consistent
    k_lo = w.shape[1] - k_hi
    assert np.array_equal(F.dequant_nvfp4(codes[:, :k_lo], frozen["lo_sf"]), q[:, :k_lo])
    assert np.array_equal(F.dequant_mxfp8(codes[:, k_lo:], frozen["hi_sf"]), q[:, k_lo:])


def test_reference_quantiser_staged_for_the_benchmark_agrees_with_the_oracle():
    """When oracle/_ref holds the staged copy of the reference's quantiser (oracle/build_ref.py), its ActQuantizer
    must return exactly what the oracle dequantises - the same statement as the fixtures, on fresh data."""
    torch = pytest.importorskip("torch")
    from oracle import build_ref
    if not build_ref.available():
        pytest.skip("oracle/_ref is not staged on this machine")
    qu, _ = build_ref.load()
    x = torch.randn(32, 512, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    q = qu.ActQuantizer()
    q.configure(bits="nvfp4", high_bits="mxfp8", high_bits_length=64)
    got = q(x).float().numpy()
    xf = F.bf16_bits_to_f32(x.view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(got, F.round_to_bf16(F.dequant_mixed(F.pack_mixed(xf, 64))))


def test_rope_oracle_equals_the_pytorch_formulation():
    """`rope_bf16` against `x.float() * cos + rotate_half(x).float() * sin` rounded to bf16, computed by PyTorch on
    the CPU (the formulation of apply_rotary_pos_emb, inference/forward_pass.py:100-109 in the reference, in
    float32), on every position of a 300-token window and bf16 inputs of mixed magnitude."""
    import torch
    g = torch.Generator().manual_seed(12)
    t, heads = 300, 3
    x = (torch.randn(2, t, heads, 128, generator=g) * torch.logspace(-3, 2, heads)[None, None, :, None]).to(torch.bfloat16)
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    ang = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    x1, x2 = x[..., :64], x[..., 64:]
    want = (x.float() * cos[None, :, None, :] + torch.cat([-x2, x1], -1).float() * sin[None, :, None, :]).to(torch.bfloat16)
    got = F.rope_bf16(x.float().numpy(), cos.numpy(), sin.numpy())
    assert np.array_equal(got, want.float().numpy())


def test_rope_oracle_against_the_reference_fixture(golden_dir):
    """`rope_bf16` against apply_rotary_pos_emb of the reference run on the same bf16-valued heads and float32
    tables (tests/golden/make_golden.py), rounded to bf16: queries and keys, positions 37..45."""
    g = np.load(os.path.join(golden_dir, "rope.npz"))
    for name in ("q", "k"):
        x = F.bf16_bits_to_f32(g[name])
        got = F.rope_bf16(x, g["cos"], g["sin"])
        assert np.array_equal(got, F.round_to_bf16(g[name + "_out"])), name
