"""CPU oracle for the mixed NVFP4 / MXFP8 quantised-linear hot path.

TEST INFRASTRUCTURE ONLY.  This module restates, in numpy float32 arithmetic, what the
reference's PyTorch fake quantiser computes, and derives from those intermediates the packed
codes and scale bytes a real packer must emit.  It is imported by the tests, by the smoke
check and by the CPU-baseline leg of the benchmark, never by the product path (the package
`plaquant_b200` raises when its CUDA library is missing instead of falling back to this).

Parity pin: `tests/golden/*.npz` were produced by running the reference's own functions
(`promix/quantize/quant_utils.py`, `inference/rotation.py`, `inference/forward_pass.py`) on
seeded inputs; `tests/test_oracle_golden.py` checks every function here against them.

Reference lines followed (paths inside the reference project):
  * E4M3 / E2M1 value grids ........ promix/quantize/quant_utils.py:444-463
  * round-to-nearest, ties-to-even . promix/quantize/quant_utils.py:466-514
  * scale round-up to E4M3 ......... promix/quantize/quant_utils.py:517-532, 587-613
  * scale round-up to E8M0 ......... promix/quantize/quant_utils.py:535-554, 557-584
  * MXFP8 fake quantiser ........... promix/quantize/quant_utils.py:660-707
  * NVFP4 fake quantiser ........... promix/quantize/quant_utils.py:710-751
  * [main | high] segment routing .. promix/quantize/quant_utils.py:182-224
  * RMSNorm ........................ inference/forward_pass.py:33-39
  * normalised Sylvester Hadamard .. inference/rotation.py:21-29, applied as
                                     (x.float() @ H).to(dtype), inference/quantize.py:447-448
  * packing conventions ............ docs/specs/spec-mxfp8-nvfp4.md:150-176 (low nibble =
                                     lower K; separate row-major scale buffers)
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

# ----------------------------------------------------------------------------------------
# Value grids (quant_utils.py:444-463).  Index in the grid == magnitude code of the format.
# ----------------------------------------------------------------------------------------
E2M1_POS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)
E2M1_MAX = F32(6.0)
E4M3_POS = np.array(
    [0.0]
    + [2.0 ** -9 * m for m in range(1, 8)]
    + [(2.0 ** (e - 7)) * (1.0 + m / 8.0) for e in range(1, 16) for m in range(8)][:-1],
    dtype=F32,
)  # 127 finite non-negative values, codes 0x00..0x7E; 0x7F is NaN
E4M3_MAX = F32(448.0)
assert E4M3_POS.size == 127 and E4M3_POS[-1] == 448.0

NVFP4_BLOCK = 16
MXFP8_BLOCK = 32
HAD_BLOCK = 128


# ----------------------------------------------------------------------------------------
# bf16 helpers (numpy has no bf16: values travel as uint16 bit patterns or as float32)
# ----------------------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest, ties to even); returns the uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> np.uint32(16)) | np.uint32(0x40), rounded).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(F32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16, returned as float32 values."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------------------
# Rounding primitives
# ----------------------------------------------------------------------------------------
def round_to_grid_rne(x: np.ndarray, grid: np.ndarray):
    """Nearest grid value of |x|, ties to the even grid index (quant_utils.py:466-514).

    Returns (index, negative) where `negative` is True only where x < 0 strictly: the
    reference multiplies the chosen magnitude by torch.sign(x), and sign(+-0) is 0, so a
    value that is exactly zero before rounding comes out as +0 whatever its sign bit was,
    while a negative value that rounds to zero comes out as -0.
    """
    x = np.asarray(x, dtype=F32)
    a = np.abs(x)
    hi = np.clip(np.searchsorted(grid, a, side="left"), 1, grid.size - 1)
    lo = hi - 1
    d_lo = np.abs(a - grid[lo])
    d_hi = np.abs(grid[hi] - a)
    pick_hi = d_hi < d_lo
    tie = np.abs(d_hi - d_lo) < F32(1e-12)
    pick_hi = np.where(tie, (lo % 2) == 1, pick_hi)
    return np.where(pick_hi, hi, lo).astype(np.uint8), x < 0


def ceil_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Smallest E4M3 grid index whose value is >= x; saturates at 448 (quant_utils.py:517-532)."""
    x = np.asarray(x, dtype=F32)
    return np.minimum(np.searchsorted(E4M3_POS, x, side="left"), E4M3_POS.size - 1).astype(np.uint8)


def e8m0_exponent_round_up(s: np.ndarray) -> np.ndarray:
    """ceil(log2(s)) for positive float32 s, from the bit pattern (exact form of
    quant_utils.py:545-547; the two agree on every bf16 block maximum, which the golden
    fixture `scales_exhaustive.npz` pins)."""
    u = np.ascontiguousarray(s, dtype=F32).view(np.uint32)
    exp = ((u >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32)
    man = (u & np.uint32(0x7FFFFF)).astype(np.int32)
    return np.where(exp == 0, -126, exp - 127 + (man != 0))  # subnormals cannot occur after the clamp


# ----------------------------------------------------------------------------------------
# Block scales
# ----------------------------------------------------------------------------------------
def _blocks(x: np.ndarray, block: int) -> np.ndarray:
    x = np.asarray(x, dtype=F32)
    assert x.shape[-1] % block == 0, f"K ({x.shape[-1]}) not divisible by block ({block})"
    return x.reshape(*x.shape[:-1], x.shape[-1] // block, block)


def nvfp4_scale_codes(x: np.ndarray) -> np.ndarray:
    """E4M3 scale byte per 16-block: ceil_E4M3(max|x| / 6), floor 2^-9 (quant_utils.py:740-743)."""
    bmax = np.abs(_blocks(x, NVFP4_BLOCK)).max(axis=-1)
    ideal = np.maximum(bmax / E2M1_MAX, F32(2.0 ** -9))
    return ceil_to_e4m3(ideal)


def mxfp8_scale_codes(x: np.ndarray) -> np.ndarray:
    """E8M0 scale byte (exponent + 127) per 32-block: 2^ceil(log2(max|x| / 448))
    (quant_utils.py:697-699 with the clamp to float32 `tiny` at :545, which makes the
    smallest scale 2^-126, byte 1, also for an all-zero block)."""
    bmax = np.abs(_blocks(x, MXFP8_BLOCK)).max(axis=-1)
    ideal = np.maximum(bmax / E4M3_MAX, F32(2.0 ** -126))
    return (e8m0_exponent_round_up(ideal) + 127).astype(np.uint8)


def e8m0_value(code: np.ndarray) -> np.ndarray:
    return np.ldexp(F32(1.0), np.asarray(code, dtype=np.int32) - 127).astype(F32)


# ----------------------------------------------------------------------------------------
# Quantisers: codes + scale bytes (what a packer stores) and the dequantised values
# ----------------------------------------------------------------------------------------
def quantize_nvfp4(x: np.ndarray):
    """-> (codes uint8 [..., K] with bit3 = sign, scale bytes uint8 [..., K/16])."""
    xb = _blocks(x, NVFP4_BLOCK)
    sc = nvfp4_scale_codes(x)
    scale = E4M3_POS[sc][..., None]
    q = np.clip(xb / scale, -E2M1_MAX, E2M1_MAX)
    idx, neg = round_to_grid_rne(q, E2M1_POS)
    codes = (idx | (neg.astype(np.uint8) << 3)).reshape(x.shape)
    return codes, sc


def quantize_mxfp8(x: np.ndarray):
    """-> (E4M3 code bytes uint8 [..., K] with bit7 = sign, E8M0 scale bytes [..., K/32])."""
    xb = _blocks(x, MXFP8_BLOCK)
    sc = mxfp8_scale_codes(x)
    scale = e8m0_value(sc)[..., None]
    with np.errstate(over="ignore"):
        q = np.clip(xb / scale, -E4M3_MAX, E4M3_MAX)
    idx, neg = round_to_grid_rne(q, E4M3_POS)
    codes = (idx | (neg.astype(np.uint8) << 7)).reshape(x.shape)
    return codes, sc


def dequant_nvfp4(codes: np.ndarray, sc: np.ndarray) -> np.ndarray:
    mag = E2M1_POS[codes & 7]
    val = np.where(codes & 8, -mag, mag).astype(F32)
    return (_blocks(val, NVFP4_BLOCK) * E4M3_POS[sc][..., None]).reshape(codes.shape)


def dequant_mxfp8(codes: np.ndarray, sc: np.ndarray) -> np.ndarray:
    mag = E4M3_POS[np.minimum(codes & 0x7F, 126)]
    val = np.where(codes & 0x80, -mag, mag).astype(F32)
    return (_blocks(val, MXFP8_BLOCK) * e8m0_value(sc)[..., None]).reshape(codes.shape)


def fake_quantize_nvfp4(x: np.ndarray) -> np.ndarray:
    return dequant_nvfp4(*quantize_nvfp4(x))


def fake_quantize_mxfp8(x: np.ndarray) -> np.ndarray:
    return dequant_mxfp8(*quantize_mxfp8(x))


# ----------------------------------------------------------------------------------------
# Packed container: the layout in HBM
# ----------------------------------------------------------------------------------------
def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """Two E2M1 codes per byte, low nibble = lower K (spec-mxfp8-nvfp4.md:161)."""
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (c[..., 0] | (c[..., 1] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    out = np.empty((*packed.shape[:-1], packed.shape[-1] * 2), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def pack_mixed(x: np.ndarray, k_hi: int) -> dict:
    """Split the last axis [main = K - k_hi | high = k_hi] (quant_utils.py:195-216) and pack:
    main -> NVFP4, high -> MXFP8.  `x` holds bf16-representable float32 values.
    Scale buffers are row-major ([rows, K_lo/16], [rows, K_hi/32])."""
    x = np.asarray(x, dtype=F32)
    x2 = x.reshape(-1, x.shape[-1])
    k = x2.shape[1]
    k_lo = k - k_hi
    assert k_lo % NVFP4_BLOCK == 0 and k_hi % MXFP8_BLOCK == 0
    lo_c, lo_s = quantize_nvfp4(x2[:, :k_lo]) if k_lo else (np.zeros((x2.shape[0], 0), np.uint8),) * 2
    hi_c, hi_s = quantize_mxfp8(x2[:, k_lo:]) if k_hi else (np.zeros((x2.shape[0], 0), np.uint8),) * 2
    return {
        "rows": x2.shape[0], "k_lo": k_lo, "k_hi": k_hi,
        "lo_codes": pack_nibbles(lo_c), "lo_sf": lo_s, "hi_codes": hi_c, "hi_sf": hi_s,
    }


def dequant_mixed(p: dict) -> np.ndarray:
    """float32 [rows, K]: what the fake quantiser would have returned for the same input."""
    parts = []
    if p["k_lo"]:
        parts.append(dequant_nvfp4(unpack_nibbles(p["lo_codes"]), p["lo_sf"]))
    if p["k_hi"]:
        parts.append(dequant_mxfp8(p["hi_codes"], p["hi_sf"]))
    return np.concatenate(parts, axis=-1)


def tile_sf(sf: np.ndarray) -> np.ndarray:
    """Row-major scale bytes [rows, n_sf] -> the 128-row x 4-scale tiled order that one
    block-scaled MMA consumes: a 512-byte chunk holds rows r0..r0+127 and scales k0..k0+3 at
    byte (r % 32) * 16 + (r % 128) // 32 * 4 + (k % 4); chunks are ordered K-fastest.
    Rows and scales are zero-padded to multiples of 128 and 4."""
    rows, n = sf.shape
    rp, npad = -(-rows // 128) * 128, -(-n // 4) * 4
    full = np.zeros((rp, npad), dtype=np.uint8)
    full[:rows, :n] = sf
    t = full.reshape(rp // 128, 4, 32, npad // 4, 4)       # [rt, r/32, r%32, kt, k%4]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(-1)  # [rt, kt, r%32, r/32, k%4]


def untile_sf(tiled: np.ndarray, rows: int, n: int) -> np.ndarray:
    rp, npad = -(-rows // 128) * 128, -(-n // 4) * 4
    t = np.asarray(tiled, dtype=np.uint8).reshape(rp // 128, npad // 4, 32, 4, 4)
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(rp, npad)[:rows, :n]


# ----------------------------------------------------------------------------------------
# Deterministic restatement of RMSNorm and the block-Hadamard rotation
#
# torch's `mean` and `@` leave the float32 summation order unspecified, so their literal
# output cannot be reproduced bit for bit by any other implementation.  The functions below
# fix one order; the CUDA kernels follow the same order and must match them exactly, and the
# tests bound the distance from the torch composition (a bf16 ulp on a small share of elements).
# ----------------------------------------------------------------------------------------
def _sumsq_det(x: np.ndarray) -> np.ndarray:
    """Row sum of squares, float32, in this order: the row is cut into chunks of 64 elements and every
    chunk into two runs of 32; inside a run the even and the odd elements are accumulated in two
    sequential chains, run sum = even + odd, chunk sum = run + run; chunks are combined 32 at a time
    (2048 elements) by a balanced pairwise tree (missing chunks count as +0); the groups of 32 chunks
    are then added left to right."""
    rows, k = x.shape
    assert k % 64 == 0
    sq = (x * x).astype(F32).reshape(rows, k // 64, 2, 16, 2)   # [.., chunk, run, pair, even/odd]
    acc = np.zeros((rows, k // 64, 2, 2), dtype=F32)
    for i in range(16):
        acc = acc + sq[:, :, :, i, :]
    run = acc[..., 0] + acc[..., 1]
    c = run[..., 0] + run[..., 1]
    nc = c.shape[1]
    pad = -(-nc // 32) * 32
    cc = np.zeros((rows, pad), dtype=F32)
    cc[:, :nc] = c
    g = cc.reshape(rows, pad // 32, 32)
    while g.shape[-1] > 1:
        g = g[..., 0::2] + g[..., 1::2]
    g = g[..., 0]
    tot = np.zeros(rows, dtype=F32)
    for w in range(g.shape[1]):
        tot = tot + g[:, w]
    return tot


def rms_norm_det(x_bf16: np.ndarray, gamma: np.ndarray, eps: float) -> np.ndarray:
    """inference/forward_pass.py:33-39 with the summation order of `_sumsq_det`:
    r = 1 / sqrt(sumsq / K + eps); y = bf16(gamma * (x * r)), all float32, each op rounded."""
    x = np.asarray(x_bf16, dtype=F32)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    var = _sumsq_det(x2) / F32(k)
    r = F32(1.0) / np.sqrt(var + F32(eps), dtype=F32)
    y = np.asarray(gamma, dtype=F32)[None, :] * (x2 * r[:, None])
    return round_to_bf16(y).reshape(x.shape)


def block_hadamard_det(x_bf16: np.ndarray) -> np.ndarray:
    """y = bf16((x.float() @ H_128) per 128-block), H = Sylvester Hadamard / sqrt(128)
    (inference/rotation.py:21-29), evaluated as seven radix-2 butterfly stages with strides
    1, 2, 4, ..., 64 (a + b, a - b; float32, each rounded) and one final multiply by
    float32(1/sqrt(128))."""
    x = np.asarray(x_bf16, dtype=F32)
    k = x.shape[-1]
    assert k % HAD_BLOCK == 0
    v = x.reshape(-1, HAD_BLOCK).copy()
    h = 1
    while h < HAD_BLOCK:
        w = v.reshape(-1, HAD_BLOCK // (2 * h), 2, h)
        a, b = w[:, :, 0, :], w[:, :, 1, :]
        v = np.stack([a + b, a - b], axis=2).reshape(-1, HAD_BLOCK)
        h *= 2
    v = v * F32(1.0 / np.sqrt(128.0))
    return round_to_bf16(v).reshape(x.shape)


def prepare_activation(x_bf16, k_hi, gamma=None, eps=1e-6, hadamard=True) -> dict:
    """[RMSNorm] -> [block-Hadamard 128] -> pack: the fused activation kernel's contract."""
    x = np.asarray(x_bf16, dtype=F32)
    x = x.reshape(-1, x.shape[-1])
    if gamma is not None:
        x = rms_norm_det(x, gamma, eps)
    if hadamard:
        x = block_hadamard_det(x)
    return pack_mixed(x, k_hi)


def linear(px: dict, pw: dict) -> np.ndarray:
    """Y = deq(X) . deq(W)^T in float32 ("dequantise, then float matmul", the parity form of
    tests/test_mixed_gemm.py:149-168 in the reference)."""
    return dequant_mixed(px) @ dequant_mixed(pw).T


# ----------------------------------------------------------------------------------------
# Element-wise steps that the fused pack entry points absorb (inference/forward_pass.py:258-269)
# ----------------------------------------------------------------------------------------
def add_bf16(residual: np.ndarray, x: np.ndarray) -> np.ndarray:
    """bf16 + bf16 as PyTorch computes it: exact float32 sum, one rounding to bf16 (returned as float32)."""
    return round_to_bf16(np.asarray(residual, dtype=F32) + np.asarray(x, dtype=F32))


def exp_det(x: np.ndarray) -> np.ndarray:
    """The float32 exponential of the SiLU prologue, operation by operation (every multiply and add is a
    separately rounded IEEE float32 operation, no fused multiply-add); the CUDA kernel follows the same list:
        x <- min(max(x, -100), 100);  n <- (x * log2(e) + 1.5 * 2^23) - 1.5 * 2^23
        r <- (x - n * 0.693359375) - n * (-2.12194440e-4)
        p <- Horner form of 1 + r + r^2/2 + ... + r^7/5040
        exp <- (p * 2^floor(n/2)) * 2^(n - floor(n/2))"""
    x = np.minimum(np.maximum(np.asarray(x, dtype=F32), F32(-100.0)), F32(100.0))
    magic = F32(12582912.0)
    n = (x * F32(1.44269502162933349609375) + magic) - magic
    r = x - n * F32(0.693359375)
    r = r - n * F32(-2.12194440e-4)
    p = np.full_like(r, F32(1.98412701138295233249664306640625e-4))
    for c in (1.388888922519981861114501953125e-3, 8.3333337679505348205566406250e-3,
              4.16666679084300994873046875e-2, 0.1666666716337203979492187500, 0.5, 1.0, 1.0):
        p = p * r + F32(c)
    ni = n.astype(np.int32)
    h = ni >> 1
    s1 = ((h + 127).astype(np.uint32) << np.uint32(23)).view(F32)
    s2 = ((ni - h + 127).astype(np.uint32) << np.uint32(23)).view(F32)
    with np.errstate(over="ignore"):
        return (p * s1) * s2


def silu_mul_bf16(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """F.silu(gate) * up on bf16 tensors: g / (1 + exp(-g)) in float32 rounded to bf16, then the product rounded
    to bf16 (inference/forward_pass.py:266-269 in the reference), with the exponential of `exp_det`.  torch's own
    float32 exp may differ from it in the last place, which survives the rounding to bf16 for about one element
    in 10^4; the kernel matches this function bit for bit."""
    g = np.asarray(gate, dtype=F32)
    with np.errstate(over="ignore"):
        s = round_to_bf16(g / (F32(1.0) + exp_det(-g)))
    return round_to_bf16(s * np.asarray(up, dtype=F32))


def rope_bf16(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotary position embedding of bf16-valued heads, float32 [..., T, heads, D] with cos / sin float32 [T, D]:
    x * cos + rotate_half(x) * sin with rotate_half(x) = [-x2 | x1], every product and the sum rounded to float32
    on its own, one rounding to bf16 (inference/forward_pass.py:100-109 in the reference; computed there in the
    model dtype, here in float32 like the CUDA kernel and the PyTorch formulation it replaces)."""
    x = x.astype(np.float32)
    d = x.shape[-1]
    rot = np.concatenate([-x[..., d // 2:], x[..., :d // 2]], axis=-1)
    c = cos.astype(np.float32)[:, None, :]
    s_ = sin.astype(np.float32)[:, None, :]
    return round_to_bf16((x * c).astype(np.float32) + (rot * s_).astype(np.float32))
