"""CPU restatement of the reference's GPTQ inner loop for the block-scaled FP formats.

TEST INFRASTRUCTURE ONLY (never imported by the product package).  Follows, in numpy float32, one column block of
`GPTQ.fasterquant` (promix/quantize/gptq.py:142-205 in the reference) with the FP branch's
`quantize_column_with_frozen_scale` (promix/quantize/quant_utils.py:616-657): the block scale of every column is
frozen beforehand, the Hessian-corrected column is divided by it, clamped, rounded to the nearest element of the
format's grid (ties to the even index) and multiplied back; the error, divided by the diagonal of the inverse
Hessian factor, is folded into the later columns.  Pinned by `tests/golden/gptq_frozen.npz`, which holds the
output of the reference's own GPTQ class on a seeded single-block problem.
"""
from __future__ import annotations

import numpy as np

from . import formats as F

F32 = np.float32


def gptq_block_frozen(w: np.ndarray, hinv: np.ndarray, lo_sf: np.ndarray, hi_sf: np.ndarray, k_hi: int, col0: int,
                      count: int):
    """Columns [col0, col0 + count) of float32 `w` [rows, k] (not modified).  Returns (q [rows, count] float32,
    err [rows, count] float32, codes [rows, count] uint8: E2M1 with bit 3 = sign for columns < k - k_hi, E4M3 with
    bit 7 = sign for the rest)."""
    rows, k = w.shape
    k_lo = k - k_hi
    w1 = np.array(w[:, col0:col0 + count], dtype=F32)
    h1 = np.asarray(hinv[col0:col0 + count, col0:col0 + count], dtype=F32)
    q1 = np.zeros_like(w1)
    e1 = np.zeros_like(w1)
    c1 = np.zeros(w1.shape, dtype=np.uint8)
    for i in range(count):
        col = col0 + i
        wi = w1[:, i].copy()
        if col < k_lo:                                   # quant_utils.py:640-657, fmt "nvfp4"
            s = F.E4M3_POS[lo_sf[:, col // 16]]
            x = np.clip(wi / s, -F.E2M1_MAX, F.E2M1_MAX)
            idx, neg = F.round_to_grid_rne(x, F.E2M1_POS)
            mag = F.E2M1_POS[idx]
            code = idx | (neg.astype(np.uint8) << 3)
        else:                                            # fmt "mxfp8"
            s = F.e8m0_value(hi_sf[:, (col - k_lo) // 32])
            with np.errstate(over="ignore"):
                x = np.clip(wi / s, -F.E4M3_MAX, F.E4M3_MAX)
            idx, neg = F.round_to_grid_rne(x, F.E4M3_POS)
            mag = F.E4M3_POS[idx]
            code = idx | (neg.astype(np.uint8) << 7)
        q = (np.where(neg, -mag, mag).astype(F32) * s).astype(F32)
        d = h1[i, i]
        err = ((wi - q) / d).astype(F32)                 # gptq.py:198-199
        q1[:, i], e1[:, i], c1[:, i] = q, err, code
        w1[:, i:] = w1[:, i:] - (err[:, None] * h1[i, i:][None, :]).astype(F32)    # gptq.py:200
    return q1, e1, c1
