"""GPTQ weight rounding for the NVFP4 / MXFP8 formats with block scales frozen on the original weight - the
reference's `GPTQ.fasterquant` FP path (promix/quantize/gptq.py:57-221 there; spec "fixed-block-scale,
Hessian-conditioned element rounding") - with the per-column inner loop on the GPU (`plq_gptq_block_frozen`).

The Hessian comes from calibration activations, which are not available offline: `hessian_from_inputs`
accumulates it from whatever inputs the caller has (the reference's `add_batch`, gptq.py:40-50), and the tests
drive the path with synthetic ones.  The result is a packed weight ready for `QuantizedLinear`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops


def hessian_from_inputs(x: torch.Tensor, h: Optional[torch.Tensor] = None, nsamples: int = 0) -> Tuple[torch.Tensor, int]:
    """Running H = 2/n * sum x^T x over calibration rows x[..., K] (gptq.py:40-50 in the reference)."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    if h is None:
        h = torch.zeros(x2.shape[1], x2.shape[1], dtype=torch.float32, device=x.device)
    batch = 1 if x.dim() == 2 else x.shape[0]
    h = h * (nsamples / (nsamples + batch))
    nsamples += batch
    xs = x2.t() * (2.0 / nsamples) ** 0.5
    return h + xs @ xs.t(), nsamples


def inverse_hessian_factor(h: torch.Tensor, percdamp: float = 0.01) -> torch.Tensor:
    """Upper Cholesky factor of the damped inverse Hessian (gptq.py:129-141): dead columns get a unit diagonal."""
    h = h.clone()
    dead = torch.diag(h) == 0
    h[dead, dead] = 1
    idx = torch.arange(h.shape[0], device=h.device)
    h[idx, idx] += percdamp * torch.mean(torch.diag(h))
    l = torch.linalg.cholesky(h)
    return torch.linalg.cholesky(torch.cholesky_inverse(l), upper=True).contiguous()


def gptq_block(w: torch.Tensor, hinv: torch.Tensor, lo_sf: torch.Tensor, hi_sf: torch.Tensor, k_hi: int, col0: int,
               count: int, q: torch.Tensor, codes: torch.Tensor) -> torch.Tensor:
    """One column block through the kernel; writes q[:, col0:col0+count] and codes, returns err [rows, count]."""
    rows, k = w.shape
    if w.dtype != torch.float32 or hinv.dtype != torch.float32 or w.stride(1) != 1 or q.stride(1) != 1:
        raise TypeError("w, hinv and q must be float32 with unit column stride")
    if hinv.stride(1) != 1:                      # e.g. the transposed view torch.linalg.cholesky(upper=True) returns
        hinv = hinv.contiguous()
    err = torch.empty(rows, count, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        st = _lib.lib().plq_gptq_block_frozen(w.data_ptr(), w.stride(0), hinv.data_ptr(), hinv.stride(0),
                                              ops._ptr(lo_sf), ops._ptr(hi_sf), rows, k, k_hi, col0, count,
                                              q.data_ptr(), q.stride(0), err.data_ptr(), codes.data_ptr(),
                                              ops._stream(w.device))
    _lib.check(st)
    return err


@torch.no_grad()
def gptq_quantize_frozen(weight: torch.Tensor, hessian: torch.Tensor, k_hi: int, blocksize: int = 128,
                         percdamp: float = 0.01, hinv: Optional[torch.Tensor] = None):
    """weight [N, K] (bf16-valued; already rotated if the layer rotates), hessian [K, K] float32 of the layer's
    (rotated) inputs.  Returns (PackedMatrix with row-major scales, dequantised float32 weight).

    The block scales are those round-to-nearest packing gives the original weight (frozen); every column is
    rounded with the earlier columns' errors folded in (the reference's loop); the columns behind a block receive
    the block's errors through one matmul."""
    if not weight.is_cuda:
        raise RuntimeError("gptq_quantize_frozen needs a CUDA tensor: plaquant_b200 has no CPU path")
    n, k = weight.shape
    if blocksize < 1 or blocksize > 128:
        raise ValueError("blocksize must be 1..128")
    frozen = ops.pack(weight.to(torch.bfloat16), k_hi, hadamard=False, sf_layout="rowmajor")   # scales of the original weight
    w = weight.float().clone()
    dead = torch.diag(hessian) == 0
    w[:, dead] = 0
    if hinv is None:
        hinv = inverse_hessian_factor(hessian, percdamp)
    q = torch.zeros_like(w)
    codes = torch.zeros(n, k, dtype=torch.uint8, device=w.device)
    for i1 in range(0, k, blocksize):
        count = min(blocksize, k - i1)
        err = gptq_block(w, hinv, frozen.lo_sf, frozen.hi_sf, k_hi, i1, count, q, codes)
        if i1 + count < k:
            w[:, i1 + count:] -= err @ hinv[i1:i1 + count, i1 + count:]          # gptq.py:207
    k_lo = k - k_hi
    lo = codes[:, :k_lo]
    packed = ops.PackedMatrix(n, k_lo, k_hi, (lo[:, 0::2] | (lo[:, 1::2] << 4)).contiguous(), frozen.lo_sf,
                              codes[:, k_lo:].contiguous(), frozen.hi_sf, ops.SF_ROWMAJOR)
    return packed, q
