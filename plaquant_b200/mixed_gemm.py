"""Module-level GEMM entry points in the call shape of the reference's `mixed_gemm` extension
(kernels/mixed_gemm/mixed_gemm.cu:346-350, 376-410 in the reference): two K phases, one output.

The reference's twelve-tensor signature carries per-token / per-channel scales, zero points and
column sums of its INT formats.  The FP block-scaled formats have none of those (no global,
per-token or per-channel scale exists on the FP path), so the four zero-point / column-sum
arguments must be None and the scale arguments carry the block-scale bytes in the tiled layout.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def fused_mixed_gemm(A_main: torch.Tensor, B_main: torch.Tensor, A_high: Optional[torch.Tensor],
                     B_high: Optional[torch.Tensor], s_x_m: torch.Tensor, s_w_m: torch.Tensor,
                     neg_zero_m=None, colsum_m=None, s_x_h: Optional[torch.Tensor] = None,
                     s_w_h: Optional[torch.Tensor] = None, neg_zero_h=None, colsum_h=None) -> torch.Tensor:
    """Y[M, N] (bf16) = deq(A_main) deq(B_main)^T + deq(A_high) deq(B_high)^T in one kernel.

    A_main u8 [M, K_lo/2] / B_main u8 [N, K_lo/2]: E2M1 codes;  s_x_m / s_w_m: E4M3 scale bytes, tiled;
    A_high u8 [M, K_hi]   / B_high u8 [N, K_hi]:   E4M3 codes;  s_x_h / s_w_h: E8M0 scale bytes, tiled.
    Activations may be [B, S, K/2]: the output is reshaped back, as the reference does (mixed_gemm.cu:282-284).
    """
    for name, v in (("neg_zero_m", neg_zero_m), ("colsum_m", colsum_m), ("neg_zero_h", neg_zero_h),
                    ("colsum_h", colsum_h)):
        if v is not None:
            raise ValueError(f"{name} belongs to the INT formats; NVFP4/MXFP8 operands are symmetric (pass None)")
    lead = A_main.shape[:-1]
    a_main = A_main.reshape(-1, A_main.shape[-1]).contiguous()
    m, n = a_main.shape[0], B_main.shape[0]
    k_lo = a_main.shape[1] * 2
    dev = a_main.device
    if A_high is None:
        a_high = torch.zeros(m, 0, dtype=torch.uint8, device=dev)
        b_high = torch.zeros(n, 0, dtype=torch.uint8, device=dev)
        s_x_h = s_w_h = torch.zeros(0, dtype=torch.uint8, device=dev)
    else:
        a_high, b_high = A_high.reshape(m, -1).contiguous(), B_high.contiguous()
    k_hi = a_high.shape[1]
    pa = ops.PackedMatrix(m, k_lo, k_hi, a_main, s_x_m.reshape(-1), a_high, s_x_h.reshape(-1), ops.SF_TILED)
    pb = ops.PackedMatrix(n, k_lo, k_hi, B_main.contiguous(), s_w_m.reshape(-1), b_high, s_w_h.reshape(-1), ops.SF_TILED)
    return ops.mixed_gemm(pa, pb).view(*lead, n)


# the reference exports five numbered variants of the same fused operation with identical signatures
fused_mixed_gemm_v2 = fused_mixed_gemm_v3 = fused_mixed_gemm_v4 = fused_mixed_gemm_v5 = fused_mixed_gemm


# `plaquant_b200.mixed_gemm` is both this module (the reference's module name) and, at package level,
# the packed-operand GEMM function; importing the module must not hide the function, so the module
# object itself is callable and forwards to it.
import sys as _sys
import types as _types


class _CallableModule(_types.ModuleType):
    def __call__(self, *args, **kwargs):
        return ops.mixed_gemm(*args, **kwargs)


_sys.modules[__name__].__class__ = _CallableModule
