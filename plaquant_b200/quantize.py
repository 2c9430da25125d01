"""`QuantizedLinear` with the reference's constructor and call shape (inference/quantize.py:389-480
in the reference), running on the B200 kernels.

In the reference this class holds INT weights and its `set_kernel("cutlass")` path raises
NotImplementedError.  Here the weights are the packed NVFP4 / MXFP8 operands and the only
implementation is the CUDA library ("b200"); asking for "pytorch" or "cutlass" raises, because
there is no fallback path.

    w_main_int    uint8 [N, K_lo/2]   E2M1 codes, two per byte
    w_main_scale  uint8 [N, K_lo/16]  E4M3 scale bytes (row-major)
    w_high_int    uint8 [N, K_hi]     E4M3 codes of the outlier columns (last K_hi of K)
    w_high_scale  uint8 [N, K_hi/32]  E8M0 scale bytes (row-major)
    a_bits / high_bits   "nvfp4" / "mxfp8" (the reference's string format identifiers,
                         promix/quantize/quant_utils.py:29)
    online_had           rotate the activations by the block-Hadamard(128) before quantising
                         (inference/quantize.py:447-448); had_matrix, if given, must be that matrix
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import ops, rotation

SUPPORTED_FP_FORMATS = ("mxfp8", "nvfp4")


def _tile_sf(sf: torch.Tensor) -> torch.Tensor:
    """Row-major scale bytes [rows, n] -> the 128 x 4 tiled order (pure data movement, done once per weight)."""
    rows, n = sf.shape
    rp, npad = -(-rows // 128) * 128, -(-n // 4) * 4
    full = torch.zeros(rp, npad, dtype=torch.uint8, device=sf.device)
    full[:rows, :n] = sf
    t = full.view(rp // 128, 4, 32, npad // 4, 4).permute(0, 3, 2, 1, 4)
    return t.contiguous().view(-1)


class QuantizedLinear:
    """One mixed NVFP4 / MXFP8 linear layer: y = x @ W^T with both operands quantised."""

    def __init__(self, w_main_int: torch.Tensor, w_main_scale: torch.Tensor,
                 w_high_int: Optional[torch.Tensor] = None, w_high_scale: Optional[torch.Tensor] = None,
                 a_bits="nvfp4", high_bits="mxfp8", a_sym: bool = False, grouped: bool = False, groupsize: int = 0,
                 clip_ratio: float = 1.0, online_had: bool = False, had_matrix: Optional[torch.Tensor] = None):
        if a_bits != "nvfp4" or (w_high_int is not None and high_bits != "mxfp8"):
            raise ValueError(f"only a_bits='nvfp4' with high_bits='mxfp8' is implemented, got {a_bits!r}/{high_bits!r}")
        if grouped or groupsize:
            raise ValueError("per-group activation quantisation belongs to the reference's INT path; "
                             "the FP formats carry their own 16/32-element block scales")
        if had_matrix is not None and not rotation.is_block_hadamard(had_matrix):
            raise ValueError("had_matrix must be the normalised block-Hadamard(128) matrix")
        self.w_main_int, self.w_main_scale = w_main_int, w_main_scale
        self.w_high_int, self.w_high_scale = w_high_int, w_high_scale
        self.high_bits_length = w_high_int.shape[1] if w_high_int is not None else 0
        self.a_bits, self.high_bits, self.a_sym = a_bits, high_bits, a_sym
        self.grouped, self.groupsize, self.clip_ratio = grouped, groupsize, clip_ratio
        self.online_had, self.had_matrix = online_had, had_matrix
        self.gemm_impl = "b200"
        self._gemm_w = self._gemv_w = None
        if w_main_int.is_cuda:
            self._prepare()

    # ---- construction from a bf16 weight ---------------------------------------------------------
    @classmethod
    def from_weight(cls, weight: torch.Tensor, high_fraction: float = 1.0 / 32, rotate: bool = True,
                    online_had: bool = True) -> "QuantizedLinear":
        """Round-to-nearest quantisation of W[N, K] (bf16, CUDA) on the device; the last
        ~high_fraction * K input channels (tp.outlier_count) become the MXFP8 subspace, the block-Hadamard(128)
        rotation is applied along K first when `rotate` (promix/quantize/rotation.py:100-116)."""
        k = weight.shape[1]
        from .tp import outlier_count
        k_hi = outlier_count(k, high_fraction)   # int(high_fraction * K), rounded up to the kernels' granularity
        p = ops.pack(weight, k_hi, hadamard=rotate, sf_layout="rowmajor")
        return cls(p.lo_codes, p.lo_sf, p.hi_codes if k_hi else None, p.hi_sf if k_hi else None,
                   online_had=online_had)

    @property
    def out_features(self) -> int:
        return self.w_main_int.shape[0]

    @property
    def in_features(self) -> int:
        return self.w_main_int.shape[1] * 2 + self.high_bits_length

    def _prepare(self) -> None:
        n, k_lo, k_hi = self.out_features, self.w_main_int.shape[1] * 2, self.high_bits_length
        dev = self.w_main_int.device
        empty = torch.zeros(n, 0, dtype=torch.uint8, device=dev)
        hi_c = self.w_high_int.contiguous() if k_hi else empty
        hi_s = self.w_high_scale.contiguous() if k_hi else empty
        lo_c, lo_s = self.w_main_int.contiguous(), self.w_main_scale.contiguous()
        self._gemv_w = ops.PackedMatrix(n, k_lo, k_hi, lo_c, lo_s, hi_c, hi_s, ops.SF_ROWMAJOR)
        self._gemm_w = ops.PackedMatrix(n, k_lo, k_hi, lo_c, _tile_sf(lo_s), hi_c,
                                        _tile_sf(hi_s) if k_hi else torch.zeros(0, dtype=torch.uint8, device=dev),
                                        ops.SF_TILED)
        # forward() declares the weights static (PLQ_GEMV_STATIC_B): the decode GEMV may then fetch them before the
        # kernels launched ahead of it have finished, so everything that produced them must be complete by now
        torch.cuda.current_stream(dev).synchronize()

    def to(self, device):
        self.w_main_int = self.w_main_int.to(device)
        self.w_main_scale = self.w_main_scale.to(device)
        if self.w_high_int is not None:
            self.w_high_int = self.w_high_int.to(device)
            self.w_high_scale = self.w_high_scale.to(device)
        if self.had_matrix is not None:
            self.had_matrix = self.had_matrix.to(device)
        if self.w_main_int.is_cuda:
            self._prepare()
        return self

    def __call__(self, x: torch.Tensor, **kw) -> torch.Tensor:
        return self.forward(x, **kw)

    def quantize_input(self, x: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6):
        """[RMSNorm] -> [Hadamard] -> pack of x[..., K] with tiled scales (what both the GEMM and the tensor-core
        GEMV read)."""
        return ops.pack(x, self.high_bits_length, hadamard=self.online_had, sf_layout="tiled", gamma=norm_weight,
                        eps=eps)

    def forward(self, x, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: bf16 [..., K] (or an already packed PackedMatrix).  `norm_weight` fuses the preceding
        RMSNorm (inference/forward_pass.py:33-39) into the quantisation kernel."""
        if self.gemm_impl != "b200":
            raise ValueError(f"Unknown gemm_impl: {self.gemm_impl}")
        if self._gemm_w is None:
            raise RuntimeError("QuantizedLinear weights are not on a CUDA device; call .to('cuda') (no CPU path)")
        if isinstance(x, ops.PackedMatrix):
            pa, lead = x, (x.rows,)
        else:
            pa, lead = self.quantize_input(x, norm_weight, eps), x.shape[:-1]
        if pa.sf_layout == ops.SF_ROWMAJOR:
            y = ops.gemv(pa, self._gemv_w, out=out)    # a caller-packed operand in the spec's row-major layout
        elif pa.rows <= 16:
            y = ops.gemv_tc(pa, self._gemm_w, out=out, static_weights=True)   # decode: stream the weights once
        else:
            y = ops.mixed_gemm(pa, self._gemm_w, out=out)
        return y.view(*lead, self.out_features)

    def set_kernel(self, impl: str = "b200"):
        """The reference switches between 'pytorch' and 'cutlass' here; this build has one implementation."""
        if impl != "b200":
            raise NotImplementedError(f"gemm_impl {impl!r}: plaquant_b200 only has the sm_100a CUDA path ('b200'), "
                                      "no PyTorch or CUTLASS fallback")
        self.gemm_impl = impl
