"""Rotation helpers with the reference's names (inference/rotation.py in the reference).

Only `get_hadamard_matrix` is on the hot path; on B200 the rotation itself is never a matmul:
it is fused into the quantise-and-pack kernel as a 128-point butterfly (plaquant_b200.pack with
hadamard=True).  The matrix is still provided because the reference API hands it around
(`QuantizedLinear(had_matrix=...)`) and tests compare against it.
"""
from __future__ import annotations

import math

import torch

HAD_BLOCK = 128


def get_hadamard_matrix(dim: int, device="cpu") -> torch.Tensor:
    """H / sqrt(dim) with H the Sylvester Hadamard matrix of order `dim` (a power of two), float32,
    so that H @ H.T = I.  Same values as inference/rotation.py:21-29 (scipy.linalg.hadamard order)."""
    assert dim > 0 and (dim & (dim - 1)) == 0, f"dim must be power of 2, got {dim}"
    h = torch.ones(1, 1, dtype=torch.float32, device=device)
    while h.shape[0] < dim:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(dim)


def is_block_hadamard(had_matrix: torch.Tensor, block: int = HAD_BLOCK) -> bool:
    """True if `had_matrix` is H_block/sqrt(block) itself or a block-diagonal repetition of it: the
    only online rotations the fused kernel implements."""
    h = get_hadamard_matrix(block, had_matrix.device)
    if had_matrix.shape == (block, block):
        return bool(torch.allclose(had_matrix.float(), h, atol=1e-6))
    k = had_matrix.shape[0]
    if had_matrix.shape != (k, k) or k % block:
        return False
    ref = torch.block_diag(*([h] * (k // block)))
    return bool(torch.allclose(had_matrix.float(), ref, atol=1e-6))
