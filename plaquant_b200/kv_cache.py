"""NVFP4 / MXFP8 key and value cache on top of the quantise-and-pack kernel.

The reference quantises keys after RoPE: Hadamard over the head dimension, then its activation quantiser on
per-head rows `k.view(-1, head_dim)` with the last `high_bits_length` channels of every head in the
high-precision format (promix/quantize/kv_quant.py:244-279, `k_groupsize != -1` branch; the FP configs
`promix/configs/*-kv4.yaml` name the formats).  With head_dim = 128 that is exactly one row of the pack kernel
per (token, head): block-Hadamard(128), NVFP4 codes + E4M3 scales for the first 128 - k_hi channels, MXFP8 codes +
E8M0 scales for the last k_hi.  The packed cache holds 0.5625 byte per NVFP4 element instead of 2; `dequantize`
returns what the reference's fake quantiser would have put in the cache.  Queries must be rotated by the same
Hadamard (`rotate_heads`), which leaves q . k unchanged up to quantisation error.
"""
from __future__ import annotations

import torch

from . import ops
from .rotation import get_hadamard_matrix


_H = {}


def quantize_heads(x: torch.Tensor, k_hi: int = 0, hadamard: bool = True) -> ops.PackedMatrix:
    """x: bf16 [..., heads, head_dim] (keys after RoPE, or values) -> packed rows, one per (token, head).
    head_dim must be 128 for the rotation; k_hi is the MXFP8 channel count per head (the reference's
    high_bits_length).  The packed formats need (head_dim - k_hi) % 64 == 0 and k_hi % 32 == 0, so with
    head_dim = 128 the choices are 0 (all NVFP4, the default) and 64; the reference's 0.125 * head_dim = 16
    does not fill a 32-element MXFP8 block."""
    d = x.shape[-1]
    if hadamard and d != 128:
        raise ValueError("the block-Hadamard rotation of the cache needs head_dim = 128")
    return ops.pack(x.reshape(-1, d), k_hi, hadamard=hadamard, sf_layout="rowmajor")


def dequantize_heads(p: ops.PackedMatrix, shape) -> torch.Tensor:
    """Packed rows -> bf16 tensor of `shape` ([..., heads, head_dim]); still in the rotated basis."""
    return ops.unpack(p).view(*shape)


def rotate_heads(q: torch.Tensor) -> torch.Tensor:
    """The same normalised Hadamard(128) on the head dimension of the queries (float32 product, one rounding:
    inference/quantize.py:447-448 in the reference)."""
    key = (q.shape[-1], q.device)
    h = _H.get(key)
    if h is None:                      # built once per device: no host-to-device copy inside a CUDA-graph capture
        h = _H[key] = get_hadamard_matrix(q.shape[-1]).to(device=q.device, dtype=torch.float32)
    return (q.float() @ h).to(q.dtype)


HEAD_DIM = 128
ROW_BYTES = HEAD_DIM // 2 + HEAD_DIM // 16      # 64 bytes of E2M1 codes + 8 E4M3 scale bytes per (token, head)


def pack_head_rows(x: torch.Tensor, hadamard: bool) -> torch.Tensor:
    """x: bf16 [..., heads, 128] -> uint8 [..., heads, 72]: the cache's storage form, per (token, head) the 64
    code bytes of the NVFP4 row followed by its 8 scale bytes (keys: `hadamard=True`, the rotation over the head
    dimension; values: False).  0.5625 byte per element instead of 2."""
    if x.shape[-1] != HEAD_DIM:
        raise ValueError("the packed key/value cache needs head_dim = 128")
    p = quantize_heads(x.contiguous(), 0, hadamard=hadamard)
    return torch.cat([p.lo_codes, p.lo_sf], 1).view(*x.shape[:-1], ROW_BYTES)


def unpack_head_rows(rows: torch.Tensor) -> torch.Tensor:
    """uint8 [..., heads, 72] -> bf16 [..., heads, 128]: the values the reference's fake quantiser leaves in its
    cache (keys still in the rotated basis).  All-zero rows (positions not written yet) give zeros."""
    flat = rows.reshape(-1, ROW_BYTES)
    n = flat.shape[0]
    empty = torch.zeros(n, 0, dtype=torch.uint8, device=rows.device)
    p = ops.PackedMatrix(n, HEAD_DIM, 0, flat[:, : HEAD_DIM // 2].contiguous(), flat[:, HEAD_DIM // 2:].contiguous(),
                         empty, empty, ops.SF_ROWMAJOR)
    return ops.unpack(p).view(*rows.shape[:-1], HEAD_DIM)
