"""Torch-tensor front end of the C-ABI kernels.  PyTorch owns device memory and streams; all
arithmetic happens in libplq_b200.so."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

SF_ROWMAJOR, SF_TILED = 0, 1
_LAYOUTS = {"rowmajor": SF_ROWMAJOR, "tiled": SF_TILED, SF_ROWMAJOR: SF_ROWMAJOR, SF_TILED: SF_TILED}


@dataclass
class PackedMatrix:
    """rows x (k_lo + k_hi) matrix in packed form (layout: include/plq.h)."""
    rows: int
    k_lo: int
    k_hi: int
    lo_codes: torch.Tensor   # u8 [rows, k_lo/2]
    lo_sf: torch.Tensor      # u8, row-major [rows, k_lo/16] or tiled (flat)
    hi_codes: torch.Tensor   # u8 [rows, k_hi]
    hi_sf: torch.Tensor      # u8, row-major [rows, k_hi/32] or tiled (flat)
    sf_layout: int

    @property
    def k(self) -> int:
        return self.k_lo + self.k_hi

    @property
    def device(self):
        return self.lo_codes.device

    def nbytes(self) -> int:
        return sum(t.numel() for t in (self.lo_codes, self.lo_sf, self.hi_codes, self.hi_sf))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: plaquant_b200 has no CPU path")


_status_words = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the GEMM kernel writes PLQ_DEV_TIMEOUT into when a bounded wait runs out."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status_words:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the status word must exist before a CUDA-graph capture: run the op once eagerly first")
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status_words[key]


def check_device_status(device=None) -> None:
    """Synchronising read of the status word; raises PlqError if a kernel reported a timeout."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    v = int(w.item())
    if v != 0:
        w.zero_()
        _lib.check(v)


def alloc_packed(rows: int, k: int, k_hi: int, sf_layout, device) -> PackedMatrix:
    layout = _LAYOUTS[sf_layout]
    k_lo = k - k_hi
    L = _lib.lib()
    u8 = dict(dtype=torch.uint8, device=device)
    if layout == SF_TILED:
        # Padding.  Rows beyond `rows` inside the last 128-row group only ever scale output rows that are not stored,
        # so they may hold anything.  Scales beyond K inside the last chunk of four meet zero codes in an MMA, and
        # 0 x NaN is NaN: they must be zero.  K_lo / 16 is always a multiple of four; K_hi / 32 need not be.
        lo_sf = torch.empty(L.plq_sf_tiled_bytes(rows, k_lo // 16), **u8)
        hi_bytes = L.plq_sf_tiled_bytes(rows, k_hi // 32)
        hi_sf = torch.zeros(hi_bytes, **u8) if (k_hi // 32) % 4 else torch.empty(hi_bytes, **u8)
    else:
        lo_sf = torch.empty(rows, k_lo // 16, **u8)
        hi_sf = torch.empty(rows, k_hi // 32, **u8)
    return PackedMatrix(rows, k_lo, k_hi, torch.empty(rows, k_lo // 2, **u8), lo_sf,
                        torch.empty(rows, k_hi, **u8), hi_sf, layout)


def pack(x: torch.Tensor, k_hi: int, hadamard: bool = False, sf_layout="tiled",
         gamma: Optional[torch.Tensor] = None, eps: float = 1e-6,
         out: Optional[PackedMatrix] = None) -> PackedMatrix:
    """[RMSNorm(gamma, eps)] -> [block-Hadamard 128] -> NVFP4 | MXFP8 pack of bf16 x[..., K]."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("x must be bfloat16")
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    p = out if out is not None else alloc_packed(rows, k, k_hi, sf_layout, x.device)
    L = _lib.lib()
    with torch.cuda.device(x.device):
        if gamma is None:
            st = L.plq_pack(_ptr(x2), rows, k, k_hi, int(hadamard), _ptr(p.lo_codes), _ptr(p.lo_sf),
                            _ptr(p.hi_codes), _ptr(p.hi_sf), p.sf_layout, _stream(x.device))
        else:
            _require_cuda(gamma, "gamma")
            if gamma.dtype != torch.bfloat16 or gamma.numel() != k:
                raise TypeError("gamma must be bfloat16 [K]")
            st = L.plq_rmsnorm_pack(_ptr(x2), _ptr(gamma.contiguous()), float(eps), rows, k, k_hi, int(hadamard),
                                    _ptr(p.lo_codes), _ptr(p.lo_sf), _ptr(p.hi_codes), _ptr(p.hi_sf), p.sf_layout,
                                    _stream(x.device))
    _lib.check(st)
    return p


def silu_mul_pack(gate_up: torch.Tensor, k_hi: int, hadamard: bool = True, sf_layout="tiled",
                  out: Optional[PackedMatrix] = None) -> PackedMatrix:
    """SiLU(gate) * up -> [block-Hadamard 128] -> pack, for gate_up[..., 2K] = [gate | up] (bf16): the input of
    down_proj without the two element-wise passes (inference/forward_pass.py:266-269 in the reference)."""
    _require_cuda(gate_up, "gate_up")
    if gate_up.dtype != torch.bfloat16 or gate_up.shape[-1] % 2:
        raise TypeError("gate_up must be bfloat16 [..., 2K]")
    k = gate_up.shape[-1] // 2
    g2 = gate_up.reshape(-1, 2 * k)
    if not g2.is_contiguous():
        g2 = g2.contiguous()
    rows = g2.shape[0]
    p = out if out is not None else alloc_packed(rows, k, k_hi, sf_layout, gate_up.device)
    with torch.cuda.device(gate_up.device):
        st = _lib.lib().plq_silu_mul_pack(_ptr(g2), g2.data_ptr() + 2 * k if rows else None, 2 * k, rows, k, k_hi,
                                          int(hadamard), _ptr(p.lo_codes), _ptr(p.lo_sf), _ptr(p.hi_codes),
                                          _ptr(p.hi_sf), p.sf_layout, _stream(gate_up.device))
    _lib.check(st)
    return p


def add_rmsnorm_pack(x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float, k_hi: int,
                     hadamard: bool = True, sf_layout="tiled", out: Optional[PackedMatrix] = None):
    """h = residual + x (bf16) -> RMSNorm(gamma, eps) -> [block-Hadamard 128] -> pack.  Returns (h, packed):
    the residual add, the norm and the quantiser of the next linear in one pass
    (inference/forward_pass.py:258-264 in the reference)."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or x.shape != residual.shape:
        raise TypeError("x and residual must be bfloat16 tensors of one shape")
    k = x.shape[-1]
    x2, r2 = x.reshape(-1, k).contiguous(), residual.reshape(-1, k).contiguous()
    rows = x2.shape[0]
    h = torch.empty_like(x2)
    p = out if out is not None else alloc_packed(rows, k, k_hi, sf_layout, x.device)
    if gamma.dtype != torch.bfloat16 or gamma.numel() != k:
        raise TypeError("gamma must be bfloat16 [K]")
    with torch.cuda.device(x.device):
        st = _lib.lib().plq_add_rmsnorm_pack(_ptr(x2), _ptr(r2), _ptr(h), _ptr(gamma.contiguous()), float(eps), rows, k,
                                             k_hi, int(hadamard), _ptr(p.lo_codes), _ptr(p.lo_sf), _ptr(p.hi_codes),
                                             _ptr(p.hi_sf), p.sf_layout, _stream(x.device))
    _lib.check(st)
    return h.view(x.shape), p


def allreduce_add_rmsnorm_pack(peer, rows: int, residual: torch.Tensor, gamma: torch.Tensor, eps: float, k_hi: int,
                               hadamard: bool = True, sf_layout="tiled", out: Optional[PackedMatrix] = None):
    """Tensor-parallel add_rmsnorm_pack: x = sum over the ranks of `peer.buffer(rows)` (each rank's partial output
    of a row-parallel linear, already written on its stream), h = residual + x, RMSNorm, rotation, pack - one
    kernel reading the peers' memory over NVLink.  `peer` is a tp.PeerReduce; returns (h, packed)."""
    _require_cuda(residual, "residual")
    k = residual.shape[-1]
    r2 = residual.reshape(-1, k).contiguous()
    if r2.shape[0] != rows or rows > peer.rows or k != peer.k or residual.dtype != torch.bfloat16:
        raise TypeError("residual must be bfloat16 [rows, k] matching the peer buffers")
    if gamma.dtype != torch.bfloat16 or gamma.numel() != k:
        raise TypeError("gamma must be bfloat16 [K]")
    h = torch.empty_like(r2)
    p = out if out is not None else alloc_packed(rows, k, k_hi, sf_layout, residual.device)
    with torch.cuda.device(residual.device):
        st = _lib.lib().plq_allreduce_add_rmsnorm_pack(
            _ptr(peer.peer_x[peer.next]), _ptr(peer.peer_flags), _ptr(peer.flags), _ptr(peer.sync), peer.world, peer.rank,
            peer.next, _ptr(r2), _ptr(h), _ptr(gamma.contiguous()), float(eps), rows, k, k_hi, int(hadamard),
            _ptr(p.lo_codes), _ptr(p.lo_sf), _ptr(p.hi_codes), _ptr(p.hi_sf), p.sf_layout,
            _ptr(status_word(residual.device)), _stream(residual.device))
    _lib.check(st)
    peer.next ^= 1
    peer.calls += 1
    return h.view(residual.shape), p


def reduce_scatter_add_rmsnorm_pack(sr, rows_total: int, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                                    hadamard: bool = True):
    """Scattered tensor-parallel add_rmsnorm_pack for prefill batches.  Every rank has written its partial output
    [rows_total, k] of a row-parallel linear into `sr.buffer(rows_total)`; this rank sums its slice of
    rows_total / world rows over the ranks, adds `residual` (its slice of the residual stream), normalises, rotates,
    quantises, and stores the packed rows into every rank's packed buffer.  `sr` is a tp.ScatterReduce.  Returns
    (h, packed): the new residual slice and the packed activations of ALL rows (complete when the kernel ends)."""
    _require_cuda(residual, "residual")
    k = residual.shape[-1]
    r2 = residual.reshape(-1, k).contiguous()
    if rows_total % sr.world != 0 or rows_total > sr.rows:
        raise ValueError(f"{rows_total} rows do not split over {sr.world} ranks within buffers of {sr.rows} rows")
    per = rows_total // sr.world
    if r2.shape[0] != per or k != sr.k or residual.dtype != torch.bfloat16:
        raise TypeError("residual must be this rank's bfloat16 [rows_total / world, k] slice")
    if gamma.dtype != torch.bfloat16 or gamma.numel() != k:
        raise TypeError("gamma must be bfloat16 [K]")
    h = torch.empty_like(r2)
    p, lo_rm, hi_rm = sr.packed(sr.next, rows_total)
    with torch.cuda.device(residual.device):
        st = _lib.lib().plq_reduce_scatter_add_rmsnorm_pack(
            _ptr(sr.peer_x[sr.next]), _ptr(sr.peer_flags), _ptr(sr.flags), _ptr(sr.sync), sr.world, sr.rank, sr.next,
            _ptr(sr.out_tbl[sr.next]), sr.rank * per, rows_total, _ptr(r2), _ptr(h), _ptr(gamma.contiguous()), float(eps),
            per, k, sr.k_hi, int(hadamard), _ptr(p.lo_codes), _ptr(lo_rm), _ptr(p.hi_codes), _ptr(hi_rm),
            _ptr(p.lo_sf), _ptr(p.hi_sf), _ptr(status_word(residual.device)), _stream(residual.device))
    _lib.check(st)
    sr.next ^= 1
    sr.calls += 1
    return h, p


def rope_kv_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int, kv_heads: int,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, pos) -> torch.Tensor:
    """RoPE on the query and key heads of `qkv` (bf16 [B, T, (heads + 2 kv_heads) * 128]) and append of the rotated
    keys and the values to `k_cache` / `v_cache` (bf16 [B, T_max, kv_heads, 128]) at positions pos .. pos + T - 1, one
    kernel.  `cos` / `sin`: float32 with T * 128 elements (one row per new position).  `pos`: an int, or a device
    int64 tensor with one element (read by the kernel: a captured decode step appends at the current position).
    Returns the rotated queries, bf16 [B, T, heads, 128]."""
    _require_cuda(qkv, "qkv")
    b, t, n = qkv.shape
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous() or n != (heads + 2 * kv_heads) * 128:
        raise TypeError("qkv must be contiguous bfloat16 [B, T, (heads + 2 kv_heads) * 128]")
    for name, c in (("cos", cos), ("sin", sin)):
        if c.dtype != torch.float32 or c.numel() != t * 128 or not c.is_contiguous():
            raise TypeError(f"{name} must be contiguous float32 with T * 128 elements")
    t_max = k_cache.shape[1]
    for name, c in (("k_cache", k_cache), ("v_cache", v_cache)):
        if c.dtype != torch.bfloat16 or not c.is_contiguous() or tuple(c.shape) != (b, t_max, kv_heads, 128):
            raise TypeError(f"{name} must be contiguous bfloat16 [B, T_max, kv_heads, 128]")
    on_device = isinstance(pos, torch.Tensor)
    if on_device and (pos.dtype != torch.int64 or pos.numel() != 1 or pos.device != qkv.device):
        raise TypeError("pos must be an int or a one-element int64 tensor on the device of qkv")
    q = torch.empty(b, t, heads, 128, dtype=torch.bfloat16, device=qkv.device)
    with torch.cuda.device(qkv.device):
        st = _lib.lib().plq_rope_kv_append(_ptr(qkv), n, _ptr(cos), _ptr(sin), b, t, heads, kv_heads, 128, _ptr(q),
                                           _ptr(k_cache), _ptr(v_cache), t_max, _ptr(pos) if on_device else None,
                                           0 if on_device else int(pos), _ptr(status_word(qkv.device)), _stream(qkv.device))
    _lib.check(st)
    return q


def unpack(p: PackedMatrix) -> torch.Tensor:
    """Dequantise to bf16 [rows, K]: the value the reference's fake quantiser returns."""
    y = torch.empty(p.rows, p.k, dtype=torch.bfloat16, device=p.device)
    with torch.cuda.device(p.device):
        st = _lib.lib().plq_unpack(_ptr(p.lo_codes), _ptr(p.lo_sf), _ptr(p.hi_codes), _ptr(p.hi_sf), p.sf_layout,
                                   p.rows, p.k_lo, p.k_hi, _ptr(y), _stream(p.device))
    _lib.check(st)
    return y


def _check_pair(a: PackedMatrix, b: PackedMatrix, layout: int) -> None:
    if (a.k_lo, a.k_hi) != (b.k_lo, b.k_hi):
        raise ValueError(f"K split mismatch: activations {a.k_lo}+{a.k_hi}, weights {b.k_lo}+{b.k_hi}")
    if a.sf_layout != layout or b.sf_layout != layout:
        raise ValueError("scale buffers are in the wrong layout for this kernel")


GEMM_VARIANTS = {None: 0, "auto": 0, "128x128": 1, "128x256": 2, "pair256x256": 3}


def mixed_gemm(a: PackedMatrix, b: PackedMatrix, out: Optional[torch.Tensor] = None,
               variant: Optional[str] = None) -> torch.Tensor:
    """y[m, n] = deq(a) @ deq(b).T, bf16, via the fused tcgen05 kernel (tiled scale layout).
    `variant` picks the tile shape ("128x128", "128x256", "pair256x256"); default: heuristic."""
    _check_pair(a, b, SF_TILED)
    y = out if out is not None else torch.empty(a.rows, b.rows, dtype=torch.bfloat16, device=a.device)
    L = _lib.lib()
    args = [_ptr(a.lo_codes), _ptr(a.lo_sf), _ptr(a.hi_codes), _ptr(a.hi_sf),
            _ptr(b.lo_codes), _ptr(b.lo_sf), _ptr(b.hi_codes), _ptr(b.hi_sf),
            a.rows, b.rows, a.k_lo, a.k_hi, _ptr(y), y.stride(0), _ptr(status_word(a.device)), _stream(a.device)]
    with torch.cuda.device(a.device):
        st = L.plq_mixed_gemm_variant(*args, GEMM_VARIANTS[variant])
    _lib.check(st)
    return y


_gemv_ws = {}


def gemv_workspace(device, n: int) -> torch.Tensor:
    """Per (device, stream) zero-initialised scratch for the GEMV's K-slice reduction; grown on demand.
    Calls on one stream are ordered, so they can share it."""
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev))
    need = _lib.lib().plq_gemv_workspace_bytes(n)
    ws = _gemv_ws.get(key)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the GEMV workspace must exist before a CUDA-graph capture: call gemv() (or "
                               "gemv_workspace()) once on this stream before capturing")
        ws = torch.zeros(need, dtype=torch.uint8, device=f"cuda:{key[0]}")
        _gemv_ws[key] = ws
    return ws


def gemv(a: PackedMatrix, b: PackedMatrix, out: Optional[torch.Tensor] = None,
         workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode path, a.rows <= 8 (row-major scale layout)."""
    _check_pair(a, b, SF_ROWMAJOR)
    y = out if out is not None else torch.empty(a.rows, b.rows, dtype=torch.bfloat16, device=a.device)
    ws = workspace if workspace is not None else gemv_workspace(a.device, b.rows)
    with torch.cuda.device(a.device):
        st = _lib.lib().plq_gemv(_ptr(a.lo_codes), _ptr(a.lo_sf), _ptr(a.hi_codes), _ptr(a.hi_sf),
                                 _ptr(b.lo_codes), _ptr(b.lo_sf), _ptr(b.hi_codes), _ptr(b.hi_sf),
                                 a.rows, b.rows, a.k_lo, a.k_hi, _ptr(y), y.stride(0), _ptr(ws), ws.numel(),
                                 _stream(a.device))
    _lib.check(st)
    return y



GEMV_STATIC_B = 1


def gemv_tc(a: PackedMatrix, b: PackedMatrix, out: Optional[torch.Tensor] = None,
            static_weights: bool = False) -> torch.Tensor:
    """Decode path on the tensor cores, a.rows <= 16; both operands with the tiled scale layout of the GEMM.
    `static_weights`: b was complete long before this call (packed at load time), so the kernel may start
    fetching it while the previous kernel of the stream is still running."""
    _check_pair(a, b, SF_TILED)
    y = out if out is not None else torch.empty(a.rows, b.rows, dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        st = _lib.lib().plq_gemv_tc(_ptr(a.lo_codes), _ptr(a.lo_sf), _ptr(a.hi_codes), _ptr(a.hi_sf),
                                    _ptr(b.lo_codes), _ptr(b.lo_sf), _ptr(b.hi_codes), _ptr(b.hi_sf),
                                    a.rows, b.rows, a.k_lo, a.k_hi, _ptr(y), y.stride(0),
                                    _ptr(status_word(a.device)), GEMV_STATIC_B if static_weights else 0,
                                    _stream(a.device))
    _lib.check(st)
    return y
