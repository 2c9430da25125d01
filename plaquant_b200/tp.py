"""Megatron-style tensor-parallel partition maps for the mixed NVFP4 / MXFP8 linears.

Column-parallel linears (fused QKV, fused gate_up) shard N and need no exchange; row-parallel
linears (O, down) shard K, every rank multiplies its K shard and the partial outputs are summed by
one all-reduce.  The K split must respect the kernels' granularity on every rank: a shard is a
whole number of 128-column Hadamard blocks (so the rotation stays rank-local), its NVFP4 part a
multiple of 64 and its MXFP8 part a multiple of 32.  Each rank therefore designates ITS OWN last
`outlier_count(K_r)` columns as the outlier subspace; the CPU oracle takes the same map, so parity
stays exact per tensor-parallel degree.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


def outlier_count(k: int, fraction: float = 1.0 / 32) -> int:
    """Smallest multiple of 32 that is >= fraction * k and leaves an NVFP4 part divisible by 64."""
    k_hi = -(-int(round(k * fraction)) // 32) * 32
    while (k - k_hi) % 64 != 0:
        k_hi += 32
    if k_hi > k:
        raise ValueError(f"K = {k} cannot be split into NVFP4 % 64 and MXFP8 % 32 parts")
    return k_hi


def shard_range(total: int, rank: int, size: int, multiple: int = 1) -> slice:
    """Contiguous equal shard [lo, hi) of `total` for `rank`; every shard is a multiple of `multiple`."""
    if total % (size * multiple) != 0:
        raise ValueError(f"{total} is not divisible into {size} shards that are multiples of {multiple}")
    per = total // size
    return slice(rank * per, (rank + 1) * per)


def column_parallel_rows(n: int, rank: int, size: int) -> slice:
    """Output rows (N) of a column-parallel weight owned by `rank` (multiple of 8: GEMM store width)."""
    return shard_range(n, rank, size, 8)


def row_parallel_cols(k: int, rank: int, size: int) -> slice:
    """Input columns (K) of a row-parallel weight owned by `rank` (whole 128-column rotation blocks)."""
    return shard_range(k, rank, size, 128)


@dataclass
class TPContext:
    """Rank / size / process group of the tensor-parallel job (size 1 = no communication)."""
    rank: int = 0
    size: int = 1
    group: Optional[object] = None

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks (NCCL over NVLink on GPUs, gloo in the CPU tests); in place."""
        if self.size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    @classmethod
    def from_env(cls) -> "TPContext":
        if dist.is_available() and dist.is_initialized():
            return cls(dist.get_rank(), dist.get_world_size(), None)
        return cls()


class PeerReduce:
    """Peer-memory plumbing of the fused all-reduce + residual + RMSNorm-quant kernel
    (`ops.allreduce_add_rmsnorm_pack`): two symmetric bf16 [rows, k] buffer sets per rank for the partial outputs,
    a symmetric int32 flag array, a local call counter, and device arrays with every rank's addresses.  Built on
    torch.distributed's symmetric memory (CUDA IPC / VMM mappings of the other ranks' allocations on one node);
    the kernel itself only does plain peer loads and flag stores, so the mappings are requested without an NVLink
    multicast binding (TORCH_SYMM_MEM_DISABLE_MULTICAST).

    Invariant.  Consecutive fused calls alternate between the two buffer sets, starting with set 0 (`next`), on
    every rank alike.  That alone keeps a fast rank from overwriting what a slower peer still reads: before rank r
    writes set b again it has completed the call in between, and that call waited until every peer had announced
    it - which a peer does only after finishing its previous call, the one that read set b.  No other collective
    is needed between the calls.  A decode step that is captured in a CUDA graph freezes `next` per call site, so
    the step must contain an even number of fused calls (`calls` counts them; `ResQForwardB200.generate` checks);
    the kernel verifies the set against its own call count and reports PLQ_DEV_PROTOCOL otherwise."""

    def __init__(self, rows: int, k: int, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # before the first symmetric allocation
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.rows, self.k, self.device = rows, k, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.x = symm_mem.empty(2, rows, k, dtype=torch.bfloat16, device=self.device)
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=self.device)
        self.x.zero_()
        self.flags.zero_()
        hx = symm_mem.rendezvous(self.x, group)
        hf = symm_mem.rendezvous(self.flags, group)
        self._handles = (hx, hf)                         # keep the mappings alive
        xs = [int(p) for p in hx.buffer_ptrs]
        fs = [int(p) for p in hf.buffer_ptrs]
        per_buf = rows * k * 2
        self.peer_x = [torch.tensor([p + b * per_buf for p in xs], dtype=torch.int64, device=self.device) for b in range(2)]
        self.peer_flags = torch.tensor(fs, dtype=torch.int64, device=self.device)
        self.sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.next = 0                                     # buffer set of the next fused call
        self.calls = 0                                    # fused calls issued (or captured) so far
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                               # nobody signals before every rank has zeroed its flags

    def buffer(self, rows: int) -> torch.Tensor:
        """The [rows, k] view of the buffer the next fused reduction will read: the row-parallel linear writes
        its output here."""
        return self.x[self.next, :rows]


class ScatterReduce:
    """Peer-memory plumbing of the scattered form of the fused reduction (`ops.reduce_scatter_add_rmsnorm_pack`), the
    prefill counterpart of `PeerReduce`: rank r sums rows [r * R / world, (r + 1) * R / world) of the ranks' partial
    outputs, keeps the residual stream for those rows only, and stores their packed codes and scale bytes into the
    packed-activation buffer of every rank (reduce-scatter in, all-gather of the 4.5-bit form out, both inside the
    RMSNorm-quant kernel, by plain peer loads and stores).  Per rank: two symmetric bf16 [rows, k] buffer sets for
    the partial outputs, two symmetric packed-activation sets (codes, and scale bytes row-major), a symmetric flag
    array, and two local sets of tiled scale buffers that the call fills from the gathered row-major ones.

    The sets alternate from call to call as in `PeerReduce`.  The kernel ends only after every rank has announced
    that its rows are in place everywhere, so when a call has completed on a rank, that rank's packed buffer is
    whole and no peer reads its partial sums of that call any more."""

    def __init__(self, rows: int, k: int, k_hi: int, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        group = group if group is not None else dist.group.WORLD
        self.rows, self.k, self.k_hi, self.device = rows, k, k_hi, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        k_lo = k - k_hi
        L = _lib.lib()
        al = lambda n: -(-n // 256) * 256
        # gathered form of the scale bytes: row-major (whole lines per warp over NVLink); each rank re-tiles locally
        sizes = [rows * k_lo // 2, rows * (k_lo // 16), rows * k_hi, rows * (k_hi // 32)]
        u8 = dict(dtype=torch.uint8, device=self.device)
        self.sf_tiled = [(torch.zeros(L.plq_sf_tiled_bytes(rows, k_lo // 16), **u8),
                          torch.zeros(L.plq_sf_tiled_bytes(rows, k_hi // 32), **u8)) for _ in range(2)]
        self._offsets = [0]
        for n in sizes:
            self._offsets.append(self._offsets[-1] + al(n))
        self._sizes, per_set = sizes, self._offsets[-1]
        self.x = symm_mem.empty(2, rows, k, dtype=torch.bfloat16, device=self.device)
        self.out = symm_mem.empty(2, per_set, dtype=torch.uint8, device=self.device)
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=self.device)
        self.out.zero_()
        self.flags.zero_()
        hx, ho, hf = (symm_mem.rendezvous(t, group) for t in (self.x, self.out, self.flags))
        self._handles = (hx, ho, hf)
        i64 = dict(dtype=torch.int64, device=self.device)
        self.peer_x = [torch.tensor([int(p) + b * rows * k * 2 for p in hx.buffer_ptrs], **i64) for b in range(2)]
        self.out_tbl = []
        for b in range(2):
            tbl = [0] * 32
            for which in range(4):
                for r, p in enumerate(ho.buffer_ptrs):
                    tbl[8 * which + r] = int(p) + b * per_set + self._offsets[which]
            self.out_tbl.append(torch.tensor(tbl, **i64))
        self.peer_flags = torch.tensor([int(p) for p in hf.buffer_ptrs], **i64)
        self.sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.next = 0
        self.calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group)

    def buffer(self, rows: int) -> torch.Tensor:
        """[rows, k] view of the partial-output buffer the next fused call reads."""
        return self.x[self.next, :rows]

    def packed(self, which: int, rows: int):
        """PackedMatrix view of the first `rows` rows of packed-activation set `which` (tiled scale layout: the
        local re-tiled copy) and the row-major gathered scale buffers behind it."""
        from . import _lib, ops
        k_lo, o, L = self.k - self.k_hi, self._offsets, _lib.lib()
        buf = self.out[which]
        lo_t, hi_t = self.sf_tiled[which]
        p = ops.PackedMatrix(
            rows, k_lo, self.k_hi,
            buf[o[0]:o[0] + rows * k_lo // 2].view(rows, k_lo // 2),
            lo_t[:L.plq_sf_tiled_bytes(rows, k_lo // 16)],
            buf[o[2]:o[2] + rows * self.k_hi].view(rows, self.k_hi),
            hi_t[:L.plq_sf_tiled_bytes(rows, self.k_hi // 32)], ops.SF_TILED)
        return p, buf[o[1]:o[1] + rows * (k_lo // 16)], buf[o[3]:o[3] + rows * (self.k_hi // 32)]
