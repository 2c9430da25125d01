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
