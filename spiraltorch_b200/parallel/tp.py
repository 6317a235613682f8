"""Tensor-parallel communication context (sequence-parallel activations).

Activations between transformer sub-blocks live as row shards ``[T/world, d]``.  A
column-parallel linear needs the gathered rows (all-gather → GEMM); a row-parallel linear
produces partial sums that are reduced and scattered back to row shards (GEMM →
reduce-scatter).  Two implementations share one interface:

* ``mode="nccl"`` – ``torch.distributed`` all-gather / reduce-scatter followed or preceded
  by the GEMM kernel.  This is the measured baseline.
* ``mode="fused"`` – the peer-memory kernels of ``csrc/comm`` where the transfer runs tile
  by tile inside the GEMM launch (see :mod:`spiraltorch_b200.parallel.fused`).

With a world size of 1 both collectives are the identity.

The reference has no tensor parallelism (its only multi-rank path is data parallel,
crates/spiral-selfsup/src/trainer/distributed.rs); this module is new functionality.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class TPContext:
    def __init__(self, group: Optional[dist.ProcessGroup] = None, mode: str = "nccl"):
        self.group = group
        if group is None or not dist.is_initialized():
            self.world, self.rank = 1, 0
        else:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.mode = mode
        self._gloo = (self.world > 1 and dist.get_backend(group) == "gloo")
        self.bytes_gathered = 0
        self.bytes_scattered = 0
        self.collective_calls = 0

    # -- row collectives -------------------------------------------------------------------
    def all_gather_rows(self, shard: torch.Tensor) -> torch.Tensor:
        """[T/world, d] → [T, d] (rank-major row order)."""
        if self.world == 1:
            return shard
        shard = shard.contiguous()
        out = torch.empty((shard.shape[0] * self.world, *shard.shape[1:]), dtype=shard.dtype,
                          device=shard.device)
        if self._gloo:  # CPU test path
            parts = list(out.chunk(self.world, dim=0))
            dist.all_gather(parts, shard, group=self.group)
        else:
            dist.all_gather_into_tensor(out, shard, group=self.group)
        self.bytes_gathered += out.numel() * out.element_size()
        self.collective_calls += 1
        return out

    def reduce_scatter_rows(self, full: torch.Tensor) -> torch.Tensor:
        """[T, d] partial sums on every rank → [T/world, d] reduced row shard."""
        if self.world == 1:
            return full
        full = full.contiguous()
        out = torch.empty((full.shape[0] // self.world, *full.shape[1:]), dtype=full.dtype,
                          device=full.device)
        if self._gloo:  # CPU test path: all-reduce then keep the local rows
            tmp = full.clone()
            dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
            out.copy_(tmp.chunk(self.world, dim=0)[self.rank])
        else:
            dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=self.group)
        self.bytes_scattered += full.numel() * full.element_size()
        self.collective_calls += 1
        return out

    def shard_slot(self, key, rows: int, K: int) -> Optional[torch.Tensor]:
        """Where a producer may write the row shard that ``ag_gemm(..., key=key)`` will gather, or ``None`` when
        the context has no preferred place (the fused context returns a view of its symmetric gather buffer)."""
        return None

    # -- parallel linears (collective + GEMM); the fused context overrides these ------------
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, key=None, **epilogue):
        """Column-parallel product ``all_gather_rows(x_shard) @ op(w)``; returns ``(y, x_full)``."""
        from ..ops.gemm import gemm
        x_full = self.all_gather_rows(x_shard)
        return gemm(x_full, w, b_mn=b_mn, **epilogue), x_full

    def gemm_rs(self, a_full: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel product ``reduce_scatter_rows(a_full @ op(w))`` (+ ``residual``)."""
        from ..ops.gemm import gemm
        if self.world == 1:
            return gemm(a_full, w, b_mn=b_mn, residual=residual)
        y = self.reduce_scatter_rows(gemm(a_full, w, b_mn=b_mn))
        return y if residual is None else y + residual

    def all_reduce_(self, t: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=op, group=self.group)
            self.collective_calls += 1
        return t
