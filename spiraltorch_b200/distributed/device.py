"""Training devices: how a trainer synchronises gradient accumulators and metrics across ranks.

Interface (crates/spiral-selfsup/src/trainer/device.rs:36-50): ``rank()``, ``world_size()``,
``synchronize_gradients(buffer)`` (all-reduce **mean**, in place, all-or-nothing) and
``aggregate_metrics(buffer, reduce)`` with ``MetricReduce.SUM | MEAN``.

* ``CpuDevice`` – world size 1, no-ops.
* ``DistributedDevice`` – ranks are threads of one process joined through a named in-memory
  rendezvous; after the sum, the mean scale is committed with a second one-element "ready"
  all-reduce so that a rank-local failure becomes ``PeerTensorFailure`` on every rank and either
  all ranks commit or none does (device.rs:147-192).
* ``ProcessGroupDevice`` – ranks are processes of a ``torch.distributed`` group (NCCL on GPUs,
  gloo on CPUs) with the same two-phase commit and a collective timeout.

Checkpoints carry the provider identity only (``{kind, contract_version, provider, rank,
world_size, state}`` with 64-bit integers as decimal strings) and are refused while a
collective is in flight (crates/st-core/src/distributed/mod.rs:33-110).
"""
from __future__ import annotations

import enum
import math
from datetime import timedelta
from typing import Callable, Optional

import torch

from . import rendezvous as rdv
from .rendezvous import (CollectiveTimeout, DistributedError, PeerTensorFailure)


class MetricReduce(enum.Enum):
    SUM = "sum"
    MEAN = "mean"


class TrainingDevice:
    def rank(self) -> int:
        raise NotImplementedError

    def world_size(self) -> int:
        raise NotImplementedError

    def synchronize_gradients(self, buffer: torch.Tensor) -> None:
        raise NotImplementedError

    def aggregate_metrics(self, buffer: torch.Tensor, reduce: MetricReduce = MetricReduce.MEAN) -> None:
        raise NotImplementedError

    def checkpoint(self) -> dict:
        return {"kind": "spiraltorch.accumulator_synchronizer", "contract_version": "v1",
                "provider": type(self).__name__, "rank": str(self.rank()), "world_size": str(self.world_size()),
                "state": {}}


class CpuDevice(TrainingDevice):
    def rank(self) -> int:
        return 0

    def world_size(self) -> int:
        return 1

    def synchronize_gradients(self, buffer) -> None:
        return None

    def aggregate_metrics(self, buffer, reduce=MetricReduce.MEAN) -> None:
        return None


class DistributedDevice(TrainingDevice):
    """Thread-rank device over :mod:`rendezvous` (``memory://`` groups)."""

    def __init__(self, group: str, rank: int, world_size: int):
        self._session = rdv.join(group, rank, world_size)
        self._timeout = rdv.DEFAULT_COLLECTIVE_TIMEOUT
        self.fail_mean_scale: Optional[Callable[[], bool]] = None   # fault-injection hook (tests)

    def with_collective_timeout(self, seconds: float) -> "DistributedDevice":
        if not seconds > 0:
            raise ValueError("collective timeout must be positive")
        self._timeout = float(seconds)
        return self

    def rank(self) -> int:
        return self._session.rank

    def world_size(self) -> int:
        return self._session.world_size

    def close(self) -> None:
        self._session.close()

    def _all_reduce(self, values: list[float]) -> list[float]:
        return self._session.all_reduce_sum(values, self._timeout)

    def synchronize_gradients(self, buffer: torch.Tensor) -> None:
        flat = buffer.detach().reshape(-1).to("cpu", torch.float64).tolist()
        summed = self._all_reduce(flat)                      # raises the same error on every rank
        ok = 1.0
        scaled = None
        try:
            if self.fail_mean_scale is not None and self.fail_mean_scale():
                raise RuntimeError("injected mean-scale failure")
            scaled = [v / self.world_size() for v in summed]
            if not all(math.isfinite(v) for v in scaled):
                raise ValueError("non-finite mean")
        except Exception:  # noqa: BLE001
            ok = 0.0
        ready = self._all_reduce([ok, float(self.rank()) if ok == 0.0 else 0.0])
        if ready[0] < self.world_size():
            failed = int(self.world_size() - ready[0])
            raise PeerTensorFailure(failed_ranks=failed, world_size=self.world_size())
        buffer.copy_(torch.tensor(scaled, dtype=buffer.dtype).reshape(buffer.shape))

    def aggregate_metrics(self, buffer: torch.Tensor, reduce: MetricReduce = MetricReduce.MEAN) -> None:
        out = self._all_reduce(buffer.detach().reshape(-1).to("cpu", torch.float64).tolist())
        if reduce is MetricReduce.MEAN:
            out = [v / self.world_size() for v in out]
        buffer.copy_(torch.tensor(out, dtype=buffer.dtype).reshape(buffer.shape))

    def checkpoint(self) -> dict:
        if self._session.in_flight():
            raise DistributedError("cannot checkpoint while a collective is in flight")
        ck = super().checkpoint()
        ck["provider"] = "spiral_selfsup.distributed"
        ck["state"] = {"group_id": self._session.group_id, "strategy": "all_reduce_mean",
                       "collective_timeout_nanos": str(int(self._timeout * 1e9))}
        return ck


class NativeDistributedDevice(DistributedDevice):
    """Thread-rank device whose all-reduce runs in the C++ host runtime on ``float32`` buffers
    (``csrc/host/host_runtime.cpp``): the wait happens outside the interpreter lock, the sum is
    accumulated in double precision, and the error vocabulary is the one of :mod:`rendezvous`."""

    def __init__(self, group: str, rank: int, world_size: int):
        from ..runtime.host import NativeRendezvous
        self._native = NativeRendezvous(group, rank, world_size)
        self._timeout = rdv.DEFAULT_COLLECTIVE_TIMEOUT
        self.fail_mean_scale = None

    def rank(self) -> int:
        return self._native.rank

    def world_size(self) -> int:
        return self._native.world_size

    def close(self) -> None:
        self._native.close()

    def _all_reduce(self, values: list[float]) -> list[float]:
        t = torch.tensor(values, dtype=torch.float32)
        self._native.all_reduce_sum_(t, self._timeout)
        return t.tolist()

    def synchronize_gradients(self, buffer: torch.Tensor) -> None:
        flat = buffer.detach().reshape(-1).to("cpu", torch.float32).contiguous().clone()
        self._native.all_reduce_sum_(flat, self._timeout)
        ok = 1.0
        try:
            if self.fail_mean_scale is not None and self.fail_mean_scale():
                raise RuntimeError("injected mean-scale failure")
            flat /= self.world_size()
            if not bool(torch.isfinite(flat).all()):
                raise ValueError("non-finite mean")
        except Exception:  # noqa: BLE001
            ok = 0.0
        ready = torch.tensor([ok], dtype=torch.float32)
        self._native.all_reduce_sum_(ready, self._timeout)
        if ready.item() < self.world_size():
            raise PeerTensorFailure(failed_ranks=int(self.world_size() - ready.item()), world_size=self.world_size())
        buffer.copy_(flat.reshape(buffer.shape).to(buffer.dtype))

    def aggregate_metrics(self, buffer: torch.Tensor, reduce: MetricReduce = MetricReduce.MEAN) -> None:
        flat = buffer.detach().reshape(-1).to("cpu", torch.float32).contiguous().clone()
        self._native.all_reduce_sum_(flat, self._timeout)
        if reduce is MetricReduce.MEAN:
            flat /= self.world_size()
        buffer.copy_(flat.reshape(buffer.shape).to(buffer.dtype))

    def checkpoint(self) -> dict:
        ck = TrainingDevice.checkpoint(self)
        ck["provider"] = "spiral_selfsup.distributed"
        ck["state"] = {"group_id": self._native.group_id, "strategy": "all_reduce_mean",
                       "collective_timeout_nanos": str(int(self._timeout * 1e9))}
        return ck


class ProcessGroupDevice(TrainingDevice):
    """Process-rank device over ``torch.distributed`` with the same all-or-nothing contract."""

    def __init__(self, group=None, timeout_s: float = rdv.DEFAULT_COLLECTIVE_TIMEOUT):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise DistributedError("torch.distributed is not initialised")
        self._dist, self._group, self._timeout = dist, group, timeout_s
        self.fail_mean_scale: Optional[Callable[[], bool]] = None

    def with_collective_timeout(self, seconds: float) -> "ProcessGroupDevice":
        self._timeout = float(seconds)
        return self

    def rank(self) -> int:
        return self._dist.get_rank(self._group)

    def world_size(self) -> int:
        return self._dist.get_world_size(self._group)

    def _all_reduce(self, t: torch.Tensor) -> None:
        work = self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM, group=self._group, async_op=True)
        try:
            done = work.wait(timeout=timedelta(seconds=self._timeout))
        except RuntimeError as exc:
            raise CollectiveTimeout(generation=-1, waited_ms=int(self._timeout * 1000)) from exc
        if done is False:
            raise CollectiveTimeout(generation=-1, waited_ms=int(self._timeout * 1000))

    def synchronize_gradients(self, buffer: torch.Tensor) -> None:
        staged = buffer.detach().clone()
        self._all_reduce(staged)
        ok = 1.0
        try:
            if self.fail_mean_scale is not None and self.fail_mean_scale():
                raise RuntimeError("injected mean-scale failure")
            staged /= self.world_size()
            if not torch.isfinite(staged).all():
                raise ValueError("non-finite mean")
        except Exception:  # noqa: BLE001
            ok = 0.0
        ready = torch.tensor([ok], dtype=torch.float32, device=buffer.device)
        self._all_reduce(ready)
        if ready.item() < self.world_size():
            raise PeerTensorFailure(failed_ranks=int(self.world_size() - ready.item()), world_size=self.world_size())
        buffer.copy_(staged)

    def aggregate_metrics(self, buffer: torch.Tensor, reduce: MetricReduce = MetricReduce.MEAN) -> None:
        staged = buffer.detach().clone()
        self._all_reduce(staged)
        if reduce is MetricReduce.MEAN:
            staged /= self.world_size()
        buffer.copy_(staged)

    def checkpoint(self) -> dict:
        ck = super().checkpoint()
        ck["provider"] = "torch.distributed"
        ck["state"] = {"backend": self._dist.get_backend(self._group), "strategy": "all_reduce_mean",
                       "collective_timeout_nanos": str(int(self._timeout * 1e9))}
        return ck
