"""GoldenRuntime / GoldenRetriever: several trainers stepping their own model on a worker pool.

Restated from crates/st-nn/src/golden.rs:45-75 (config), :598-700 (construction), :720-766
(``sync_z_barycenter``), :784-900 (``run_epoch`` with dropout tolerance) and :1158-1212 (report).
Workers are native threads of :class:`~spiraltorch_b200.runtime.host.WorkerPool`; a worker that
raises is either fatal (default) or recorded as a *dropout* when ``allow_dropout`` is set, as long
as ``min_successful_workers`` still finished.
"""
from __future__ import annotations

import math
import queue
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

import torch

from ..nn.trainer import EpochStats, ModuleTrainer
from ..ops.rank import plan_rank
from ..tensor import Tensor, TensorError
from .host import WorkerFailure, WorkerPool


@dataclass
class GoldenRuntimeConfig:
    worker_threads: int = 0
    thread_name: str = "golden-runtime"


class GoldenRuntime:
    """Thread pool façade: ``spawn_blocking(fn)`` → handle with ``join()``; ``reduce``."""

    def __init__(self, config: Optional[GoldenRuntimeConfig] = None):
        self.config = config or GoldenRuntimeConfig()
        self._pool = WorkerPool(self.config.worker_threads, self.config.thread_name)

    def worker_count(self) -> int:
        return self._pool.workers

    def spawn_blocking(self, fn: Callable[..., Any], *args, **kw):
        return self._pool.spawn(fn, *args, **kw)

    def reduce(self, items: Sequence, map_fn: Callable, fold_fn: Callable, identity):
        """Tree-free parallel map + sequential fold (deterministic in the item order)."""
        mapped = [h.join() for h in [self._pool.spawn(map_fn, it) for it in items]]
        acc = identity
        for m in mapped:
            acc = fold_fn(acc, m)
        return acc

    def stats(self) -> dict:
        return self._pool.stats()

    def close(self) -> None:
        self._pool.close()


@dataclass
class GoldenRetrieverConfig:
    workers: int = 0
    runtime: Optional[GoldenRuntimeConfig] = None
    sync_blackcat_minutes: bool = False
    sync_heuristics_log: bool = False
    coordinate_blackcat: bool = False
    exploration_bias: float = 1.0
    optimization_boost: float = 1.0
    synergy_bias: float = 1.0
    reinforcement_bias: float = 1.0
    allow_dropout: bool = False
    min_successful_workers: int = 1


@dataclass
class GoldenDropoutRecord:
    worker: int
    error: str


@dataclass
class GoldenBlackcatPulse:
    exploration_drive: float = 0.0
    optimization_gain: float = 0.0
    synergy_score: float = 0.0
    reinforcement_weight: float = 0.0
    mean_support: float = 0.0
    mean_reward: float = 0.0
    dominant_plan: Optional[str] = None
    worker_count: int = 0


@dataclass
class CouncilDigest:
    epoch: int
    average_loss: float
    workers: int
    dropouts: int


@dataclass
class GoldenEpochReport:
    workers: int
    batches: int
    total_loss: float
    average_loss: float
    per_worker: list = field(default_factory=list)
    moderator_minutes: list = field(default_factory=list)
    heuristics_log: list = field(default_factory=list)
    cooperative_pulse: Optional[GoldenBlackcatPulse] = None
    council_snapshot: Optional[dict] = None
    dropouts: list = field(default_factory=list)


class GoldenRetriever:
    def __init__(self, config: GoldenRetrieverConfig, trainers: Sequence[ModuleTrainer]):
        if not trainers:
            raise TensorError("golden retriever requires at least one trainer")
        if config.workers and config.workers != len(trainers):
            raise TensorError(f"golden retriever configured for {config.workers} workers but got {len(trainers)} trainers")
        self.config = config
        self._trainers = list(trainers)
        self._locks = [threading.Lock() for _ in trainers]
        rc = config.runtime or GoldenRuntimeConfig(worker_threads=len(trainers))
        self._runtime = GoldenRuntime(rc)
        self.allow_dropout = config.allow_dropout
        self.min_successful_workers = max(1, config.min_successful_workers)
        self._last_dropouts: list[GoldenDropoutRecord] = []
        self._epoch = 0
        self._digest_subscribers: list[queue.Queue] = []
        self._last_council: Optional[dict] = None

    # ---- accessors ---------------------------------------------------------------------------
    def workers(self) -> int:
        return len(self._trainers)

    def runtime(self) -> GoldenRuntime:
        return self._runtime

    def coordination_biases(self) -> tuple[float, float, float, float]:
        c = self.config
        return (c.exploration_bias, c.optimization_boost, c.synergy_bias, c.reinforcement_bias)

    def last_dropouts(self) -> list[GoldenDropoutRecord]:
        return list(self._last_dropouts)

    def last_council_snapshot(self) -> Optional[dict]:
        return self._last_council

    def subscribe_digest(self) -> "queue.Queue[CouncilDigest]":
        q: queue.Queue = queue.Queue()
        self._digest_subscribers.append(q)
        return q

    # ---- reductions --------------------------------------------------------------------------
    def sync_z_barycenter(self, partials: Sequence[Tensor], rank: int) -> Tensor:
        """Mean of the workers' tensors scaled by ``1 + tanh(log2(tile_cols) / rank)``."""
        if not partials:
            raise TensorError("golden_z_barycenter: empty input")
        shape = partials[0].shape()
        for t in partials[1:]:
            if t.shape() != shape:
                raise TensorError(f"shape mismatch: {shape} vs {t.shape()}")
        acc = torch.stack([t._t.float() for t in partials]).mean(0)
        rank = max(1, int(rank))
        plan = plan_rank("topk", shape[0], shape[1], min(rank, shape[1]))
        tile_cols = max(2, plan.workgroup * 2 if plan.kernel == "smem_bitonic" else plan.workgroup)
        guard = math.tanh(math.log2(tile_cols) * (1.0 / rank))
        return Tensor._wrap(acc * (1.0 + guard))

    # ---- epoch -------------------------------------------------------------------------------
    def run_epoch(self, modules: Sequence, losses: Sequence, loaders: Sequence, schedules: Sequence) -> GoldenEpochReport:
        n = len(self._trainers)
        if not (len(modules) == len(losses) == len(loaders) == len(schedules) == n):
            raise TensorError(f"golden retriever requires {n} modules, losses, loaders, and schedules")
        self._last_dropouts = []
        self._epoch += 1

        def work(i: int) -> EpochStats:
            with self._locks[i]:
                return self._trainers[i].train_epoch(modules[i], losses[i], loaders[i], schedules[i])

        handles = [(i, self._runtime.spawn_blocking(work, i)) for i in range(n)]
        stats, successes, dropouts = [], [], []
        for i, h in handles:
            try:
                stats.append(h.join())
                successes.append(i)
            except WorkerFailure as exc:
                if not self.allow_dropout:
                    # the remaining workers still finish on the pool; their results are dropped
                    for _, rest in handles[i + 1:]:
                        try:
                            rest.join()
                        except WorkerFailure:
                            pass
                    raise TensorError(f"golden retriever worker {i} failed during epoch: {exc}") from exc
                dropouts.append(GoldenDropoutRecord(i, str(exc)))
        self._last_dropouts = dropouts
        if len(stats) < self.min_successful_workers:
            msg = (f"golden retriever completed {len(stats)} of {n} workers "
                   f"(minimum required {self.min_successful_workers})")
            if dropouts:
                msg += "; dropouts -> " + ", ".join(f"worker {d.worker}: {d.error}" for d in dropouts)
            raise TensorError(msg)

        total_loss, batches = self._runtime.reduce(stats, lambda s: (s.total_loss, s.batches),
                                                   lambda a, b: (a[0] + b[0], a[1] + b[1]), (0.0, 0))
        avg = total_loss / batches if batches else 0.0
        pulse = None
        if self.config.coordinate_blackcat:
            c = self.config
            pulse = GoldenBlackcatPulse(exploration_drive=c.exploration_bias, optimization_gain=c.optimization_boost,
                                        synergy_score=c.synergy_bias * len(successes) / n,
                                        reinforcement_weight=c.reinforcement_bias, mean_support=len(successes) / n,
                                        mean_reward=-avg, worker_count=len(successes))
        self._last_council = {"epoch": self._epoch, "workers": successes, "average_loss": avg,
                              "dropouts": [d.worker for d in dropouts]}
        digest = CouncilDigest(self._epoch, avg, len(successes), len(dropouts))
        for q in self._digest_subscribers:
            q.put(digest)
        return GoldenEpochReport(workers=len(stats), batches=batches, total_loss=total_loss, average_loss=avg,
                                 per_worker=stats, cooperative_pulse=pulse, council_snapshot=self._last_council,
                                 dropouts=dropouts)

    def close(self) -> None:
        self._runtime.close()
