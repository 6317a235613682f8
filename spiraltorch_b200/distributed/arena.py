"""Single-process collectives with transactional semantics, the sharded SGD reducer built on them
and gossip ("ameba") gradient propagation over a neighbour graph.

Restated from crates/st-core/src/distributed/collective.rs:34-440 (``CollectiveArena``: all-reduce
sum / broadcast that validate everything first and mutate nothing on error, execution reports with
SHA-256 digests of inputs and outputs, asynchronous gradient queue with a lease that is restored
unless committed), trainer.rs:96-600 (``DistributedTrainer``: ``p -= lr/world * Σ g`` over shards,
async gradient merge) and autograd.rs:77-660 (``AmebaAutograd``: a seeded gradient updates its
agent and is forwarded, damped, to the neighbours it did not come from, until it falls under the
tolerance or reaches ``max_hops``; a round is committed atomically).
"""
from __future__ import annotations

import copy
import hashlib
import math
import struct
import threading
from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

CONTRACT_VERSION = "spiraltorch.collective.v1"


class CollectiveError(ValueError):
    def __init__(self, kind: str, message: str, **fields):
        super().__init__(message)
        self.kind, self.fields = kind, fields


@dataclass
class CollectiveExecutionReport:
    operation: str
    participants: int
    width: int
    input_values: int
    output_values: int
    input_sha256: str
    output_sha256: str
    committed: bool = True
    kind: str = "spiraltorch.collective_execution"
    contract_version: str = CONTRACT_VERSION
    semantic_owner: str = "st-core"
    numeric_kernel: str = "sum_axis0"
    selected_backend: str = "cpu"

    def validate(self) -> None:
        if self.participants <= 0:
            raise CollectiveError("InvalidReport", "invalid collective execution report at participants: must be positive")
        if self.input_values != self.participants * self.width and self.operation == "all_reduce_sum":
            raise CollectiveError("InvalidReport", "invalid collective execution report at input_values: count mismatch")
        for name in ("input_sha256", "output_sha256"):
            v = getattr(self, name)
            if len(v) != 64 or any(c not in "0123456789abcdef" for c in v):
                raise CollectiveError("InvalidReport", f"invalid collective execution report at {name}: not a sha256 hex digest")


def _digest(domain: str, rows: Sequence[Sequence[float]]) -> str:
    h = hashlib.sha256(domain.encode())
    h.update(struct.pack("<QQ", len(rows), len(rows[0]) if rows else 0))
    for r in rows:
        h.update(struct.pack(f"<{len(r)}f", *r))
    return h.hexdigest()


def _check_finite(op: str, participant: int, values: Sequence[float]) -> None:
    for i, v in enumerate(values):
        if not math.isfinite(v):
            raise CollectiveError("NonFiniteInput", f"{op} participant {participant} contained non-finite value at "
                                  f"index {i}: {v}", operation=op, participant=participant, index=i, value=v)


class GradientLease:
    """Batches taken from the queue; they go back to its front unless :meth:`commit` is called."""

    def __init__(self, arena: "CollectiveArena", batches: list):
        self._arena, self._batches, self._committed = arena, batches, False

    def batches(self) -> list:
        return self._batches

    def is_empty(self) -> bool:
        return not self._batches

    def commit(self) -> None:
        self._committed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False

    def release(self) -> None:
        if not self._committed and self._batches:
            with self._arena._lock:
                self._arena._queue.extendleft(reversed(self._batches))
            self._batches = []
        self._committed = True

    def __del__(self):
        try:
            self.release()
        except Exception:  # noqa: BLE001
            pass


class CollectiveArena:
    def __init__(self):
        self._queue: deque = deque()
        self._lock = threading.Lock()

    def all_reduce_sum(self, tensors: list) -> CollectiveExecutionReport:
        """Replace every participant's row by the element-wise sum; on error nothing changes."""
        if not tensors:
            raise CollectiveError("EmptyParticipants", "all-reduce requires at least one participant")
        width = len(tensors[0])
        for p, t in enumerate(tensors):
            if len(t) != width:
                raise CollectiveError("ShapeMismatch", f"collective participant {p} has width {len(t)}, expected the "
                                      f"canonical width {width}", participant=p, expected=width, got=len(t))
            _check_finite("all_reduce_sum", p, t)
        in_digest = _digest("all_reduce_input", tensors)
        total = torch.tensor(tensors, dtype=torch.float32).sum(0)
        bad = (~torch.isfinite(total)).nonzero()
        if bad.numel():
            i = int(bad[0])
            raise CollectiveError("NonFiniteReduction", f"all-reduce sum became non-finite at index {i}: {float(total[i])}",
                                  index=i, value=float(total[i]))
        out = total.tolist()
        for t in tensors:
            t[:] = out
        return CollectiveExecutionReport("all_reduce_sum", len(tensors), width, len(tensors) * width, len(tensors) * width,
                                         in_digest, _digest("all_reduce_output", [out]))

    def broadcast(self, root: Sequence[float], targets: list) -> CollectiveExecutionReport:
        _check_finite("broadcast", 0, root)
        for p, t in enumerate(targets):
            if len(t) != len(root):
                raise CollectiveError("ShapeMismatch", f"collective participant {p} has width {len(t)}, expected the "
                                      f"canonical width {len(root)}", participant=p, expected=len(root), got=len(t))
        for t in targets:
            t[:] = list(root)
        d = _digest("broadcast", [list(root)])
        return CollectiveExecutionReport("broadcast", max(1, len(targets)), len(root), len(root), len(targets) * len(root),
                                         d, d, numeric_kernel="copy")

    def enqueue_gradient(self, gradient: Sequence[float]) -> None:
        if len(gradient) == 0:
            raise CollectiveError("EmptyGradient", "gradient batches must contain at least one value")
        _check_finite("enqueue_gradient", 0, gradient)
        with self._lock:
            self._queue.append(list(gradient))

    def drain_gradients(self) -> list:
        with self._lock:
            out = [v for g in self._queue for v in g]
            self._queue.clear()
        return out

    def lease_gradient_batches(self) -> GradientLease:
        with self._lock:
            batches = list(self._queue)
            self._queue.clear()
        return GradientLease(self, batches)

    def pending(self) -> int:
        with self._lock:
            return len(self._queue)


class DistributedTrainerError(ValueError):
    pass


class DistributedTrainer:
    def __init__(self, shards: int, shard_dim: int, learning_rate: float):
        if shards <= 0 or shard_dim <= 0:
            raise DistributedTrainerError("trainer needs at least one shard with at least one parameter")
        if not (learning_rate > 0 and math.isfinite(learning_rate)):
            raise DistributedTrainerError(f"learning rate must be positive, got {learning_rate}")
        self._arena = CollectiveArena()
        self._params = [[0.0] * shard_dim for _ in range(shards)]
        self._shard_dim, self._lr = shard_dim, learning_rate
        self.last_report: Optional[CollectiveExecutionReport] = None

    def parameters(self) -> list:
        return [v for shard in self._params for v in shard]

    def broadcast_parameters(self, root: Sequence[float]) -> None:
        if len(root) != self._shard_dim:
            raise DistributedTrainerError(f"root has {len(root)} values, expected {self._shard_dim}")
        try:
            self._arena.broadcast(root, self._params)
        except CollectiveError as e:
            raise DistributedTrainerError(str(e)) from e

    def apply_step(self, gradients: list) -> None:
        """All-reduce the per-shard gradients and apply ``p -= lr / shards * Σ g`` to every shard.
        ``gradients`` is left untouched; on any error the parameters are too."""
        if len(gradients) != len(self._params):
            raise DistributedTrainerError(f"expected {len(self._params)} gradient shards, got {len(gradients)}")
        for g in gradients:
            if len(g) != self._shard_dim:
                raise DistributedTrainerError(f"expected gradients of width {self._shard_dim}, got {len(g)}")
        work = [list(g) for g in gradients]
        try:
            self.last_report = self._arena.all_reduce_sum(work)
        except CollectiveError as e:
            raise DistributedTrainerError(str(e)) from e
        scale = -(self._lr / len(self._params))
        nxt = [[p + scale * s for p, s in zip(shard, work[0])] for shard in self._params]
        for shard in nxt:
            for i, v in enumerate(shard):
                if not math.isfinite(v):
                    raise DistributedTrainerError(f"parameter update became non-finite at index {i}")
        self._params = nxt

    def submit_async_gradient(self, gradient: Sequence[float]) -> None:
        total = len(self._params) * self._shard_dim
        if len(gradient) != total:
            raise DistributedTrainerError(f"async gradient has {len(gradient)} values, expected {total}")
        try:
            self._arena.enqueue_gradient(gradient)
        except CollectiveError as e:
            raise DistributedTrainerError(str(e)) from e

    def merge_async_gradients(self) -> bool:
        """Apply the mean of all queued full-parameter gradients; the queue is only consumed when
        the merge succeeds."""
        with self._arena.lease_gradient_batches() as lease:
            if lease.is_empty():
                lease.commit()
                return False
            batches = lease.batches()
            mean = torch.tensor(batches, dtype=torch.float32).mean(0)
            flat = torch.tensor(self.parameters(), dtype=torch.float32) - self._lr * mean
            if not bool(torch.isfinite(flat).all()):
                raise DistributedTrainerError("async merge produced a non-finite parameter")
            vals = flat.tolist()
            self._params = [vals[i * self._shard_dim:(i + 1) * self._shard_dim] for i in range(len(self._params))]
            lease.commit()
            return True


# ---- gossip autograd ----------------------------------------------------------------------------------
class AutogradError(ValueError):
    pass


@dataclass
class AgentConfig:
    id: int
    dimension: int
    neighbors: list = field(default_factory=list)
    learning_rate: float = 0.01
    damping: float = 0.5
    weights: Optional[list] = None

    def with_neighbors(self, neighbors) -> "AgentConfig":
        self.neighbors = list(neighbors)
        return self

    def with_learning_rate(self, rate: float) -> "AgentConfig":
        self.learning_rate = rate
        return self

    def with_damping(self, damping: float) -> "AgentConfig":
        self.damping = damping
        return self

    def with_weights(self, weights) -> "AgentConfig":
        self.weights = list(weights)
        return self


class AmebaAutograd:
    def __init__(self, max_hops: int, tolerance: float):
        if not math.isfinite(tolerance):
            raise AutogradError("tolerance must be finite")
        if tolerance < 0:
            raise AutogradError(f"tolerance must not be negative, got {tolerance}")
        self._agents: dict[int, dict] = {}
        self._pending: deque = deque()
        self.max_hops, self.tolerance = max_hops, tolerance

    def register_agent(self, cfg: AgentConfig) -> None:
        if cfg.id in self._agents:
            raise AutogradError(f"agent {cfg.id} is already registered")
        weights = list(cfg.weights) if cfg.weights is not None else [0.0] * cfg.dimension
        if not weights:
            raise AutogradError(f"agent {cfg.id} has no parameters")
        if not (cfg.learning_rate > 0 and math.isfinite(cfg.learning_rate)):
            raise AutogradError(f"learning rate must be positive, got {cfg.learning_rate}")
        if not math.isfinite(cfg.damping) or not 0.0 <= cfg.damping <= 1.0:
            raise AutogradError(f"damping must lie in [0, 1], got {cfg.damping}")
        if any(not math.isfinite(w) for w in weights):
            raise AutogradError("weights must be finite")
        if cfg.id in cfg.neighbors:
            raise AutogradError(f"agent {cfg.id} lists itself as a neighbour")
        if len(set(cfg.neighbors)) != len(cfg.neighbors):
            raise AutogradError(f"agent {cfg.id} lists a neighbour twice")
        self._agents[cfg.id] = {"neighbors": list(cfg.neighbors), "lr": cfg.learning_rate, "damping": cfg.damping,
                                "weights": weights}

    def validate_topology(self) -> None:
        for aid in sorted(self._agents):
            a = self._agents[aid]
            for n in a["neighbors"]:
                if n not in self._agents:
                    raise AutogradError(f"agent {aid} references unknown neighbour {n}")
                if len(self._agents[n]["weights"]) != len(a["weights"]):
                    raise AutogradError(f"agents {aid} and {n} have different dimensions")

    def seed_gradient(self, agent_id: int, gradient: Sequence[float]) -> None:
        if agent_id not in self._agents:
            raise AutogradError(f"unknown agent {agent_id}")
        if len(gradient) != len(self._agents[agent_id]["weights"]):
            raise AutogradError(f"gradient has {len(gradient)} values, expected {len(self._agents[agent_id]['weights'])}")
        if any(not math.isfinite(g) for g in gradient):
            raise AutogradError("gradient must be finite")
        self._pending.append((agent_id, agent_id, 0, list(gradient)))

    def _handle(self, agents: dict, pending: deque, msg) -> None:
        src, dst, hops, payload = msg
        a = agents[dst]
        nxt = [w - a["lr"] * g for w, g in zip(a["weights"], payload)]
        if any(not math.isfinite(v) for v in nxt):
            raise AutogradError(f"weight update of agent {dst} became non-finite")
        a["weights"] = nxt
        signal = sum(abs(g) for g in payload)
        if (signal < self.tolerance and hops > 0) or hops >= self.max_hops:
            return
        neighbors = [n for n in a["neighbors"] if n != src]
        if not neighbors:
            return
        fwd = [g * a["damping"] for g in payload]
        if sum(abs(g) for g in fwd) < self.tolerance:
            return
        for n in neighbors:
            pending.append((dst, n, hops + 1, list(fwd)))

    def _round(self, agents: dict, pending: deque) -> int:
        n = len(pending)
        for _ in range(n):
            self._handle(agents, pending, pending.popleft())
        return n

    def propagate_round(self) -> int:
        """Process the messages pending at the start of the round; committed only if all succeed."""
        self.validate_topology()
        agents, pending = copy.deepcopy(self._agents), copy.deepcopy(self._pending)
        n = self._round(agents, pending)
        self._agents, self._pending = agents, pending
        return n

    def drain(self) -> int:
        self.validate_topology()
        agents, pending = copy.deepcopy(self._agents), copy.deepcopy(self._pending)
        total = 0
        while pending:
            total += self._round(agents, pending)
        self._agents, self._pending = agents, pending
        return total

    def pending_messages(self) -> int:
        return len(self._pending)

    def weights(self, agent_id: int) -> list:
        if agent_id not in self._agents:
            raise AutogradError(f"unknown agent {agent_id}")
        return list(self._agents[agent_id]["weights"])
