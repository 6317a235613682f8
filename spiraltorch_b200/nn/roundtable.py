"""Roundtable node: decision summaries exchanged between trainers and the conductor that turns
agreeing summaries into heuristic proposals.

Reference behaviour: crates/st-nn/src/roundtable.rs:42-160 (DistMode / DistConfig / connectors),
:273-410 (OutcomeBand, DecisionEvent, MetaSummary, Wilson bounds), :415-560 (HeurOp log),
:571-650 (RoundtableNode), :656-750 (MetaConductor, local simulation).  The reference describes the
transports (meta endpoints, cloud queues) without implementing one; here a node hands its summaries
to any callable, and :func:`exchange_summaries` all-gathers them over ``torch.distributed`` so that
every rank's conductor sees the same evidence.
"""
from __future__ import annotations

import hashlib
import json
import math
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

LOCAL_ONLY, PERIODIC_META, FULLY_GLOBAL = "local", "periodic_meta", "fully_global"


@dataclass
class DistConfig:
    node_id: str = "local"
    mode: str = LOCAL_ONLY
    push_interval: float = 30.0              # seconds
    meta_endpoints: List[str] = field(default_factory=list)
    summary_window: int = 32
    cloud_targets: List[Tuple[str, ...]] = field(default_factory=list)

    def __post_init__(self):
        if self.mode not in (LOCAL_ONLY, PERIODIC_META, FULLY_GLOBAL):
            raise ValueError(f"unknown dist mode {self.mode!r}")

    def with_cloud_target(self, *target: str) -> "DistConfig":
        if tuple(target) not in self.cloud_targets:
            self.cloud_targets.append(tuple(target))
        return self

    def with_azure_event_hub(self, namespace: str, hub: str) -> "DistConfig":
        return self.with_cloud_target("azure_event_hub", namespace, hub)

    def with_azure_storage_queue(self, account: str, queue: str) -> "DistConfig":
        return self.with_cloud_target("azure_storage_queue", account, queue)

    def with_aws_kinesis(self, region: str, stream: str) -> "DistConfig":
        return self.with_cloud_target("aws_kinesis", region, stream)

    def with_aws_sqs(self, region: str, queue: str) -> "DistConfig":
        return self.with_cloud_target("aws_sqs", region, queue)


def outcome_band(above: float, here: float, beneath: float) -> str:
    if above >= here and above >= beneath:
        return "above"
    return "here" if here >= beneath else "beneath"


def wilson_bounds(p_hat: float, n: float, z: float = 1.0) -> Tuple[float, float]:
    denom = 1.0 + z * z / n
    centre = p_hat + z * z / (2.0 * n)
    margin = math.sqrt(max(p_hat * (1.0 - p_hat) + z * z / (4.0 * n), 0.0)) * z / math.sqrt(n)
    clamp = lambda v: min(max(v, 0.0), 1.0)  # noqa: E731
    return clamp((centre - margin) / denom), clamp((centre + margin) / denom)


@dataclass
class DecisionEvent:
    plan_signature: str
    script_hint: str
    rank_kind: str
    winner: str
    score: float
    wilson_low: float
    wilson_high: float
    psi_total: Optional[float]
    band_energy: Tuple[float, float, float]
    drift: float
    z_signal: float
    timestamp: float
    sequence: int

    def reliability(self) -> float:
        window = max(abs(self.wilson_high - self.wilson_low), 1e-4)
        psi_scale = max(self.psi_total if self.psi_total is not None else 1.0, 0.1)
        z_factor = min(max(1.0 + self.z_signal * 0.5, 0.25), 1.75)
        return min(max(self.score / psi_scale, 0.0), 1.0) * (1.0 - min(window, 1.0)) * z_factor


@dataclass
class MetaSummary:
    node_id: str
    plan_signature: str
    script_hint: str
    rank_kind: str
    winner: str
    mean_score: float
    wilson_low: float
    wilson_high: float
    mean_psi: float
    mean_z: float
    support: float
    events: int
    issued_at: float

    @classmethod
    def from_events(cls, node_id: str, events: Sequence[DecisionEvent]) -> Optional["MetaSummary"]:
        if not events:
            return None
        n = len(events)
        counts: Dict[str, int] = {}
        for e in events:
            counts[e.winner] = counts.get(e.winner, 0) + 1
        dominant = max(counts.items(), key=lambda kv: kv[1])[0]
        mean_score = sum(e.score for e in events) / n
        has_psi = any(e.psi_total is not None for e in events)
        lo, hi = wilson_bounds(min(max(mean_score, 0.0), 1.0), max(float(n), 1.0), 1.0)
        first = events[0]
        return cls(node_id, first.plan_signature, first.script_hint, first.rank_kind, dominant, mean_score, lo, hi,
                   sum(e.psi_total or 0.0 for e in events) / n if has_psi else 0.0,
                   sum(e.z_signal for e in events) / n, max(sum(e.reliability() for e in events), 0.0), n,
                   max(e.timestamp for e in events))


@dataclass
class HeurOp:
    origin: str
    kind: str                                 # append_soft | retract | annotate
    script: str = ""
    weight: float = 0.0
    script_hash: int = 0
    note: str = ""
    issued_at: float = 0.0

    def fingerprint(self) -> int:
        blob = json.dumps([self.origin, self.kind, self.script, repr(float(self.weight)), self.script_hash, self.note,
                           repr(float(self.issued_at))])
        return int.from_bytes(hashlib.sha256(blob.encode()).digest()[:8], "little")


@dataclass
class GlobalProposal:
    proposal_id: str
    ops: List[HeurOp]
    evidence: List[MetaSummary]


class HeurOpLog:
    """Append-only, de-duplicated (by fingerprint) log of heuristic operations; merges are idempotent."""

    def __init__(self):
        self.entries: List[HeurOp] = []
        self._fingerprints = set()

    def append(self, op: HeurOp) -> None:
        fp = op.fingerprint()
        if fp not in self._fingerprints:
            self._fingerprints.add(fp)
            self.entries.append(op)

    def merge(self, other: "HeurOpLog") -> None:
        for op in other.entries:
            self.append(op)

    def high_watermark(self) -> int:
        return len(self.entries)

    def missing_ranges(self) -> List[Tuple[int, int]]:
        return [(0, 0)] if not self.entries else []

    def top_winners(self, limit: int) -> List[HeurOp]:
        soft = [op for op in self.entries if op.kind == "append_soft"]
        soft.sort(key=lambda op: (-op.weight, op.issued_at))
        return soft[:max(limit, 0)]


class RoundtableNode:
    """Buffers decision events and emits a :class:`MetaSummary` when the window fills or the push
    interval has passed.  In ``local`` mode nothing is recorded."""

    def __init__(self, config: Optional[DistConfig] = None, clock: Callable[[], float] = time.monotonic,
                 sink: Optional[Callable[[MetaSummary], None]] = None):
        self.config = config or DistConfig()
        self._clock, self._sink = clock, sink
        self.pending: deque = deque()
        self._last_flush = clock()
        self._next_sequence = 0

    def record_decision(self, plan_signature: str, script_hint: str, rank_kind: str, winner: str, score: float,
                        psi_total: Optional[float] = None, band_energy: Tuple[float, float, float] = (0.0, 0.0, 0.0),
                        drift: float = 0.0, z_signal: float = 0.0) -> Optional[MetaSummary]:
        if self.config.mode == LOCAL_ONLY:
            return None
        score = min(max(score, 0.0), 1.0)
        lo, hi = wilson_bounds(score, 1.0, 1.0)
        self.pending.append(DecisionEvent(plan_signature, script_hint, rank_kind, winner, score, lo, hi, psi_total,
                                          tuple(band_energy), drift, z_signal, time.time(), self._next_sequence))
        self._next_sequence += 1
        if len(self.pending) >= self.config.summary_window or self._clock() - self._last_flush >= self.config.push_interval:
            self._last_flush = self._clock()
            batch = list(self.pending)
            self.pending.clear()
            summary = MetaSummary.from_events(self.config.node_id, batch)
            if summary is not None and self._sink is not None:
                self._sink(summary)
            return summary
        return None

    def drain(self) -> None:
        self.pending.clear()

    def retune(self, push_interval: float, summary_window: int) -> None:
        self.config.push_interval = max(push_interval, 0.010)
        self.config.summary_window = max(int(summary_window), 1)
        if len(self.pending) >= self.config.summary_window:
            self._last_flush = self._clock() - self.config.push_interval


class MetaConductor:
    """Keeps the latest summary per (plan, node); once at least ``participation`` nodes back a plan
    with total support ≥ ``threshold`` it emits a proposal to append the plan's script as a soft rule
    with weight ``min(support / threshold, 2)`` and clears the evidence."""

    def __init__(self, threshold: float, participation: int):
        self.threshold, self.participation = threshold, participation
        self.plans: Dict[str, Dict[str, object]] = {}

    def ingest(self, summary: MetaSummary) -> Optional[GlobalProposal]:
        entry = self.plans.setdefault(summary.plan_signature, {"script_hint": summary.script_hint, "evidence": {}})
        entry["script_hint"] = summary.script_hint
        evidence: Dict[str, MetaSummary] = entry["evidence"]          # type: ignore[assignment]
        evidence[summary.node_id] = summary
        support = sum(max(s.support, 0.0) * min(max(1.0 + s.mean_z * 0.4, 0.3), 1.7) for s in evidence.values())
        if len(evidence) >= self.participation and support >= self.threshold:
            op = HeurOp("meta", "append_soft", script=str(entry["script_hint"]), weight=min(support / self.threshold, 2.0),
                        issued_at=time.time())
            proposal = GlobalProposal(f"proposal-{op.fingerprint()}", [op], list(evidence.values()))
            evidence.clear()
            return proposal
        return None


def simulate_proposal_locally(proposal: GlobalProposal, log: HeurOpLog) -> Tuple[bool, Dict[str, float]]:
    """Previews a proposal: returns the metrics it would set and leaves a ``local-preview`` annotation in the log."""
    metrics: Dict[str, float] = {}
    for op in proposal.ops:
        if op.kind == "append_soft":
            metrics[op.script] = op.weight
        elif op.kind == "retract":
            metrics[f"retract:{op.script_hash}"] = 1.0
        else:
            metrics[f"annotate:{op.script_hash}"] = float(len(op.note))
    first = proposal.ops[0].fingerprint() if proposal.ops else 0
    log.append(HeurOp("local-preview", "annotate", script_hash=first, note="preview", issued_at=time.time()))
    return True, metrics


def exchange_summaries(local: Optional[MetaSummary], group=None) -> List[MetaSummary]:
    """All-gathers one optional summary per rank (``torch.distributed``, any backend) and returns the
    non-empty ones in rank order.  Without an initialised process group the local summary is returned."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return [local] if local is not None else []
    gathered: List[Optional[dict]] = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, asdict(local) if local is not None else None, group=group)
    return [MetaSummary(**g) for g in gathered if g is not None]
