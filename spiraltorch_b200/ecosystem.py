"""Ecosystem registry: a process-wide, bounded record of what the heuristics decided (which launch choice, from which
source), what the roundtable scheduled, what the cloud connectors did and which metrics were emitted, with per-metric
digests (count, sum, extremes, first / last) grouped by name and sorted tags.

Reference parity: crates/st-core/src/ecosystem/mod.rs (`HeuristicSource` :10-29, `HeuristicChoiceSummary` :32-74,
`HeuristicDecision` :76-96, `MetricSample` / `MetricDigest` :99-167, roundtable / rank / distribution summaries
:170-239, `CloudConnector` :241-286, `ConnectorEvent` :288-303, `EcosystemCapacity` :326-345, `EcosystemRegistry`
:374-469, digests :507-585).
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field, replace
from typing import Callable, Deque, Dict, List, Optional, Tuple

HEURISTIC_SOURCES = ("soft_logic", "dsl", "kv", "generated", "fallback")


@dataclass
class HeuristicChoiceSummary:
    use_two_stage: bool
    workgroup: int
    lanes: int
    channel_stride: int
    algo_hint: Optional[str] = None
    compaction_tile: int = 0
    fft_tile_cols: int = 0
    fft_radix: int = 0
    fft_segments: int = 0


@dataclass
class HeuristicDecision:
    subsystem: str
    kind: str
    rows: int
    cols: int
    k: int
    choice: HeuristicChoiceSummary
    score_hint: Optional[float] = None
    source: str = "fallback"
    issued_at: float = field(default_factory=time.time)

    def __post_init__(self):
        if self.source not in HEURISTIC_SOURCES:
            raise ValueError(f"unknown heuristic source {self.source!r}; one of {HEURISTIC_SOURCES}")

    def issued_at_secs(self) -> float:
        return self.issued_at


@dataclass
class MetricSample:
    name: str
    value: float
    unit: Optional[str] = None
    tags: Dict[str, str] = field(default_factory=dict)
    issued_at: float = field(default_factory=time.time)

    def with_tag(self, key: str, value: str) -> "MetricSample":
        self.tags[key] = value
        return self

    def with_unit(self, unit: str) -> "MetricSample":
        self.unit = unit
        return self

    def issued_at_secs(self) -> float:
        return self.issued_at


@dataclass
class MetricDigest:
    name: str
    tags: List[Tuple[str, str]]
    unit: Optional[str]
    count: int
    sum: float
    min: float
    max: float
    average: float
    first_at: float
    last_value: float
    last_at: float


@dataclass
class RoundtableConfigSummary:
    top_k: int
    mid_k: int
    bottom_k: int
    here_tolerance: float


@dataclass
class RankPlanSummary:
    kind: str
    rows: int
    cols: int
    k: int
    workgroup: int = 0
    lanes: int = 0
    channel_stride: int = 0
    tile: int = 0
    compaction_tile: int = 0
    subgroup: bool = False
    fft_tile: int = 0
    fft_radix: int = 0
    fft_segments: int = 0


@dataclass
class CloudConnector:
    """``kind``: ``azure_event_hub`` (namespace, hub), ``azure_storage_queue`` (account, queue), ``aws_kinesis`` (region,
    stream) or ``aws_sqs`` (region, queue); ``scope`` / ``target`` are those two names in order."""
    kind: str
    scope: str
    target: str

    _KINDS = {"azure_event_hub": ("azure", "event_hub"), "azure_storage_queue": ("azure", "storage_queue"),
              "aws_kinesis": ("aws", "kinesis"), "aws_sqs": ("aws", "sqs")}

    def __post_init__(self):
        if self.kind not in self._KINDS:
            raise ValueError(f"unknown connector kind {self.kind!r}; one of {tuple(self._KINDS)}")

    def provider(self) -> str:
        return self._KINDS[self.kind][0]

    def service(self) -> str:
        return self._KINDS[self.kind][1]

    def descriptor(self) -> str:
        return f"{self.scope}/{self.target}"


@dataclass
class DistributionSummary:
    node_id: str
    mode: str
    summary_window: int
    push_interval_ms: int
    meta_endpoints: List[str] = field(default_factory=list)
    cloud_targets: List[CloudConnector] = field(default_factory=list)


@dataclass
class ConnectorEvent:
    name: str
    stage: str
    metadata: Dict[str, str] = field(default_factory=dict)
    issued_at: float = field(default_factory=time.time)

    def issued_at_secs(self) -> float:
        return self.issued_at


@dataclass
class RoundtableSummary:
    rows: int
    cols: int
    config: RoundtableConfigSummary
    plans: List[RankPlanSummary] = field(default_factory=list)
    autopilot_enabled: bool = False
    distribution: Optional[DistributionSummary] = None
    issued_at: float = field(default_factory=time.time)

    def issued_at_secs(self) -> float:
        return self.issued_at


@dataclass
class EcosystemCapacity:
    heuristics: int = 2048
    roundtables: int = 256
    connectors: int = 512
    metrics: int = 4096


@dataclass
class EcosystemReport:
    heuristics: List[HeuristicDecision]
    roundtables: List[RoundtableSummary]
    connectors: List[ConnectorEvent]
    metrics: List[MetricSample]
    metric_digests: List[MetricDigest]


def summarise_metrics(samples) -> List[MetricDigest]:
    """One digest per (name, sorted tags), in sorted key order; the first unit seen for a key is kept."""
    acc: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], MetricDigest] = {}
    for s in samples:
        key = (s.name, tuple(sorted(s.tags.items())))
        d = acc.get(key)
        if d is None:
            acc[key] = MetricDigest(s.name, list(key[1]), s.unit, 1, s.value, s.value, s.value, s.value, s.issued_at, s.value, s.issued_at)
        else:
            d.count += 1
            d.sum += s.value
            d.min, d.max = min(d.min, s.value), max(d.max, s.value)
            d.last_value, d.last_at = s.value, s.issued_at
            d.unit = d.unit if d.unit is not None else s.unit
            d.average = d.sum / d.count
    return [acc[k] for k in sorted(acc)]


class EcosystemRegistry:
    """Bounded queues behind one lock; the oldest entries fall off first, and a capacity of zero keeps nothing."""

    _global: Optional["EcosystemRegistry"] = None
    _global_lock = threading.Lock()

    def __init__(self, capacity: Optional[EcosystemCapacity] = None):
        self._lock = threading.Lock()
        self._capacity = capacity or EcosystemCapacity()
        self._heuristics: Deque[HeuristicDecision] = deque()
        self._roundtables: Deque[RoundtableSummary] = deque()
        self._connectors: Deque[ConnectorEvent] = deque()
        self._metrics: Deque[MetricSample] = deque()

    @classmethod
    def global_(cls) -> "EcosystemRegistry":
        with cls._global_lock:
            if cls._global is None:
                cls._global = cls()
            return cls._global

    def _enforce(self) -> None:
        for q, cap in ((self._heuristics, self._capacity.heuristics), (self._roundtables, self._capacity.roundtables),
                       (self._connectors, self._capacity.connectors), (self._metrics, self._capacity.metrics)):
            if cap <= 0:
                q.clear()
            while len(q) > cap > 0:
                q.popleft()

    def _push(self, q: Deque, item) -> None:
        with self._lock:
            q.append(item)
            self._enforce()

    def record_heuristic(self, decision: HeuristicDecision) -> None:
        self._push(self._heuristics, decision)

    def record_roundtable(self, summary: RoundtableSummary) -> None:
        self._push(self._roundtables, summary)

    def record_connector(self, event: ConnectorEvent) -> None:
        self._push(self._connectors, event)

    def record_metric(self, sample: MetricSample) -> None:
        self._push(self._metrics, sample)

    def configure(self, mutator: Callable[[EcosystemCapacity], None]) -> None:
        """Lets ``mutator`` edit the capacities in place; if it raises, the previous capacities stay."""
        with self._lock:
            trial = replace(self._capacity)
            mutator(trial)
            self._capacity = trial
            self._enforce()

    def capacity(self) -> EcosystemCapacity:
        with self._lock:
            return replace(self._capacity)

    def snapshot(self) -> EcosystemReport:
        with self._lock:
            metrics = list(self._metrics)
            return EcosystemReport(list(self._heuristics), list(self._roundtables), list(self._connectors), metrics, summarise_metrics(metrics))

    def drain(self) -> EcosystemReport:
        with self._lock:
            report = EcosystemReport(list(self._heuristics), list(self._roundtables), list(self._connectors), list(self._metrics),
                                     summarise_metrics(self._metrics))
            for q in (self._heuristics, self._roundtables, self._connectors, self._metrics):
                q.clear()
            return report
