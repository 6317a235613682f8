"""Meta-narrative layer: narrative beats live in a causal set (a DAG of events), a temporal engine releases them in an
order that respects the dependencies, and a sheaf of weighted tag sections — optionally gated by the Z-space signature
of the observed Maxwell pulse — decides which tags and how much intensity a released beat carries.

Parity: crates/st-logic/src/meta_layer.rs — `CausalSet` (:122-395: insert / add_dependency with cycle refusal / resolve /
validate), `TemporalLogicEngine` (:397-520: frontier in readiness order, `next_matching`), `MeaningSection` /
`MeaningSheaf::collapse` (:583-717), `ToposLogicBridge` (:720-750), `NarrativeBeat` / `ZSpaceGate` (:768-885),
`MetaNarrativeLayer::next_with_pulse` (:887-945); `ZSpace` from crates/st-logic/src/quantum_reality.rs:970-1027.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, List, Optional, Sequence, Set, Tuple, TypeVar

from .theory import MaxwellZPulse

T = TypeVar("T")
EPS = 2.220446049250313e-16


class CausalError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


class CausalInvariantError(AssertionError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass
class CausalNode(Generic[T]):
    id: str
    payload: T
    parents: Set[str] = field(default_factory=set)

    def parent_ids(self) -> List[str]:
        return sorted(self.parents)


class CausalSet(Generic[T]):
    """Live events with their parents, a successor index over live events, and the set of resolved ids.  A dependency on
    an already resolved event is recorded but never blocks."""

    def __init__(self):
        self.nodes: Dict[str, CausalNode[T]] = {}
        self.successors: Dict[str, Set[str]] = {}
        self.resolved: Set[str] = set()

    def __len__(self) -> int:
        return len(self.nodes)

    def is_empty(self) -> bool:
        return not self.nodes

    def resolved_len(self) -> int:
        return len(self.resolved)

    def was_resolved(self, event_id: str) -> bool:
        return event_id in self.resolved

    def insert(self, event_id: str, payload: T) -> None:
        if not event_id.strip():
            raise CausalError("empty_event_id", "causal event identifier cannot be empty")
        if event_id in self.nodes:
            raise CausalError("duplicate_event", f"causal event `{event_id}` is already registered")
        if event_id in self.resolved:
            raise CausalError("resolved_event", f"causal event `{event_id}` has already been resolved")
        self.successors.setdefault(event_id, set())
        self.nodes[event_id] = CausalNode(event_id, payload)

    def _ensure_live(self, event_id: str) -> None:
        if event_id in self.nodes:
            return
        if event_id in self.resolved:
            raise CausalError("resolved_event", f"causal event `{event_id}` has already been resolved")
        raise CausalError("unknown_event", f"causal event `{event_id}` is not registered")

    def _reaches(self, start: str, target: str) -> bool:
        stack, seen = [start], set()
        while stack:
            cur = stack.pop()
            if cur in seen:
                continue
            seen.add(cur)
            if cur == target:
                return True
            stack.extend(self.successors.get(cur, ()))
        return False

    def add_dependency(self, earlier: str, later: str) -> None:
        if earlier == later:
            raise CausalError("self_dependency", "causal event cannot depend on itself")
        if earlier in self.nodes:
            live = True
        elif earlier in self.resolved:
            live = False
        else:
            raise CausalError("unknown_event", f"causal event `{earlier}` is not registered")
        self._ensure_live(later)
        if live and self._reaches(later, earlier):
            raise CausalError("cyclic_dependency", f"causal relation `{earlier}` -> `{later}` would create a cycle")
        self.nodes[later].parents.add(earlier)
        if live:
            self.successors.setdefault(earlier, set()).add(later)

    def get(self, event_id: str) -> Optional[CausalNode[T]]:
        return self.nodes.get(event_id)

    def is_ready(self, event_id: str) -> bool:
        node = self.nodes.get(event_id)
        return node is not None and all(p in self.resolved for p in node.parents)

    def ready_ids(self) -> List[str]:
        return [i for i in sorted(self.nodes) if self.is_ready(i)]

    def resolve(self, event_id: str) -> Optional[Tuple[str, T]]:
        node = self.nodes.pop(event_id, None)
        if node is None:
            return None
        self.successors.pop(event_id, None)
        for parent in node.parents:
            self.successors.get(parent, set()).discard(event_id)
        self.resolved.add(node.id)
        return node.id, node.payload

    take = resolve

    def validate(self) -> None:
        for key, node in self.nodes.items():
            if key != node.id:
                raise CausalInvariantError("node_id_mismatch", f"causal node key `{key}` does not match embedded identifier `{node.id}`")
            if key in self.resolved:
                raise CausalInvariantError("resolved_node", f"resolved causal event `{key}` is still live")
            if key not in self.successors:
                raise CausalInvariantError("missing_successor_index", f"live causal event `{key}` has no successor index")
            for parent in node.parents:
                if parent in self.resolved:
                    continue
                if parent not in self.nodes:
                    raise CausalInvariantError("dangling_parent", f"causal event `{key}` references unknown parent `{parent}`")
                if key not in self.successors.get(parent, ()):
                    raise CausalInvariantError("missing_successor_link", f"causal event `{key}` references live parent `{parent}` without a successor link")
        for parent, children in self.successors.items():
            if parent not in self.nodes:
                raise CausalInvariantError("unknown_successor_index", f"successor index exists for non-live event `{parent}`")
            for child in children:
                if child not in self.nodes:
                    raise CausalInvariantError("unknown_successor", f"causal successor `{parent}` -> `{child}` points to a non-live child")
                if parent not in self.nodes[child].parents:
                    raise CausalInvariantError("missing_parent_link", f"causal successor `{parent}` -> `{child}` is missing from the child parent set")
        indegree = {i: sum(p in self.nodes for p in n.parents) for i, n in self.nodes.items()}
        ready = [i for i, d in indegree.items() if d == 0]
        visited = 0
        while ready:
            cur = ready.pop()
            visited += 1
            for child in self.successors.get(cur, ()):
                if indegree.get(child, 0) > 0:
                    indegree[child] -= 1
                    if indegree[child] == 0:
                        ready.append(child)
        if visited != len(self.nodes):
            raise CausalInvariantError("cyclic_graph", "causal graph contains a dependency cycle")


class TemporalLogicEngine(Generic[T]):
    """Releases ready events; among ready events the one that became ready first goes first."""

    def __init__(self, causal: Optional[CausalSet[T]] = None):
        self.causal: CausalSet[T] = causal or CausalSet()
        self.frontier: List[str] = []
        self._refresh()

    from_causal_set = classmethod(lambda cls, causal: cls(causal))

    def _refresh(self) -> None:
        self.frontier = [i for i in self.frontier if self.causal.is_ready(i)]
        for i in self.causal.ready_ids():
            if i not in self.frontier:
                self.frontier.append(i)

    def pending(self) -> int:
        return len(self.causal)

    def insert_event(self, event_id: str, payload: T) -> None:
        self.causal.insert(event_id, payload)
        self._refresh()

    def add_dependency(self, earlier: str, later: str) -> None:
        self.causal.add_dependency(earlier, later)
        self._refresh()

    def discard_event(self, event_id: str) -> Optional[Tuple[str, T]]:
        out = self.causal.resolve(event_id)
        self._refresh()
        return out

    def was_resolved(self, event_id: str) -> bool:
        return self.causal.was_resolved(event_id)

    def payload(self, event_id: str) -> Optional[T]:
        node = self.causal.get(event_id)
        return None if node is None else node.payload

    def next_matching(self, predicate: Callable[[T], bool]) -> Optional[Tuple[str, T]]:
        self._refresh()
        for i in self.frontier:
            node = self.causal.get(i)
            if node is not None and self.causal.is_ready(i) and predicate(node.payload):
                self.frontier.remove(i)
                out = self.causal.resolve(i)
                self._refresh()
                return out
        return None

    def next_ready(self) -> Optional[Tuple[str, T]]:
        return self.next_matching(lambda _p: True)

    def validate(self) -> None:
        self.causal.validate()
        seen = set()
        for i in self.frontier:
            if i in seen:
                raise CausalInvariantError("duplicate_frontier_event", f"causal frontier contains duplicate event `{i}`")
            seen.add(i)
            if self.causal.get(i) is None:
                raise CausalInvariantError("unknown_frontier_event", f"causal frontier contains non-live event `{i}`")
            if not self.causal.is_ready(i):
                raise CausalInvariantError("blocked_frontier_event", f"causal frontier contains blocked event `{i}`")
        for i in self.causal.ready_ids():
            if i not in seen:
                raise CausalInvariantError("missing_frontier_event", f"ready causal event `{i}` is missing from the frontier")


# ---- Z-space signatures -------------------------------------------------------------------------------------------------------
@dataclass
class ZSpace:
    signature: List[float]

    @classmethod
    def from_pulse(cls, pulse: MaxwellZPulse) -> "ZSpace":
        return cls([float(pulse.blocks), pulse.mean, pulse.standard_error, pulse.z_score, float(pulse.band_energy[0]),
                    float(pulse.band_energy[1]), float(pulse.band_energy[2]), float(pulse.z_bias)])

    def norm(self) -> float:
        return math.sqrt(sum(v * v for v in self.signature))

    def cosine_similarity(self, other: "ZSpace") -> float:
        return signature_similarity(self.signature, other)


def signature_similarity(expected: Sequence[float], observed: ZSpace) -> float:
    en, on = math.sqrt(sum(v * v for v in expected)), observed.norm()
    if en <= EPS or on <= EPS:
        return 0.0
    return min(max(sum(a * b for a, b in zip(expected, observed.signature)) / (en * on), -1.0), 1.0)


def _clean(labels: Sequence[str]) -> List[str]:
    return [s.strip() for s in labels if s.strip()]


class MeaningSection:
    """Tags with a weight, valid over a cover of contexts (``*`` = everywhere), optionally only while the observed
    signature stays similar enough to an expected one (the weight is then scaled by the similarity)."""

    def __init__(self, cover: Sequence[str], tags: Sequence[str], weight: float):
        self.cover = _clean(cover) or ["*"]
        self.tags = sorted(set(_clean(tags)))
        self.weight = max(float(weight), 0.0)
        self.zspace_signature: Optional[List[float]] = None
        self.min_similarity = 0.0

    @classmethod
    def for_open(cls, open_: str, tags: Sequence[str], weight: float) -> "MeaningSection":
        return cls([open_], tags, weight)

    def with_zspace_signature(self, signature: Sequence[float], min_similarity: float) -> "MeaningSection":
        self.zspace_signature, self.min_similarity = list(signature), min(max(min_similarity, 0.0), 1.0)
        return self

    def supports(self, open_: str) -> bool:
        return any(c == "*" or c == open_ for c in self.cover)


class MeaningSheaf:
    def __init__(self):
        self.sections: List[MeaningSection] = []

    def add_section(self, section: MeaningSection) -> None:
        self.sections.append(section)

    def with_section(self, section: MeaningSection) -> "MeaningSheaf":
        self.add_section(section)
        return self

    def collapse(self, open_: str, threshold: float, zspace: Optional[ZSpace] = None) -> Tuple[List[Tuple[str, float]], float]:
        """``([(tag, weight)] by decreasing weight, total weight)`` of the tags whose summed weight reaches `threshold`."""
        agg: Dict[str, float] = {}
        for sec in self.sections:
            if not sec.supports(open_):
                continue
            w = sec.weight
            if sec.zspace_signature is not None:
                if zspace is None:
                    continue
                sim = signature_similarity(sec.zspace_signature, zspace)
                if sim < sec.min_similarity:
                    continue
                w *= sim
            if w <= 0.0:
                continue
            for tag in sec.tags:
                agg[tag] = agg.get(tag, 0.0) + w
        entries = sorted(((t, w) for t, w in sorted(agg.items()) if w >= threshold), key=lambda e: -e[1])
        return entries, sum(w for _, w in entries)


class ToposLogicBridge:
    def __init__(self):
        self.sheaves: Dict[str, MeaningSheaf] = {}

    def attach(self, event_id: str, sheaf: MeaningSheaf) -> None:
        self.sheaves[event_id] = sheaf

    def resolve(self, event_id: str, open_: str, threshold: float, zspace: Optional[ZSpace] = None):
        sheaf = self.sheaves.get(event_id)
        return ([], 0.0) if sheaf is None else sheaf.collapse(open_, threshold, zspace)


@dataclass
class ZSpaceGate:
    signature: List[float]
    min_similarity: float = 0.0
    min_norm: float = 0.0

    def __post_init__(self):
        self.min_similarity, self.min_norm = min(max(self.min_similarity, 0.0), 1.0), max(self.min_norm, 0.0)

    def allows(self, observed: ZSpace) -> bool:
        return signature_similarity(self.signature, observed) >= self.min_similarity and observed.norm() >= self.min_norm


class NarrativeBeat:
    def __init__(self, channel: Optional[str], context: str, base_tags: Sequence[str]):
        self.channel, self.context = channel, context
        self.base_tags = sorted(set(_clean(base_tags)))
        self.intensity_scale, self.floor, self.sheaf_threshold = 1.0, 0.0, 0.0
        self.zspace_gate: Optional[ZSpaceGate] = None

    def with_channel(self, channel: str) -> "NarrativeBeat":
        self.channel = channel
        return self

    def with_intensity_scale(self, scale: float) -> "NarrativeBeat":
        self.intensity_scale = max(scale, 0.0)
        return self

    def with_floor(self, floor: float) -> "NarrativeBeat":
        self.floor = max(floor, 0.0)
        return self

    def with_sheaf_threshold(self, threshold: float) -> "NarrativeBeat":
        self.sheaf_threshold = max(threshold, 0.0)
        return self

    def with_zspace_gate(self, signature: Sequence[float], min_similarity: float, min_norm: float) -> "NarrativeBeat":
        self.zspace_gate = ZSpaceGate(list(signature), min_similarity, min_norm)
        return self

    def matches(self, channel: str, zspace: ZSpace) -> bool:
        return (self.channel is None or self.channel == channel) and (self.zspace_gate is None or self.zspace_gate.allows(zspace))


@dataclass
class ResolvedNarrative:
    event_id: str
    channel: str
    tags: List[str]
    intensity: float
    z_space: ZSpace


class MetaNarrativeLayer:
    def __init__(self, engine: Optional[TemporalLogicEngine] = None, bridge: Optional[ToposLogicBridge] = None):
        self.engine: TemporalLogicEngine[NarrativeBeat] = engine or TemporalLogicEngine()
        self.bridge = bridge or ToposLogicBridge()

    from_parts = classmethod(lambda cls, engine, bridge: cls(engine, bridge))

    def engine_mut(self) -> TemporalLogicEngine:
        return self.engine

    def bridge_mut(self) -> ToposLogicBridge:
        return self.bridge

    def next_with_pulse(self, channel: str, pulse: MaxwellZPulse) -> Optional[ResolvedNarrative]:
        """Releases the first ready beat that accepts this channel and pulse: intensity is ``max(|z| * scale, floor)``,
        boosted by ``1 + sheaf weight`` when the event's sheaf contributes tags."""
        observed = ZSpace.from_pulse(pulse)
        hit = self.engine.next_matching(lambda beat: beat.matches(channel, observed))
        if hit is None:
            return None
        event_id, beat = hit
        base = max(pulse.magnitude() * beat.intensity_scale, beat.floor)
        sheaf_tags, sheaf_weight = self.bridge.resolve(event_id, beat.context, beat.sheaf_threshold, observed)
        tags = sorted(set(beat.base_tags) | {t for t, _ in sheaf_tags})
        return ResolvedNarrative(event_id, beat.channel or channel, tags, base * (1.0 + sheaf_weight) if sheaf_weight > 0.0 else base, observed)
