"""Soft-rule scoring, beam selection, the SpiralK block IR, phase synchronisation and refract
lowering.

Restated from
* crates/st-softlogic/src/lib.rs:13-140 — ``SoftMode`` {Sum, Normalize, Softmax, Prob},
  ``apply_softmode``, ``beam_select`` (NaN scores rank last);
* crates/st-softlogic/src/spiralk/ir.rs — ``RefractBlock`` / ``SyncBlock`` / ``FeedbackBlock``;
* crates/st-sync/src/lib.rs:36-221 — ``PhaseSync.merge``: candidates inside the tolerance window win,
  score = 0.6·trust + 0.3·phase term + 0.1·tanh(resonance), ties by trust, phase delta, resonance;
* crates/st-refract/src/lib.rs:25-70 — lowering a refract block onto a backend object with
  begin / commit / rollback;
* crates/st-zeta/src/lib.rs — feedback blocks emitted as telemetry events.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from . import plugin

F32_EPS = 1.1920929e-07


@dataclass
class SoftRule:
    name: str
    weight: float
    score: float


@dataclass
class SolveCfg:
    noise: float = 0.0
    seed: int = 0
    beam: Optional[int] = None
    soft_mode: str = "sum"


@dataclass
class Ctx:
    rows: int
    cols: int
    k: int
    sg: bool = True


def _safe_sigmoid(x: float) -> float:
    if x > 20.0:
        return 1.0
    if x < -20.0:
        return 0.0
    return 1.0 / (1.0 + math.exp(-x))


def apply_softmode(rules: Sequence[SoftRule], mode: str) -> float:
    mode = mode.lower()
    if not rules:
        return 0.0
    if mode == "sum":
        return sum(r.weight * r.score for r in rules)
    if mode == "normalize":
        sw = max(sum(abs(r.weight) for r in rules), 1e-6)
        return sum(r.weight / sw * r.score for r in rules)
    if mode == "softmax":
        m = max(r.score for r in rules)
        ex = [math.exp(r.score - m) for r in rules]
        z = max(sum(ex), 1e-6)
        return sum(r.weight * e / z for r, e in zip(rules, ex))
    if mode == "prob":
        p_none = 1.0
        for r in rules:
            pw = min(max(_safe_sigmoid(r.score) * min(max(r.weight, 0.0), 1.0), 0.0), 1.0)
            p_none *= 1.0 - pw
        q = min(max(1.0 - p_none, 1e-6), 1.0 - 1e-6)
        return math.log(q / (1.0 - q))
    raise ValueError(f"unknown soft mode '{mode}'")


def beam_select(seed, expand: Callable, score_fn: Callable, beam_k: int, max_depth: int):
    """Beam search: at every depth expand head + tail, keep the best ``beam_k`` (NaN last)."""
    head, tail = seed, []
    for _ in range(max_depth):
        pool = []
        for cand in [head] + tail:
            for c in expand(cand):
                pool.append((c, score_fn(c)))
        if not pool:
            break
        pool.sort(key=lambda n: (math.isnan(n[1]), -n[1] if not math.isnan(n[1]) else 0.0))
        head = pool[0][0]
        tail = [c for c, _ in pool[1:max(1, beam_k)]]
    return head


# ---- SpiralK block IR --------------------------------------------------------------------------
PRECISIONS = ("fp32", "fp16", "bf16")
LAYOUTS = ("nhwc", "nchw", "blocked")
BACKENDS = ("wgpu", "mps", "cuda", "cpu")


@dataclass
class RefractOpPolicy:
    op: str
    flags: list = field(default_factory=list)


@dataclass
class RefractBlock:
    name: str
    target: tuple               # ("graph", name) | ("prsn", name)
    precision: Optional[str] = None
    layout: Optional[str] = None
    schedule: Optional[str] = None
    backend: Optional[str] = None
    policies: list = field(default_factory=list)


@dataclass
class SyncBlock:
    name: str
    pairs: list
    tolerance: float = 0.0


@dataclass
class FeedbackBlock:
    name: str
    export_path: str
    metrics: list = field(default_factory=list)


# ---- st-sync -----------------------------------------------------------------------------------
@dataclass
class PhaseCandidate:
    graph_id: str
    phase_delta: float
    trust: float
    resonance: float


@dataclass
class PhaseSelection:
    graph_id: str
    pairs: list
    score: float
    phase_delta: float
    trust: float
    resonance: float


def _nonneg_finite(label: str, v: float) -> None:
    if not math.isfinite(v):
        raise ValueError(f"{label} must be finite")
    if v < 0:
        raise ValueError(f"{label} must not be negative")


class PhaseSync:
    def __init__(self, default_tolerance: float = 0.05):
        self.default_tolerance = default_tolerance

    @classmethod
    def try_new(cls, default_tolerance: float) -> "PhaseSync":
        _nonneg_finite("default tolerance", default_tolerance)
        return cls(default_tolerance)

    @staticmethod
    def _score(c: PhaseCandidate, tol: float) -> float:
        trust = min(max(c.trust, 0.0), 1.0)
        phase = min(max((tol - c.phase_delta) / tol, 0.0), 1.0) if tol > 0 else 1.0 / (1.0 + c.phase_delta)
        return 0.6 * trust + 0.3 * phase + 0.1 * max(math.tanh(c.resonance), 0.0)

    @staticmethod
    def _tie_break(cur: PhaseCandidate, best: PhaseCandidate) -> bool:
        if cur.trust > best.trust + F32_EPS:
            return True
        same_trust = abs(cur.trust - best.trust) <= F32_EPS
        if same_trust and cur.phase_delta + F32_EPS < best.phase_delta:
            return True
        return same_trust and abs(cur.phase_delta - best.phase_delta) <= F32_EPS and cur.resonance > best.resonance

    def _validate(self, sync: SyncBlock, candidates: Sequence[PhaseCandidate]) -> None:
        if not sync.name.strip():
            raise ValueError("sync block name must not be empty")
        if not sync.pairs:
            raise ValueError(f"sync block '{sync.name}' must specify at least one pair")
        seen = set()
        for i, p in enumerate(sync.pairs):
            if not p.strip():
                raise ValueError(f"sync block '{sync.name}' contains an empty pair at index {i}")
            if p in seen:
                raise ValueError(f"sync block '{sync.name}' contains duplicate pair '{p}'")
            seen.add(p)
        _nonneg_finite("sync tolerance", sync.tolerance)
        _nonneg_finite("default tolerance", self.default_tolerance)
        ids = set()
        for i, c in enumerate(candidates):
            if not c.graph_id.strip():
                raise ValueError(f"candidate at index {i} has an empty graph id")
            if c.graph_id in ids:
                raise ValueError(f"candidate graph id '{c.graph_id}' is duplicated")
            ids.add(c.graph_id)
            _nonneg_finite(f"candidate '{c.graph_id}': candidate phase delta", c.phase_delta)
            for label, v in (("trust", c.trust), ("resonance", c.resonance)):
                if not math.isfinite(v):
                    raise ValueError(f"candidate '{c.graph_id}': candidate {label} must be finite")

    def merge(self, sync: SyncBlock, candidates: Sequence[PhaseCandidate]) -> Optional[PhaseSelection]:
        self._validate(sync, candidates)
        if not candidates:
            return None
        tol = sync.tolerance if sync.tolerance > 0 else max(self.default_tolerance, 0.0)
        best, best_within, best_score = None, False, -math.inf
        for c in candidates:
            within = tol <= 0 or c.phase_delta <= tol
            score = self._score(c, tol)
            if best is None or (within and not best_within):
                choose = True
            elif within == best_within:
                choose = score > best_score + F32_EPS or (abs(score - best_score) <= F32_EPS and self._tie_break(c, best))
            else:
                choose = False
            if choose:
                best, best_within, best_score = c, within, score
        return PhaseSelection(best.graph_id, list(sync.pairs), best_score, best.phase_delta, best.trust, best.resonance)


# ---- st-refract ----------------------------------------------------------------------------------
_IDENT = re.compile(r"^[A-Za-z_][A-Za-z0-9_\-\.]*$")


class KdslBackend:
    """Receiver of a lowered refract block; every hook defaults to a no-op."""

    def begin_refract(self, block): ...
    def select_target(self, target): ...
    def set_precision(self, precision): ...
    def set_layout(self, layout): ...
    def set_schedule(self, schedule): ...
    def select_backend(self, backend): ...
    def tune_op(self, op, flags): ...
    def commit_refract(self, block): ...
    def rollback_refract(self, block): ...


def validate_refract_block(block: RefractBlock) -> None:
    def ident(v, what):
        if not v or not _IDENT.match(v):
            raise ValueError(f"invalid {what} '{v}'")

    ident(block.name, "block name")
    kind, name = block.target
    if kind not in ("graph", "prsn"):
        raise ValueError(f"unknown target kind '{kind}'")
    ident(name, f"{kind} target")
    if block.schedule is not None:
        ident(block.schedule, "schedule")
    if block.precision is not None and block.precision not in PRECISIONS:
        raise ValueError(f"unknown precision '{block.precision}'")
    if block.layout is not None and block.layout not in LAYOUTS:
        raise ValueError(f"unknown layout '{block.layout}'")
    if block.backend is not None and block.backend not in BACKENDS:
        raise ValueError(f"unknown backend '{block.backend}'")
    seen = set()
    for pol in block.policies:
        ident(pol.op, "policy op")
        if pol.op in seen:
            raise ValueError(f"duplicate policy for op '{pol.op}'")
        seen.add(pol.op)


def lower_refract(block: RefractBlock, backend: KdslBackend) -> None:
    """Apply ``block`` to ``backend``; any failure (including in ``commit``) triggers ``rollback``
    and is re-raised with the block name."""
    validate_refract_block(block)
    backend.begin_refract(block)
    try:
        backend.select_target(block.target)
        if block.precision is not None:
            backend.set_precision(block.precision)
        if block.layout is not None:
            backend.set_layout(block.layout)
        if block.schedule is not None:
            backend.set_schedule(block.schedule)
        if block.backend is not None:
            backend.select_backend(block.backend)
        for pol in block.policies:
            backend.tune_op(pol.op, list(pol.flags))
        backend.commit_refract(block)
    except Exception as exc:
        try:
            backend.rollback_refract(block)
        except Exception as rb:  # noqa: BLE001
            raise RuntimeError(f"refract block '{block.name}' failed ({exc}); rollback also failed ({rb})") from exc
        raise RuntimeError(f"refract block '{block.name}' failed: {exc}") from exc


# ---- st-zeta -------------------------------------------------------------------------------------
def emit_feedback(block: FeedbackBlock, values: dict) -> dict:
    """Publish the metrics a feedback block names as one ``Telemetry`` event; returns the payload.
    Metrics without a finite value are reported under ``missing``."""
    present, missing = {}, []
    for m in block.metrics:
        v = values.get(m)
        if v is None or not math.isfinite(float(v)):
            missing.append(m)
        else:
            present[m] = float(v)
    payload = {"feedback": block.name, "export_path": block.export_path, "metrics": present, "missing": missing}
    plugin.publish("Telemetry", payload)
    return payload
