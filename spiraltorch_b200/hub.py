"""Process-wide telemetry blackboard: the latest value of every cross-subsystem signal (psi reading / events / spiral
advisory, soft-logic Z feedback, real-gradient pulse, desire step, chrono loop, collapse pulse, maintainer report,
region attribution reports, psychoid reading), bounded histories (atlas route, dashboard frames, loopback envelopes,
config diffs) and the atlas frame that every producer's fragment is merged into.  All access is under one re-entrant
lock; observers are called outside of it.

Parity: crates/st-core/src/telemetry/hub.rs — psi store and `PsiMetricsSubscription` (:130-310, :392-570), atlas frame,
route (capacity 24), observers and `merge_atlas_fragment` (:314-360, :850-955), dashboard ring of 64 (:812-832),
`SoftlogicZFeedback` and its atlas metrics (:608-700, :1441-1530), `RealGradPulse` (:1137-1228), desire step store
(:758-800, :1238-1280), chrono loop (:1283-1291), `LoopbackEnvelope` buffer of 64 (:1295-1400, :1902-1930),
`CollapsePulse` (:1932-1965), region reports (:988-1052), config diff events (:366-392, :575-592).
"""
from __future__ import annotations

import math
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from . import observability
from .telemetry import AtlasFragment, AtlasFrame, AtlasRoute, AtlasRouteSummary, ChronoLoopSignal, DashboardRing, MaintainerReport
from .zpulse import ZScale, source_label

ATLAS_ROUTE_CAPACITY = 24
DASHBOARD_CAPACITY = 64
LOOPBACK_CAPACITY = 64

_lock = threading.RLock()


def telemetry_guard():
    """The hub's lock, for callers that must read several slots consistently (``with hub.telemetry_guard(): ...``)."""
    return _lock


# ---- records ---------------------------------------------------------------------------------------------------------------
@dataclass
class SoftlogicZFeedback:
    psi_total: float = 0.0
    weighted_loss: float = 0.0
    band_energy: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    drift: float = 0.0
    z_signal: float = 0.0
    scale: Optional[ZScale] = None
    events: List[str] = field(default_factory=list)
    attributions: List[Tuple[str, float]] = field(default_factory=list)
    elliptic: Optional[dict] = None          # curvature_radius, geodesic_radius, normalized_radius, spin_alignment, sheet_index, ...

    def has_event(self, tag: str) -> bool:
        return tag in self.events

    def push_event(self, tag: str) -> None:
        self.events.append(str(tag))

    def set_events(self, events) -> None:
        self.events = [str(e) for e in events]

    def set_attributions(self, attributions) -> None:
        self.attributions = [(source_label(s), max(float(w), 0.0)) for s, w in attributions]


@dataclass
class RealGradPulse:
    lebesgue_measure: float = 0.0
    monad_energy: float = 0.0
    z_energy: float = 0.0
    residual_ratio: float = 0.0
    lebesgue_ratio: float = 0.0
    ramanujan_pi: float = 0.0
    tolerance: float = 0.0
    convergence_error: float = 0.0
    iterations: int = 0
    dominated: bool = False
    converged: bool = False
    gradient_norm: float = 0.0
    gradient_sparsity: float = 1.0
    rolling_gradient_norm: float = 0.0
    rolling_residual_ratio: float = 0.0
    transparency: Optional[dict] = None

    def gradient_summary(self) -> dict:
        return {"norm": max(self.gradient_norm, 0.0), "sparsity": min(max(self.gradient_sparsity, 0.0), 1.0)}


@dataclass
class DesireStepTelemetry:
    timestamp: float
    entropy: float
    temperature: float
    hypergrad_penalty: float
    avoidance_energy: float
    logit_energy: float
    phase: str
    alpha: float
    beta: float
    gamma: float
    lam: float
    avoidance: Optional[dict] = None         # {"tokens": [...], "scores": [...]}
    trigger: Optional[dict] = None           # {"mean_penalty", "mean_entropy", "temperature", "samples"}
    trigger_emitted: bool = False
    psi_total: Optional[float] = None
    psi_breakdown: Dict[str, float] = field(default_factory=dict)
    psi_events: list = field(default_factory=list)
    z_feedback: Optional[SoftlogicZFeedback] = None


@dataclass
class LoopbackEnvelope:
    loop_signal: ChronoLoopSignal
    timestamp: float = 0.0
    source: Optional[str] = None
    support: float = 1.0
    collapse_total: Optional[float] = None
    z_signal: Optional[float] = None
    script_hint: Optional[str] = None

    def __post_init__(self):
        if not self.timestamp:
            self.timestamp = self.loop_signal.summary.latest_timestamp
        if not math.isfinite(self.support):
            self.support = 1.0
        self.collapse_total = self.collapse_total if self.collapse_total is not None and math.isfinite(self.collapse_total) else None
        self.z_signal = self.z_signal if self.z_signal is not None and math.isfinite(self.z_signal) else None


@dataclass
class CollapsePulse:
    step: int
    total: float
    command: dict                           # {"kind": "collapse" | "bloom" | "none", ...}
    loop_signal: Optional[ChronoLoopSignal] = None


@dataclass
class ConfigDiffEvent:
    layer: str                              # "base" | "site" | "run"
    path: str
    previous: object = None
    current: object = None


@dataclass
class AttributionReport:
    rows: int
    cols: int
    values: List[float]
    algorithm: str = "unknown"
    layer: Optional[str] = None
    target: Optional[str] = None
    steps: Optional[int] = None
    extras: dict = field(default_factory=dict)


@dataclass
class PsiMetricsFrame:
    reading: Optional[object] = None
    events: list = field(default_factory=list)
    spiral: Optional[object] = None
    tuning: Optional[object] = None


# ---- state -----------------------------------------------------------------------------------------------------------------
class _State:
    def __init__(self):
        self.slots: Dict[str, object] = {}
        self.psi_events: list = []
        self.atlas: Optional[AtlasFrame] = None
        self.route: deque = deque()
        self.dashboard = DashboardRing(DASHBOARD_CAPACITY)
        self.loopback: deque = deque()
        self.config_events: List[ConfigDiffEvent] = []
        self.atlas_observers: Dict[int, Callable[[AtlasFrame], None]] = {}
        self.psi_subscribers: Dict[int, PsiMetricsFrame] = {}
        self.next_id = 1


_state = _State()


def reset() -> None:
    """Forgets everything (observers and subscriptions included)."""
    global _state
    with _lock:
        _state = _State()


def _slot_set(name: str, value) -> None:
    with _lock:
        _state.slots[name] = value


def _slot_get(name: str):
    with _lock:
        return _state.slots.get(name)


def _slot_clear(name: str) -> bool:
    with _lock:
        return _state.slots.pop(name, None) is not None


# ---- psi -------------------------------------------------------------------------------------------------------------------
def _psi_frame() -> PsiMetricsFrame:
    return PsiMetricsFrame(_state.slots.get("psi"), list(_state.psi_events), _state.slots.get("psi_spiral"), _state.slots.get("psi_tuning"))


def _refresh_psi_subscribers() -> None:
    frame = _psi_frame()
    for f in _state.psi_subscribers.values():
        f.reading, f.events, f.spiral, f.tuning = frame.reading, list(frame.events), frame.spiral, frame.tuning


class PsiMetricsSubscription:
    """A live view of the psi slots; `snapshot()` returns the state as of the latest store.  `close()` (or garbage
    collection) detaches it."""

    def __init__(self, sid: Optional[int], frame: PsiMetricsFrame):
        self._id, self._frame = sid, frame

    @classmethod
    def detached(cls, frame: PsiMetricsFrame) -> "PsiMetricsSubscription":
        return cls(None, frame)

    def snapshot(self) -> PsiMetricsFrame:
        with _lock:
            f = self._frame
            return PsiMetricsFrame(f.reading, list(f.events), f.spiral, f.tuning)

    def close(self) -> None:
        if self._id is not None:
            with _lock:
                _state.psi_subscribers.pop(self._id, None)
            self._id = None

    __del__ = close


def subscribe_psi_metrics() -> PsiMetricsSubscription:
    with _lock:
        sid, _state.next_id = _state.next_id, _state.next_id + 1
        frame = _psi_frame()
        _state.psi_subscribers[sid] = frame
        return PsiMetricsSubscription(sid, frame)


def psi_subscriber_count() -> int:
    with _lock:
        return len(_state.psi_subscribers)


def set_last_psi(reading) -> None:
    with _lock:
        _state.slots["psi"] = reading
        _refresh_psi_subscribers()
    frag = AtlasFragment()
    frag.push_metric("psi.total", reading.total)
    for comp, value in reading.breakdown.items():
        frag.push_metric(f"psi.{getattr(comp, 'name', str(comp)).lower()}", value)
    if getattr(reading, "step", 0):
        frag.timestamp = float(reading.step)
    merge_atlas_fragment(frag)


def get_last_psi():
    return _slot_get("psi")


def clear_last_psi() -> None:
    with _lock:
        _state.slots.pop("psi", None)
        _refresh_psi_subscribers()


def set_last_psi_events(events: Sequence) -> None:
    with _lock:
        _state.psi_events = list(events)
        _refresh_psi_subscribers()
    if events:
        frag = AtlasFragment()
        frag.push_metric("psi.events", float(len(events)))
        for e in events:
            frag.push_note(str(e))
        merge_atlas_fragment(frag)


def get_last_psi_events() -> list:
    with _lock:
        return list(_state.psi_events)


def clear_last_psi_events() -> None:
    with _lock:
        _state.psi_events = []
        _refresh_psi_subscribers()


def set_last_psi_spiral(advisory) -> None:
    with _lock:
        _state.slots["psi_spiral"] = advisory
        _refresh_psi_subscribers()


def get_last_psi_spiral():
    return _slot_get("psi_spiral")


def set_last_psi_spiral_tuning(tuning) -> None:
    with _lock:
        _state.slots["psi_tuning"] = tuning
        _refresh_psi_subscribers()


def get_last_psi_spiral_tuning():
    return _slot_get("psi_tuning")


def clear_last_psi_spiral() -> None:
    with _lock:
        _state.slots.pop("psi_spiral", None)
        _refresh_psi_subscribers()


def clear_last_psi_spiral_tuning() -> None:
    with _lock:
        _state.slots.pop("psi_tuning", None)
        _refresh_psi_subscribers()


def set_last_psychoid(reading) -> None:
    _slot_set("psychoid", reading)


def get_last_psychoid():
    return _slot_get("psychoid")


# ---- config diffs -----------------------------------------------------------------------------------------------------------
def record_config_events(events: Sequence[ConfigDiffEvent]) -> None:
    with _lock:
        _state.config_events.extend(events)


def get_config_events() -> List[ConfigDiffEvent]:
    with _lock:
        return list(_state.config_events)


# ---- atlas -----------------------------------------------------------------------------------------------------------------
class AtlasFrameSubscription:
    def __init__(self, oid: int):
        self._id: Optional[int] = oid

    def close(self) -> None:
        if self._id is not None:
            with _lock:
                _state.atlas_observers.pop(self._id, None)
            self._id = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def register_atlas_frame_observer(callback: Callable[[AtlasFrame], None]) -> AtlasFrameSubscription:
    """`callback(frame)` runs after every store or merge, outside the hub's lock; keep the returned handle alive."""
    with _lock:
        oid, _state.next_id = _state.next_id, _state.next_id + 1
        _state.atlas_observers[oid] = callback
    return AtlasFrameSubscription(oid)


def atlas_observer_count() -> int:
    with _lock:
        return len(_state.atlas_observers)


def _copy_frame(frame: AtlasFrame) -> AtlasFrame:
    import copy
    return copy.deepcopy(frame)


def _publish_frame(frame: AtlasFrame) -> None:
    with _lock:
        if frame.timestamp > 0.0:
            _state.route.append(_copy_frame(frame))
            while len(_state.route) > ATLAS_ROUTE_CAPACITY:
                _state.route.popleft()
        observers = list(_state.atlas_observers.values())
    for cb in observers:
        cb(frame)


def set_atlas_frame(frame: AtlasFrame) -> None:
    with _lock:
        _state.atlas = _copy_frame(frame)
    _publish_frame(frame)


def get_atlas_frame() -> Optional[AtlasFrame]:
    with _lock:
        return None if _state.atlas is None else _copy_frame(_state.atlas)


def clear_atlas() -> None:
    with _lock:
        _state.atlas = None
        _state.route.clear()


def clear_atlas_route() -> None:
    with _lock:
        _state.route.clear()


def get_atlas_route(limit: Optional[int] = None) -> AtlasRoute:
    route = AtlasRoute()
    if limit == 0:
        return route
    with _lock:
        frames = list(_state.route)
    route.frames = frames if limit is None else frames[-limit:]
    return route


def get_atlas_route_summary(limit: Optional[int] = None) -> AtlasRouteSummary:
    return get_atlas_route(limit).summary()


def merge_atlas_fragment(fragment: AtlasFragment) -> None:
    if fragment.is_empty():
        return
    with _lock:
        if _state.atlas is not None:
            _state.atlas.merge_fragment(fragment)
            updated = _copy_frame(_state.atlas)
        else:
            updated = AtlasFrame.from_fragment(fragment)
            if updated is not None:
                _state.atlas = _copy_frame(updated)
    if updated is not None:
        _publish_frame(updated)


# ---- dashboard -------------------------------------------------------------------------------------------------------------
def push_dashboard_frame(frame) -> None:
    with _lock:
        _state.dashboard.push(frame)


def latest_dashboard_frame():
    with _lock:
        return _state.dashboard.latest()


def snapshot_dashboard_frames(limit: int) -> list:
    """The newest ``limit`` frames, newest first."""
    with _lock:
        frames = list(_state.dashboard)[::-1][:max(limit, 0)] if limit > 0 else []
    observability.emit_tensor_op("dashboard_snapshot_export", (limit,), (len(frames),))
    observability.emit_tensor_op_meta("dashboard_snapshot_export", lambda: {
        "backend": "host", "kind": "dashboard_snapshot_export", "requested_limit": limit, "returned_frames": len(frames),
        "metrics": sum(len(f.metrics) for f in frames), "events": sum(len(f.events) for f in frames)})
    return frames


# ---- maintainer, soft-logic feedback, region reports ---------------------------------------------------------------------------
def set_maintainer_report(report: MaintainerReport) -> None:
    _slot_set("maintainer", report)
    frag = AtlasFragment(maintainer_status=report.status, suggested_max_scale=report.suggested_max_scale, suggested_pressure=report.suggested_pressure)
    if report.diagnostic:
        frag.maintainer_diagnostic = report.diagnostic
        frag.push_note(f"maintainer.diagnostic:{report.diagnostic}")
    frag.push_note(f"maintainer.status:{report.status}")
    frag.push_metric("maintainer.average_drift", report.average_drift)
    frag.push_metric("maintainer.mean_energy", report.mean_energy)
    frag.push_metric("maintainer.mean_decay", report.mean_decay)
    frag.push_metric("maintainer.should_rewrite", 1.0 if report.should_rewrite() else 0.0)
    for name, peak in (("drift_peak", report.drift_peak), ("energy_peak", report.energy_peak)):
        if peak is not None:
            frag.push_metric(f"maintainer.{name}.frequency", peak.frequency)
            frag.push_metric(f"maintainer.{name}.magnitude", peak.magnitude)
            frag.push_metric(f"maintainer.{name}.phase", peak.phase)
    if report.spiralk_script:
        frag.script_hint = report.spiralk_script
    merge_atlas_fragment(frag)


def get_maintainer_report() -> Optional[MaintainerReport]:
    return _slot_get("maintainer")


def _softlogic_metrics(frag: AtlasFragment, prefix: str, fb: SoftlogicZFeedback) -> None:
    above, here, beneath = fb.band_energy
    for name, v in (("psi_total", fb.psi_total), ("weighted_loss", fb.weighted_loss), ("band.above", above), ("band.here", here),
                    ("band.beneath", beneath), ("band.total", above + here + beneath), ("drift", fb.drift), ("z_signal", fb.z_signal)):
        frag.push_metric(f"{prefix}.{name}", v)
    if fb.scale is not None:
        frag.push_metric(f"{prefix}.scale.physical", fb.scale.physical_radius)
        frag.push_metric(f"{prefix}.scale.log", fb.scale.log_radius)
    frag.push_metric(f"{prefix}.events", float(len(fb.events)))
    for e in fb.events:
        if e:
            frag.push_note(f"{prefix}.event:{e}")
    if fb.attributions:
        for source, w in fb.attributions:
            frag.push_metric(f"{prefix}.attribution.{source_label(source)}", w)
        frag.push_metric(f"{prefix}.attribution.total", sum(max(w, 0.0) for _, w in fb.attributions))
    for key, v in (fb.elliptic or {}).items():
        if isinstance(v, (int, float)):
            frag.push_metric(f"{prefix}.elliptic.{key}", float(v))


def set_softlogic_z(feedback: SoftlogicZFeedback) -> None:
    _slot_set("softlogic_z", feedback)
    frag = AtlasFragment(z_signal=feedback.z_signal)
    _softlogic_metrics(frag, "softlogic", feedback)
    if feedback.scale is not None:
        frag.push_note(f"softlogic.scale.radius:{feedback.scale.physical_radius:.3f}@{feedback.scale.log_radius:.3f}")
    merge_atlas_fragment(frag)


def get_softlogic_z() -> Optional[SoftlogicZFeedback]:
    return _slot_get("softlogic_z")


def clear_softlogic_z() -> bool:
    return _slot_clear("softlogic_z")


def _region_slot(slot: str):
    def setter(report: AttributionReport) -> None:
        fin = [v for v in report.values if math.isfinite(v)]
        observability.emit_tensor_op(f"region_{slot}_report_store", (report.rows, report.cols), (len(report.values),))
        observability.emit_tensor_op_meta(f"region_{slot}_report_store", lambda: {
            "backend": "host", "kind": f"region_{slot}_report_store", "slot": slot.replace("loss_", "") if slot != "loss" else "loss",
            "algorithm": report.algorithm, "rows": report.rows, "cols": report.cols, "values": len(report.values),
            "finite_values": len(fin), "non_finite_values": len(report.values) - len(fin), "positive_values": sum(v > 0 for v in fin),
            "negative_values": sum(v < 0 for v in fin), "mean_value": sum(fin) / len(fin) if fin else 0.0,
            "max_abs_value": max((abs(v) for v in fin), default=0.0)})
        _slot_set(f"region_{slot}", report)
    return setter, (lambda: _slot_get(f"region_{slot}")), (lambda: _slot_clear(f"region_{slot}"))


set_region_loss_report, get_region_loss_report, clear_region_loss_report = _region_slot("loss")
set_region_loss_trend_report, get_region_loss_trend_report, clear_region_loss_trend_report = _region_slot("loss_trend")
set_region_loss_volatility_report, get_region_loss_volatility_report, clear_region_loss_volatility_report = _region_slot("loss_volatility")


# ---- real-gradient pulse, desire step, chrono loop, loopback, collapse -------------------------------------------------------
def set_last_realgrad(pulse: RealGradPulse) -> None:
    _slot_set("realgrad", pulse)
    frag = AtlasFragment(timestamp=float(pulse.iterations) if pulse.iterations > 0 else None)
    for name in ("lebesgue_measure", "monad_energy", "z_energy", "residual_ratio", "lebesgue_ratio", "ramanujan_pi", "tolerance",
                 "convergence_error", "gradient_norm", "gradient_sparsity", "rolling_gradient_norm", "rolling_residual_ratio"):
        frag.push_metric(f"realgrad.{name}", getattr(pulse, name))
    frag.push_metric("realgrad.iterations", float(pulse.iterations))
    frag.push_metric("realgrad.dominated", 1.0 if pulse.dominated else 0.0)
    frag.push_metric("realgrad.converged", 1.0 if pulse.converged else 0.0)
    for key, v in (pulse.transparency or {}).items():
        if isinstance(v, (int, float)):
            frag.push_metric(f"realgrad.transparency.{key}", float(v))
    merge_atlas_fragment(frag)


def get_last_realgrad() -> Optional[RealGradPulse]:
    return _slot_get("realgrad")


def set_last_desire_step(step: DesireStepTelemetry) -> None:
    _slot_set("desire_step", step)
    frag = AtlasFragment()
    for name in ("entropy", "temperature", "hypergrad_penalty", "avoidance_energy", "logit_energy", "alpha", "beta", "gamma"):
        frag.push_metric(f"desire.{name}", getattr(step, name))
    frag.push_metric("desire.lambda", step.lam)
    for name, v in (("alpha", step.alpha), ("beta", step.beta), ("gamma", step.gamma), ("lambda", step.lam)):
        frag.push_metric(f"desire.weights.{name}", v)
    frag.push_metric("desire.trigger_emitted", 1.0 if step.trigger_emitted else 0.0)
    frag.push_note(f"desire.phase:{step.phase}")
    if step.trigger:
        for key in ("mean_penalty", "mean_entropy", "temperature", "samples"):
            frag.push_metric(f"desire.trigger.{key}", float(step.trigger.get(key, 0.0)))
    if step.avoidance:
        scores = list(step.avoidance.get("scores", []))
        frag.push_metric("desire.avoidance.tokens", float(len(step.avoidance.get("tokens", []))))
        if scores:
            frag.push_metric("desire.avoidance.score_mean", sum(scores) / len(scores))
            frag.push_metric("desire.avoidance.score_max", max(scores))
            frag.push_metric("desire.avoidance.score_min", min(scores))
    if step.z_feedback is not None:
        _softlogic_metrics(frag, "desire.z_feedback", step.z_feedback)
        frag.z_signal = step.z_feedback.z_signal
    for comp, v in step.psi_breakdown.items():
        frag.push_metric(f"desire.psi.{getattr(comp, 'name', str(comp)).lower()}", v)
    if step.psi_total is not None:
        frag.push_metric("desire.psi.total", step.psi_total)
    if math.isfinite(step.timestamp) and step.timestamp > 0:
        frag.timestamp = float(step.timestamp)
    if step.psi_events:
        frag.push_metric("desire.psi.events", float(len(step.psi_events)))
        for e in step.psi_events:
            frag.push_note(f"desire.psi.event:{e}")
    merge_atlas_fragment(frag)


def get_last_desire_step() -> Optional[DesireStepTelemetry]:
    return _slot_get("desire_step")


def clear_last_desire_step() -> None:
    _slot_clear("desire_step")


def set_chrono_loop(signal: ChronoLoopSignal) -> None:
    _slot_set("chrono_loop", signal)


def get_chrono_loop() -> Optional[ChronoLoopSignal]:
    return _slot_get("chrono_loop")


def push_loopback_envelope(envelope: LoopbackEnvelope) -> None:
    with _lock:
        _state.loopback.append(envelope)
        while len(_state.loopback) > LOOPBACK_CAPACITY:
            _state.loopback.popleft()
    s = envelope.loop_signal.summary
    frag = AtlasFragment(timestamp=envelope.timestamp, summary=s, harmonics=envelope.loop_signal.harmonics, loop_support=envelope.support,
                         collapse_total=envelope.collapse_total, z_signal=envelope.z_signal, script_hint=envelope.script_hint)
    if envelope.source:
        frag.push_note(f"source:{envelope.source}")
    frag.push_metric("loop.frames", float(s.frames))
    frag.push_metric("loop.energy", s.mean_energy)
    frag.push_metric("loop.drift", s.mean_drift)
    if envelope.collapse_total is not None:
        frag.push_metric("collapse.total", envelope.collapse_total)
    if envelope.z_signal is not None:
        frag.push_metric("z.bias", envelope.z_signal)
    merge_atlas_fragment(frag)


def drain_loopback_envelopes(limit: int) -> List[LoopbackEnvelope]:
    """Removes and returns up to ``limit`` of the oldest envelopes."""
    out = []
    with _lock:
        while _state.loopback and len(out) < limit:
            out.append(_state.loopback.popleft())
    return out


def peek_loopback_envelopes(limit: int) -> List[LoopbackEnvelope]:
    with _lock:
        return list(_state.loopback)[:max(limit, 0)]


def set_collapse_pulse(pulse: CollapsePulse) -> None:
    _slot_set("collapse", pulse)
    frag = AtlasFragment(timestamp=float(pulse.step) if pulse.step > 0 else None, collapse_total=pulse.total)
    frag.push_metric("collapse.total", pulse.total)
    frag.push_metric("collapse.step", float(pulse.step))
    frag.push_note(f"collapse.command:{pulse.command.get('kind', 'none')}")
    for key, v in pulse.command.items():
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            frag.push_metric(f"collapse.command.{key}", float(v))
    if pulse.loop_signal is not None:
        frag.summary, frag.harmonics = pulse.loop_signal.summary, pulse.loop_signal.harmonics
    merge_atlas_fragment(frag)


def get_collapse_pulse() -> Optional[CollapsePulse]:
    return _slot_get("collapse")
