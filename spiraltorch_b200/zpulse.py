"""Z pulses and their conductor.  Every subsystem that has an opinion about the Z-space bias (microlocal gauges, the
Maxwell bridge, graph flows, the desire pipeline, gradient meters) emits `ZPulse` records; `ZConductor` fuses the pulses
that are due at a step into one `ZFused` control value with sign-flip hysteresis, a slew limit, a budget clamp and
per-source latency alignment against the microlocal anchor.

Parity: crates/st-core/src/theory/zpulse.rs — `ZScale` (:29-121), `ZSupport` (:125-190), `ZSource` (:194-203), `ZPulse`
(:207-308), `ZEmitter` (:311-322), `ZFrequencyConfig` / `ZAdaptiveGainCfg` / `LatencyAlignerCfg` (:326-424), the latency
aligner state machine (:444-585), `ZConductorCfg` / `ZFused` / `ZConductor::{ingest, step, step_from_registry}`
(:587-856), `derive_quality` (:878-889), `ZRegistry` (:1079-1114), `DesireEmitter` (:1118-1160); and
crates/st-core/src/theory/scale_persistence.rs — `zpulse_scale_stack` (:24-50), `zpulse_coherence_levels` (:51-62).
Host-side control logic: scalars per step, no device work.
"""
from __future__ import annotations

import math
import threading
from collections import deque
from dataclasses import dataclass, field, replace
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from . import observability

EPS = 1.1920929e-07                     # f32 epsilon: the thresholds below are the reference's f32 ones
SOURCES = ("microlocal", "maxwell", "graph", "desire", "gw", "realgrad")


def _finite(v: float) -> bool:
    return isinstance(v, (int, float)) and math.isfinite(v)


@dataclass(frozen=True)
class ZScale:
    """A physical radius with its logarithm carried along, so that blends stay consistent in both."""
    physical_radius: float
    log_radius: float

    @classmethod
    def new(cls, physical_radius: float) -> Optional["ZScale"]:
        if _finite(physical_radius) and physical_radius > 0.0:
            return cls(float(physical_radius), math.log(physical_radius))
        return None

    @classmethod
    def from_log(cls, log_radius: float) -> Optional["ZScale"]:
        if not _finite(log_radius):
            return None
        try:
            p = math.exp(log_radius)
        except OverflowError:
            return None
        return cls(p, float(log_radius)) if p > 0.0 and math.isfinite(p) else None

    @classmethod
    def from_components(cls, physical_radius: float, log_radius: float) -> Optional["ZScale"]:
        if _finite(physical_radius) and physical_radius > 0.0 and _finite(log_radius):
            return cls(float(physical_radius), float(log_radius))
        return None

    def value(self) -> float:
        return self.physical_radius

    @staticmethod
    def lerp(a: "ZScale", b: "ZScale", t: float) -> "ZScale":
        t = min(max(t, 0.0), 1.0)
        out = ZScale.from_components(a.physical_radius + (b.physical_radius - a.physical_radius) * t,
                                     a.log_radius + (b.log_radius - a.log_radius) * t)
        return out or (a if t < 0.5 else b)

    @staticmethod
    def weighted_average(weights: Iterable[Tuple["ZScale", float]]) -> Optional["ZScale"]:
        sp = sl = total = 0.0
        for scale, w in weights:
            if not _finite(w) or w <= 0.0:
                continue
            sp, sl, total = sp + scale.physical_radius * w, sl + scale.log_radius * w, total + w
        return ZScale.from_components(sp / total, sl / total) if total > 0.0 else None


ZScale.ONE = ZScale(1.0, 0.0)


def _nonneg(v: float) -> float:
    return max(float(v), 0.0) if _finite(v) else 0.0


@dataclass(frozen=True)
class ZSupport:
    leading: float = 0.0
    central: float = 0.0
    trailing: float = 0.0

    @classmethod
    def new(cls, leading: float, central: float, trailing: float) -> "ZSupport":
        return cls(_nonneg(leading), _nonneg(central), _nonneg(trailing))

    @classmethod
    def from_band_energy(cls, bands: Sequence[float]) -> "ZSupport":
        return cls.new(*bands)

    def total(self) -> float:
        return self.leading + self.central + self.trailing

    def is_empty(self) -> bool:
        return self.leading <= EPS and self.central <= EPS and self.trailing <= EPS

    def max_component(self) -> float:
        return max(abs(self.leading), abs(self.central), abs(self.trailing))


def source_label(source: str) -> str:
    """Known sources keep their name; anything else is ``other.<tag>``."""
    s = str(source).lower()
    return s if s in SOURCES or s.startswith("other.") else f"other.{s}"


@dataclass
class ZPulse:
    source: str = "microlocal"
    ts: int = 0
    tempo: float = 0.0
    band_energy: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    density_fluctuation: float = 0.0
    drift: float = 0.0
    z_bias: float = 0.0
    support: ZSupport = field(default_factory=ZSupport)
    scale: Optional[ZScale] = None
    quality: float = 0.0
    stderr: float = 0.0
    latency_ms: float = 0.0

    def __post_init__(self):
        self.source = source_label(self.source)
        if not isinstance(self.support, ZSupport):
            self.support = ZSupport.new(*self.support)
        self.band_energy = tuple(float(b) for b in self.band_energy)

    def support_mass(self) -> float:
        return self.support.total()

    def total_energy(self) -> float:
        return sum(self.band_energy)

    def normalised_drift(self) -> float:
        a, _, b = self.band_energy
        return (a - b) / max(self.total_energy(), 1e-6)

    def is_empty(self) -> bool:
        return self.support.is_empty() and self.total_energy() <= EPS

    @staticmethod
    def density_fluctuation_for(band_energy: Sequence[float]) -> float:
        """Standard deviation of the three band energies over their sum, in [0, 1]."""
        bands = [max(b, 0.0) if _finite(b) else 0.0 for b in band_energy]
        total = sum(bands)
        if total <= EPS:
            return 0.0
        mean = total / 3.0
        var = sum((b - mean) ** 2 for b in bands) / 3.0
        f = min(max(math.sqrt(var) / (total + 1e-6), 0.0), 1.0)
        return f if math.isfinite(f) else 0.0

    def features(self) -> List[float]:
        """The eight features the scale-persistence analysis stacks per pulse."""
        return [self.total_energy(), self.drift, self.z_bias, self.support_mass(), self.tempo, self.quality, self.latency_ms,
                self.density_fluctuation]


def derive_quality(pulse: ZPulse) -> float:
    """Quality for a pulse that did not bring one: 0.4 tanh(energy / (stderr + 1)) + 0.3 support / (support + 1) +
    0.3 drift / (drift + 1), discounted by up to 20 % for density fluctuation."""
    support = max(pulse.support_mass(), 1e-6)
    energy = max(pulse.total_energy(), 1e-6)
    drift, stderr = abs(pulse.drift), max(abs(pulse.stderr), 1e-6)
    base = 0.4 * math.tanh(energy / (stderr + 1.0)) + 0.3 * min(support / (support + 1.0), 1.0) + 0.3 * min(drift / (drift + 1.0), 1.0)
    return min(max(min(max(base, 0.0), 1.0) * (1.0 - min(max(pulse.density_fluctuation, 0.0), 1.0) * 0.2), 0.0), 1.0)


class ZEmitter:
    """A source of pulses: `tick(now)` is called until it returns ``None``."""

    def name(self) -> str:
        raise NotImplementedError

    def tick(self, now: int) -> Optional[ZPulse]:
        raise NotImplementedError

    def quality_hint(self) -> Optional[float]:
        return None


@dataclass(frozen=True)
class ZFrequencyConfig:
    smoothing: float = 0.0
    minimum_energy: float = 0.0

    @classmethod
    def new(cls, smoothing: float, minimum_energy: float) -> "ZFrequencyConfig":
        return cls(min(max(smoothing, 0.0), 1.0), max(minimum_energy, 0.0))


@dataclass(frozen=True)
class ZAdaptiveGainCfg:
    gain_floor: float = 0.0
    gain_ceil: float = 1.0
    responsiveness: float = 0.0

    @classmethod
    def new(cls, gain_floor: float, gain_ceil: float, responsiveness: float) -> "ZAdaptiveGainCfg":
        floor = max(gain_floor, 0.0)
        return cls(floor, max(gain_ceil, floor), min(max(responsiveness, 0.0), 1.0))


@dataclass(frozen=True)
class LatencyAlignerCfg:
    window: int = 128
    hop: int = 1
    max_lag_steps: int = 48
    alpha: float = 0.25
    coherence_min: float = 0.2
    hold_steps: int = 2
    fractional: bool = False

    @classmethod
    def balanced(cls) -> "LatencyAlignerCfg":
        return cls()

    @classmethod
    def from_steps(cls, max_lag_steps: int, alpha: float, coherence_min: float, hold_steps: int) -> "LatencyAlignerCfg":
        return cls(max_lag_steps=max_lag_steps, alpha=alpha, coherence_min=coherence_min, hold_steps=hold_steps)

    def with_window(self, window: int) -> "LatencyAlignerCfg":
        return replace(self, window=max(int(window), 1))

    def with_hop(self, hop: int) -> "LatencyAlignerCfg":
        return replace(self, hop=max(int(hop), 1))


def _lerp(a: float, b: float, t: float) -> float:
    return a + (b - a) * min(max(t, 0.0), 1.0)


def _round_half_away(x: float) -> float:
    return math.copysign(math.floor(abs(x) + 0.5), x)


def shift_timestamp(ts: int, lag: float, hop: int) -> int:
    if not _finite(lag):
        return ts
    return max(ts + int(_round_half_away(lag / max(hop, 1))), 0)


class _LatencyAligner:
    """Per-source lag against the microlocal anchor.  A pulse that carries `latency_ms` seeds its source's lag; otherwise
    the lag follows the timestamp distance to the anchor (clamped, rounded unless `fractional`, smoothed by `alpha`),
    at most once per `hold_steps` conductor steps."""

    def __init__(self, cfg: LatencyAlignerCfg):
        self.cfg = cfg
        self.last: Dict[str, Tuple[int, float]] = {}                    # source -> (ts, strength)
        self.lags: Dict[str, List] = {}                                 # source -> [lag, frames_since_update, seeded]
        self.pending_events: List[str] = []

    def record(self, pulse: ZPulse) -> None:
        prev = self.last.get(pulse.source)
        if prev is not None and pulse.ts < prev[0]:
            self.pending_events.append(f"latency.invalid_ts:{pulse.source}")
            return
        if _finite(pulse.latency_ms) and abs(pulse.latency_ms) > EPS:
            self.lags[pulse.source] = [float(pulse.latency_ms), 0, True]
            self.pending_events.append(f"latency.seeded:{pulse.source}:{pulse.latency_ms:.2f}")
        self.last[pulse.source] = (pulse.ts, max(pulse.support_mass(), 1e-6))

    def _increment_all(self) -> None:
        for est in self.lags.values():
            est[1] += 1

    def prepare(self, now: int, events: List[str]) -> None:
        events.extend(self.pending_events)
        self.pending_events = []
        anchor = self.last.get("microlocal")
        if anchor is None:
            self._increment_all()
            return
        if self.cfg.coherence_min > 1.0:                                # an unreachable coherence bar: nothing is adjusted
            events.extend(f"latency.low_coherence:{s}" for s in self.last if s != "microlocal")
            self._increment_all()
            return
        hop, max_lag = float(max(self.cfg.hop, 1)), float(max(self.cfg.max_lag_steps, 1))
        for source, (ts, _) in list(self.last.items()):
            if source == "microlocal":
                continue
            est = self.lags.setdefault(source, [0.0, 0, False])
            if est[2]:
                est[2] = False
                if self.cfg.hold_steps > 0:
                    events.append(f"latency.held:{source}")
                    est[1] = max(est[1], 1)
                    continue
            if est[1] != 0 and est[1] < self.cfg.hold_steps:
                events.append(f"latency.held:{source}")
                continue
            clamped = min(max(float(ts - anchor[0]), -max_lag), max_lag)
            units = (clamped if self.cfg.fractional else _round_half_away(clamped)) * hop
            est[0] = units if est[1] == 0 else _lerp(est[0], units, self.cfg.alpha)
            est[1] = 0
            events.append(f"latency.adjusted:{source}:{est[0]:.2f}")
        self._increment_all()
        self.last["microlocal"] = (now, anchor[1])

    def apply(self, pulse: ZPulse) -> None:
        est = self.lags.get(pulse.source)
        if est is not None and math.isfinite(est[0]):
            pulse.latency_ms = est[0]
            pulse.ts = shift_timestamp(pulse.ts, est[0], self.cfg.hop)

    def lag_for(self, source: str) -> Optional[float]:
        est = self.lags.get(source_label(source))
        return None if est is None else est[0]


@dataclass
class ZConductorCfg:
    alpha_fast: float = 0.35
    alpha_slow: float = 0.12
    flip_hold: int = 3
    slew_max: float = 0.35
    z_budget: float = 1.2
    robust_delta: float = 0.25
    latency_align: bool = True
    latency: Optional[LatencyAlignerCfg] = field(default_factory=LatencyAlignerCfg.balanced)


@dataclass
class ZFused:
    ts: int = 0
    z: float = 0.0
    support: float = 0.0
    drift: float = 0.0
    quality: float = 0.0
    density_fluctuation: float = 0.0
    events: List[str] = field(default_factory=list)
    attributions: List[Tuple[str, float]] = field(default_factory=list)


def _sign(v: float) -> float:
    return 0.0 if v == 0.0 or v != v else math.copysign(1.0, v)


class ZConductor:
    def __init__(self, cfg: Optional[ZConductorCfg] = None):
        self.cfg = cfg or ZConductorCfg()
        self.freq: Optional[ZFrequencyConfig] = None
        self.adaptive: Optional[ZAdaptiveGainCfg] = None
        self.latency: Optional[_LatencyAligner] = _LatencyAligner(self.cfg.latency or LatencyAlignerCfg.balanced())
        self.pending: deque = deque()
        self.last_step: Optional[int] = None
        self.last_z = 0.0
        self.hold_until: Optional[int] = None
        self.pending_flip_sign: Optional[float] = None

    def set_frequency_config(self, cfg: Optional[ZFrequencyConfig]) -> None:
        self.freq = cfg

    def set_adaptive_gain_config(self, cfg: Optional[ZAdaptiveGainCfg]) -> None:
        self.adaptive = cfg

    def set_latency_aligner(self, cfg: Optional[LatencyAlignerCfg]) -> None:
        self.latency = None if cfg is None else _LatencyAligner(cfg)

    def latency_for(self, source: str) -> Optional[float]:
        return None if self.latency is None else self.latency.lag_for(source)

    def ingest(self, pulse: ZPulse) -> None:
        pulse = replace(pulse)
        pulse.quality = derive_quality(pulse) if not _finite(pulse.quality) or pulse.quality <= 0.0 else min(max(pulse.quality, 0.0), 1.0)
        if self.latency is not None:
            self.latency.record(pulse)
        self.pending.append(pulse)

    def step(self, now: int) -> ZFused:
        self.last_step = now
        events: List[str] = []
        if self.latency is not None:
            self.latency.prepare(now, events)
        pending_before = len(self.pending)
        ready, retained = [], deque()
        while self.pending:
            pulse = self.pending.popleft()
            if self.cfg.latency_align and self.latency is not None:
                self.latency.apply(pulse)
            (ready if pulse.ts <= now else retained).append(pulse)
        self.pending = retained
        total = wz = wq = qw = dsum = dw = dens = densw = 0.0
        attributions: List[Tuple[str, float]] = []
        for p in ready:
            if p.is_empty():
                continue
            support = max(p.support_mass(), 0.0)
            total += support
            wz += p.z_bias * support
            w = max(support, 1e-6)
            wq, qw = wq + p.quality * w, qw + w
            dq = max(p.quality, 1e-6)
            dsum, dw = dsum + p.normalised_drift() * dq, dw + dq
            dens, densw = dens + p.density_fluctuation * support, densw + support
            attributions.append((p.source, support))
        attributions.sort(key=lambda a: -a[1])
        raw_z = wz / total if total > 0.0 else 0.0
        fused = ZFused(now, 0.0, total, min(max(dsum / dw, -1.0), 1.0) if dw > 0.0 else 0.0,
                       min(max(wq / qw, 0.0), 1.0) if qw > 0.0 else 0.0, min(max(dens / densw, 0.0), 1.0) if densw > 0.0 else 0.0,
                       events, attributions)
        incoming = _sign(raw_z)
        if self.hold_until is not None:
            if now < self.hold_until:
                fused.events.append("flip-held")
                raw_z = self.last_z
            else:
                self.hold_until = None
                if self.pending_flip_sign is not None:
                    fused.events.append("sign-flip")
                    raw_z = math.copysign(max(abs(raw_z), self.cfg.robust_delta), self.pending_flip_sign)
                    self.pending_flip_sign = None
        elif incoming != 0.0 and _sign(self.last_z) != 0.0 and incoming != _sign(self.last_z):
            self.hold_until = now + self.cfg.flip_hold
            self.pending_flip_sign = incoming
            fused.events.append("flip-held")
            raw_z = self.last_z
        alpha = min(max(self.cfg.alpha_fast if _sign(self.last_z) == incoming else self.cfg.alpha_slow, 0.0), 1.0)
        target = _lerp(self.last_z, raw_z, alpha)
        delta = target - self.last_z
        if abs(delta) > self.cfg.slew_max:
            target = self.last_z + math.copysign(self.cfg.slew_max, delta)
        target = min(max(target, -self.cfg.z_budget), self.cfg.z_budget)
        self.last_z = fused.z = target
        if fused.density_fluctuation > 0.45:
            fused.events.append(f"density.fluctuation:{fused.density_fluctuation:.3f}")
        self._emit(pending_before, len(ready), fused)
        return fused

    def step_from_registry(self, registry: "ZRegistry", now: int) -> ZFused:
        for pulse in registry.gather(now):
            self.ingest(pulse)
        return self.step(now)

    def _emit(self, pending_before: int, ready: int, fused: ZFused) -> None:
        observability.emit_tensor_op("zpulse_conductor_step", (pending_before, max(ready, 1)), (1, max(len(fused.attributions), 1)))

        def meta():
            by_source: Dict[str, float] = {}
            for s, v in fused.attributions:
                by_source[s] = by_source.get(s, 0.0) + max(v, 0.0)
            lags = [abs(e[0]) for e in (self.latency.lags.values() if self.latency else []) if math.isfinite(e[0])]
            out = {"backend": "host", "kind": "zpulse_conductor_step", "ts": fused.ts, "pending_before": pending_before,
                   "ready_count": ready, "retained_count": len(self.pending), "event_count": len(fused.events),
                   "latency_event_count": sum(e.startswith("latency.") for e in fused.events),
                   "flip_event_count": sum(e in ("flip-held", "sign-flip") for e in fused.events),
                   "density_event_count": sum(e.startswith("density.") for e in fused.events),
                   "attribution_count": len(fused.attributions), "top_source": fused.attributions[0][0] if fused.attributions else "none",
                   "top_source_support": fused.attributions[0][1] if fused.attributions else 0.0, "z": fused.z, "abs_z": abs(fused.z),
                   "support": fused.support, "drift": fused.drift, "quality": fused.quality, "density_fluctuation": fused.density_fluctuation,
                   "alpha_fast": self.cfg.alpha_fast, "alpha_slow": self.cfg.alpha_slow, "flip_hold": self.cfg.flip_hold,
                   "slew_max": self.cfg.slew_max, "z_budget": self.cfg.z_budget, "robust_delta": self.cfg.robust_delta,
                   "latency_align": self.cfg.latency_align, "latency_configured": self.latency is not None,
                   "latency_source_count": len(self.latency.lags) if self.latency else 0,
                   "latency_abs_mean": sum(lags) / len(lags) if lags else 0.0, "latency_abs_max": max(lags, default=0.0),
                   "frequency_configured": self.freq is not None, "adaptive_configured": self.adaptive is not None}
            out.update({f"source_{s}_support": by_source.get(s, 0.0) for s in SOURCES})
            return out
        observability.emit_tensor_op_meta("zpulse_conductor_step", meta)


class ZRegistry:
    def __init__(self):
        self.emitters: List[ZEmitter] = []

    def register(self, emitter: ZEmitter) -> None:
        self.emitters.append(emitter)

    def gather(self, now: int) -> List[ZPulse]:
        pulses = []
        for emitter in self.emitters:
            while True:
                pulse = emitter.tick(now)
                if pulse is None:
                    break
                if pulse.quality <= 0.0 and emitter.quality_hint() is not None:
                    pulse.quality = emitter.quality_hint()
                pulses.append(pulse)
        return pulses


class DesireEmitter(ZEmitter):
    """A thread-safe queue; whatever goes through comes out tagged as a desire pulse."""

    def __init__(self):
        self._queue: deque = deque()
        self._lock = threading.Lock()

    def name(self) -> str:
        return "desire"

    def enqueue(self, pulse: ZPulse) -> None:
        with self._lock:
            self._queue.append(pulse)

    def extend(self, pulses: Iterable[ZPulse]) -> None:
        with self._lock:
            self._queue.extend(pulses)

    def tick(self, now: int) -> Optional[ZPulse]:
        with self._lock:
            if not self._queue:
                return None
            return replace(self._queue.popleft(), source="desire")


# ---- scale persistence of a pulse train -----------------------------------------------------------------------------------
FEATURE_DIM = 8


def zpulse_scale_stack(pulses: Sequence[ZPulse], scales: Sequence[float], threshold: float, metric: str = "euclidean"):
    """Stacks the eight features of every pulse into a ``[pulses, 8]`` semantic field and measures at which scales
    neighbouring pulses differ by more than `threshold`."""
    from .frac import ScaleStack
    data = torch.tensor([p.features() for p in pulses], dtype=torch.float32).reshape(len(pulses), FEATURE_DIM)
    stack = ScaleStack.from_semantic_field(data, scales, threshold, 1, metric)
    observability.emit_tensor_op("zpulse_scale_stack", (len(pulses), FEATURE_DIM), (len(stack.samples), 2))
    observability.emit_tensor_op_meta("zpulse_scale_stack", lambda: {
        "backend": "torch", "kind": "zpulse_scale_stack", "pulse_count": len(pulses), "feature_dim": FEATURE_DIM,
        "scale_count": len(scales), "threshold": threshold, "metric": metric, "sample_count": len(stack.samples),
        **{f"source_{s}_count": sum(p.source == s for p in pulses) for s in SOURCES[:4]},
        "source_other_count": sum(p.source not in SOURCES[:4] for p in pulses)})
    return stack


def zpulse_coherence_levels(pulses: Sequence[ZPulse], scales: Sequence[float], threshold: float, metric: str, levels: Sequence[float]):
    """For each level, the smallest scale at which that fraction of the pulse train is already interface (or ``None``)."""
    return zpulse_scale_stack(pulses, scales, threshold, metric).coherence_profile(levels)
