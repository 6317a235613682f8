"""Robotics runtime: sensor fusion, desire energies, stability telemetry, a learning-rate
controller, safety plugins and a bounded trajectory recorder.

Restated from crates/st-robotics/src: ``SensorFusionHub`` (sensors.rs:119-300 — per-channel bias /
scale calibration, exponential smoothing, staleness health), ``ZSpaceGeometry.metric_norm``
(geometry.rs:50-97), ``Desire`` / ``DesireLagrangianField`` (desire.rs:8-90), ``PsiTelemetry``
(telemetry.rs:18-125 — stability = 1/(1+σ) of the energy window, anomaly tags, failsafe),
``PolicyGradientController`` (policy.rs:8-35), ``RoboticsRuntime.step`` (runtime.rs:66-101) and
``SafetyPlugin`` (safety.rs:12-30).
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional


class RoboticsError(ValueError):
    pass


@dataclass
class ChannelHealth:
    stale: bool
    optional: bool


@dataclass
class FusedFrame:
    coordinates: dict
    timestamp: float
    health: dict

    def norm(self, channel: str) -> Optional[float]:
        v = self.coordinates.get(channel)
        return None if v is None else math.sqrt(sum(x * x for x in v))


class _Channel:
    def __init__(self, dimension: int):
        self.dimension = dimension
        self.bias = [0.0] * dimension
        self.scale = 1.0
        self.alpha: Optional[float] = None
        self.state: Optional[list] = None
        self.optional = False
        self.max_staleness: Optional[float] = None
        self.last_update: Optional[float] = None

    def apply(self, values, now: float):
        out = [(v - b) * self.scale for v, b in zip(values, self.bias)]
        if self.alpha is not None:
            if self.state is not None:
                out = [self.alpha * v + (1.0 - self.alpha) * s for v, s in zip(out, self.state)]
            self.state = list(out)
        stale = self.max_staleness is not None and self.last_update is not None and \
            now - self.last_update > self.max_staleness
        self.last_update = now
        return out, stale


class SensorFusionHub:
    def __init__(self, clock: Callable[[], float] = time.monotonic):
        self._channels: dict[str, _Channel] = {}
        self._clock = clock

    def register_channel(self, name: str, dimension: int, smoothing: Optional[float] = None, optional: bool = False,
                         max_staleness: Optional[float] = None) -> None:
        if dimension <= 0:
            raise RoboticsError(f"channel '{name}' must have a positive dimension")
        if name in self._channels:
            raise RoboticsError(f"channel '{name}' already exists")
        ch = _Channel(dimension)
        if smoothing is not None:
            self._set_smoothing(name, ch, smoothing)
        if max_staleness is not None:
            if max_staleness <= 0:
                raise RoboticsError(f"channel '{name}': staleness threshold {max_staleness} must be positive")
            ch.max_staleness = max(max_staleness, 1e-3)
        ch.optional = optional
        self._channels[name] = ch

    @staticmethod
    def _set_smoothing(name: str, ch: _Channel, alpha: float) -> None:
        if not 0.0 < alpha <= 1.0:
            raise RoboticsError(f"channel '{name}': smoothing coefficient {alpha} is outside (0, 1]")
        ch.alpha, ch.state = alpha, None

    def _get(self, name: str) -> _Channel:
        if name not in self._channels:
            raise RoboticsError(f"channel '{name}' is not registered")
        return self._channels[name]

    def calibrate(self, name: str, bias=None, scale: Optional[float] = None) -> None:
        ch = self._get(name)
        if bias is not None:
            if len(bias) != ch.dimension:
                raise RoboticsError(f"channel '{name}': bias has {len(bias)} values, expected {ch.dimension}")
            ch.bias = [float(b) for b in bias]
        if scale is not None:
            ch.scale = float(scale)

    def configure_smoothing(self, name: str, smoothing: Optional[float]) -> None:
        ch = self._get(name)
        if smoothing is None:
            ch.alpha, ch.state = None, None
        else:
            self._set_smoothing(name, ch, smoothing)

    def fuse(self, payloads: dict) -> FusedFrame:
        now = self._clock()
        coords, health = {}, {}
        for name, ch in self._channels.items():
            if name in payloads:
                values = list(payloads[name])
                if len(values) != ch.dimension:
                    raise RoboticsError(f"channel '{name}': got {len(values)} values, expected {ch.dimension}")
                coords[name], stale = ch.apply(values, now)
                health[name] = ChannelHealth(stale, ch.optional)
            elif ch.optional:
                stale = ch.max_staleness is not None and (ch.last_update is None or now - ch.last_update > ch.max_staleness)
                health[name] = ChannelHealth(stale, True)
            else:
                raise RoboticsError(f"missing payload for required channel '{name}'")
        return FusedFrame(coords, now, health)


class ZSpaceGeometry:
    def __init__(self, kind: str = "euclidean", curvature: float = 0.0, metric=None, time_dilation: float = 1.0):
        self.kind, self.curvature, self.metric, self.time_dilation = kind, curvature, metric, time_dilation

    @classmethod
    def euclidean(cls):
        return cls()

    @classmethod
    def non_euclidean(cls, curvature: float):
        return cls("non_euclidean", curvature)

    @classmethod
    def general_relativity(cls, metric, time_dilation: float):
        return cls("general_relativity", 0.0, [list(r) for r in metric], time_dilation)

    def metric_norm(self, vector) -> float:
        if not vector:
            return 0.0
        e = math.sqrt(sum(v * v for v in vector))
        if self.kind == "euclidean":
            return e
        if self.kind == "non_euclidean":
            c = self.curvature
            if abs(c) < 1e-6:
                return e
            if c > 0:
                return e * (1.0 + c * e * e / 6.0)
            return e / max(1.0 + abs(c) * e * e / 6.0, 1e-6)
        acc = 0.0
        for i, vi in enumerate(vector):
            for j, vj in enumerate(vector):
                try:
                    g = self.metric[i][j]
                except (IndexError, TypeError):
                    g = 1.0 if i == j else 0.0
                acc += vi * g * vj
        return math.sqrt(abs(acc)) * max(self.time_dilation, 1e-6)


@dataclass
class Desire:
    target_norm: float
    tolerance: float
    weight: float

    def energy(self, norm: float) -> float:
        return max(abs(norm - self.target_norm) - self.tolerance, 0.0) * self.weight


@dataclass
class EnergyReport:
    total: float = 0.0
    per_channel: dict = field(default_factory=dict)
    gravitational: float = 0.0
    gravitational_per_channel: dict = field(default_factory=dict)


class DesireLagrangianField:
    def __init__(self, desires: dict, geometry: Optional[ZSpaceGeometry] = None, gravity: Optional[Callable] = None):
        self.desires, self.geometry, self.gravity = dict(desires), geometry or ZSpaceGeometry(), gravity

    def energy(self, frame: FusedFrame) -> EnergyReport:
        rep = EnergyReport()
        for name, desire in self.desires.items():
            v = frame.coordinates.get(name)
            if v is None:
                continue
            e = desire.energy(self.geometry.metric_norm(v))
            rep.per_channel[name] = e
            rep.total += e
            if self.gravity is not None:
                g = float(self.gravity(name, v))
                rep.gravitational_per_channel[name] = g
                rep.gravitational += g
        rep.total += rep.gravitational
        return rep


@dataclass
class TelemetryReport:
    energy: float
    stability: float
    failsafe: bool
    anomalies: list


class PsiTelemetry:
    def __init__(self, window: int = 8, stability_threshold: float = 0.5, failure_energy: float = 5.0,
                 norm_limit: float = 10.0, geometry: Optional[ZSpaceGeometry] = None):
        self.window, self.stability_threshold = max(1, window), stability_threshold
        self.failure_energy, self.norm_limit = failure_energy, norm_limit
        self.geometry = geometry or ZSpaceGeometry()
        self._history: deque = deque(maxlen=self.window)

    def observe(self, frame: FusedFrame, energy: EnergyReport) -> TelemetryReport:
        self._history.append(energy.total)
        if len(self._history) < 2:
            stability = 1.0
        else:
            mean = sum(self._history) / len(self._history)
            stability = 1.0 / (1.0 + math.sqrt(sum((v - mean) ** 2 for v in self._history) / len(self._history)))
        anomalies = set()
        if stability < self.stability_threshold:
            anomalies.add("instability")
        if energy.total > self.failure_energy:
            anomalies.add("energy_overflow")
        if abs(energy.gravitational) > self.failure_energy:
            anomalies.add("gravity_overflow")
        for v in frame.coordinates.values():
            if self.geometry.metric_norm(v) > self.norm_limit:
                anomalies.add("norm_overflow")
        for name, h in frame.health.items():
            if h.stale:
                anomalies.add(f"stale:{name}")
                stability *= 0.5
        failsafe = "norm_overflow" in anomalies or energy.total > self.failure_energy or \
            abs(energy.gravitational) > self.failure_energy
        return TelemetryReport(energy.total, stability, failsafe, sorted(anomalies))


class PolicyGradientController:
    def __init__(self, base_learning_rate: float, smoothing: float):
        self.base_learning_rate, self.smoothing, self.gauge = base_learning_rate, smoothing, 0.0

    def update(self, energy: EnergyReport, telemetry: TelemetryReport) -> dict:
        self.gauge = self.gauge * self.smoothing + telemetry.stability * (1.0 - self.smoothing)
        return {"learning_rate": self.base_learning_rate / (1.0 + max(energy.total, 0.0)), "gauge": self.gauge}


@dataclass
class SafetyReview:
    plugin: str
    refused: bool
    hazard: float = 0.0
    flagged: list = field(default_factory=list)


class SafetyPlugin:
    name = "safety"

    def review(self, frame: FusedFrame, energy: EnergyReport, telemetry: TelemetryReport) -> SafetyReview:
        raise NotImplementedError


class DriftSafetyPlugin(SafetyPlugin):
    """Refuses when a channel's desire energy, scaled by instability, passes the hazard cut."""

    def __init__(self, name: str = "drift", hazard_cut: float = 0.8):
        self.name, self._hazard_cut, self._thresholds = name, hazard_cut, {}

    def set_hazard_cut(self, hazard_cut: float) -> None:
        self._hazard_cut = hazard_cut

    def hazard_cut(self) -> float:
        return self._hazard_cut

    def set_threshold(self, channel: str, hazard: float) -> None:
        self._thresholds[channel] = hazard

    def thresholds(self) -> dict:
        return dict(self._thresholds)

    def review(self, frame, energy, telemetry) -> SafetyReview:
        flagged, worst = [], 0.0
        for ch, e in energy.per_channel.items():
            hazard = 1.0 - math.exp(-max(e, 0.0)) * min(max(telemetry.stability, 0.0), 1.0)
            worst = max(worst, hazard)
            if hazard >= self._thresholds.get(ch, self._hazard_cut):
                flagged.append(ch)
        return SafetyReview(self.name, bool(flagged), worst, sorted(flagged))


@dataclass
class RuntimeStep:
    frame: FusedFrame
    energy: EnergyReport
    telemetry: TelemetryReport
    commands: dict
    halted: bool
    safety: list


class TrajectoryRecorder:
    def __init__(self, capacity: int):
        self._steps: deque = deque(maxlen=max(1, capacity))

    def push(self, step: RuntimeStep) -> None:
        self._steps.append(step)

    def __len__(self) -> int:
        return len(self._steps)

    def is_empty(self) -> bool:
        return not self._steps

    def drain(self) -> list:
        out = list(self._steps)
        self._steps.clear()
        return out


class RoboticsRuntime:
    def __init__(self, sensors: SensorFusionHub, desires: DesireLagrangianField, telemetry: PsiTelemetry):
        self._sensors, self._desires, self._telemetry = sensors, desires, telemetry
        self._policy: Optional[PolicyGradientController] = None
        self._safety: list[SafetyPlugin] = []
        self._recorder: Optional[TrajectoryRecorder] = None

    def attach_policy_gradient(self, controller: PolicyGradientController) -> None:
        self._policy = controller

    def attach_safety_plugin(self, plugin: SafetyPlugin) -> None:
        self._safety.append(plugin)

    def clear_safety_plugins(self) -> None:
        self._safety.clear()

    def sensors(self) -> SensorFusionHub:
        return self._sensors

    def desires(self) -> DesireLagrangianField:
        return self._desires

    def telemetry(self) -> PsiTelemetry:
        return self._telemetry

    def enable_recording(self, capacity: int) -> None:
        self._recorder = TrajectoryRecorder(capacity)

    def recording_len(self) -> int:
        return 0 if self._recorder is None else len(self._recorder)

    def drain_trajectory(self) -> list:
        return [] if self._recorder is None else self._recorder.drain()

    def step(self, payloads: dict) -> RuntimeStep:
        frame = self._sensors.fuse(payloads)
        energy = self._desires.energy(frame)
        report = self._telemetry.observe(frame, energy)
        commands = {}
        if self._policy is not None:
            commands.update(self._policy.update(energy, report))
        halted = report.failsafe
        reviews = []
        for p in self._safety:
            r = p.review(frame, energy, report)
            halted = halted or r.refused
            reviews.append(r)
        if halted:
            commands["halt"] = 1.0
        step = RuntimeStep(frame, energy, report, commands, halted, reviews)
        if self._recorder is not None:
            self._recorder.push(step)
        return step
