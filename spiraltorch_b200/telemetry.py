"""Telemetry: monitoring hub (feature drift + performance regression alerts), metric exporters,
a chrono timeline of per-step observations, and device-timed step metrics.

Restated from crates/st-core/src/telemetry/monitoring.rs:14-690 (``DriftDetector`` with a frozen
Welford baseline and a 32-sample window, ``PerformanceMonitor`` with three consecutive failures
before a critical alert, ``MonitoringHub`` with an alert ring and exporter fan-out; gauge names
``runtime_step_time_ms`` / ``runtime_mem_peak_mb`` / ``runtime_retry_rate`` / ``runtime_reward`` /
``extra_*`` / ``performance_*``) and crates/st-core/src/telemetry/chrono.rs:431-740
(``ChronoTimeline``: bounded frame history with summaries).  The Prometheus exporter writes the text
exposition format; nothing here needs a network.
"""
from __future__ import annotations

import math
import re
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

from . import plugin
from .nn.trainer import StepMetrics

EPS = 1e-9
DEFAULT_WINDOW = 32
DEFAULT_ALERT_CAP = 256


@dataclass
class AlertRecord:
    severity: str            # "info" | "warning" | "critical"
    kind: str                # "feature_drift" | "performance_regression"
    message: str
    fields: dict = field(default_factory=dict)
    timestamp: float = field(default_factory=time.monotonic)


class _RunningStats:
    __slots__ = ("count", "mean", "m2")

    def __init__(self):
        self.count, self.mean, self.m2 = 0, 0.0, 0.0

    def update(self, v: float) -> None:
        self.count += 1
        d = v - self.mean
        self.mean += d / self.count
        self.m2 += d * (v - self.mean)

    def stddev(self) -> float:
        return math.sqrt(self.m2 / (self.count - 1)) if self.count >= 2 else 0.0


class _FeatureWindow:
    def __init__(self, capacity: int, warmup: int):
        self.history: deque = deque()
        self.capacity, self.warmup = capacity, warmup
        self.baseline = _RunningStats()
        self.sum = 0.0
        self.frozen = False

    def update(self, v: float) -> None:
        if len(self.history) == self.capacity:
            self.sum -= self.history.popleft()
        self.history.append(v)
        self.sum += v
        if not self.frozen:
            self.baseline.update(v)
            if self.baseline.count >= self.warmup:
                self.frozen = True

    def ready(self) -> bool:
        return self.frozen and len(self.history) >= min(self.warmup, self.capacity)

    def z_score(self) -> float:
        if not self.ready():
            return 0.0
        mean = self.sum / len(self.history)
        return abs(mean - self.baseline.mean) / max(self.baseline.stddev(), EPS)


class DriftDetector:
    def __init__(self, z_threshold: float, warmup: int):
        self.z_threshold, self.warmup = z_threshold, warmup
        self._features: dict[str, _FeatureWindow] = {}

    def observe(self, features: dict) -> list[AlertRecord]:
        alerts = []
        for name, value in features.items():
            w = self._features.setdefault(name, _FeatureWindow(DEFAULT_WINDOW, self.warmup))
            w.update(float(value))
            z = w.z_score()
            if math.isfinite(z) and z >= self.z_threshold:
                alerts.append(AlertRecord("warning", "feature_drift",
                                          f"Feature drift detected for `{name}` (z-score {z:.2f} ≥ {self.z_threshold:.2f})",
                                          {"feature": name, "z_score": z, "threshold": self.z_threshold}))
        return alerts


HIGHER_IS_BETTER, LOWER_IS_BETTER = "higher_is_better", "lower_is_better"


class _PerformanceTarget:
    def __init__(self, name: str, direction: str, tolerance: float, warmup: int):
        self.name, self.direction, self.tolerance, self.warmup = name, direction, tolerance, warmup
        self.stats = _RunningStats()
        self.latest: Optional[float] = None
        self.consecutive_failures = 0
        self.required_failures = 3

    def update(self, value: float) -> Optional[AlertRecord]:
        self.latest = value
        self.stats.update(value)
        if self.stats.count < self.warmup:
            return None
        base = self.stats.mean
        if abs(base) <= EPS:
            drift = 0.0
        elif self.direction == HIGHER_IS_BETTER:
            drift = (base - value) / max(base, EPS)
        else:
            drift = (value - base) / max(base, EPS)
        self.consecutive_failures = self.consecutive_failures + 1 if drift > self.tolerance else 0
        if self.consecutive_failures < self.required_failures:
            return None
        self.consecutive_failures = 0
        side = "below" if self.direction == HIGHER_IS_BETTER else "above"
        return AlertRecord("critical", "performance_regression",
                           f"Performance regression on `{self.name}` — value {value:.4f} is {drift * 100:.1f}% {side} "
                           f"baseline {base:.4f}",
                           {"metric": self.name, "delta_ratio": drift, "tolerance": self.tolerance})


class PerformanceMonitor:
    def __init__(self, default_warmup: int):
        self._targets = {
            "step_loss": _PerformanceTarget("step_loss", LOWER_IS_BETTER, 0.25, default_warmup),
            "loss_weighted": _PerformanceTarget("loss_weighted", LOWER_IS_BETTER, 0.25, default_warmup),
            "reward": _PerformanceTarget("reward", HIGHER_IS_BETTER, 0.2, default_warmup),
        }

    def with_target(self, name: str, direction: str, tolerance: float, warmup: int) -> "PerformanceMonitor":
        self._targets[name] = _PerformanceTarget(name, direction, tolerance, warmup)
        return self

    def observe(self, metrics: dict, reward: float) -> list[AlertRecord]:
        alerts = []
        for name, target in self._targets.items():
            if name == "reward":
                value = reward
            elif name in metrics:
                value = metrics[name]
            else:
                continue
            a = target.update(float(value))
            if a is not None:
                alerts.append(a)
        return alerts

    def latest_values(self) -> dict:
        return {n: t.latest for n, t in self._targets.items() if t.latest is not None}


# ---- exporters -----------------------------------------------------------------------------------
class MetricsExporter:
    def record_gauge(self, name: str, value: float, labels: Iterable[tuple[str, str]] = ()) -> None:
        raise NotImplementedError


class PrometheusExporter(MetricsExporter):
    """Keeps the latest value of every gauge; ``render()`` returns the text exposition format
    (``# TYPE <name> gauge`` + one sample line per label set), ``write(path)`` stores it durably."""

    def __init__(self, namespace: str = "spiraltorch"):
        self.namespace = namespace
        self._gauges: dict[str, dict[tuple, float]] = {}
        self._lock = threading.Lock()

    def record_gauge(self, name, value, labels=()):
        key = tuple(sorted(labels))
        with self._lock:
            self._gauges.setdefault(f"{self.namespace}_{name}", {})[key] = float(value)

    def render(self) -> str:
        lines = []
        with self._lock:
            for name in sorted(self._gauges):
                lines.append(f"# TYPE {name} gauge")
                for key, v in sorted(self._gauges[name].items()):
                    lab = "{" + ",".join(f'{k}="{val}"' for k, val in key) + "}" if key else ""
                    lines.append(f"{name}{lab} {v!r}")
        return "\n".join(lines) + "\n"

    def write(self, path) -> None:
        from .config import atomic_write
        atomic_write(path, self.render())


class CallbackExporter(MetricsExporter):
    """Forwards every gauge to a callable (the hook an OpenTelemetry meter would be attached to)."""

    def __init__(self, fn: Callable[[str, float, tuple], None]):
        self._fn = fn

    def record_gauge(self, name, value, labels=()):
        self._fn(name, float(value), tuple(labels))


def _sanitize(name: str) -> str:
    return re.sub(r"[^A-Za-z0-9]", "_", name)


class MonitoringHub:
    def __init__(self, drift_threshold: float = 3.0, drift_warmup: int = 16, perf_warmup: int = 16):
        self.drift = DriftDetector(drift_threshold, drift_warmup)
        self.performance = PerformanceMonitor(perf_warmup)
        self._exporters: list[MetricsExporter] = []
        self._alerts: deque = deque(maxlen=DEFAULT_ALERT_CAP)
        self._last_observation: Optional[float] = None

    def with_exporter(self, exporter: MetricsExporter) -> "MonitoringHub":
        self._exporters.append(exporter)
        return self

    register_exporter = with_exporter

    def reconfigure(self, drift_threshold: float, drift_warmup: int, perf_warmup: int) -> None:
        exporters = self._exporters
        self.__init__(drift_threshold, drift_warmup, perf_warmup)
        self._exporters = exporters

    def observe(self, metrics: StepMetrics, reward: float = 0.0) -> list[AlertRecord]:
        self._last_observation = time.monotonic()
        alerts = self.drift.observe(metrics.extra) + self.performance.observe(metrics.extra, reward)
        self._alerts.extend(alerts)
        latest = self.performance.latest_values()
        for ex in self._exporters:
            ex.record_gauge("runtime_step_time_ms", metrics.step_time_ms)
            ex.record_gauge("runtime_mem_peak_mb", metrics.mem_peak_mb)
            ex.record_gauge("runtime_retry_rate", metrics.retry_rate)
            ex.record_gauge("runtime_reward", reward)
            for k, v in metrics.extra.items():
                ex.record_gauge("extra_" + _sanitize(k), v)
            for k, v in latest.items():
                ex.record_gauge("performance_" + _sanitize(k), v)
        if alerts and plugin.has_listeners("Telemetry"):
            for a in alerts:
                plugin.publish("Telemetry", {"alert": a.kind, "severity": a.severity, "message": a.message, **a.fields})
        return alerts

    def latest_alerts(self) -> list[AlertRecord]:
        return list(self._alerts)

    def last_observation(self) -> Optional[float]:
        return self._last_observation


# ---- chrono timeline -------------------------------------------------------------------------------
@dataclass
class ChronoFrame:
    step: int
    timestamp: float
    dt: float
    observed_curvature: float = 0.0
    total_energy: float = 0.0
    homotopy_energy: float = 0.0
    functor_energy: float = 0.0
    recursive_energy: float = 0.0
    projection_energy: float = 0.0
    infinity_energy: float = 0.0
    curvature_drift: float = 0.0
    energy_decay: float = 0.0

    def _ratio(self, part: float) -> float:
        return part / self.total_energy if self.total_energy > 0 else 0.0

    def homotopy_ratio(self) -> float:
        return self._ratio(self.homotopy_energy)

    def functor_ratio(self) -> float:
        return self._ratio(self.functor_energy)

    def recursive_ratio(self) -> float:
        return self._ratio(self.recursive_energy)

    def projection_ratio(self) -> float:
        return self._ratio(self.projection_energy)

    def infinity_ratio(self) -> float:
        return self._ratio(self.infinity_energy)


@dataclass
class ChronoSummary:
    frames: int
    duration: float
    latest_timestamp: float
    mean_drift: float
    mean_abs_drift: float
    drift_std: float
    mean_energy: float
    energy_std: float
    mean_decay: float
    min_energy: float
    max_energy: float


class ChronoTimeline:
    """Bounded history of per-step frames; ``record(dt, metrics)`` derives curvature drift and
    energy decay against the previous frame."""

    def __init__(self, capacity: int = 256):
        self._capacity = max(1, capacity)
        self._frames: deque = deque(maxlen=self._capacity)
        self._step = 0
        self._time = 0.0

    with_capacity = classmethod(lambda cls, capacity: cls(capacity))

    def capacity(self) -> int:
        return self._capacity

    def __len__(self) -> int:
        return len(self._frames)

    def is_empty(self) -> bool:
        return not self._frames

    def reset(self) -> None:
        self._frames.clear()
        self._step, self._time = 0, 0.0

    def frames(self):
        return iter(self._frames)

    def latest(self) -> Optional[ChronoFrame]:
        return self._frames[-1] if self._frames else None

    def record(self, dt: float, metrics: dict) -> ChronoFrame:
        dt = dt if (math.isfinite(dt) and dt > 0) else 1e-6
        m = {k: (float(v) if math.isfinite(float(v)) else 0.0) for k, v in metrics.items()}
        prev = self.latest()
        self._time += dt
        curv = m.get("observed_curvature", 0.0)
        energy = max(0.0, m.get("total_energy", 0.0))
        drift = (curv - prev.observed_curvature) / dt if prev else 0.0
        decay = (prev.total_energy - energy) / dt if prev else 0.0
        f = ChronoFrame(self._step, self._time, dt, curv, energy, max(0.0, m.get("homotopy_energy", 0.0)),
                        max(0.0, m.get("functor_energy", 0.0)), max(0.0, m.get("recursive_energy", 0.0)),
                        max(0.0, m.get("projection_energy", 0.0)), max(0.0, m.get("infinity_energy", 0.0)), drift, decay)
        self._step += 1
        self._frames.append(f)
        return f

    def summarise(self, window: int) -> Optional[ChronoSummary]:
        fr = list(self._frames)[-max(1, window):]
        if not fr:
            return None
        n = len(fr)
        drifts = [f.curvature_drift for f in fr]
        energies = [f.total_energy for f in fr]
        md = sum(drifts) / n
        me = sum(energies) / n
        return ChronoSummary(n, fr[-1].timestamp - fr[0].timestamp + fr[0].dt, fr[-1].timestamp, md,
                             sum(abs(d) for d in drifts) / n, math.sqrt(sum((d - md) ** 2 for d in drifts) / n), me,
                             math.sqrt(sum((e - me) ** 2 for e in energies) / n), sum(f.energy_decay for f in fr) / n,
                             min(energies), max(energies))

    def rewind_steps(self, steps: int) -> int:
        k = min(steps, len(self._frames))
        for _ in range(k):
            self._frames.pop()
        if self._frames:
            self._step, self._time = self._frames[-1].step + 1, self._frames[-1].timestamp
        else:
            self._step, self._time = 0, 0.0
        return k


# ---- device-timed step metrics ----------------------------------------------------------------------
class StepTimer:
    """Measures a training step with CUDA events on the current stream (wall clock on CPU) and
    turns it into :class:`StepMetrics` (``step_time_ms``, ``mem_peak_mb``)."""

    def __init__(self, device=None):
        import torch
        self._torch = torch
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._cuda = self.device.type == "cuda"

    def __enter__(self):
        t = self._torch
        if self._cuda:
            t.cuda.reset_peak_memory_stats(self.device)
            self._e0, self._e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self._cuda:
            self._e1.record()
        else:
            self._t1 = time.perf_counter()
        return False

    def metrics(self, **extra) -> StepMetrics:
        t = self._torch
        if self._cuda:
            self._e1.synchronize()
            ms = self._e0.elapsed_time(self._e1)
            peak = t.cuda.max_memory_allocated(self.device) / 2 ** 20
        else:
            ms, peak = (self._t1 - self._t0) * 1e3, 0.0
        return StepMetrics(step_time_ms=ms, mem_peak_mb=peak, retry_rate=0.0, extra={k: float(v) for k, v in extra.items()})
