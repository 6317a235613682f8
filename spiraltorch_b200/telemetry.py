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
import json
import re
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

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

    def serve(self, port: int = 9464, host: str = "127.0.0.1"):
        """Serve `render()` at `/metrics` from a daemon thread; returns the server (`.shutdown()` stops it,
        `.server_address[1]` is the bound port — pass `port=0` for an ephemeral one)."""
        from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
        exporter = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802
                if self.path.split("?")[0] not in ("/metrics", "/"):
                    self.send_error(404)
                    return
                body = exporter.render().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *args):
                pass

        server = ThreadingHTTPServer((host, port), Handler)
        threading.Thread(target=server.serve_forever, daemon=True).start()
        return server


class CallbackExporter(MetricsExporter):
    """Forwards every gauge to a callable (the hook an OpenTelemetry meter would be attached to)."""

    def __init__(self, fn: Callable[[str, float, tuple], None]):
        self._fn = fn

    def record_gauge(self, name, value, labels=()):
        self._fn(name, float(value), tuple(labels))


class OtelExporter(MetricsExporter):
    """OpenTelemetry metrics without the SDK: gauges keep their latest value, counters accumulate, and
    ``payload()`` renders both as an OTLP/JSON ``ExportMetricsServiceRequest`` (``resourceMetrics`` →
    ``scopeMetrics`` → ``metrics`` with ``gauge`` / monotonic cumulative ``sum`` data points) that ``write(path)``
    stores durably and ``post(endpoint)`` sends to an OTLP/HTTP collector (``/v1/metrics``) with the standard
    library.  Plays the role of the reference's ``OtelExporter`` over an ``opentelemetry`` meter
    (crates/st-core/src/telemetry/monitoring.rs:526-575)."""

    def __init__(self, service_name: str = "spiraltorch", scope: str = "spiraltorch_b200.telemetry"):
        self.service_name, self.scope = service_name, scope
        self._gauges: dict = {}
        self._counters: dict = {}
        self._lock = threading.Lock()
        self._start_ns = time.time_ns()

    def record_gauge(self, name, value, labels=()):
        with self._lock:
            self._gauges[(name, tuple(sorted(labels)))] = (float(value), time.time_ns())

    def record_counter(self, name, value, labels=()):
        key = (name, tuple(sorted(labels)))
        with self._lock:
            total = self._counters.get(key, (0.0, 0))[0] + max(float(value), 0.0)
            self._counters[key] = (total, time.time_ns())

    @staticmethod
    def _attrs(labels) -> list:
        return [{"key": k, "value": {"stringValue": str(v)}} for k, v in labels]

    def payload(self) -> dict:
        metrics: dict = {}
        with self._lock:
            for (name, labels), (v, ts) in sorted(self._gauges.items()):
                m = metrics.setdefault(("g", name), {"name": name, "description": f"Gauge for {name}", "gauge": {"dataPoints": []}})
                m["gauge"]["dataPoints"].append({"asDouble": v, "timeUnixNano": str(ts), "attributes": self._attrs(labels)})
            for (name, labels), (v, ts) in sorted(self._counters.items()):
                m = metrics.setdefault(("c", name), {"name": name, "description": f"Counter for {name}",
                                                     "sum": {"dataPoints": [], "isMonotonic": True,
                                                             "aggregationTemporality": 2}})
                m["sum"]["dataPoints"].append({"asDouble": v, "startTimeUnixNano": str(self._start_ns),
                                               "timeUnixNano": str(ts), "attributes": self._attrs(labels)})
        return {"resourceMetrics": [{
            "resource": {"attributes": [{"key": "service.name", "value": {"stringValue": self.service_name}}]},
            "scopeMetrics": [{"scope": {"name": self.scope}, "metrics": list(metrics.values())}]}]}

    def write(self, path) -> None:
        from .config import atomic_write
        atomic_write(path, json.dumps(self.payload(), sort_keys=True))

    def post(self, endpoint: str, timeout: float = 5.0) -> int:
        """POST the payload to ``endpoint`` (e.g. ``http://127.0.0.1:4318/v1/metrics``); returns the HTTP status."""
        import urllib.request
        req = urllib.request.Request(endpoint, data=json.dumps(self.payload()).encode(),
                                     headers={"Content-Type": "application/json"}, method="POST")
        with urllib.request.urlopen(req, timeout=timeout) as resp:      # noqa: S310 - caller-provided collector URL
            return resp.status


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


# ---- chrono harmonics, loop signal, time warps, maintainer ------------------------------------------------
@dataclass
class ChronoPeak:
    frequency: float = 0.0
    magnitude: float = 0.0
    phase: float = 0.0


@dataclass
class ChronoHarmonics:
    """Magnitude spectra ``|DFT| / n`` of the drift and energy series of a window of frames (the first ``bins``
    bins), with the strongest non-DC bin of each.  Parity: crates/st-core/src/telemetry/chrono.rs:55-151,258-300."""
    frames: int
    duration: float
    sample_rate: float
    nyquist: float
    drift_power: List[float]
    energy_power: List[float]
    dominant_drift: Optional[ChronoPeak]
    dominant_energy: Optional[ChronoPeak]

    @staticmethod
    def _spectrum(series: List[float], bins: int) -> List[float]:
        import torch
        x = torch.tensor(series, dtype=torch.float64)
        return (torch.fft.rfft(x).abs()[:bins] / len(series)).tolist()

    @staticmethod
    def _peak(power: List[float], sample_rate: float, samples: int) -> Optional[ChronoPeak]:
        best, best_v = None, 0.0
        for k, v in enumerate(power):
            if k and math.isfinite(v) and v > best_v:
                best, best_v = k, v
        return None if best is None else ChronoPeak(sample_rate * best / samples, best_v, 0.0)

    @classmethod
    def from_frames(cls, frames: Sequence[ChronoFrame], bins: int) -> Optional["ChronoHarmonics"]:
        n = len(frames)
        if n < 2 or bins <= 0:
            return None
        duration = sum(max(f.dt, 1.1920929e-07) for f in frames)
        if not math.isfinite(duration) or duration <= 1.1920929e-07:
            return None
        rate = n / duration
        bins = min(bins, n // 2 + 1)
        dp = cls._spectrum([f.curvature_drift for f in frames], bins)
        ep = cls._spectrum([f.total_energy for f in frames], bins)
        out = cls(n, duration, rate, 0.5 * rate, dp, ep, cls._peak(dp, rate, n), cls._peak(ep, rate, n))
        from . import observability
        observability.emit_tensor_op("chrono_harmonics_summary", (n, bins), (2, bins))
        observability.emit_tensor_op_meta("chrono_harmonics_summary", lambda: {
            "backend": "torch", "kind": "chrono_harmonics_summary", "frames": n, "bins": bins, "duration": duration,
            "sample_rate": rate, "nyquist": 0.5 * rate, "drift_power_total": sum(dp), "energy_power_total": sum(ep),
            "has_dominant_drift": out.dominant_drift is not None, "has_dominant_energy": out.dominant_energy is not None,
            "dominant_drift_frequency": out.dominant_drift.frequency if out.dominant_drift else 0.0,
            "dominant_energy_frequency": out.dominant_energy.frequency if out.dominant_energy else 0.0})
        return out


def _clampf(v: float, lo: float, hi: float) -> float:
    return min(max(v, lo), hi)


@dataclass
class ChronoLoopSignal:
    """A summary with its harmonics and the SpiralK hints derived from them (radix / segments / tile_cols from the
    drift and energy statistics, kl / wg from the dominant peaks).  Parity: chrono.rs:157-256."""
    summary: ChronoSummary
    harmonics: Optional[ChronoHarmonics] = None
    spiralk_script: Optional[str] = None
    spiralk_hints: list = field(default_factory=list)

    def __post_init__(self):
        from .kdsl_rewrite import HeuristicHint, synthesize_program
        s, hints = self.summary, []
        drift = _clampf(s.mean_abs_drift, 0.0, 4.0)
        band = max(s.max_energy - s.min_energy, 0.0)
        hints.append(HeuristicHint("radix", f"{_clampf(2.0 + drift * 4.0, 2.0, 16.0):.3f}", _clampf(0.25 + drift, 0.25, 0.9), "true"))
        hints.append(HeuristicHint("segments", f"{_clampf(1.0 + band ** 0.25 * 2.0, 1.0, 8.0):.3f}", 0.3 + min(drift, 1.0) * 0.2, "true"))
        hints.append(HeuristicHint("tile_cols", f"{_clampf(64.0 + s.mean_energy * 8.0, 32.0, 512.0):.3f}",
                                   _clampf(0.3 + math.sqrt(band) * 0.1, 0.3, 1.1), "true"))
        h = self.harmonics
        if h is not None and h.dominant_drift is not None:
            hints.append(HeuristicHint("kl", f"{_clampf(1.0 + h.dominant_drift.frequency * max(h.duration, 1e-3), 1.0, 9.0):.3f}",
                                       _clampf(h.dominant_drift.magnitude, 0.05, 1.2), "true"))
        if h is not None and h.dominant_energy is not None:
            hints.append(HeuristicHint("wg", f"{_clampf(128.0 + h.dominant_energy.frequency * 48.0, 64.0, 2048.0):.3f}",
                                       _clampf(h.dominant_energy.magnitude, 0.05, 1.5), "true"))
        self.spiralk_hints = hints
        self.spiralk_script = synthesize_program("", hints) if hints else None


class TemporalWarpError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass(frozen=True)
class TemporalWarp:
    """``t -> pivot + (t - pivot) * scale + offset`` with a positive finite scale.  Parity: crates/st-core/src/util/timewarp.rs."""
    scale: float = 1.0
    offset: float = 0.0
    pivot: float = 0.0

    def validate(self) -> None:
        if not all(math.isfinite(v) for v in (self.scale, self.offset, self.pivot)):
            raise TemporalWarpError("non_finite", "warp components must be finite")
        if self.scale <= 0.0:
            raise TemporalWarpError("invalid_scale", f"warp scale must be positive, got {self.scale}")

    @classmethod
    def dilation(cls, factor: float) -> "TemporalWarp":
        return cls(factor, 0.0, 0.0)

    @classmethod
    def translation(cls, offset: float) -> "TemporalWarp":
        return cls(1.0, offset, 0.0)

    @classmethod
    def fit_span(cls, source_start: float, source_end: float, target_start: float, target_end: float) -> "TemporalWarp":
        if not all(math.isfinite(v) for v in (source_start, source_end, target_start, target_end)):
            raise TemporalWarpError("non_finite", "spans must be finite")
        src, dst = source_end - source_start, target_end - target_start
        if abs(src) <= 1.1920929e-07:
            if abs(dst) <= 1.1920929e-07:
                return cls(1.0, target_start - source_start, 0.0)
            raise TemporalWarpError("degenerate", "cannot stretch an empty span")
        scale = dst / src
        if scale <= 0.0:
            raise TemporalWarpError("invalid_scale", f"warp scale must be positive, got {scale}")
        return cls(scale, target_start - source_start * scale, 0.0)

    def apply(self, t: float) -> float:
        return self.pivot + (t - self.pivot) * self.scale + self.offset


def _timeline_harmonics(self, window: int, bins: int) -> Optional[ChronoHarmonics]:
    fr = list(self._frames)[-max(1, window):]
    return ChronoHarmonics.from_frames(fr, bins) if fr else None


def _timeline_loop_signal(self, window: int, bins: int) -> Optional[ChronoLoopSignal]:
    if not self._frames:
        return None
    window = min(max(1, window), len(self._frames))
    summary = self.summarise(window)
    return ChronoLoopSignal(summary, None if window < 2 else self.harmonics(window, max(bins, 1)))


def _timeline_warp(self, warp: TemporalWarp) -> None:
    """Re-times every frame; ``dt`` follows the warped axis and the energy decay rate is divided by the scale."""
    if not self._frames:
        raise TemporalWarpError("empty", "the timeline has no frames")
    warp.validate()
    frames = list(self._frames)
    axis = [frames[0].timestamp - frames[0].dt] + [f.timestamp for f in frames]
    if not all(math.isfinite(t) for t in axis):
        raise TemporalWarpError("non_finite", "timestamps must be finite")
    if any(b < a for a, b in zip(axis, axis[1:])):
        raise TemporalWarpError("non_monotonic", "timestamps must not decrease")
    warped = [warp.apply(t) for t in axis]
    if not all(math.isfinite(t) for t in warped):
        raise TemporalWarpError("non_finite", "the warp leaves the representable range")
    prev = warped[0]
    for f, t in zip(frames, warped[1:]):
        f.dt, f.timestamp = max(t - prev, 1.1920929e-07), t
        f.energy_decay /= warp.scale
        prev = t
    self._time = prev


def _timeline_dilate(self, factor: float) -> None:
    self.warp_time_axis(TemporalWarp.dilation(factor))


def _timeline_shift(self, offset: float) -> None:
    if not math.isfinite(offset):
        raise TemporalWarpError("non_finite", "offset must be finite")
    self.warp_time_axis(TemporalWarp.translation(offset))


def _timeline_align(self, progress: float, window: float) -> None:
    """Stretches the recorded span onto ``[0, window * progress]``."""
    if not self._frames:
        raise TemporalWarpError("empty", "the timeline has no frames")
    if not (math.isfinite(progress) and math.isfinite(window)):
        raise TemporalWarpError("non_finite", "progress and window must be finite")
    first, last = self._frames[0], self._frames[-1]
    target = max(max(window, 1.1920929e-07) * max(progress, 0.0), 1.1920929e-07)
    self.warp_time_axis(TemporalWarp.fit_span(first.timestamp - first.dt, last.timestamp, 0.0, target))


ChronoTimeline.harmonics = _timeline_harmonics
ChronoTimeline.loop_signal = _timeline_loop_signal
ChronoTimeline.warp_time_axis = _timeline_warp
ChronoTimeline.dilate = _timeline_dilate
ChronoTimeline.shift = _timeline_shift
ChronoTimeline.align_to_progress = _timeline_align


def chrono_summary_from_frames(frames: Sequence[ChronoFrame]) -> Optional[ChronoSummary]:
    t = ChronoTimeline(max(len(frames), 1))
    t._frames.extend(frames)
    return t.summarise(len(frames)) if frames else None


MAINTAINER_STATUSES = ("stable", "dormant", "clamp", "rewrite")


@dataclass
class MaintainerConfig:
    jitter_threshold: float = 0.35
    growth_threshold: float = 0.05
    energy_floor: float = 1e-3
    clamp_min: float = 2.0
    clamp_max: float = 3.0
    pressure_step: float = 0.12
    window: int = 32

    def sanitise(self) -> "MaintainerConfig":
        def pos(v, d, strict=True):
            return v if math.isfinite(v) and (v > 0.0 if strict else v >= 0.0) else d
        lo = self.clamp_min if math.isfinite(self.clamp_min) else 2.0
        hi = self.clamp_max if math.isfinite(self.clamp_max) else 3.0
        return MaintainerConfig(pos(self.jitter_threshold, 0.35), pos(self.growth_threshold, 0.05), pos(self.energy_floor, 1e-3, False),
                                min(lo, hi), max(lo, hi), pos(self.pressure_step, 0.12), max(int(self.window), 1))


@dataclass
class MaintainerReport:
    status: str
    average_drift: float = 0.0
    mean_energy: float = 0.0
    mean_decay: float = 0.0
    drift_peak: Optional[ChronoPeak] = None
    energy_peak: Optional[ChronoPeak] = None
    suggested_max_scale: Optional[float] = None
    suggested_pressure: Optional[float] = None
    diagnostic: str = ""
    spiralk_script: Optional[str] = None

    def should_rewrite(self) -> bool:
        return self.status == "rewrite"


class Maintainer:
    """Reads the tail of a chrono timeline and decides whether the temporal dynamics are stable, dormant (no energy),
    need a clamp (curvature jitter or a strong drift harmonic) or a rewrite (energy growth or a strong energy harmonic),
    with a suggested scale clamp and pressure.  Parity: crates/st-core/src/telemetry/maintainer.rs:108-265."""

    def __init__(self, config: Optional[MaintainerConfig] = None):
        self.config = (config or MaintainerConfig()).sanitise()

    def assess(self, frames: Sequence[ChronoFrame]) -> MaintainerReport:
        frames = list(frames)
        c = self.config
        if not frames:
            return self._emit(0, 0, MaintainerReport("dormant", diagnostic="No temporal frames recorded; timeline is dormant."))
        tail = frames[-max(min(c.window, len(frames)), 1):]
        s = chrono_summary_from_frames(tail)
        h = ChronoHarmonics.from_frames(tail, 16)
        dpk, epk = (h.dominant_drift if h else None), (h.dominant_energy if h else None)
        growth = max(-s.mean_decay, 0.0)
        status = "dormant" if s.mean_energy <= c.energy_floor else "stable"
        reasons, scale, pressure = [], None, None
        if s.mean_abs_drift > c.jitter_threshold:
            status = "clamp"
            scale = _clampf(c.clamp_min + s.mean_abs_drift / (c.jitter_threshold + 1.1920929e-07), c.clamp_min, c.clamp_max)
            reasons.append(f"curvature jitter {s.mean_abs_drift:.3f} exceeds threshold {c.jitter_threshold:.3f}")
        if growth > c.growth_threshold:
            status = "rewrite"
            pressure = min(c.pressure_step * (1.0 + growth / c.growth_threshold), 1.0)
            reasons.append(f"energy growth {growth:.3f} exceeds threshold {c.growth_threshold:.3f}")
        elif status == "clamp":
            pressure = min(c.pressure_step * (1.0 + s.mean_abs_drift / c.jitter_threshold), 1.0)
        if dpk is not None and dpk.magnitude > c.jitter_threshold:
            status = "clamp"
            reasons.append(f"drift harmonic {dpk.frequency:.2f}Hz magnitude {dpk.magnitude:.3f}")
            scale = scale if scale is not None else c.clamp_max
        if epk is not None and epk.magnitude > c.growth_threshold:
            status = "rewrite"
            reasons.append(f"energy harmonic {epk.frequency:.2f}Hz magnitude {epk.magnitude:.3f}")
            pressure = min(c.pressure_step * (1.0 + epk.magnitude / c.growth_threshold), 1.0)
        if not reasons:
            reasons.append(f"timeline energy below floor; drift {s.mean_abs_drift:.3f}±{s.drift_std:.3f}" if status == "dormant" else
                           f"temporal dynamics within expected range (drift {s.mean_abs_drift:.3f}±{s.drift_std:.3f}, "
                           f"energy {s.mean_energy:.3f}±{s.energy_std:.3f})")
        return self._emit(len(frames), len(tail), MaintainerReport(status, s.mean_abs_drift, s.mean_energy, s.mean_decay, dpk, epk, scale, pressure,
                                                                   "; ".join(reasons), ChronoLoopSignal(s, h).spiralk_script))

    @staticmethod
    def _emit(frames: int, window: int, report: MaintainerReport) -> MaintainerReport:
        from . import observability
        observability.emit_tensor_op("timeline_maintainer_assessment", (frames, window), (1, 8))
        observability.emit_tensor_op_meta("timeline_maintainer_assessment", lambda: {
            "backend": "host", "kind": "timeline_maintainer_assessment", "frames": frames, "window": window, "status": report.status,
            "average_drift": report.average_drift, "mean_energy": report.mean_energy, "mean_decay": report.mean_decay,
            "should_rewrite": report.should_rewrite(), "has_suggested_max_scale": report.suggested_max_scale is not None,
            "has_suggested_pressure": report.suggested_pressure is not None})
        return report


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


# ----------------------------------------------------------------------------------------------
# Atlas: frames of named metrics grouped into districts, bounded routes and their summaries
# (crates/st-core/src/telemetry/atlas.rs:129-700, :1070-1400, :2007-2030)
# ----------------------------------------------------------------------------------------------

_SURFACE = {"py", "python", "bindings", "session", "timeline", "config", "psychoid", "canvas"}
_CONCOURSE = {"trainer", "maintainer", "atlas", "loop", "chrono", "policy", "resonator", "softlogic", "psi", "desire"}
_SUBSTRATE = {"tensor", "backend", "core", "z", "collapse", "geometry", "kdsl", "realgrad"}


def metric_root_token(name: str) -> str:
    """Leading namespace token of a metric id: ``psi.total`` → ``psi``, ``canvas_energy`` → ``canvas``."""
    import re
    return next((t for t in re.split(r"[.:/\-_]", name.strip()) if t), "")


def infer_district(name: str) -> str:
    token = metric_root_token(name).lower()
    if token in _SURFACE:
        return "Surface"
    if token in _CONCOURSE:
        return "Concourse"
    if token in _SUBSTRATE:
        return "Substrate"
    return "Unknown"


@dataclass
class AtlasFrame:
    timestamp: float
    loop_support: float = 0.0
    collapse_total: Optional[float] = None
    z_signal: Optional[float] = None
    script_hint: Optional[str] = None
    metrics: Dict[str, float] = field(default_factory=dict)
    districts: Dict[str, str] = field(default_factory=dict)      # explicit district per metric
    notes: List[str] = field(default_factory=list)
    concepts: List[tuple] = field(default_factory=list)          # (term, sense)
    chrono_summary: Optional["ChronoSummary"] = None
    harmonics: Optional[object] = None
    maintainer_status: Optional[str] = None
    maintainer_diagnostic: Optional[str] = None
    suggested_max_scale: Optional[float] = None
    suggested_pressure: Optional[float] = None

    def __post_init__(self):
        if not math.isfinite(self.timestamp):
            self.timestamp = 0.0

    @classmethod
    def from_fragment(cls, fragment: "AtlasFragment") -> Optional["AtlasFrame"]:
        if fragment.is_empty():
            return None
        frame = cls(0.0)
        frame.merge_fragment(fragment)
        return frame if frame.timestamp > 0.0 else None

    def merge_fragment(self, fragment: "AtlasFragment") -> None:
        """Folds a producer's partial view in: the timestamp only moves forward, loop support accumulates, scalars and
        texts are replaced when the fragment carries a usable value, metrics replace by name, notes and concepts are
        appended once.  Parity: crates/st-core/src/telemetry/atlas.rs:337-409."""
        if fragment.is_empty():
            return
        ts = fragment.timestamp if fragment.timestamp is not None else (fragment.summary.latest_timestamp if fragment.summary else None)
        if ts is not None and math.isfinite(ts):
            self.timestamp = max(ts, 1.1920929e-07) if self.timestamp <= 0.0 else max(self.timestamp, ts)
        if fragment.summary is not None:
            self.chrono_summary = fragment.summary
        if fragment.harmonics is not None:
            self.harmonics = fragment.harmonics
        if fragment.loop_support is not None and math.isfinite(fragment.loop_support):
            self.loop_support += max(fragment.loop_support, 0.0)
        for name in ("collapse_total", "z_signal", "suggested_max_scale", "suggested_pressure"):
            v = getattr(fragment, name)
            if v is not None and math.isfinite(v):
                setattr(self, name, float(v))
        for name in ("script_hint", "maintainer_diagnostic"):
            v = getattr(fragment, name)
            if v is not None and v.strip():
                setattr(self, name, v.strip())
        if fragment.maintainer_status is not None:
            self.maintainer_status = fragment.maintainer_status
        for name, value, district in fragment.metrics:
            self.push_metric(name, value, district)
        for note in fragment.notes:
            if note not in self.notes:
                self.notes.append(note)
        for concept in fragment.concepts:
            if concept not in self.concepts:
                self.concepts.append(concept)
        if self.timestamp <= 0.0:
            self.timestamp = 1.1920929e-07

    def push_metric(self, name: str, value: float, district: Optional[str] = None) -> None:
        if math.isfinite(value):
            self.metrics[name] = float(value)
            if district:
                self.districts[name] = district

    def metric_value(self, name: str) -> Optional[float]:
        return self.metrics.get(name)

    def metrics_with_prefix(self, prefix: str) -> Dict[str, float]:
        return {k: v for k, v in self.metrics.items() if k.startswith(prefix)}

    def district_of(self, name: str) -> str:
        return self.districts.get(name) or infer_district(name)


@dataclass
class AtlasFragment:
    """What one producer knows about the current atlas frame."""
    timestamp: Optional[float] = None
    summary: Optional["ChronoSummary"] = None
    harmonics: Optional[object] = None
    loop_support: Optional[float] = None
    collapse_total: Optional[float] = None
    z_signal: Optional[float] = None
    script_hint: Optional[str] = None
    maintainer_status: Optional[str] = None
    maintainer_diagnostic: Optional[str] = None
    suggested_max_scale: Optional[float] = None
    suggested_pressure: Optional[float] = None
    metrics: List[tuple] = field(default_factory=list)          # (name, value, district or None)
    notes: List[str] = field(default_factory=list)
    concepts: List[tuple] = field(default_factory=list)

    def is_empty(self) -> bool:
        scalars = (self.timestamp, self.summary, self.harmonics, self.loop_support, self.collapse_total, self.z_signal, self.script_hint,
                   self.maintainer_status, self.maintainer_diagnostic, self.suggested_max_scale, self.suggested_pressure)
        return all(v is None for v in scalars) and not self.metrics and not self.notes and not self.concepts

    def push_metric(self, name: str, value: float, district: Optional[str] = None) -> None:
        name = str(name).strip()
        if name and isinstance(value, (int, float)) and math.isfinite(value):
            self.metrics.append((name, float(value), district))

    def push_note(self, note: str) -> None:
        note = str(note).strip()
        if note:
            self.notes.append(note)

    def push_concept(self, term: str, sense: str) -> None:
        self.concepts.append((term, sense))


class AtlasRoute:
    """Bounded sequence of frames; frames without a positive timestamp are dropped."""

    def __init__(self):
        self.frames: List[AtlasFrame] = []

    def __len__(self) -> int:
        return len(self.frames)

    def latest(self) -> Optional[AtlasFrame]:
        return self.frames[-1] if self.frames else None

    def push_bounded(self, frame: AtlasFrame, capacity: int = 0) -> None:
        if frame.timestamp <= 0.0:
            return
        self.frames.append(frame)
        if capacity > 0 and len(self.frames) > capacity:
            del self.frames[: len(self.frames) - capacity]

    def summary(self) -> "AtlasRouteSummary":
        return AtlasRouteSummary(self.frames)


class AtlasRouteSummary:
    """Loop-support statistics, collapse / z-signal trends (latest − first), per-district metric
    focus (coverage, mean, latest, delta, momentum = delta / (coverage − 1), std) and concept counts."""

    def __init__(self, frames: Sequence[AtlasFrame]):
        self.frames = len(frames)
        self.latest_timestamp = frames[-1].timestamp if frames else 0.0
        loops = [max(f.loop_support, 0.0) for f in frames]
        self.loop_min = min(loops) if loops else 0.0
        self.loop_max = max(loops) if loops else 0.0
        self.mean_loop = sum(loops) / len(loops) if loops else 0.0
        self.loop_std = math.sqrt(max(sum(l * l for l in loops) / len(loops) - self.mean_loop ** 2, 0.0)) if loops else 0.0
        self.loop_trend = loops[-1] - loops[0] if len(loops) > 1 else None
        collapse = [f.collapse_total for f in frames if f.collapse_total is not None and math.isfinite(f.collapse_total)]
        zsig = [f.z_signal for f in frames if f.z_signal is not None and math.isfinite(f.z_signal)]
        self.latest_collapse_total = collapse[-1] if collapse else None
        self.collapse_trend = collapse[-1] - collapse[0] if len(collapse) > 1 else None
        self.latest_z_signal = zsig[-1] if zsig else None
        self.z_signal_trend = zsig[-1] - zsig[0] if len(zsig) > 1 else None
        self.script_hint = next((f.script_hint for f in reversed(frames) if f.script_hint), None)
        self.total_notes = sum(len(f.notes) for f in frames)
        self.latest_notes = [n for f in frames for n in f.notes][-16:]
        series: Dict[tuple, List[float]] = {}
        for f in frames:
            for name, value in f.metrics.items():
                series.setdefault((f.district_of(name), name), []).append(value)
        self.districts: Dict[str, List[dict]] = {}
        for (district, name), vals in sorted(series.items()):
            mean = sum(vals) / len(vals)
            delta = vals[-1] - vals[0]
            self.districts.setdefault(district, []).append({
                "name": name, "coverage": len(vals), "mean": mean, "latest": vals[-1], "delta": delta,
                "momentum": delta / (len(vals) - 1) if len(vals) > 1 else 0.0,
                "std_dev": math.sqrt(max(sum(v * v for v in vals) / len(vals) - mean * mean, 0.0))})
        self.concept_counts: Dict[tuple, int] = {}
        for f in frames:
            for term, sense in f.concepts:
                self.concept_counts[(term, sense)] = self.concept_counts.get((term, sense), 0) + 1

    def is_empty(self) -> bool:
        return self.frames == 0

    def latest_note(self) -> Optional[str]:
        return self.latest_notes[-1] if self.latest_notes else None

    def beacons(self, limit: int = 0) -> List[dict]:
        """Metrics that moved, strongest first (intensity = max(|delta|, |momentum|))."""
        out = []
        for district, focus_list in self.districts.items():
            for fc in focus_list:
                intensity = max(abs(fc["delta"]), abs(fc["momentum"]))
                if fc["coverage"] == 0 or intensity <= 1e-6:
                    continue
                trend = "steady" if abs(fc["delta"]) <= 1e-6 else ("rising" if fc["delta"] > 0 else "falling")
                vol = fc["std_dev"]
                variance = ("with calm variance" if vol <= 1e-6 else "with mild variance" if vol < 0.25
                            else "with adaptive variance" if vol < 0.75 else "with turbulent variance")
                verb = {"rising": "is surging", "falling": "is easing", "steady": "holds steady"}[trend]
                tempo = "flat momentum" if abs(fc["momentum"]) <= 1e-6 else "momentum"
                out.append({"district": district, "metric": fc["name"], "coverage": fc["coverage"], "mean": fc["mean"],
                            "latest": fc["latest"], "delta": fc["delta"], "momentum": fc["momentum"],
                            "volatility": vol, "intensity": intensity, "trend": trend,
                            "narrative": f"{district}::{fc['name']} {verb} (Δ {fc['delta']:+.3f}, {tempo} "
                                         f"{fc['momentum']:+.3f}, σ {vol:.3f}) {variance}."})
        out.sort(key=lambda b: (-b["intensity"], b["metric"]))
        return out[:limit] if limit > 0 else out

    def beacon_for(self, metric: str) -> Optional[dict]:
        return next((b for b in self.beacons() if b["metric"] == metric), None)

    def concept_heatmap(self) -> dict:
        senses: Dict[str, int] = {}
        terms: Dict[str, int] = {}
        for (term, sense), n in self.concept_counts.items():
            senses[sense] = senses.get(sense, 0) + n
            terms[term] = terms.get(term, 0) + n
        return {"sense_counts": senses, "term_counts": terms, "total_mentions": sum(terms.values()),
                "total_terms": len(terms)}

    def flux(self) -> Optional[dict]:
        if self.frames == 0:
            return None
        heat = self.concept_heatmap()
        return {"coverage": self.frames, "loop_range": max(self.loop_max - self.loop_min, 0.0),
                "loop_variability": self.loop_std, "collapse_drift": self.collapse_trend or 0.0,
                "z_signal_drift": self.z_signal_trend or 0.0, "note_density": self.total_notes / self.frames,
                "concept_density": heat["total_mentions"] / self.frames}

    def to_json(self) -> dict:
        return {"frames": self.frames, "latest_timestamp": self.latest_timestamp, "mean_loop": self.mean_loop,
                "loop_std": self.loop_std, "loop_min": self.loop_min, "loop_max": self.loop_max,
                "latest_collapse_total": self.latest_collapse_total, "collapse_trend": self.collapse_trend,
                "latest_z_signal": self.latest_z_signal, "z_signal_trend": self.z_signal_trend,
                "script_hint": self.script_hint, "total_notes": self.total_notes, "latest_notes": self.latest_notes,
                "districts": self.districts, "beacons": self.beacons(8), "flux": self.flux()}


# ----------------------------------------------------------------------------------------------
# Dashboard frames (crates/st-core/src/telemetry/dashboard.rs:13-400)
# ----------------------------------------------------------------------------------------------
SEVERITIES = ("info", "warning", "critical")


@dataclass
class DashboardMetric:
    name: str
    value: float
    unit: Optional[str] = None
    trend: Optional[float] = None

    def with_unit(self, unit: str) -> "DashboardMetric":
        self.unit = unit
        return self

    def with_trend(self, trend: float) -> "DashboardMetric":
        self.trend = float(trend)
        return self


@dataclass
class DashboardEvent:
    message: str
    severity: str = "info"

    def __post_init__(self):
        if self.severity not in SEVERITIES:
            raise ValueError(f"unknown severity {self.severity!r}; expected one of {SEVERITIES}")


@dataclass
class DashboardFrame:
    timestamp: float
    metrics: list = field(default_factory=list)
    events: list = field(default_factory=list)

    def push_metric(self, metric: DashboardMetric) -> None:
        self.metrics.append(metric)

    def push_event(self, event: DashboardEvent) -> None:
        self.events.append(event)


@dataclass
class MetricAggregate:
    name: str
    mean: float
    min: float
    max: float
    latest: float
    samples: int


@dataclass
class DashboardSummary:
    frame_count: int
    span_seconds: float
    metrics: list
    events: dict

    def is_empty(self) -> bool:
        return self.frame_count == 0

    def top_metric(self) -> Optional[MetricAggregate]:
        """The metric with the widest range over the summarised frames (ties: the later name)."""
        return max(self.metrics, key=lambda m: (abs(m.max - m.min), m.name), default=None)


class DashboardRing:
    """Bounded history of frames; `summarize(limit)` aggregates the newest `limit` frames per metric
    name (mean / min / max / latest / samples) and counts events per severity."""

    def __init__(self, capacity: int):
        from collections import deque
        self.capacity = max(int(capacity), 1)
        self._frames = deque(maxlen=self.capacity)

    def push(self, frame: DashboardFrame) -> None:
        self._frames.append(frame)

    def latest(self) -> Optional[DashboardFrame]:
        return self._frames[-1] if self._frames else None

    def __len__(self) -> int:
        return len(self._frames)

    def __iter__(self):
        return iter(self._frames)

    def summarize(self, limit: Optional[int] = None) -> Optional[DashboardSummary]:
        if not self._frames:
            return None
        take = list(self._frames)[-max(limit or len(self._frames), 1):][::-1]          # newest first
        acc, events = {}, {}
        for f in take:
            for m in f.metrics:
                a = acc.setdefault(m.name, {"latest": m.value, "sum": 0.0, "min": m.value, "max": m.value, "n": 0})
                a["sum"] += m.value
                a["n"] += 1
                a["min"], a["max"] = min(a["min"], m.value), max(a["max"], m.value)
            for e in f.events:
                events[e.severity] = events.get(e.severity, 0) + 1
        metrics = [MetricAggregate(k, a["sum"] / a["n"], a["min"], a["max"], a["latest"], a["n"]) for k, a in sorted(acc.items())]
        return DashboardSummary(len(take), abs(take[0].timestamp - take[-1].timestamp), metrics, events)


class DashboardBuilder:
    """Collects the metrics / events of one frame; `finish_with_latency` adds `frame_latency_ms`."""

    def __init__(self, start: Optional[float] = None):
        import time
        self._clock = time.time
        self._start = self._clock() if start is None else float(start)
        self._metrics, self._events = [], []

    def record_metric(self, metric: DashboardMetric) -> None:
        self._metrics.append(metric)

    def record_event(self, message: str, severity: str = "info") -> None:
        self._events.append(DashboardEvent(message, severity))

    def finish(self) -> DashboardFrame:
        return DashboardFrame(self._start, self._metrics, self._events)

    def finish_with_latency(self) -> DashboardFrame:
        self._metrics.append(DashboardMetric("frame_latency_ms", (self._clock() - self._start) * 1e3, "ms"))
        return self.finish()


# ----------------------------------------------------------------------------------------------
# Z-space partial fusion (crates/st-core/src/telemetry/zspace_fusion.rs:160-1300)
# ----------------------------------------------------------------------------------------------
class ZSpaceFusionError(ValueError):
    pass


_METRIC_ALIASES = {"velocity": "speed", "mem": "memory", "stab": "stability", "frac_reg": "frac", "fractality": "frac",
                   "drift": "drs", "grad": "gradient", "curvature_radius": "elliptic_curvature",
                   "elliptic_curvature_radius": "elliptic_curvature", "geodesic_radius": "elliptic_geodesic",
                   "normalized_radius": "elliptic_normalized", "spin_alignment": "elliptic_alignment",
                   "normal_bias": "elliptic_bias", "sheet_position": "elliptic_sheet_position",
                   "sheet_index": "elliptic_sheet_index", "sheet_count": "elliptic_sheet_count",
                   "topological_sector": "elliptic_sector", "homology_index": "elliptic_homology",
                   "resonance_heat": "elliptic_resonance", "noise_density": "elliptic_noise"}
_METRIC_FAMILIES = ("canvas_", "hypergrad_", "realgrad_", "import_", "elliptic_", "coherence_")
_METRIC_BASE = ("speed", "memory", "stability", "frac", "drs", "gradient")


def canonical_metric_name(name: str) -> Optional[str]:
    """Canonical spelling of a Z-space metric label (aliases folded, case ignored); None when unknown."""
    if len(name) > 128:
        return None
    n = name.lower()
    n = _METRIC_ALIASES.get(n, n)
    return n if n in _METRIC_BASE or n.startswith(_METRIC_FAMILIES) else None


@dataclass
class ZSpaceTelemetrySummary:
    count: int = 0
    l1: float = 0.0
    l2: float = 0.0
    linf: float = 0.0
    mean: float = 0.0
    variance: float = 0.0
    energy: float = 0.0
    amplitude: float = 0.0
    positive: float = 0.0
    negative: float = 0.0
    balance: float = 0.0
    focus: float = 0.0

    @classmethod
    def from_values(cls, values: Iterable[float]) -> "ZSpaceTelemetrySummary":
        d = [float(v) for v in values]
        if not d:
            return cls()
        if not all(math.isfinite(v) for v in d):
            raise ZSpaceFusionError("telemetry summary: non-finite value")
        n, energy = len(d), sum(v * v for v in d)
        mean = sum(d) / n
        pos, neg = sum(v for v in d if v > 0), -sum(v for v in d if v < 0)
        bal = (pos - neg) / (pos + neg + 1e-9)
        return cls(n, sum(abs(v) for v in d), math.sqrt(energy), max(abs(v) for v in d), mean,
                   sum((v - mean) ** 2 for v in d) / n, energy, max(d) - min(d), pos, neg, bal, math.tanh(1.5 * bal))


def _weighted_median(pairs: list) -> float:
    pairs = sorted(pairs)
    half, acc = 0.5 * sum(w for _, w in pairs), 0.0
    for i, (v, w) in enumerate(pairs):
        acc += w
        if acc > half + 1e-15:
            return v
        if abs(acc - half) <= 1e-15 and i + 1 < len(pairs):
            return 0.5 * (v + pairs[i + 1][0])           # balanced boundary: interpolate the neighbours
    return pairs[-1][0]


def fuse_zspace_partials(partials: Sequence[Optional[dict]], weights: Optional[Sequence[float]] = None,
                         strategy: str = "mean", gradient_alignment: str = "strict",
                         metric_gradient_dimension: Optional[int] = None) -> dict:
    """Fuse partial observations `{"metrics": {...}, "weight": w, "origin": ..., "gradient": [...]}`.

    Metric labels are canonicalised; partials that are `None` or carry a non-positive weight are audited
    and skipped.  `strategy`: mean (weighted), last, max, min, median (weighted), sum (weighted).
    Gradients are weight-averaged; with `gradient_alignment="strict"` differing lengths are an error,
    with "pad_zero" shorter ones are zero-padded.  A partial without a gradient contributes the projection
    of its canonical metrics when `metric_gradient_dimension` is given."""
    if strategy not in ("mean", "last", "max", "min", "median", "sum"):
        raise ZSpaceFusionError(f"unknown fusion strategy {strategy!r}")
    if gradient_alignment not in ("strict", "pad_zero"):
        raise ZSpaceFusionError(f"unknown gradient alignment {gradient_alignment!r}")
    if weights is not None:
        if len(weights) != len(partials):
            raise ZSpaceFusionError(f"weights has {len(weights)} entries, expected {len(partials)}")
        if not all(math.isfinite(w) for w in weights):
            raise ZSpaceFusionError("non-finite weight")
    if metric_gradient_dimension is not None and not 1 <= metric_gradient_dimension <= 65536:
        raise ZSpaceFusionError(f"invalid metric gradient dimension {metric_gradient_dimension}")
    agg: Dict[str, list] = {}
    grads, sources = [], []
    for i, part in enumerate(partials):
        if part is None:
            sources.append({"index": i, "status": "null"})
            continue
        w = float(weights[i] if weights is not None else part.get("weight", 1.0))
        if not math.isfinite(w):
            raise ZSpaceFusionError(f"non-finite weight at {i}")
        if w <= 0:
            sources.append({"index": i, "status": "suppressed", "weight": w, "origin": part.get("origin")})
            continue
        canon = {}
        for k, v in part.get("metrics", {}).items():
            c = canonical_metric_name(k)
            if c is None:
                continue
            v = float(v)
            if not math.isfinite(v):
                raise ZSpaceFusionError(f"non-finite metric {k!r} in partial {i}")
            canon[c] = v
            agg.setdefault(c, []).append((v, w))
        g, replaced = part.get("gradient"), False
        if g is None and metric_gradient_dimension is not None and canon:
            from .api_llm import metric_gradient_projection
            g, replaced = metric_gradient_projection(canon, metric_gradient_dimension)["gradient"], True
        if g is not None:
            g = [float(x) for x in g]
            if not all(math.isfinite(x) for x in g):
                raise ZSpaceFusionError(f"non-finite gradient in partial {i}")
            grads.append((g, w))
        sources.append({"index": i, "status": "active", "weight": w, "origin": part.get("origin"),
                        "metric_count": len(canon), "gradient_dim": len(g) if g is not None else 0,
                        "gradient_replaced_by_metric_projection": replaced})
    fused = {}
    for name, pairs in sorted(agg.items()):
        tot = sum(w for _, w in pairs)
        fused[name] = {"mean": sum(v * w for v, w in pairs) / tot, "last": pairs[-1][0], "max": max(v for v, _ in pairs),
                       "min": min(v for v, _ in pairs), "median": _weighted_median(pairs),
                       "sum": math.fsum(v * w for v, w in pairs)}[strategy]
    gradient = None
    if grads:
        dims = {len(g) for g, _ in grads}
        if len(dims) > 1 and gradient_alignment == "strict":
            raise ZSpaceFusionError(f"gradient dimensions differ: {sorted(dims)}")
        dim, tot = max(dims), sum(w for _, w in grads)
        gradient = [sum((g[j] if j < len(g) else 0.0) * w for g, w in grads) / tot for j in range(dim)]
    return {"kind": "spiraltorch.zspace_partial_fusion", "strategy": strategy, "metrics": fused, "gradient": gradient,
            "gradient_summary": ZSpaceTelemetrySummary.from_values(gradient or []), "sources": sources,
            "active_count": sum(s["status"] == "active" for s in sources),
            "suppressed_count": sum(s["status"] == "suppressed" for s in sources),
            "null_count": sum(s["status"] == "null" for s in sources)}
