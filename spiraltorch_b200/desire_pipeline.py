"""Desire automation and pipeline: drives a :class:`DesireLagrangian` step by step, watches the integration
phase for sustained repression pressure and fans every step (and every rewrite trigger) out to sinks - a JSONL
logbook that can be replayed, an in-process channel, the telemetry bus, trigger and trainer bridges.

Restated from crates/st-nn/src/language: ``DesireAutomation`` (automation.rs:122-330: phase-dependent mixing of
avoidance heat / desire bias into the desire vector with weights 0.35 / 0.65, the trigger rule - integration
phase, at least ``min_samples`` penalties, mean penalty at or above ``score_thresh``, cool-down elapsed),
``SelfRewriteCfg`` (crates/st-core/src/config/self_rewrite.rs:11-25), ``DesireLogbook`` / ``DesireLogReplay``
(logbook.rs:17-120), ``DesirePipelineSink`` / ``DesireChannelSink`` / ``DesireTelemetrySink`` /
``DesireTriggerBuffer`` / ``DesireTrainerBridge`` / ``DesirePipelineBuilder`` / ``DesirePipeline``
(pipeline.rs:40-1060,1122-1300).
"""
from __future__ import annotations

import json
import math
import queue
import threading
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

import torch

from . import plugin
from .language import INTEGRATION, OBSERVATION, DesireLagrangian, DesireSolution, DesireWeights

OBSERVATION_MIX, INTEGRATION_MIX = 0.35, 0.65
HISTORY_LIMIT, TRIGGER_EXPORT = 256, 12


@dataclass
class SelfRewriteCfg:
    score_thresh: float = 0.02
    min_samples: int = 30
    cooldown_sec: float = 300.0


@dataclass
class DesireAvoidanceReport:
    tokens: list              # token ids with the highest avoidance heat, hottest first
    scores: list
    observation_steps: int = 0


@dataclass
class DesireRewriteTrigger:
    report: DesireAvoidanceReport
    mean_penalty: float
    mean_entropy: float
    temperature: float
    samples: int


@dataclass
class DesireAutomatedStep:
    solution: DesireSolution
    trigger: Optional[DesireRewriteTrigger] = None


class DesireAutomation:
    def __init__(self, desire: DesireLagrangian, cfg: Optional[SelfRewriteCfg] = None):
        self.desire, self.cfg = desire, cfg or SelfRewriteCfg()
        self.penalties: deque = deque()
        self.entropies: deque = deque()
        self.last_trigger: Optional[float] = None
        self.vector = torch.zeros(desire.vocab_size())
        self.trigger_count = 0
        self._observation_steps = 0

    def desire_vector(self) -> list:
        return self.vector.tolist()

    def mean_penalty(self) -> float:
        return sum(self.penalties) / len(self.penalties) if self.penalties else 0.0

    def mean_entropy(self) -> float:
        return sum(self.entropies) / len(self.entropies) if self.entropies else 0.0

    def penalty_samples(self) -> int:
        return len(self.penalties)

    def report(self, limit: int) -> DesireAvoidanceReport:
        heat = self.desire.avoidance_heat
        k = max(0, min(limit, int((heat > 0).sum())))
        top = torch.topk(heat, k) if k else None
        return DesireAvoidanceReport([] if top is None else top.indices.tolist(),
                                     [] if top is None else top.values.tolist(), self._observation_steps)

    def step(self, lm_logits, previous_token: int, concept_hint, now: Optional[float] = None) -> DesireAutomatedStep:
        return self._drive(self.desire.step_with_scheduler(lm_logits, previous_token, concept_hint), now)

    def step_with_weights(self, lm_logits, previous_token: int, concept_hint, weights: DesireWeights,
                          now: Optional[float] = None) -> DesireAutomatedStep:
        return self._drive(self.desire.step(lm_logits, previous_token, concept_hint, weights), now)

    def _drive(self, solution: DesireSolution, now: Optional[float]) -> DesireAutomatedStep:
        now = time.monotonic() if now is None else now
        if solution.phase == OBSERVATION:
            self._observation_steps += 1
            self._mix(self.desire.avoidance_heat, OBSERVATION_MIX)
        else:
            self._mix(self.desire.desire_bias, INTEGRATION_MIX)
        return DesireAutomatedStep(solution, self._evaluate(now, solution))

    def _mix(self, source: torch.Tensor, mix: float) -> None:
        total = float(source.sum())
        if total <= 1e-6:
            self.vector.mul_(1.0 - mix)
            return
        self.vector = self.vector * (1.0 - mix) + mix * (source / total).clamp(min=0.0)
        norm = float(self.vector.sum())
        if norm > 1e-6:
            self.vector /= norm

    def _evaluate(self, now: float, solution: DesireSolution) -> Optional[DesireRewriteTrigger]:
        if solution.phase != INTEGRATION:
            return None
        limit = max(self.cfg.min_samples, HISTORY_LIMIT)
        for store, v in ((self.penalties, solution.hypergrad_penalty), (self.entropies, solution.entropy)):
            if v == v and abs(v) != float("inf"):
                store.append(max(0.0, float(v)))
                while len(store) > limit:
                    store.popleft()
        if len(self.penalties) < max(1, self.cfg.min_samples) or self.mean_penalty() < self.cfg.score_thresh:
            return None
        if self.last_trigger is not None and now < self.last_trigger + self.cfg.cooldown_sec:
            return None
        trig = DesireRewriteTrigger(self.report(TRIGGER_EXPORT), self.mean_penalty(), self.mean_entropy(),
                                    solution.temperature, len(self.penalties))
        self.last_trigger = now
        self.trigger_count += 1
        self.penalties.clear()
        self.entropies.clear()
        return trig


# ---- logbook ---------------------------------------------------------------------------------------------------
def _step_to_doc(step: DesireAutomatedStep) -> dict:
    return {"solution": asdict(step.solution), "trigger": None if step.trigger is None else asdict(step.trigger)}


def _step_from_doc(doc: dict) -> DesireAutomatedStep:
    sol = dict(doc["solution"])
    sol["weights"] = DesireWeights(**sol["weights"])
    trig = doc.get("trigger")
    if trig is not None:
        trig = dict(trig)
        trig["report"] = DesireAvoidanceReport(**trig["report"])
        trig = DesireRewriteTrigger(**trig)
    return DesireAutomatedStep(DesireSolution(**sol), trig)


@dataclass
class DesireLogRecord:
    ordinal: int
    timestamp_ms: int
    step: DesireAutomatedStep


class DesireLogbook:
    """Append-only JSON-lines log of automated steps; ordinals continue across re-opens of the same file."""

    def __init__(self, path, flush_every: int = 1):
        self.path = Path(path)
        self.flush_every = max(1, flush_every)
        self._ordinal = 0
        if self.path.exists():
            with open(self.path, "r", encoding="utf-8") as f:
                self._ordinal = sum(1 for line in f if line.strip())
        self._fh = open(self.path, "a", encoding="utf-8")
        self._pending = 0

    def ordinal(self) -> int:
        return self._ordinal

    def record(self, step: DesireAutomatedStep, timestamp: Optional[float] = None) -> None:
        ts = time.time() if timestamp is None else timestamp
        self._fh.write(json.dumps({"ordinal": self._ordinal, "timestamp_ms": int(ts * 1e3), **_step_to_doc(step)}) + "\n")
        self._ordinal += 1
        self._pending += 1
        if self._pending >= self.flush_every:
            self.flush()

    record_now = record

    def flush(self) -> None:
        self._fh.flush()
        self._pending = 0

    def close(self) -> None:
        self.flush()
        self._fh.close()


class DesireLogReplay:
    def __init__(self, path):
        self.path = Path(path)
        if not self.path.exists():
            raise FileNotFoundError(f"desire logbook {self.path} does not exist")

    @classmethod
    def open(cls, path) -> "DesireLogReplay":
        return cls(path)

    def __iter__(self):
        with open(self.path, "r", encoding="utf-8") as f:
            for n, line in enumerate(f):
                if not line.strip():
                    continue
                try:
                    doc = json.loads(line)
                    yield DesireLogRecord(int(doc["ordinal"]), int(doc["timestamp_ms"]), _step_from_doc(doc))
                except (ValueError, KeyError, TypeError) as exc:
                    raise ValueError(f"desire logbook {self.path} line {n + 1} is malformed: {exc}") from exc


# ---- sinks -----------------------------------------------------------------------------------------------------
class DesirePipelineSink:
    def on_step(self, step: DesireAutomatedStep, timestamp: float) -> None: ...
    def on_trigger(self, trigger: DesireRewriteTrigger, timestamp: float) -> None: ...
    def flush(self) -> None: ...


class _LogbookSink(DesirePipelineSink):
    def __init__(self, logbook: DesireLogbook):
        self.logbook = logbook

    def on_step(self, step, timestamp):
        self.logbook.record(step, timestamp)

    def flush(self):
        self.logbook.flush()


class DesireChannelSink(DesirePipelineSink):
    """Events as ``("step" | "trigger", payload, timestamp)`` tuples on a thread-safe queue."""

    def __init__(self, sender: Optional[queue.Queue] = None):
        self.queue = sender if sender is not None else queue.Queue()

    def on_step(self, step, timestamp):
        self.queue.put(("step", step, timestamp))

    def on_trigger(self, trigger, timestamp):
        self.queue.put(("trigger", trigger, timestamp))


class DesireTelemetrySink(DesirePipelineSink):
    """Publishes ``DesireStep`` / ``DesireTrigger`` on the plugin event bus."""

    def on_step(self, step, timestamp):
        s = step.solution
        plugin.publish("DesireStep", {"phase": s.phase, "temperature": s.temperature, "entropy": s.entropy,
                                      "hypergrad_penalty": s.hypergrad_penalty, "alpha": s.weights.alpha,
                                      "beta": s.weights.beta, "gamma": s.weights.gamma, "lambda": s.weights.lam,
                                      "triggered": step.trigger is not None})

    def on_trigger(self, trigger, timestamp):
        plugin.publish("DesireTrigger", {"mean_penalty": trigger.mean_penalty, "mean_entropy": trigger.mean_entropy,
                                         "temperature": trigger.temperature, "samples": trigger.samples,
                                         "tokens": list(trigger.report.tokens)})


@dataclass
class DesireTriggerEvent:
    trigger: DesireRewriteTrigger
    timestamp: float


class DesireTriggerBuffer(DesirePipelineSink):
    def __init__(self):
        self._events: list = []
        self._lock = threading.Lock()

    def on_trigger(self, trigger, timestamp):
        with self._lock:
            self._events.append(DesireTriggerEvent(trigger, timestamp))

    def __len__(self):
        with self._lock:
            return len(self._events)

    def is_empty(self) -> bool:
        return len(self) == 0

    def drain(self) -> list:
        with self._lock:
            out, self._events = self._events, []
        return out


@dataclass
class DesireTrainerEvent:
    timestamp: float
    phase: str
    temperature: float
    entropy: float
    hypergrad_penalty: float
    weights: DesireWeights
    trigger: Optional[DesireRewriteTrigger]


@dataclass
class DesireTrainerSummary:
    total: int = 0
    observation: int = 0
    injection: int = 0
    integration: int = 0
    triggers: int = 0
    mean_entropy: float = 0.0
    mean_temperature: float = 0.0
    mean_penalty: float = 0.0
    mean_alpha: float = 0.0
    mean_beta: float = 0.0
    mean_gamma: float = 0.0
    mean_lambda: float = 0.0
    trigger_mean_penalty: float = 0.0

    @classmethod
    def from_events(cls, events: list) -> Optional["DesireTrainerSummary"]:
        if not events:
            return None
        n = len(events)
        trig = [e.trigger for e in events if e.trigger is not None]
        mean = lambda f: sum(f(e) for e in events) / n       # noqa: E731
        return cls(n, sum(e.phase == "observation" for e in events), sum(e.phase == "injection" for e in events),
                   sum(e.phase == "integration" for e in events), len(trig), mean(lambda e: e.entropy),
                   mean(lambda e: e.temperature), mean(lambda e: e.hypergrad_penalty), mean(lambda e: e.weights.alpha),
                   mean(lambda e: e.weights.beta), mean(lambda e: e.weights.gamma), mean(lambda e: e.weights.lam),
                   sum(t.mean_penalty for t in trig) / len(trig) if trig else 0.0)


class DesireTrainerBridge(DesirePipelineSink):
    """Queue between the pipeline and a trainer: the trainer drains the events (or their summary) once per step."""

    def __init__(self):
        self._events: list = []
        self._lock = threading.Lock()

    def on_step(self, step, timestamp):
        s = step.solution
        with self._lock:
            self._events.append(DesireTrainerEvent(timestamp, s.phase, s.temperature, s.entropy, s.hypergrad_penalty,
                                                   s.weights, step.trigger))

    def __len__(self):
        with self._lock:
            return len(self._events)

    def is_empty(self) -> bool:
        return len(self) == 0

    def drain(self) -> list:
        with self._lock:
            out, self._events = self._events, []
        return out

    def drain_summary(self) -> Optional[DesireTrainerSummary]:
        return DesireTrainerSummary.from_events(self.drain())

    def checkpoint(self) -> list:
        with self._lock:
            return [asdict(e) for e in self._events]

    def restore_checkpoint(self, doc: list) -> None:
        events = []
        for d in doc:
            d = dict(d)
            d["weights"] = DesireWeights(**d["weights"])
            if d.get("trigger") is not None:
                t = dict(d["trigger"])
                t["report"] = DesireAvoidanceReport(**t["report"])
                d["trigger"] = DesireRewriteTrigger(**t)
            events.append(DesireTrainerEvent(**d))
        with self._lock:
            self._events = events


# ---- roundtable bridge --------------------------------------------------------------------------------------------
@dataclass
class DesireRoundtableImpulse:
    multipliers: tuple      # (above, here, beneath) band multipliers, each in [0.35, 1.65]
    drift: float            # tanh(lambda) * drift_gain, in [-1, 1]
    timestamp: float


@dataclass
class DesireRoundtableEvent:
    timestamp: float
    solution: DesireSolution
    trigger: Optional[DesireRewriteTrigger]
    multipliers: tuple
    drift: float


_RT_SUMS = ("entropy", "temperature", "alpha", "beta", "gamma", "lambda", "above", "here", "beneath", "drift")


@dataclass
class DesireRoundtableSummary:
    steps: int = 0
    triggers: int = 0
    mean_entropy: float = 0.0
    mean_temperature: float = 0.0
    mean_alpha: float = 0.0
    mean_beta: float = 0.0
    mean_gamma: float = 0.0
    mean_lambda: float = 0.0
    mean_above: float = 0.0
    mean_here: float = 0.0
    mean_beneath: float = 0.0
    mean_drift: float = 0.0
    last_timestamp: float = 0.0

    @classmethod
    def from_events(cls, events: list) -> "DesireRoundtableSummary":
        return _summary_from_pending(_absorb(None, events))


def _absorb(pending: Optional[dict], events: list) -> dict:
    p = dict(pending) if pending else {"steps": 0, "triggers": 0, "last_timestamp": 0.0, **{f"sum_{k}": 0.0 for k in _RT_SUMS}}
    for e in events:
        w = e.solution.weights
        p["steps"] += 1
        p["triggers"] += int(e.trigger is not None)
        for k, v in zip(_RT_SUMS, (e.solution.entropy, e.solution.temperature, w.alpha, w.beta, w.gamma, w.lam, *e.multipliers, e.drift)):
            p[f"sum_{k}"] += v
        p["last_timestamp"] = max(p["last_timestamp"], e.timestamp)
    return p


def _summary_from_pending(p: dict) -> DesireRoundtableSummary:
    n = max(p["steps"], 1)
    return DesireRoundtableSummary(p["steps"], p["triggers"], *[p[f"sum_{k}"] / n for k in _RT_SUMS], p["last_timestamp"])


class DesireRoundtableBridge(DesirePipelineSink):
    """Projects each desire step onto the roundtable: the (alpha, gamma, beta) weights become barycentric band
    multipliers ``1 + blend * (share - 1/3)`` for (above, here, beneath), the lambda weight becomes a drift
    (crates/st-nn/src/language/pipeline.rs:1583-1890, 2057-2124).  The trainer reads the latest impulse per step and
    drains the event queue (or its summary) when it reports; ``propose`` / ``observe`` make it a cooperative agent
    whose blend and drift gain react to team reward and credit."""

    def __init__(self, blend: float = 0.35, drift_gain: float = 0.35):
        self._lock = threading.Lock()
        self._blend = self._drift_gain = 0.35
        self._latest: Optional[DesireRoundtableImpulse] = None
        self._pending: Optional[dict] = None
        self._events: list = []
        self.set_blend(blend)
        self.set_drift_gain(drift_gain)

    def blend(self) -> float:
        return self._blend

    def drift_gain(self) -> float:
        return self._drift_gain

    def set_blend(self, v: float) -> None:
        if math.isfinite(v):
            self._blend = min(max(float(v), 0.0), 1.0)

    def set_drift_gain(self, v: float) -> None:
        if math.isfinite(v):
            self._drift_gain = min(max(float(v), 0.0), 1.0)

    def with_blend(self, v: float) -> "DesireRoundtableBridge":
        self.set_blend(v)
        return self

    def with_drift_gain(self, v: float) -> "DesireRoundtableBridge":
        self.set_drift_gain(v)
        return self

    @staticmethod
    def project(weights: DesireWeights, blend: float, drift_gain: float, timestamp: float) -> DesireRoundtableImpulse:
        above, here, beneath = max(weights.alpha, 0.0), max(weights.gamma, 0.0), max(weights.beta, 0.0)
        total = max(above + here + beneath, 1e-6)
        mult = tuple(min(max(1.0 + blend * (v / total - 1.0 / 3.0), 0.35), 1.65) for v in (above, here, beneath))
        return DesireRoundtableImpulse(mult, min(max(math.tanh(weights.lam) * drift_gain, -1.0), 1.0), timestamp)

    def on_step(self, step, timestamp):
        with self._lock:
            imp = self.project(step.solution.weights, self._blend, self._drift_gain, timestamp)
            self._events.append(DesireRoundtableEvent(timestamp, step.solution, step.trigger, imp.multipliers, imp.drift))
            self._latest = imp

    def impulse(self) -> Optional[DesireRoundtableImpulse]:
        return self._latest

    def __len__(self):
        with self._lock:
            return len(self._events) + (self._pending["steps"] if self._pending else 0)

    def is_empty(self) -> bool:
        return len(self) == 0

    def drain(self) -> list:
        with self._lock:
            out, self._events = self._events, []
        return out

    def drain_summary(self) -> Optional[DesireRoundtableSummary]:
        with self._lock:
            p = _absorb(self._pending, self._events)
            self._pending, self._events = None, []
        return None if p["steps"] == 0 else _summary_from_pending(p)

    def checkpoint(self) -> dict:
        """Blend, drift gain, latest impulse and the queue folded into running sums (events themselves are not kept)."""
        with self._lock:
            p = _absorb(self._pending, self._events)
            latest = None if self._latest is None else {"multipliers": list(self._latest.multipliers), "drift": self._latest.drift,
                                                        "timestamp": self._latest.timestamp}
            return {"blend": self._blend, "drift_gain": self._drift_gain, "latest": latest,
                    "pending_summary": p if p["steps"] else None}

    def restore_checkpoint(self, doc: dict) -> None:
        """Validates everything first; a rejected document leaves the bridge unchanged."""
        def finite(name, v, lo=None, hi=None):
            if not isinstance(v, (int, float)) or not math.isfinite(v) or (lo is not None and v < lo) or (hi is not None and v > hi):
                raise ValueError(f"desire roundtable checkpoint: '{name}' is out of its domain ({v})")
            return float(v)
        blend, gain = finite("blend", doc.get("blend"), 0.0, 1.0), finite("drift_gain", doc.get("drift_gain"), 0.0, 1.2)
        latest = None
        if doc.get("latest") is not None:
            lt = doc["latest"]
            if len(lt.get("multipliers", ())) != 3:
                raise ValueError("desire roundtable checkpoint: 'latest.multipliers' needs three values")
            latest = DesireRoundtableImpulse(tuple(finite("latest.multipliers", m, 0.35, 1.65) for m in lt["multipliers"]),
                                             finite("latest.drift", lt.get("drift"), -1.0, 1.0), finite("latest.timestamp", lt.get("timestamp"), 0.0))
        pending = None
        if doc.get("pending_summary") is not None:
            ps = doc["pending_summary"]
            pending = {"steps": int(ps["steps"]), "triggers": int(ps["triggers"]), "last_timestamp": finite("pending.last_timestamp", ps["last_timestamp"], 0.0),
                       **{f"sum_{k}": finite(f"pending.sum_{k}", ps[f"sum_{k}"]) for k in _RT_SUMS}}
            if pending["steps"] <= 0 or not 0 <= pending["triggers"] <= pending["steps"]:
                raise ValueError("desire roundtable checkpoint: pending step / trigger counts are inconsistent")
        with self._lock:
            self._blend, self._drift_gain, self._latest, self._pending, self._events = blend, gain, latest, pending, []

    # cooperative agent ---------------------------------------------------------------------------------------------
    def propose(self) -> tuple:
        """``(z_bias, weight)``: the latest drift, weighted by the mean multiplier in [0.05, 2]; neutral ``(0, 1)`` before any step."""
        imp = self._latest
        if imp is None:
            return 0.0, 1.0
        return imp.drift, min(max(sum(imp.multipliers) / 3.0, 0.05), 2.0)

    def observe(self, team_reward: float, credit: float) -> None:
        r, c = math.tanh(team_reward), math.tanh(credit)
        with self._lock:
            b = self._blend + (-r * 0.05 if r < 0 else -r * 0.03) + (-c * 0.04 if c < 0 else -c * 0.02)
            self._blend = min(max(b, 0.05), 0.95)
            g = self._drift_gain * ((1.0 - 0.08 * c) if c > 0 else (1.0 + 0.05 * -c))
            self._drift_gain = min(max(g * (1.0 - 0.03 * abs(r)), 0.1), 1.2)


# ---- psi bridge ---------------------------------------------------------------------------------------------------
def record_step_with_psi(step: DesireAutomatedStep, timestamp: float):
    """Builds the step's telemetry sample with the psi reading, psi events and soft-logic Z feedback that the
    telemetry hub holds at this moment, stores it as the hub's latest desire step, and returns
    ``(sample, reading, z_feedback)``.  Parity: crates/st-nn/src/language/pipeline.rs:150-231."""
    from . import hub
    s = step.solution
    with hub.telemetry_guard():
        reading, events, z = hub.get_last_psi(), hub.get_last_psi_events(), hub.get_softlogic_z()
    avoid = getattr(s, "avoidance", None)
    offsets = getattr(s, "logit_offsets", None)
    sample = hub.DesireStepTelemetry(
        timestamp=timestamp, entropy=s.entropy, temperature=s.temperature, hypergrad_penalty=s.hypergrad_penalty,
        avoidance_energy=float(sum(abs(float(v)) for v in avoid.scores)) if avoid is not None else 0.0,
        logit_energy=float(torch.as_tensor(offsets).abs().sum()) if offsets is not None else 0.0, phase=s.phase,
        alpha=s.weights.alpha, beta=s.weights.beta, gamma=s.weights.gamma, lam=s.weights.lam,
        avoidance={"tokens": list(avoid.tokens), "scores": [float(v) for v in avoid.scores]} if avoid is not None else None,
        trigger=None if step.trigger is None else {"mean_penalty": step.trigger.mean_penalty, "mean_entropy": step.trigger.mean_entropy,
                                                   "temperature": step.trigger.temperature, "samples": step.trigger.samples},
        trigger_emitted=step.trigger is not None, psi_total=None if reading is None else reading.total,
        psi_breakdown={} if reading is None else dict(reading.breakdown), psi_events=list(events), z_feedback=z)
    hub.set_last_desire_step(sample)
    return sample, reading, z


@dataclass
class DesirePsiEvent:
    timestamp: float
    solution: DesireSolution
    trigger: Optional[DesireRewriteTrigger]
    telemetry: object
    reading: object
    z_feedback: object
    events: list


@dataclass
class DesirePsiSummary:
    steps: int = 0
    triggers: int = 0
    psi_samples: int = 0
    mean_psi_total: float = 0.0
    component_means: dict = field(default_factory=dict)
    threshold_crossings: dict = field(default_factory=dict)          # component -> (ups, downs)
    mean_entropy: float = 0.0
    mean_temperature: float = 0.0
    mean_hypergrad_penalty: float = 0.0
    mean_z_signal: float = 0.0
    last_timestamp: float = 0.0

    @classmethod
    def from_events(cls, events: list) -> "DesirePsiSummary":
        n = len(events)
        comp_sum, comp_n, crossings = {}, {}, {}
        psi_samples = psi_total = z_n = z_sum = 0.0
        for e in events:
            t = e.telemetry
            if t.psi_total is not None:
                psi_samples, psi_total = psi_samples + 1, psi_total + t.psi_total
                for c, v in t.psi_breakdown.items():
                    comp_sum[c], comp_n[c] = comp_sum.get(c, 0.0) + v, comp_n.get(c, 0) + 1
            if e.z_feedback is not None:
                z_n, z_sum = z_n + 1, z_sum + e.z_feedback.z_signal
            for ev in t.psi_events:
                up, down = crossings.get(ev.component, (0, 0))
                crossings[ev.component] = (up + 1, down) if ev.up else (up, down + 1)
        mean = lambda f: sum(f(e.telemetry) for e in events) / n if n else 0.0       # noqa: E731
        return cls(n, sum(e.trigger is not None for e in events), int(psi_samples), psi_total / psi_samples if psi_samples else 0.0,
                   {c: comp_sum[c] / comp_n[c] for c in comp_sum}, crossings, mean(lambda t: t.entropy), mean(lambda t: t.temperature),
                   mean(lambda t: max(t.hypergrad_penalty, 0.0)), z_sum / z_n if z_n else 0.0, max((e.timestamp for e in events), default=0.0))


class DesirePsiBridge(DesirePipelineSink):
    """Pairs every desire step with the psi reading and Z feedback current at that moment; a trainer drains the events
    (or their summary) once per step.  Parity: crates/st-nn/src/language/pipeline.rs:2288-2470."""

    def __init__(self):
        self._events: list = []
        self._lock = threading.Lock()

    def on_step(self, step, timestamp):
        sample, reading, z = record_step_with_psi(step, timestamp)
        with self._lock:
            self._events.append(DesirePsiEvent(timestamp, step.solution, step.trigger, sample, reading, z, list(sample.psi_events)))

    def __len__(self):
        with self._lock:
            return len(self._events)

    def is_empty(self) -> bool:
        return len(self) == 0

    def drain(self) -> list:
        with self._lock:
            out, self._events = self._events, []
        return out

    def drain_summary(self) -> Optional[DesirePsiSummary]:
        events = self.drain()
        return DesirePsiSummary.from_events(events) if events else None


class DesireTelemetryBundle:
    """The bridges a pipeline should feed, handed around as one object."""

    def __init__(self, trainer: Optional[DesireTrainerBridge] = None, roundtable: Optional[DesireRoundtableBridge] = None, psi=None):
        self.trainer, self.roundtable, self.psi = trainer, roundtable, psi

    def with_trainer_bridge(self, bridge) -> "DesireTelemetryBundle":
        self.trainer = bridge
        return self

    def with_roundtable_bridge(self, bridge) -> "DesireTelemetryBundle":
        self.roundtable = bridge
        return self

    def with_psi_bridge(self, bridge) -> "DesireTelemetryBundle":
        self.psi = bridge
        return self

    def trainer_bridge(self):
        return self.trainer

    def roundtable_bridge(self):
        return self.roundtable

    def psi_bridge(self):
        return self.psi

    def sinks(self) -> list:
        return [b for b in (self.trainer, self.roundtable, self.psi) if b is not None]


# ---- pipeline --------------------------------------------------------------------------------------------------
class DesirePipelineBuilder:
    def __init__(self, automation: DesireAutomation):
        self.automation, self.sinks = automation, []

    def with_sink(self, sink: DesirePipelineSink) -> "DesirePipelineBuilder":
        self.sinks.append(sink)
        return self

    def with_logbook(self, logbook: DesireLogbook): return self.with_sink(_LogbookSink(logbook))                 # noqa: E704
    def with_channel(self, sender: queue.Queue): return self.with_sink(DesireChannelSink(sender))                # noqa: E704
    def with_telemetry(self): return self.with_sink(DesireTelemetrySink())                                        # noqa: E704
    def with_trainer_bridge(self, bridge: DesireTrainerBridge): return self.with_sink(bridge)                    # noqa: E704
    def with_trigger_buffer(self, buffer: DesireTriggerBuffer): return self.with_sink(buffer)                    # noqa: E704
    def with_roundtable_bridge(self, bridge: "DesireRoundtableBridge"): return self.with_sink(bridge)            # noqa: E704
    def with_psi_bridge(self, bridge: "DesirePsiBridge"): return self.with_sink(bridge)                          # noqa: E704

    def with_telemetry_bundle(self, bundle: "DesireTelemetryBundle") -> "DesirePipelineBuilder":
        for sink in bundle.sinks():
            self.with_sink(sink)
        return self

    def build(self) -> "DesirePipeline":
        pipe = DesirePipeline(self.automation)
        pipe.sinks = list(self.sinks)
        return pipe


class DesirePipeline:
    def __init__(self, automation: DesireAutomation):
        self.automation = automation
        self.sinks: list = []

    @staticmethod
    def builder(automation: DesireAutomation) -> DesirePipelineBuilder:
        return DesirePipelineBuilder(automation)

    def attach_sink(self, sink: DesirePipelineSink) -> None:
        self.sinks.append(sink)

    def attach_logbook(self, logbook): self.attach_sink(_LogbookSink(logbook))            # noqa: E704
    def attach_channel(self, sender): self.attach_sink(DesireChannelSink(sender))         # noqa: E704
    def attach_telemetry(self): self.attach_sink(DesireTelemetrySink())                   # noqa: E704
    def attach_trainer_bridge(self, bridge): self.attach_sink(bridge)                     # noqa: E704
    def attach_roundtable_bridge(self, bridge): self.attach_sink(bridge)                  # noqa: E704
    def attach_psi_bridge(self, bridge): self.attach_sink(bridge)                         # noqa: E704

    def sink_count(self) -> int:
        return len(self.sinks)

    def _dispatch(self, step: DesireAutomatedStep, timestamp: float) -> DesireAutomatedStep:
        first = None
        for sink in self.sinks:
            try:
                sink.on_step(step, timestamp)
                if step.trigger is not None:
                    sink.on_trigger(step.trigger, timestamp)
            except Exception as exc:  # noqa: BLE001 - every sink sees the step; the first failure is reported after
                first = first or exc
        if first is not None:
            raise first
        return step

    def step_at(self, lm_logits, previous_token: int, concept_hint, now: float, timestamp: float) -> DesireAutomatedStep:
        return self._dispatch(self.automation.step(lm_logits, previous_token, concept_hint, now), timestamp)

    def step_with_weights_at(self, lm_logits, previous_token: int, concept_hint, weights: DesireWeights, now: float,
                             timestamp: float) -> DesireAutomatedStep:
        return self._dispatch(self.automation.step_with_weights(lm_logits, previous_token, concept_hint, weights, now),
                              timestamp)

    def step_realtime(self, lm_logits, previous_token: int, concept_hint) -> DesireAutomatedStep:
        return self.step_at(lm_logits, previous_token, concept_hint, time.monotonic(), time.time())

    def step_with_weights_realtime(self, lm_logits, previous_token, concept_hint, weights) -> DesireAutomatedStep:
        return self.step_with_weights_at(lm_logits, previous_token, concept_hint, weights, time.monotonic(), time.time())

    def replay(self, replay: DesireLogReplay) -> int:
        """Feeds recorded steps to the sinks again (the automation itself is not re-run); returns their count."""
        n = 0
        for rec in replay:
            self._dispatch(rec.step, rec.timestamp_ms / 1e3)
            n += 1
        return n

    def flush(self) -> None:
        for sink in self.sinks:
            sink.flush()
