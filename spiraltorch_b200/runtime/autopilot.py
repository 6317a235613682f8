"""Autopilot: closed-world runtime knob tuning on top of the BlackCat contextual bandit.

One suggest / report cycle per training step: ``build_context`` turns the workload (batch, tiles, depth,
device load, named extras) and the device capabilities into the bandit's feature vector; ``suggest`` asks
BlackCat for one value per knob (under ``AutoMode.HINT`` the persisted choices break ties between
equivalent arms); ``report`` credits the step's :class:`StepMetrics` to that selection, folds the step into a
bounded observation window and durably commits the device profile (median step latency, p95 peak memory,
mean retry rate over the last 128 steps) to ``<profile_dir>/<profile_key>.json``.

Restated from crates/st-core/src/runtime/autopilot.rs: ``AutoMode`` :61, ``KnobSpec`` :73, ``AutoConfig``
:84, ``DeviceProfile`` :109, ``AutopilotReport`` :122, the error vocabulary :133-190, ``Autopilot`` :297
(``try_build_context`` :471, ``try_suggest`` :567, ``abandon_suggestion`` :654, ``try_report`` :667), the
Hyndman-Fan type-7 quantile :1055 and the compensated mean used for the retry rate.
"""
from __future__ import annotations

import enum
import json
import math
import os
from collections import deque
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Sequence

from .. import plugin
from ..nn.trainer import StepMetrics
from .blackcat import BlackCat, BlackCatError

PROFILE_CONTRACT = "st-core.runtime.autopilot.profile"
PROFILE_SCHEMA_VERSION = 2
CONTEXT_CONTRACT = "st-core.runtime.autopilot.context"
CONTEXT_SCHEMA_VERSION = 2
BASE_CONTEXT_FEATURES = ("intercept", "batch", "tiles", "depth", "device_lane_width_over_1024",
                         "device_max_workgroup_over_4096", "device_load", "device_subgroup")
PROFILE_WINDOW = 128
QUANTILE_ESTIMATOR = "exact_hyndman_fan_type_7"
RETRY_ESTIMATOR = "window_neumaier_arithmetic_mean"


class AutoMode(enum.Enum):
    AUTO = "Auto"       # fully automatic; environment / CLI values are hints only
    HINT = "Hint"       # persisted choices win among equivalent arms, the bandit decides otherwise
    OFF = "Off"         # no dynamic tuning


class AutopilotError(ValueError):
    """Rejected at the Autopilot boundary; ``kind`` names the rule that refused the call."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass
class KnobSpec:
    id: str
    domain: Sequence[str]
    default_idx: int = 0


@dataclass
class AutoConfig:
    mode: AutoMode = AutoMode.AUTO
    knobs: Sequence[KnobSpec] = ()
    feat_dim: int = len(BASE_CONTEXT_FEATURES)
    extra_features: Sequence[str] = ()


@dataclass
class DeviceProfile:
    chosen: dict = field(default_factory=dict)
    step_ms_p50: float = 0.0
    mem_mb_p95: float = 0.0
    retry_rate: float = 0.0


@dataclass
class AutopilotReport:
    reward: float
    profile: DeviceProfile
    sample_count: int


def quantile_type7(values: Sequence[float], probability: float) -> float:
    """Hyndman-Fan type 7 (linear interpolation between order statistics); 0 for an empty window."""
    if not values:
        return 0.0
    xs = sorted(values)
    h = (len(xs) - 1) * probability
    lo = int(math.floor(h))
    hi = min(lo + 1, len(xs) - 1)
    return xs[lo] + (h - lo) * (xs[hi] - xs[lo])


def neumaier_mean(values: Sequence[float]) -> float:
    if not values:
        return 0.0
    total, comp = 0.0, 0.0
    for v in values:
        t = total + v
        comp += (total - t) + v if abs(total) >= abs(v) else (v - t) + total
        total = t
    return (total + comp) / len(values)


class ProfileHistory:
    """The last ``PROFILE_WINDOW`` observations of each metric."""

    def __init__(self):
        self.step_ms: deque = deque(maxlen=PROFILE_WINDOW)
        self.mem_mb: deque = deque(maxlen=PROFILE_WINDOW)
        self.retry: deque = deque(maxlen=PROFILE_WINDOW)

    def copy(self) -> "ProfileHistory":
        h = ProfileHistory()
        h.step_ms.extend(self.step_ms); h.mem_mb.extend(self.mem_mb); h.retry.extend(self.retry)
        return h

    def push(self, m: StepMetrics) -> None:
        self.step_ms.append(float(m.step_time_ms)); self.mem_mb.append(float(m.mem_peak_mb))
        self.retry.append(float(m.retry_rate))

    def sample_count(self) -> int:
        return len(self.step_ms)

    def profile(self, chosen: dict) -> DeviceProfile:
        return DeviceProfile(dict(chosen), quantile_type7(list(self.step_ms), 0.5),
                             quantile_type7(list(self.mem_mb), 0.95), neumaier_mean(list(self.retry)))


def default_profile_dir() -> Path:
    return Path.home() / ".spiraltorch" / "profile.d"


def _reject(stage: str, error: Exception) -> None:
    if plugin.has_listeners("AutopilotRejected"):
        plugin.publish("AutopilotRejected", {"stage": stage, "error": str(error), "kind": getattr(error, "kind", "")})


class Autopilot:
    def __init__(self, caps, cfg: AutoConfig, runtime: BlackCat, profile_dir=None):
        """``caps``: a device-capability record with ``backend``, ``lane_width``, ``max_workgroup`` and
        ``subgroup`` (``device_caps.DeviceCaps``)."""
        if cfg.feat_dim <= 0:
            raise AutopilotError("InvalidFeatureDim", "feat_dim must be positive")
        base = min(cfg.feat_dim, len(BASE_CONTEXT_FEATURES))
        extras = list(cfg.extra_features)
        if base + len(extras) != cfg.feat_dim:
            raise AutopilotError("FeatureSchemaMismatch",
                                 f"feat_dim {cfg.feat_dim} does not equal {base} base features + {len(extras)} extras")
        if len(set(extras)) != len(extras) or any((not e) or e in BASE_CONTEXT_FEATURES for e in extras):
            raise AutopilotError("DuplicateFeature", "extra feature names must be unique, non-empty and not base names")
        if runtime.context_dim != cfg.feat_dim:
            raise AutopilotError("FeatureSchemaMismatch",
                                 f"BlackCat expects {runtime.context_dim} features, the Autopilot builds {cfg.feat_dim}")
        domains = runtime.choice_domains()
        self.knobs: dict = {}
        for k in cfg.knobs:
            dom = [str(v) for v in k.domain]
            if not dom or len(set(dom)) != len(dom) or not 0 <= k.default_idx < len(dom):
                raise AutopilotError("InvalidKnob", f"knob '{k.id}' needs a non-empty, duplicate-free domain and a valid default")
            if k.id in self.knobs:
                raise AutopilotError("InvalidKnob", f"knob '{k.id}' declared twice")
            if k.id in domains and any(v not in dom for v in domains[k.id]):
                raise AutopilotError("InvalidKnob", f"BlackCat may emit values outside the declared domain of '{k.id}'")
            self.knobs[k.id] = (dom, dom[k.default_idx])
        self.caps, self.runtime, self.mode = caps, runtime, cfg.mode
        self.feat_dim, self.extra_features = cfg.feat_dim, extras
        self.profile_dir = Path(profile_dir) if profile_dir is not None else default_profile_dir()
        backend = getattr(caps, "backend", "cuda")
        self.profile_key = f"{backend}-lw{getattr(caps, 'lane_width', 32)}-wg{getattr(caps, 'max_workgroup', 1024)}" \
                           f"-f{cfg.feat_dim}"
        self.profile, self.history = self._load_profile()
        self.picks: dict = {}
        self.suggestion_ready = False

    # ---- persistence ---------------------------------------------------------------------------------------
    def profile_path(self) -> Path:
        return self.profile_dir / f"{self.profile_key}.json"

    def _load_profile(self):
        path = self.profile_path()
        try:
            doc = json.loads(path.read_text())
            if doc.get("contract") != PROFILE_CONTRACT or doc.get("schema_version") != PROFILE_SCHEMA_VERSION \
                    or doc.get("sample_capacity") != PROFILE_WINDOW:
                raise ValueError("foreign or outdated profile")
            samples = doc["samples"]
            lens = {len(samples[k]) for k in ("step_ms", "mem_mb", "retry_rate")}
            if len(lens) != 1 or max(lens) > PROFILE_WINDOW:
                raise ValueError("metric sample counts disagree or exceed the window")
            h = ProfileHistory()
            for a, b, c in zip(samples["step_ms"], samples["mem_mb"], samples["retry_rate"]):
                if not all(math.isfinite(float(v)) and float(v) >= 0 for v in (a, b, c)):
                    raise ValueError("non-finite sample")
                h.push(StepMetrics(float(a), float(b), float(c)))
            return h.profile({str(k): str(v) for k, v in doc.get("chosen", {}).items()}), h
        except (OSError, ValueError, KeyError, TypeError):
            return DeviceProfile(), ProfileHistory()      # a missing or corrupt profile is replaced by an empty one

    def _save_profile(self, profile: DeviceProfile, history: ProfileHistory) -> None:
        doc = {"contract": PROFILE_CONTRACT, "schema_version": PROFILE_SCHEMA_VERSION, "profile_key": self.profile_key,
               "sample_capacity": PROFILE_WINDOW,
               "estimators": {"step_ms_p50": QUANTILE_ESTIMATOR, "mem_mb_p95": QUANTILE_ESTIMATOR,
                              "retry_rate": RETRY_ESTIMATOR},
               "chosen": dict(sorted(profile.chosen.items())),
               "profile": {"step_ms_p50": profile.step_ms_p50, "mem_mb_p95": profile.mem_mb_p95,
                           "retry_rate": profile.retry_rate},
               "samples": {"step_ms": list(history.step_ms), "mem_mb": list(history.mem_mb),
                           "retry_rate": list(history.retry)}}
        self.profile_dir.mkdir(parents=True, exist_ok=True)
        tmp = self.profile_path().with_suffix(f".tmp{os.getpid()}")
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(doc, f, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self.profile_path())

    # ---- context -----------------------------------------------------------------------------------------
    def context_features(self) -> list:
        return list(BASE_CONTEXT_FEATURES[:min(self.feat_dim, len(BASE_CONTEXT_FEATURES))]) + list(self.extra_features)

    def try_build_context(self, batch: int, tiles: int, depth: int, device_load: float, extras=()) -> list:
        try:
            for name, v in (("batch", batch), ("tiles", tiles), ("depth", depth)):
                if int(v) <= 0:
                    raise AutopilotError("NonPositiveWorkload", f"{name} must be positive")
            if not (math.isfinite(device_load) and device_load >= 0):
                raise AutopilotError("InvalidValue", "device_load must be finite and non-negative")
            provided: dict = {}
            for name, value in extras:
                if name in provided:
                    raise AutopilotError("DuplicateFeature", f"feature '{name}' given twice")
                if not math.isfinite(value):
                    raise AutopilotError("InvalidValue", f"extras.{name} must be finite")
                provided[name] = float(value)
            for name in provided:
                if name not in self.extra_features:
                    raise AutopilotError("UnexpectedFeature", f"feature '{name}' is not part of the schema")
            for name in self.extra_features:
                if name not in provided:
                    raise AutopilotError("MissingFeature", f"feature '{name}' is missing")
        except AutopilotError as exc:
            _reject("context", exc)
            raise
        ctx = [1.0, float(batch), float(tiles), float(depth), getattr(self.caps, "lane_width", 32) / 1024.0,
               getattr(self.caps, "max_workgroup", 1024) / 4096.0, float(device_load),
               1.0 if getattr(self.caps, "subgroup", True) else 0.0]
        ctx = ctx[:min(self.feat_dim, len(BASE_CONTEXT_FEATURES))]
        ctx.extend(provided[name] for name in self.extra_features)
        return ctx

    def build_context(self, batch, tiles, depth, device_load, extras=()) -> list:
        try:
            return self.try_build_context(batch, tiles, depth, device_load, extras)
        except AutopilotError:
            return []            # an unusable context: the guarded suggestion path rejects it

    # ---- suggest / report --------------------------------------------------------------------------------
    def try_suggest(self, context) -> dict:
        if self.mode is AutoMode.OFF:
            self.suggestion_ready = False
            self.picks = {}
            return self.picks
        if self.suggestion_ready:
            err = AutopilotError("PendingSuggestion", "the previous suggestion has not been reported or abandoned")
            _reject("suggest", err)
            raise err
        domains = self.runtime.choice_domains()
        hints = {}
        if self.mode is AutoMode.HINT:
            hints = {k: v for k, v in self.profile.chosen.items() if v in domains.get(k, ())}
        try:
            runtime_picks = self.runtime.try_choose_with_hints(context, hints)
        except BlackCatError as exc:
            err = AutopilotError("BlackCat", str(exc))
            _reject("suggest", err)
            raise err from exc
        try:
            picks = self._resolve(runtime_picks)
        except AutopilotError as exc:
            self.runtime.abandon_pending_selection()
            _reject("suggest", exc)
            raise
        self.picks, self.suggestion_ready = picks, True
        if plugin.has_listeners("AutopilotSuggest"):
            plugin.publish("AutopilotSuggest", {
                "profile_key": self.profile_key, "mode": self.mode.value, "context": list(context),
                "context_contract": CONTEXT_CONTRACT, "context_schema_version": CONTEXT_SCHEMA_VERSION,
                "base_context_features": list(BASE_CONTEXT_FEATURES), "context_features": self.context_features(),
                "hints": dict(sorted(hints.items())), "picks": dict(sorted(picks.items())),
                "bandit_selection": self.runtime.last_selection_witness(),
                "profile_contract": PROFILE_CONTRACT, "profile_schema_version": PROFILE_SCHEMA_VERSION})
        return self.picks

    def suggest(self, context) -> dict:
        try:
            return self.try_suggest(context)
        except AutopilotError:
            if not self.suggestion_ready:
                self.picks = {}
            return self.picks

    def abandon_suggestion(self) -> Optional[int]:
        if not self.suggestion_ready:
            return None
        sel = self.runtime.abandon_pending_selection()
        if sel is None:
            return None
        self.suggestion_ready, self.picks = False, {}
        return sel

    def _resolve(self, runtime_picks: dict) -> dict:
        if not self.knobs:
            return dict(runtime_picks)
        for k in runtime_picks:
            if k not in self.knobs:
                raise AutopilotError("UndeclaredKnob", f"BlackCat emitted a value for undeclared knob '{k}'")
        out = {}
        for kid, (domain, default) in self.knobs.items():
            choice = runtime_picks.get(kid)
            if choice is None and self.mode is AutoMode.HINT:
                choice = self.profile.chosen.get(kid)
            if choice is None:
                choice = default
            if choice not in domain:
                raise AutopilotError("InvalidKnobChoice", f"'{choice}' is outside the domain of knob '{kid}'")
            out[kid] = choice
        return out

    def try_report(self, metrics: StepMetrics) -> Optional[AutopilotReport]:
        if self.mode is AutoMode.OFF:
            return None
        if not self.suggestion_ready:
            err = AutopilotError("MissingSuggestion", "report without a pending suggestion")
            _reject("report", err)
            raise err
        for name, v in (("step_time_ms", metrics.step_time_ms), ("mem_peak_mb", metrics.mem_peak_mb),
                        ("retry_rate", metrics.retry_rate)):
            if not (math.isfinite(v) and v >= 0):
                err = AutopilotError("InvalidValue", f"{name} must be finite and non-negative")
                _reject("report", err)
                raise err
        next_history = self.history.copy()
        next_history.push(metrics)
        next_profile = next_history.profile(self.picks)
        try:
            reward = self.runtime.try_post_step(metrics)
        except BlackCatError as exc:
            err = AutopilotError("BlackCat", str(exc))
            _reject("report", err)
            raise err from exc
        self.suggestion_ready = False
        try:
            self._save_profile(next_profile, next_history)
        except OSError as exc:
            err = AutopilotError("ProfileCommit", f"reward {reward} was credited but the profile was not saved: {exc}")
            _reject("profile_commit", err)
            raise err from exc
        self.history, self.profile = next_history, next_profile
        report = AutopilotReport(reward, next_profile, next_history.sample_count())
        if plugin.has_listeners("AutopilotReport"):
            plugin.publish("AutopilotReport", {
                "profile_key": self.profile_key, "mode": self.mode.value, "reward": reward,
                "picks": dict(sorted(self.picks.items())),
                "metrics": {"step_time_ms": metrics.step_time_ms, "mem_peak_mb": metrics.mem_peak_mb,
                            "retry_rate": metrics.retry_rate, "extra": dict(metrics.extra)},
                "profile": {"step_ms_p50": next_profile.step_ms_p50, "mem_mb_p95": next_profile.mem_mb_p95,
                            "retry_rate": next_profile.retry_rate, "sample_count": report.sample_count,
                            "sample_capacity": PROFILE_WINDOW,
                            "estimators": {"step_ms_p50": QUANTILE_ESTIMATOR, "mem_mb_p95": QUANTILE_ESTIMATOR,
                                           "retry_rate": RETRY_ESTIMATOR}},
                "profile_contract": PROFILE_CONTRACT, "profile_schema_version": PROFILE_SCHEMA_VERSION})
        return report

    def report(self, metrics: StepMetrics) -> None:
        try:
            self.try_report(metrics)
        except AutopilotError:
            pass

    def profile_sample_count(self) -> int:
        return self.history.sample_count()
