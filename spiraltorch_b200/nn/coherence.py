"""Attention-free Z-space coherence sequencer with its measurement engine, pre-discard policy / regulator,
diagnostics and stage-trace recorder.

Parity: crates/st-nn/src/zspace_coherence/coherence_engine.rs (`CoherenceEngine::measure_phases` :472-572,
linguistic profiles :135-228, contour :365-419, channel reports :421-466), sequencer.rs (`PreDiscardPolicy::apply`
:725-857, `PreDiscardRegulator::observe` :1181-1298, `ZSpaceCoherenceSequencer` :1616-2240, semantic window
:2369-2526, Maxwell pulse summary :2528-2594) and trace.rs (`ZSpaceTraceRecorder` :744-1000,
`coherence_relation_tensor` :1002-1030).

The pipeline per call is: project rows into the Poincare ball and saturate, measure one weight per channel (RMS of
the channel's columns, biased by curvature / profiles, normalised to a distribution), optionally discard weak
channels, then aggregate: scale each channel's columns by its weight, and smooth along the feature axis with a
forward and a reverse first-order recurrence of coefficient ``fractional_order``.

Device mapping: the projection, the per-channel reduction and the aggregate run as tensor ops on the input's device.
The two recurrences are linear in the row, so they are folded into one ``[dim, dim]`` matrix (built once per
``(dim, order)`` and cached) and the whole aggregate becomes ``(x * column_weight) @ M`` — one GEMM instead of
``2 * dim`` dependent steps.  Only the channel-weight vector (``dim / 8`` floats) comes back to the host, because the
discard policy, diagnostics and plugins are host-side control logic.
"""
from __future__ import annotations

import json
import math
import os
import threading
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import zspace_coherence as zc
from ..tensor import Tensor, TensorError
from ..theory import MaxwellZPulse
from ..topos import OpenCartesianTopos

_F32_EPS = 1.1920929e-07

# ---- concepts, backends, profiles ------------------------------------------------------------------------------------
DOMAIN_CONCEPTS = ("membrane", "grain_boundary", "neuronal_pattern", "droplet_coalescence")
_BACKEND_CAPS = {          # label -> (fft, gpu, timeseries, columnar)
    "pure_rust": (False, False, False, False), "fftw": (True, False, True, False), "cufft": (True, True, True, False),
    "polars": (False, False, True, True), "arrow": (False, False, True, True), "webgpu": (True, True, True, False),
}


@dataclass(frozen=True)
class CoherenceBackend:
    """Label of the runtime a sequencer bridges to; labels outside the known set are custom (no capabilities)."""
    name: str = "pure_rust"

    def label(self) -> str:
        return self.name

    def is_accelerated(self) -> bool:
        return self.name in _BACKEND_CAPS and self.name != "pure_rust"

    def capabilities(self) -> dict:
        fft, gpu, ts, col = _BACKEND_CAPS.get(self.name, (False, False, False, False))
        return {"fft": fft, "gpu": gpu, "timeseries": ts, "columnar": col}


def _positive(label: str, v: float) -> float:
    if not math.isfinite(v) or v <= 0:
        raise TensorError(f"non-positive coherence for {label}: {v}")
    return float(v)


class DomainLinguisticProfile:
    """Biases channel weights towards a domain's harmonic structure: per channel a multiplier
    ``emphasis * shape(concept, (channel + 0.5) / channels)`` or an explicit ``harmonic_bias`` table (its last
    entry extends to further channels)."""

    def __init__(self, concept: str, emphasis: float = 1.0, harmonic_bias: Optional[Sequence[float]] = None,
                 descriptor: Optional[str] = None):
        self.concept = str(concept)
        self.emphasis = _positive("emphasis", emphasis)
        if harmonic_bias is not None:
            if len(harmonic_bias) == 0:
                raise TensorError("empty input: harmonic_bias")
            harmonic_bias = [_positive("harmonic_bias", b) for b in harmonic_bias]
        self.harmonic_bias = harmonic_bias
        self.descriptor = descriptor

    def with_emphasis(self, emphasis: float) -> "DomainLinguisticProfile":
        return DomainLinguisticProfile(self.concept, emphasis, self.harmonic_bias, self.descriptor)

    def with_harmonic_bias(self, bias: Sequence[float]) -> "DomainLinguisticProfile":
        return DomainLinguisticProfile(self.concept, self.emphasis, bias, self.descriptor)

    def with_descriptor(self, descriptor: str) -> "DomainLinguisticProfile":
        return DomainLinguisticProfile(self.concept, self.emphasis, self.harmonic_bias, descriptor)

    def harmonic_bias_len(self) -> Optional[int]:
        return None if self.harmonic_bias is None else len(self.harmonic_bias)

    def harmonic_multiplier(self, channel: int, total: int) -> float:
        if self.harmonic_bias:
            b = self.harmonic_bias[channel] if channel < len(self.harmonic_bias) else self.harmonic_bias[-1]
            return max(b * self.emphasis, 1e-6)
        h = (channel + 0.5) / max(total, 1)
        base = {"membrane": 1.15 - 0.35 * h, "grain_boundary": 0.85 + 0.65 * h,
                "neuronal_pattern": 0.75 + 0.9 * abs(h - 0.5),
                "droplet_coalescence": 0.95 + 0.55 * (1.0 - abs(2.0 * h - 1.0))}.get(self.concept, 1.0)
        return max(base * self.emphasis, 1e-6)

    def multipliers(self, total: int) -> List[float]:
        return [self.harmonic_multiplier(c, total) for c in range(total)]


@dataclass(frozen=True)
class LinguisticContour:
    coherence_strength: float      # sum p^2
    articulation_bias: float       # strength * sqrt(|curvature|), clamped to [0, 4]
    prosody_index: float           # centroid / (channels - 1)
    timbre_spread: float           # sqrt(weighted variance of the channel index / channels)


@dataclass(frozen=True)
class LinguisticChannelReport:
    channel: int
    weight: float
    backend: CoherenceBackend
    dominant_concept: Optional[str]
    emphasis: float
    descriptor: Optional[str]


CoherenceChannelReport = LinguisticChannelReport


class CoherenceEngine:
    """Measures one non-negative weight per feature channel; the weights sum to one."""

    def __init__(self, dim: int, curvature: float, num_channels: Optional[int] = None):
        if dim <= 0:
            raise TensorError("invalid dimensions: coherence engine needs dim > 0")
        if curvature >= 0:
            raise TensorError(f"non-hyperbolic curvature {curvature}")
        if num_channels is not None and num_channels <= 0:
            raise TensorError("empty input: maxwell_channels")
        self.dim, self.curvature = int(dim), float(curvature)
        self.num_channels = int(num_channels) if num_channels else max(dim // 64, 1)
        self.backend = CoherenceBackend()
        self.linguistic_profiles: List[DomainLinguisticProfile] = []

    def with_channel_count(self, n: int) -> "CoherenceEngine":
        if n <= 0:
            raise TensorError("empty input: maxwell_channels")
        self.num_channels = int(n)
        return self

    def set_backend(self, backend) -> None:
        self.backend = backend if isinstance(backend, CoherenceBackend) else CoherenceBackend(str(backend))

    def register_linguistic_profile(self, profile: DomainLinguisticProfile) -> None:
        self.linguistic_profiles.append(profile)

    def clear_linguistic_profiles(self) -> None:
        self.linguistic_profiles.clear()

    def is_accelerated(self) -> bool:
        return self.backend.is_accelerated()

    def curvature_bias(self) -> float:
        return 1.0 + min(math.sqrt(abs(self.curvature)), 4.0)

    def channel_width(self) -> int:
        return -(-self.dim // self.num_channels)

    def _channel_bias(self) -> List[float]:
        bias = [self.curvature_bias() * (1.05 if self.is_accelerated() else 1.0)] * self.num_channels
        for p in self.linguistic_profiles:
            bias = [b * m for b, m in zip(bias, p.multipliers(self.num_channels))]
        return bias

    def measure_phases(self, x) -> List[float]:
        t = x.torch() if isinstance(x, Tensor) else torch.as_tensor(x, dtype=torch.float32)
        if t.dim() != 2 or t.shape[1] != self.dim:
            raise TensorError(f"shape mismatch: input {tuple(t.shape)} against dim {self.dim}")
        t = t.float()
        rows, n, cw = t.shape[0], self.num_channels, self.channel_width()
        colsq = (t * t).sum(0)                                                # [dim], one pass over the input
        pad = n * cw - self.dim
        if pad > 0:
            colsq = torch.cat([colsq, colsq.new_zeros(pad)])
        energy = colsq.reshape(n, cw).sum(1)
        width = torch.tensor([max(min((c + 1) * cw, self.dim) - c * cw, 0) for c in range(n)], dtype=torch.float32, device=t.device)
        samples = width * rows
        rms = torch.sqrt(energy / samples.clamp(min=1.0))
        rms = torch.where(torch.isfinite(rms), rms, torch.zeros_like(rms))
        bias = torch.tensor(self._channel_bias(), dtype=torch.float32, device=t.device)
        w = torch.where(width > 0, (rms * bias).clamp(min=1e-6), torch.full_like(rms, 1e-6))
        total = float(w.sum())
        if not math.isfinite(total) or total <= _F32_EPS:
            raise TensorError(f"non-positive coherence: {total}")
        return (w / max(total, 1e-6)).tolist()

    def derive_linguistic_contour(self, weights: Sequence[float]) -> LinguisticContour:
        if len(weights) == 0:
            raise TensorError("empty input: linguistic_contour_weights")
        if len(weights) != self.num_channels:
            raise TensorError(f"data length mismatch: expected {self.num_channels}, got {len(weights)}")
        for w in weights:
            if not math.isfinite(w) or w < 0:
                raise TensorError(f"non-positive coherence: {w}")
        total = float(sum(weights))
        if not math.isfinite(total) or total <= 0:
            raise TensorError(f"non-positive coherence: {total}")
        p = [w / total for w in weights]
        conc = sum(v * v for v in p)
        centroid = sum(v * i for i, v in enumerate(p))
        prosody = min(max(centroid / max(self.num_channels - 1, 1), 0.0), 1.0) if self.num_channels > 1 else 0.5
        var = sum(v * (i - centroid) ** 2 for i, v in enumerate(p))
        return LinguisticContour(conc, min(max(conc * math.sqrt(abs(self.curvature)), 0.0), 4.0), prosody,
                                 math.sqrt(var / max(self.num_channels, 1)))

    def describe_channels(self, weights: Sequence[float]) -> List[LinguisticChannelReport]:
        if len(weights) != self.num_channels:
            raise TensorError(f"data length mismatch: expected {self.num_channels}, got {len(weights)}")
        if any((not math.isfinite(w)) or w < 0 for w in weights):
            raise TensorError("non-positive coherence: -1")
        out = []
        for c, w in enumerate(weights):
            best = None
            for p in self.linguistic_profiles:
                e = p.harmonic_multiplier(c, self.num_channels)
                if best is None or e > best[1]:
                    best = (p.concept, e, p.descriptor)
            concept, emphasis, desc = best if best else (None, 1.0, None)
            out.append(LinguisticChannelReport(c, float(w), self.backend, concept, emphasis, desc))
        return out


# ---- pre-discard ------------------------------------------------------------------------------------------------------
def _score(v: float) -> float:
    return max(v, 0.0) if math.isfinite(v) else 0.0


def _repairs(values: Sequence[float]) -> Tuple[int, int]:
    nf = sum(1 for v in values if not math.isfinite(v))
    neg = sum(1 for v in values if math.isfinite(v) and v < 0)
    return nf, neg


@dataclass(frozen=True)
class PreDiscardTelemetry:
    dominance_ratio: float
    energy_floor: float
    discarded: int
    preserved: int
    used_fallback: bool
    survivor_energy: float
    discarded_energy: float
    dominant_weight: float
    repaired_non_finite: int = 0
    repaired_negative: int = 0

    @property
    def total(self) -> int:
        return self.discarded + self.preserved

    @property
    def preserved_ratio(self) -> float:
        return self.preserved / self.total if self.total else 0.0

    @property
    def discarded_ratio(self) -> float:
        return self.discarded / self.total if self.total else 0.0

    @property
    def total_energy(self) -> float:
        return self.survivor_energy + self.discarded_energy

    @property
    def survivor_energy_ratio(self) -> float:
        t = self.total_energy
        return min(max(self.survivor_energy / t, 0.0), 1.0) if t > _F32_EPS and math.isfinite(t) else 0.0

    @property
    def discarded_energy_ratio(self) -> float:
        t = self.total_energy
        return min(max(self.discarded_energy / t, 0.0), 1.0) if t > _F32_EPS and math.isfinite(t) else 0.0

    @property
    def repairs_total(self) -> int:
        return self.repaired_non_finite + self.repaired_negative

    def summary(self) -> dict:
        return {"dominance_ratio": self.dominance_ratio, "energy_floor": self.energy_floor, "discarded": self.discarded,
                "preserved": self.preserved, "used_fallback": self.used_fallback, "survivor_energy": self.survivor_energy,
                "discarded_energy": self.discarded_energy, "dominant_weight": self.dominant_weight,
                "preserved_ratio": self.preserved_ratio, "survivor_energy_ratio": self.survivor_energy_ratio,
                "repaired_non_finite": self.repaired_non_finite, "repaired_negative": self.repaired_negative,
                "repairs_total": self.repairs_total}


def _telemetry(policy, discarded, preserved, fallback, surv, disc, dominant, repairs=(0, 0)) -> PreDiscardTelemetry:
    dominant = min(max(dominant, 0.0), 1.0) if math.isfinite(dominant) else 0.0
    if dominant <= _F32_EPS:
        dominant = 0.0
    return PreDiscardTelemetry(policy.dominance_ratio, policy.energy_floor, discarded, preserved, fallback, surv, disc, dominant,
                               repairs[0], repairs[1])


class PreDiscardPolicy:
    """Keeps the channels whose weight is at least ``(1 - dominance_ratio)`` of the strongest one (or above the energy
    floor when even the strongest is below it), never fewer than ``min_channels``, and renormalises the survivors."""

    def __init__(self, dominance_ratio: float, energy_floor: float = 0.0, min_channels: int = 1):
        if not math.isfinite(dominance_ratio) or dominance_ratio < 0:
            raise TensorError(f"non-positive coherence: {dominance_ratio}")
        if not math.isfinite(energy_floor) or energy_floor < 0:
            raise TensorError(f"non-positive coherence: {energy_floor}")
        self.dominance_ratio = min(float(dominance_ratio), 1.0)
        self.energy_floor = float(energy_floor)
        self.min_channels = max(int(min_channels), 1)

    def with_energy_floor(self, floor: float) -> "PreDiscardPolicy":
        return PreDiscardPolicy(self.dominance_ratio, floor, self.min_channels)

    def with_min_channels(self, n: int) -> "PreDiscardPolicy":
        return PreDiscardPolicy(self.dominance_ratio, self.energy_floor, n)

    def apply(self, original: Sequence[float]):
        """Returns ``(filtered weights, telemetry, survivor indices, discarded indices)``."""
        n = len(original)
        if n == 0:
            return [], _telemetry(self, 0, 0, True, 0.0, 0.0, 0.0), [], []
        repairs = _repairs(original)
        scores = [_score(v) for v in original]
        order = sorted(range(n), key=lambda i: -scores[i])            # stable: ties keep the lower index first
        dominant = max(scores[order[0]], 1e-6)
        threshold = dominant * max(1.0 - self.dominance_ratio, 0.0)
        keep = [s >= threshold or (s >= self.energy_floor and dominant <= self.energy_floor) for s in scores]
        if sum(keep) < min(self.min_channels, n):
            for i in order[:min(self.min_channels, n)]:
                keep[i] = True
        surv = [i for i in range(n) if keep[i]]
        disc = [i for i in range(n) if not keep[i]]
        surv_e = sum(scores[i] for i in surv)
        disc_e = sum(scores[i] for i in disc)
        total_e = surv_e + disc_e
        share = min(max(dominant / total_e, 0.0), 1.0) if math.isfinite(total_e) and total_e > _F32_EPS else 0.0
        if surv_e <= _F32_EPS or not math.isfinite(surv_e):
            return [1.0 / n] * n, _telemetry(self, 0, n, True, total_e, 0.0, share, repairs), list(range(n)), []
        filtered = [scores[i] / surv_e if keep[i] else 0.0 for i in range(n)]
        return filtered, _telemetry(self, len(disc), len(surv), False, surv_e, disc_e, share, repairs), surv, disc


class PreDiscardRegulator:
    """Closed-loop offset on the policy's dominance ratio.  Each observation compares the smoothed preserved-channel
    ratio and survivor-energy ratio with their targets; the weighted error (zero inside the deadband) drives a step
    ``-aggressiveness * (error + momentum * trend + integral_gain * integral)``, scaled by a confidence factor from the
    dominant weight, reduced by a fallback penalty, clamped to ``max_step``; the offset stays inside its bounds and
    relaxes towards zero by ``equilibrium_decay`` when the error is zero."""

    def __init__(self, target_preserved_ratio: float, target_survivor_energy_ratio: float):
        for v in (target_preserved_ratio, target_survivor_energy_ratio):
            if not math.isfinite(v) or v < 0:
                raise TensorError(f"non-positive coherence: {v}")
        self.target_preserved_ratio = min(float(target_preserved_ratio), 1.0)
        self.target_survivor_energy_ratio = min(float(target_survivor_energy_ratio), 1.0)
        self.smoothing, self.trend_smoothing, self.aggressiveness, self.max_step = 0.25, 0.5, 0.5, 0.2
        self.min_offset, self.max_offset = -0.5, 0.5
        self.channel_weight, self.energy_weight = 0.5, 0.5
        self.fallback_penalty, self.fallback_gain, self.fallback_smoothing = 0.1, 0.0, 0.0
        self.momentum = self.deadband = self.equilibrium_decay = 0.0
        self.confidence_floor = self.confidence_gain = 0.0
        self.integral_gain = self.integral_limit = self.integral_decay = 0.0
        self.offset = 0.0
        self._preserved_ema = self._energy_ema = self._trend_ema = None
        self._fallback_state = self._integral_state = self._last_error = None
        self.observations = 0

    @staticmethod
    def _unit(v: float) -> float:
        if not (isinstance(v, (int, float)) and 0.0 <= v <= 1.0):
            raise TensorError(f"non-positive coherence: {v}")
        return float(v)

    @staticmethod
    def _nonneg(v: float, strict: bool = False) -> float:
        if not math.isfinite(v) or v < 0 or (strict and v <= 0):
            raise TensorError(f"non-positive coherence: {v}")
        return float(v)

    def with_smoothing(self, s):
        self.smoothing = self._unit(s)
        return self

    def with_error_weights(self, channel_weight, energy_weight):
        cw, ew = self._nonneg(channel_weight), self._nonneg(energy_weight)
        if cw + ew <= _F32_EPS:
            raise TensorError("non-positive coherence: error weights sum to zero")
        self.channel_weight, self.energy_weight = cw, ew
        return self

    def with_fallback_penalty(self, p):
        self.fallback_penalty = self._nonneg(p)
        return self

    def with_fallback_memory(self, gain, smoothing):
        self.fallback_gain, self.fallback_smoothing = self._nonneg(gain), self._unit(smoothing)
        return self

    def with_aggressiveness(self, a):
        self.aggressiveness = self._nonneg(a, strict=True)
        return self

    def with_trend_smoothing(self, s):
        self.trend_smoothing = self._unit(s)
        return self

    def with_max_step(self, s):
        self.max_step = min(self._nonneg(s, strict=True), 1.0)
        return self

    def with_bounds(self, lo, hi):
        if not (math.isfinite(lo) and math.isfinite(hi)) or lo > hi:
            raise TensorError(f"non-positive coherence: {min(lo, hi)}")
        self.min_offset, self.max_offset = float(lo), float(hi)
        return self

    def with_momentum(self, m):
        self.momentum = self._nonneg(m)
        return self

    def with_deadband(self, d):
        self.deadband = self._nonneg(d)
        return self

    def with_equilibrium_decay(self, d):
        self.equilibrium_decay = self._unit(d)
        return self

    def with_confidence_scaling(self, floor, gain):
        self.confidence_floor, self.confidence_gain = self._unit(floor), self._nonneg(gain)
        return self

    def with_integral_control(self, gain, limit, decay):
        self.integral_gain, self.integral_limit, self.integral_decay = self._nonneg(gain), self._nonneg(limit), self._unit(decay)
        return self

    @staticmethod
    def _ema(prev, value, smoothing):
        if prev is None:
            return value
        return value if smoothing <= _F32_EPS else prev + smoothing * (value - prev)

    def next_policy(self, base: PreDiscardPolicy) -> PreDiscardPolicy:
        ratio = min(max(base.dominance_ratio + self.offset, 0.0), 1.0)
        return PreDiscardPolicy(ratio, base.energy_floor, base.min_channels)

    def observe(self, t: PreDiscardTelemetry) -> None:
        self._preserved_ema = self._ema(self._preserved_ema, t.preserved_ratio, self.smoothing)
        self._energy_ema = self._ema(self._energy_ema, t.survivor_energy_ratio, self.smoothing)
        tw = self.channel_weight + self.energy_weight
        raw = 0.0 if tw <= _F32_EPS else (self.channel_weight * (self._preserved_ema - self.target_preserved_ratio)
                                          + self.energy_weight * (self._energy_ema - self.target_survivor_energy_ratio)) / tw
        err = 0.0 if (self.deadband > 0 and abs(raw) <= self.deadband) else raw
        if self._last_error is not None:
            self._trend_ema = self._ema(self._trend_ema, err - self._last_error, self.trend_smoothing)
            trend = self._trend_ema if math.isfinite(self._trend_ema) else 0.0
        else:
            self._trend_ema, trend = 0.0, 0.0
        self._last_error = err
        step = -self.aggressiveness * err
        if self.momentum > 0:
            step -= self.aggressiveness * self.momentum * trend
        if self.confidence_floor > 0 or self.confidence_gain > 0:
            conf = t.dominant_weight if math.isfinite(t.dominant_weight) else 0.0
            conf = min(max(conf, 0.0), 1.0)
            scale = 1.0
            if self.confidence_floor > 0:
                if conf < self.confidence_floor:
                    scale *= min(max(conf / max(self.confidence_floor, _F32_EPS), 0.0), 1.0)
                elif self.confidence_gain > 0:
                    scale *= 1.0 + self.confidence_gain * (conf - self.confidence_floor)
            elif self.confidence_gain > 0:
                scale *= 1.0 + self.confidence_gain * conf
            step *= scale
        quiet = abs(err) <= _F32_EPS and not t.used_fallback
        if self.integral_gain > 0:
            integral = (self._integral_state or 0.0) + err
            if self.integral_limit > 0:
                integral = min(max(integral, -self.integral_limit), self.integral_limit)
            if self.integral_decay > 0 and quiet:
                integral *= 1.0 - self.integral_decay
                if abs(integral) < 1e-6:
                    integral = 0.0
            self._integral_state = integral
            step -= self.aggressiveness * self.integral_gain * integral
        signal = 1.0 if t.used_fallback else 0.0
        if self.fallback_gain > 0 or self.fallback_smoothing > 0:
            self._fallback_state = signal if self.fallback_smoothing <= _F32_EPS else self._ema(self._fallback_state, signal, self.fallback_smoothing)
            state = self._fallback_state
        else:
            state = signal
        pressure = signal + self.fallback_gain * state
        if pressure > 0:
            step -= self.fallback_penalty * pressure
        step = min(max(step, -self.max_step), self.max_step)
        nxt = min(max(self.offset + step, self.min_offset), self.max_offset)
        if self.equilibrium_decay > 0 and quiet:
            nxt *= 1.0 - self.equilibrium_decay
            if abs(nxt) < 1e-6:
                nxt = 0.0
        self.offset = nxt
        self.observations += 1


@dataclass(frozen=True)
class PreDiscardSnapshot:
    step: int
    telemetry: PreDiscardTelemetry
    survivors: Tuple[int, ...]
    discarded: Tuple[int, ...]
    filtered: Tuple[float, ...]


# ---- diagnostics -------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CoherenceSignature:
    dominant_channel: Optional[int]
    energy_ratio: float
    entropy: float
    normalized_entropy: float
    concentration: float
    effective_channels: float
    channels: int
    mean_coherence: float
    swap_invariant: bool
    classification: zc.ClassificationPayload

    @property
    def label(self) -> str:
        return self.classification.label

    @property
    def classification_reason(self) -> str:
        return self.classification.reason


@dataclass(frozen=True)
class CoherenceObservation:
    """Either undetermined (no channels, or background energy) or a signature."""
    signature: Optional[CoherenceSignature] = None

    @property
    def is_signature(self) -> bool:
        return self.signature is not None

    def lift_to_label(self) -> str:
        return "background" if self.signature is None else self.signature.label


is_swap_invariant = zc.is_swap_invariant


@dataclass
class CoherenceDiagnostics:
    channel_weights: List[float]
    normalized_weights: List[float]
    normalization: float
    fractional_order: float
    repaired_non_finite_weights: int
    repaired_negative_weights: int
    dominant_channel: Optional[int]
    mean_coherence: float
    z_bias: float
    energy_ratio: float
    entropy: float
    aggregated: Tensor
    channel_reports: List[LinguisticChannelReport] = field(default_factory=list)
    pre_discard: Optional[PreDiscardTelemetry] = None

    @property
    def coherence(self) -> List[float]:
        return self.channel_weights

    @property
    def coherence_entropy(self) -> float:
        return self.entropy

    @property
    def repaired_weights_total(self) -> int:
        return self.repaired_non_finite_weights + self.repaired_negative_weights

    def preserved_channels(self) -> int:
        return sum(1 for w in self.channel_weights if w > 0)

    def discarded_channels(self) -> int:
        return max(len(self.channel_weights) - self.preserved_channels(), 0)

    def distribution_summary(self) -> zc.DistributionSummary:
        return zc.summarize_distribution(self.normalized_weights)

    def distribution_witness(self) -> zc.DistributionWitness:
        return zc.build_distribution_witness(self.normalized_weights)

    def control_summary(self) -> zc.ControlPayload:
        return zc.derive_control(self.distribution_summary(), self.energy_ratio, self.mean_coherence)

    def classify(self, policy: Optional[zc.ClassificationPolicy] = None) -> zc.ClassificationPayload:
        self.distribution_summary()
        return zc.classify(self.energy_ratio, zc.is_swap_invariant(self.normalized_weights), policy)

    def observation_with_policy(self, policy: Optional[zc.ClassificationPolicy] = None) -> CoherenceObservation:
        if not self.channel_weights:
            return CoherenceObservation()
        dist = self.distribution_summary()
        cls = zc.classify(self.energy_ratio, zc.is_swap_invariant(self.normalized_weights), policy)
        if cls.label == "background":
            return CoherenceObservation()
        return CoherenceObservation(CoherenceSignature(self.dominant_channel, self.energy_ratio, self.entropy, dist.normalized_entropy,
                                                       dist.concentration, dist.effective_channels, dist.channels, self.mean_coherence,
                                                       cls.swap_invariant, cls))

    def observation(self) -> CoherenceObservation:
        try:
            return self.observation_with_policy()
        except zc.CoherenceProjectionError:
            return CoherenceObservation()

    def project_to_zspace_partial(self, config: Optional[zc.ProjectionConfig] = None,
                                  contour: Optional[LinguisticContour] = None) -> zc.ProjectionPayload:
        d = zc.DiagnosticsInput(self.mean_coherence, self.entropy, self.energy_ratio, self.z_bias, self.fractional_order,
                                list(self.normalized_weights), self.preserved_channels(), self.discarded_channels(), self.dominant_channel)
        c = None if contour is None else zc.ContourInput(contour.coherence_strength, contour.prosody_index, contour.articulation_bias,
                                                         contour.timbre_spread)
        return zc.project(d, self.channel_weights, c, config)

    def summary(self) -> dict:
        out = {"dominant_channel": self.dominant_channel, "mean_coherence": self.mean_coherence, "energy_ratio": self.energy_ratio,
               "entropy": self.entropy, "z_bias": self.z_bias, "fractional_order": self.fractional_order,
               "normalization": self.normalization, "preserved_channels": self.preserved_channels(),
               "discarded_channels": self.discarded_channels(), "repaired_weights_total": self.repaired_weights_total}
        try:
            dist = self.distribution_summary()
            cls = self.classify()
            out.update(normalized_entropy=dist.normalized_entropy, concentration=dist.concentration,
                       effective_channels=dist.effective_channels, distribution_channels=dist.channels,
                       distribution_weight_mass=dist.weight_mass, swap_invariant=cls.swap_invariant,
                       classification_kind=cls.label, classification_reason=cls.reason,
                       distribution_witness=self.distribution_witness().as_dict())
        except zc.CoherenceProjectionError:
            pass
        if self.pre_discard is not None:
            out["pre_discard"] = self.pre_discard.summary()
        return out


# ---- the sequencer -----------------------------------------------------------------------------------------------------
_SMOOTHING_CACHE: Dict[tuple, torch.Tensor] = {}


def _smoothing_matrix(dim: int, order: float, device) -> torch.Tensor:
    """``M`` with ``row @ M`` equal to the forward recurrence ``a_j = a_{j-1} + order (v_j - a_{j-1})`` (``a_0 = v_0``)
    followed by the same recurrence run from the last column backwards."""
    key = (dim, round(order, 9), str(device))
    m = _SMOOTHING_CACHE.get(key)
    if m is None:
        f, q = float(order), 1.0 - float(order)
        idx = torch.arange(dim, dtype=torch.float64)
        lag = idx[None, :] - idx[:, None]                                    # lag[k, j] = j - k
        fwd = torch.where(lag >= 0, f * q ** lag.clamp(min=0), torch.zeros_like(lag))      # weight of v_k in a_j, k >= 1
        fwd[0, :] = q ** idx                                                 # v_0 enters with weight q^j
        bwd = torch.where(lag <= 0, f * q ** (-lag).clamp(min=0), torch.zeros_like(lag))   # weight of a_k in b_j, k <= dim-2
        bwd[dim - 1, :] = q ** (dim - 1 - idx)
        m = (fwd @ bwd).float().to(device)
        if len(_SMOOTHING_CACHE) > 16:
            _SMOOTHING_CACHE.clear()
        _SMOOTHING_CACHE[key] = m
    return m


class ZSpaceCoherenceSequencer:
    """Sequence mixer that replaces attention with coherence-weighted channel aggregation."""

    STAGES = ("Projected", "CoherenceMeasured", "PreDiscardApplied", "Aggregated", "LanguageBridged", "BackendConfigured",
              "LinguisticProfileRegistered", "LinguisticProfilesCleared", "SemanticWindowDerived", "SemanticDistributionDerived",
              "CanonicalConceptSelected", "MaxwellBridgeEmitted", "LinguisticContourEmitted", "ChannelsDescribed",
              "SemanticWindowFused", "PsiTelemetryPublished")

    def __init__(self, dim: int, num_heads: int, curvature: float, topos: OpenCartesianTopos):
        if num_heads <= 0:
            raise TensorError("empty input: maxwell_heads")
        if dim <= 0 or dim % num_heads:
            raise TensorError(f"invalid dimensions: dim {dim} is not a multiple of {num_heads} heads")
        if abs(topos.curvature - curvature) > 1e-6:
            raise TensorError(f"curvature mismatch: expected {curvature}, got {topos.curvature}")
        self.dim, self.num_heads, self.curvature, self.topos = int(dim), int(num_heads), float(curvature), topos
        self.coherence_engine = CoherenceEngine(dim, curvature, max(dim // 8, 1, num_heads))
        self._plugins: List = []
        self._pre_discard: Optional[PreDiscardPolicy] = None
        self._regulator: Optional[PreDiscardRegulator] = None
        self._journal: deque = deque(maxlen=32)
        self._journal_step = 0
        self._lock = threading.Lock()

    # -- configuration -------------------------------------------------------------------------------------------
    def set_backend(self, backend) -> None:
        self.coherence_engine.set_backend(backend)
        self._dispatch("BackendConfigured", backend=self.coherence_engine.backend)

    def backend(self) -> CoherenceBackend:
        return self.coherence_engine.backend

    def enable_pre_discard(self, policy: PreDiscardPolicy, regulator: Optional[PreDiscardRegulator] = None) -> None:
        self._pre_discard = policy
        if regulator is not None:
            self._regulator = regulator

    enable_pre_discard_with_regulator = enable_pre_discard

    def set_pre_discard_regulator(self, regulator: PreDiscardRegulator) -> None:
        self._regulator = regulator

    def clear_pre_discard_regulator(self) -> None:
        self._regulator = None

    def disable_pre_discard(self) -> None:
        self._pre_discard = self._regulator = None

    def pre_discard_policy(self) -> Optional[PreDiscardPolicy]:
        return self._pre_discard

    def pre_discard_regulator(self) -> Optional[PreDiscardRegulator]:
        return self._regulator

    def configure_pre_discard_memory(self, limit: int) -> None:
        with self._lock:
            self._journal = deque(self._journal, maxlen=max(int(limit), 1)) if limit > 0 else deque(maxlen=0)

    def pre_discard_snapshots(self) -> List[PreDiscardSnapshot]:
        with self._lock:
            return list(self._journal)

    def clear_pre_discard_snapshots(self) -> None:
        with self._lock:
            self._journal.clear()

    def register_plugin(self, plugin) -> None:
        """``plugin`` has ``name`` and ``on_stage(stage: str, payload: dict)``; a raising plugin aborts the call."""
        self._plugins.append(plugin)

    def install_trace_recorder(self, config: Optional["ZSpaceTraceConfig"] = None) -> "ZSpaceTraceRecorder":
        rec = ZSpaceTraceRecorder(config)
        self.register_plugin(rec)
        return rec

    def clear_plugins(self) -> None:
        self._plugins.clear()

    def plugin_names(self) -> List[str]:
        return [getattr(p, "name", type(p).__name__) for p in self._plugins]

    def register_linguistic_profile(self, profile: DomainLinguisticProfile) -> None:
        self.coherence_engine.register_linguistic_profile(profile)
        self._dispatch("LinguisticProfileRegistered", profile=profile)

    def clear_linguistic_profiles(self) -> None:
        self.coherence_engine.clear_linguistic_profiles()
        self._dispatch("LinguisticProfilesCleared")

    def linguistic_profiles(self) -> List[DomainLinguisticProfile]:
        return list(self.coherence_engine.linguistic_profiles)

    def maxwell_channels(self) -> int:
        return self.coherence_engine.num_channels

    def canonical_domain_concept(self) -> str:
        if self.curvature < -0.5:
            return "neuronal_pattern" if self.num_heads > 16 else "membrane"
        if self.curvature > 0.5:
            return "droplet_coalescence" if self.num_heads > 8 else "grain_boundary"
        return "neuronal_pattern" if self.num_heads >= 12 else "membrane"

    def fractional_order(self) -> float:
        c = abs(self.curvature)
        k, lo, hi = {"membrane": (1.0, 0.1, 0.85), "grain_boundary": (0.8, 0.15, 0.9), "neuronal_pattern": (0.6, 0.2, 0.95),
                     "droplet_coalescence": (1.2, 0.05, 0.8)}[self.canonical_domain_concept()]
        return min(max(1.0 / (1.0 + c * k), lo), hi)

    def _dispatch(self, stage: str, **payload) -> None:
        for p in self._plugins:
            p.on_stage(stage, payload)

    # -- the pipeline --------------------------------------------------------------------------------------------
    @staticmethod
    def _raw(x) -> torch.Tensor:
        return (x.torch() if isinstance(x, Tensor) else torch.as_tensor(x, dtype=torch.float32)).float()

    def project_to_zspace(self, x) -> Tensor:
        t = self._raw(x)
        if t.dim() != 2 or t.shape[1] != self.dim:
            raise TensorError(f"shape mismatch: input {tuple(t.shape)} against dim {self.dim}")
        p = Tensor._wrap(t).project_to_poincare(self.curvature).torch()
        p = self.topos.saturate(p)
        self.topos.guard_tensor("zspace_coherence_project_to_zspace", p)
        return Tensor._wrap(p)

    def _run_pre_discard(self, coherence: List[float]):
        if self._pre_discard is None:
            return coherence, None
        policy = self._regulator.next_policy(self._pre_discard) if self._regulator is not None else self._pre_discard
        filtered, tel, surv, disc = policy.apply(coherence)
        if self._regulator is not None:
            self._regulator.observe(tel)
        self._dispatch("PreDiscardApplied", original=coherence, filtered=filtered, telemetry=tel, survivors=surv, discarded=disc)
        with self._lock:
            if self._journal.maxlen:
                self._journal.append(PreDiscardSnapshot(self._journal_step, tel, tuple(surv), tuple(disc), tuple(filtered)))
            self._journal_step += 1
        return filtered, tel

    def _aggregate(self, x, weights: Sequence[float]):
        if len(weights) == 0:
            raise TensorError("empty input: coherence_weights")
        n = self.coherence_engine.num_channels
        if len(weights) != n:
            raise TensorError(f"data length mismatch: expected {n}, got {len(weights)}")
        t = self._raw(x)
        cw = -(-self.dim // n)
        repairs = _repairs(weights)
        clean = [_score(w) for w in weights]
        norm = max(sum(clean), 1e-6)
        order = self.fractional_order()
        col = torch.tensor(clean, dtype=torch.float32, device=t.device).repeat_interleave(cw)[:self.dim] / norm
        agg = (t * col) @ _smoothing_matrix(self.dim, order, t.device)
        agg = self.topos.saturate(agg)
        self.topos.guard_tensor("zspace_coherence_geometric_aggregate", agg)
        return agg, norm, order, max(cw, 1), repairs

    def geometric_aggregate(self, x, coherence_weights: Sequence[float]) -> Tensor:
        return Tensor._wrap(self._aggregate(x, coherence_weights)[0])

    def summarise_maxwell_pulse(self, aggregated, coherence: Sequence[float]) -> MaxwellZPulse:
        a = self._raw(aggregated).double()
        n = max(a.numel(), 1)
        mean = float(a.mean()) if a.numel() else 0.0
        std = float(a.var(unbiased=False).sqrt()) if a.numel() else 0.0
        se = std / math.sqrt(n)
        third = max(len(coherence) // 3, 1)
        above, here, beneath = sum(coherence[:third]), sum(coherence[third:2 * third]), sum(coherence[2 * third:])
        zb = (above - beneath) * math.sqrt(abs(self.curvature))
        return MaxwellZPulse(int(a.shape[0]) if a.dim() else 0, mean, se, mean / se if se > 0 else 0.0,
                             (float(above), float(here), float(beneath)), zb if math.isfinite(zb) else 0.0)

    def _diagnostics(self, agg: torch.Tensor, weights, cw, norm, order, repairs, pre) -> CoherenceDiagnostics:
        w = list(weights)
        nw = [max(v, 0.0) for v in w]
        s = sum(nw)
        nw = [v / s for v in nw] if s > 0 else ([1.0 / len(nw)] * len(nw) if nw else [])
        mean = sum(w) / len(w) if w else 0.0
        finite = [(v, i) for i, v in enumerate(w) if math.isfinite(v)]
        dom = max(finite, key=lambda p: (p[0], p[1]))[1] if finite else None      # ties: the later channel, as max_by does
        absum = agg.abs().sum(0)
        total = max(float(absum.sum()), 1e-6)
        de = float(absum[dom * cw:min((dom + 1) * cw, self.dim)].sum()) if dom is not None else 0.0
        entropy = -sum(v * math.log(v) for v in nw if math.isfinite(v) and v > 0)
        zb = self.summarise_maxwell_pulse(agg, w).z_bias
        return CoherenceDiagnostics(w, nw, norm, order, repairs[0], repairs[1], dom, mean, zb, min(max(de / total, 0.0), 1.0),
                                    entropy, Tensor._wrap(agg), [], pre)

    def forward_with_diagnostics(self, x):
        """Returns ``(aggregated, channel weights, diagnostics)``."""
        z = self.project_to_zspace(x)
        self._dispatch("Projected", input=x, projected=z)
        coherence = self.coherence_engine.measure_phases(z)
        self._dispatch("CoherenceMeasured", z_space=z, coherence=coherence)
        coherence, pre = self._run_pre_discard(coherence)
        agg, norm, order, cw, repairs = self._aggregate(z, coherence)
        diag = self._diagnostics(agg, coherence, cw, norm, order, repairs, pre)
        diag.channel_reports = self.coherence_engine.describe_channels(coherence)
        out = Tensor._wrap(agg)
        self._dispatch("Aggregated", aggregated=out, coherence=coherence, diagnostics=diag)
        return out, coherence, diag

    def forward_with_coherence(self, x):
        out, coherence, _ = self.forward_with_diagnostics(x)
        return out, coherence

    def diagnostics(self, x) -> CoherenceDiagnostics:
        return self.forward_with_diagnostics(x)[2]

    def forward(self, x) -> Tensor:
        return self.forward_with_diagnostics(x)[0]

    __call__ = forward

    def backward(self, _input, grad_output):
        """The sequencer has no parameters and passes the gradient through unchanged."""
        return grad_output

    def parameters(self) -> list:
        return []

    def state_dict(self) -> list:
        return []

    def load_state_dict(self, state) -> None:
        if state:
            raise TensorError("the coherence sequencer has no parameters to load")

    def emit_linguistic_contour(self, x) -> LinguisticContour:
        coherence, _ = self._run_pre_discard(self.coherence_engine.measure_phases(x))
        contour = self.coherence_engine.derive_linguistic_contour(coherence)
        self._dispatch("LinguisticContourEmitted", coherence=coherence, contour=contour)
        return contour

    def describe_channels(self, x) -> List[LinguisticChannelReport]:
        coherence, _ = self._run_pre_discard(self.coherence_engine.measure_phases(x))
        reports = self.coherence_engine.describe_channels(coherence)
        self._dispatch("ChannelsDescribed", coherence=coherence, reports=reports)
        return reports

    # -- language bridges ----------------------------------------------------------------------------------------
    def derive_semantic_window(self, aggregated, coherence: Sequence[float], tokens: int) -> List[Tuple[int, float]]:
        """Splits the feature axis into ``tokens`` bands; each band with positive mean |activation| becomes
        ``(token, energy * weight of the channel under the band's centre)``, normalised to sum to one (floor 1e-6)."""
        a = self._raw(aggregated)
        if tokens <= 0 or not len(coherence) or a.numel() == 0:
            return []
        rows, cols = a.shape
        tw, cw = -(-cols // tokens), -(-cols // len(coherence))
        colabs = a.abs().sum(0).tolist()
        window = []
        for tok in range(tokens):
            s = tok * tw
            if s >= cols:
                break
            e = min((tok + 1) * tw, cols)
            energy = sum(colabs[s:e]) / ((e - s) * rows)
            if not math.isfinite(energy) or energy <= 0:
                continue
            ch = ((s + e - 1) // 2) // cw
            w = max(energy * (coherence[ch] if ch < len(coherence) else 1.0 / len(coherence)), 0.0)
            if w > 0:
                window.append((tok, w))
        tot = sum(w for _, w in window)
        if tot > 0:
            window = [(t, max(w / tot, 1e-6)) for t, w in window]
        return window

    @staticmethod
    def fuse_distributions(lhs: Sequence[float], rhs: Sequence[float]) -> List[float]:
        n = max(len(lhs), len(rhs), 1)
        get = lambda v, i: max(v[i], 0.0) if i < len(v) else 1e-6                     # noqa: E731
        fused = [get(lhs, i) + get(rhs, i) for i in range(n)]
        s = sum(fused)
        return [max(v / s, 1e-6) for v in fused] if s > 0 and math.isfinite(s) else [1.0 / n] * n

    def forward_with_language_bridges(self, x, semantics, maxwell_bridge):
        """Returns ``(aggregated, coherence, concept distribution, narrative hint or None, pulse)``."""
        agg, coherence = self.forward_with_coherence(x)
        tokens = semantics.vocab_size()
        window = self.derive_semantic_window(agg, coherence, tokens)
        self._dispatch("SemanticWindowDerived", window=window, tokens=tokens)
        if window:
            dist = [float(v) for v in semantics.infer_from_window(window, 1e-6).tolist()]
        else:
            c = max(semantics.concept_count(), 1)
            dist = [1.0 / c] * c
        self._dispatch("SemanticDistributionDerived", window=window, distribution=dist)
        pulse = self.summarise_maxwell_pulse(agg, coherence)
        channel = self.canonical_domain_concept()
        self._dispatch("CanonicalConceptSelected", concept=channel, channel=channel)
        emission = maxwell_bridge.emit(channel, pulse)
        narrative = None
        if emission is not None:
            hint, narrative = emission
            self._dispatch("MaxwellBridgeEmitted", channel=channel, pulse=pulse, hint=hint, narrative=narrative)
            dist = self.fuse_distributions(dist, hint.as_distribution(semantics))
        self._dispatch("SemanticWindowFused", concept=dist)
        self._dispatch("LanguageBridged", aggregated=agg, coherence=coherence, concept=dist, narrative=narrative, pulse=pulse)
        return agg, coherence, dist, narrative, pulse


# ---- trace recorder ----------------------------------------------------------------------------------------------------
@dataclass
class ZSpaceTraceConfig:
    capacity: int = 256
    max_vector_len: int = 256
    publish_plugin_events: bool = field(
        default_factory=lambda: os.environ.get("SPIRAL_ZSPACE_TRACE_PUBLISH", "").strip().lower() in ("1", "true", "on"))


TRACE_SCHEMA = "spiraltorch.zspace_trace"
TRACE_SCHEMA_VERSION = 1


class ZSpaceTraceRecorder:
    """Sequencer plugin that keeps the last ``capacity`` stage events as JSON-ready dicts (vectors cut to
    ``max_vector_len``), counts what it dropped, writes JSONL, and optionally republishes each record on the plugin
    bus as a ``ZSpaceTrace`` custom event."""

    name = "zspace_trace"

    def __init__(self, config: Optional[ZSpaceTraceConfig] = None):
        self.config = config or ZSpaceTraceConfig()
        self._events: deque = deque()
        self._next_step = 0
        self._dropped = 0
        self._lock = threading.Lock()

    def _vec(self, v) -> list:
        return [float(a) for a in list(v)[:max(self.config.max_vector_len, 1)]]

    @staticmethod
    def _shape(t) -> list:
        return list(t.shape()) if isinstance(t, Tensor) else list(getattr(t, "shape", ()))

    @staticmethod
    def _pulse(p: MaxwellZPulse) -> dict:
        return {"blocks": p.blocks, "mean": p.mean, "standard_error": p.standard_error, "z_score": p.z_score,
                "band_energy": list(p.band_energy), "z_bias": p.z_bias}

    def _snapshot(self, stage: str, p: dict) -> dict:
        if stage == "Projected":
            return {"input_shape": self._shape(p["input"]), "projected_shape": self._shape(p["projected"])}
        if stage == "CoherenceMeasured":
            return {"coherence": self._vec(p["coherence"])}
        if stage == "Aggregated":
            return {"aggregated_shape": self._shape(p["aggregated"]), "coherence": self._vec(p["coherence"]),
                    "diagnostics": p["diagnostics"].summary()}
        if stage == "PreDiscardApplied":
            lim = max(self.config.max_vector_len, 1)
            return {"original": self._vec(p["original"]), "filtered": self._vec(p["filtered"]), "telemetry": p["telemetry"].summary(),
                    "survivors": list(p["survivors"])[:lim], "discarded": list(p["discarded"])[:lim]}
        if stage == "LanguageBridged":
            n = p.get("narrative")
            return {"coherence": self._vec(p["coherence"]), "concept": {"distribution": self._vec(p["concept"])},
                    "narrative": None if n is None else n.summary().as_dict(), "pulse": self._pulse(p["pulse"])}
        if stage == "BackendConfigured":
            return {"backend": p["backend"].label()}
        if stage == "LinguisticProfileRegistered":
            pr = p["profile"]
            return {"profile": {"concept": pr.concept, "emphasis": pr.emphasis, "harmonic_bias_len": pr.harmonic_bias_len(),
                                "descriptor": pr.descriptor}}
        if stage == "SemanticWindowDerived":
            return {"window": [[int(t), float(w)] for t, w in p["window"][:max(self.config.max_vector_len, 1)]], "tokens": p["tokens"]}
        if stage == "SemanticDistributionDerived":
            return {"distribution": self._vec(p["distribution"]),
                    "window": [[int(t), float(w)] for t, w in p["window"][:max(self.config.max_vector_len, 1)]]}
        if stage == "CanonicalConceptSelected":
            return {"concept": p["concept"], "channel": p["channel"]}
        if stage == "MaxwellBridgeEmitted":
            n = p.get("narrative")
            return {"channel": p["channel"], "pulse": self._pulse(p["pulse"]), "hint": p["hint"].snapshot(self.config.max_vector_len),
                    "narrative": None if n is None else n.summary().as_dict()}
        if stage == "LinguisticContourEmitted":
            c = p["contour"]
            return {"coherence": self._vec(p["coherence"]), "contour": {"coherence_strength": c.coherence_strength,
                    "articulation_bias": c.articulation_bias, "prosody_index": c.prosody_index, "timbre_spread": c.timbre_spread}}
        if stage == "ChannelsDescribed":
            return {"coherence": self._vec(p["coherence"]),
                    "reports": [{"channel": r.channel, "weight": r.weight, "backend": r.backend.label(),
                                 "dominant_concept": r.dominant_concept, "emphasis": r.emphasis, "descriptor": r.descriptor}
                                for r in p["reports"][:max(self.config.max_vector_len, 1)]]}
        if stage == "SemanticWindowFused":
            return {"concept": {"distribution": self._vec(p["concept"])}}
        if stage == "PsiTelemetryPublished":
            return {"pulse": self._pulse(p["pulse"]), "events": len(p.get("events", ())), "reading_present": p.get("reading") is not None}
        return {}

    def on_stage(self, stage: str, payload: dict) -> None:
        with self._lock:
            step = self._next_step
            self._next_step += 1
            record = {"schema": TRACE_SCHEMA, "schema_version": TRACE_SCHEMA_VERSION, "kind": stage, "step": step,
                      "payload": self._snapshot(stage, payload)}
            self._events.append(record)
            while len(self._events) > max(self.config.capacity, 1):
                self._events.popleft()
                self._dropped += 1
        if self.config.publish_plugin_events:
            from .. import plugin
            if plugin.has_listeners("ZSpaceTrace"):
                plugin.publish("ZSpaceTrace", {"record": record})

    def snapshot(self) -> dict:
        with self._lock:
            return {"dropped_events": self._dropped, "events": list(self._events)}

    def records(self) -> List[dict]:
        return self.snapshot()["events"]

    def clear(self) -> None:
        with self._lock:
            self._events.clear()
            self._dropped = self._next_step = 0

    def write_jsonl(self, path) -> None:
        with open(path, "w") as f:
            for r in self.records():
                f.write(json.dumps(r) + "\n")


def coherence_relation_tensor(coherence: Sequence[float]) -> Tensor:
    """``n x n`` outer product of the weights scaled by their maximum (non-finite entries count as zero)."""
    if len(coherence) == 0:
        raise TensorError("empty input: coherence")
    c = torch.as_tensor(list(coherence), dtype=torch.float32)
    c = torch.where(torch.isfinite(c), c, torch.zeros_like(c))
    c = (c / max(float(c.max()), 1e-6)).clamp(0.0, 1.0)
    return Tensor._wrap(torch.outer(c, c))
