"""Microlocal interface gauges: detect where a phase-field mask has an interface, lift the detection to a Z pulse and
fuse the pulses of several gauges through the Z conductor.

Parity: crates/st-core/src/theory/microlocal.rs — `InterfaceGauge::analyze*` (:58-240: per cell the largest one-sided
difference, the interface flag against the threshold, the second-difference vector, the boundary-aware Laplacian, the
bounded mean curvature, the label-signed curvature and the unit orientation), `MicrolocalGaugeBank` (:242-345),
`InterfaceZLift::project` (:399-575), `InterfaceZPulse::{aggregate, lerp, scaled,
into_softlogic_feedback}` (:577-757), `MicrolocalFeedback` (:806-900), quality policies `Default / Fixed / Composite /
Band / Budget` (:900-1082), `InterfaceZConductor::{apply_feedback, step}` (:1119-1440).

The gauge is a stencil over the whole mask: here it is a handful of shifted tensor differences on whichever device holds
the mask (any number of dimensions), not a loop over cells.  With an `EllipticWarp` on the lift the mean orientation is
read on a curved chart (`elliptic.py`) and its sheet / spin / heat telemetry shapes the bands and the bias.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import observability
from .elliptic import EllipticAccumulator, EllipticTelemetry, EllipticWarp
from .hub import SoftlogicZFeedback
from .theory import LeechProjector
from .zpulse import ZConductor, ZEmitter, ZPulse, ZRegistry, ZScale, ZSupport, source_label

EPS = 1.1920929e-07


def unit_sphere_area(dim: int) -> float:
    return 0.0 if dim == 0 else 2.0 * math.pi ** (dim / 2.0) / math.gamma(dim / 2.0)


@dataclass
class InterfaceSignature:
    r_machine: torch.Tensor                      # 1 where an interface passes, else 0
    raw_density: torch.Tensor                    # largest one-sided difference per cell
    perimeter_density: torch.Tensor              # kappa_d on interface cells
    mean_curvature: torch.Tensor                 # min(|laplacian| / 4, kappa_d)
    signed_mean_curvature: Optional[torch.Tensor]
    orientation: Optional[torch.Tensor]          # [dim, *mask.shape]
    kappa_d: float
    radius: int
    physical_radius: float

    def has_interface(self) -> bool:
        return bool((self.r_machine > 0).any())


def _shift_pairs(mask: torch.Tensor, axis: int):
    """Forward and backward one-sided differences along `axis`, zero where the neighbour does not exist, and the
    masks of where each exists."""
    d = torch.diff(mask, dim=axis)                                   # x[i+1] - x[i] at position i
    zero = torch.zeros_like(mask.narrow(axis, 0, 1))
    fwd = torch.cat([d, zero], dim=axis)                             # defined for i < n - 1
    bwd = torch.cat([zero, d], dim=axis)                             # x[i] - x[i-1], defined for i > 0
    n = mask.shape[axis]
    idx = torch.arange(n, device=mask.device)
    shape = [1] * mask.dim()
    shape[axis] = n
    return fwd, bwd, (idx < n - 1).reshape(shape), (idx > 0).reshape(shape)


class InterfaceGauge:
    def __init__(self, grid_spacing: float, physical_radius: float, threshold: float = 0.25):
        self.grid_spacing, self._physical_radius, self._threshold = max(grid_spacing, EPS), max(physical_radius, EPS), max(threshold, 0.0)

    def with_threshold(self, threshold: float) -> "InterfaceGauge":
        self._threshold = max(threshold, 0.0)
        return self

    def physical_radius(self) -> float:
        return self._physical_radius

    def threshold(self) -> float:
        return self._threshold

    def scale_threshold(self, scale: float) -> None:
        if scale > 0.0:
            self._threshold = max(self._threshold * scale, 0.0)

    def analyze(self, mask) -> InterfaceSignature:
        return self.analyze_with_radius(mask, None, self._physical_radius)

    def analyze_with_label(self, mask, c_prime=None) -> InterfaceSignature:
        return self.analyze_with_radius(mask, c_prime, self._physical_radius)

    def analyze_multiradius(self, mask, c_prime, radii: Sequence[float]) -> List[InterfaceSignature]:
        return [self.analyze_with_radius(mask, c_prime, r) for r in radii]

    def analyze_with_radius(self, mask, c_prime, physical_radius: float) -> InterfaceSignature:
        mask = torch.as_tensor(mask, dtype=torch.float32)
        if mask.dim() == 0:
            raise ValueError("mask must have positive dimension")
        if c_prime is not None:
            c_prime = torch.as_tensor(c_prime, dtype=torch.float32, device=mask.device)
            if c_prime.shape != mask.shape:
                raise ValueError("c' must match mask shape")
        steps = max(int(math.floor(physical_radius / self.grid_spacing + 0.5)), 1)
        dim = mask.dim()
        kappa = unit_sphere_area(dim)
        variation = torch.zeros_like(mask)
        interface = torch.zeros_like(mask, dtype=torch.bool)
        laplacian = torch.zeros_like(mask)
        second = []
        for axis in range(dim):
            fwd, bwd, has_f, has_b = _shift_pairs(mask, axis)
            variation = torch.maximum(variation, torch.maximum(fwd.abs(), bwd.abs()))
            interface |= (has_f & (fwd.abs() >= self._threshold)) | (has_b & (bwd.abs() >= self._threshold))
            second.append(fwd - bwd)                                  # forward + backward - 2 centre where both exist
            laplacian = laplacian + torch.where(has_f & has_b, fwd - bwd, torch.zeros_like(mask))
        r_machine = interface.to(mask.dtype)
        signed = orient = None
        if c_prime is not None:
            signed = laplacian * torch.sign(c_prime)
            g = torch.stack(second)
            norm = g.pow(2).sum(0).sqrt()
            orient = torch.where(norm > 0, g / norm.clamp(min=1e-6), g)
        return InterfaceSignature(r_machine, variation, r_machine * kappa, (laplacian.abs() * 0.25).clamp(max=kappa), signed, orient,
                                  kappa, steps, float(physical_radius))


class MicrolocalGaugeBank:
    """Gauges by id, in registration order."""

    def __init__(self):
        self._gauges: Dict[str, InterfaceGauge] = {}

    def register(self, gauge_id: str, gauge: InterfaceGauge) -> bool:
        if gauge_id in self._gauges:
            return False
        self._gauges[gauge_id] = gauge
        return True

    def with_registered(self, gauge_id: str, gauge: InterfaceGauge) -> "MicrolocalGaugeBank":
        self.register(gauge_id, gauge)
        return self

    def get(self, gauge_id: str) -> Optional[InterfaceGauge]:
        return self._gauges.get(gauge_id)

    def remove(self, gauge_id: str) -> Optional[InterfaceGauge]:
        return self._gauges.pop(gauge_id, None)

    def ids(self) -> List[str]:
        return list(self._gauges)

    def items(self):
        return list(self._gauges.items())

    def __len__(self) -> int:
        return len(self._gauges)

    def is_empty(self) -> bool:
        return not self._gauges

    def to_vec(self) -> List[InterfaceGauge]:
        return list(self._gauges.values())

    def analyze_all(self, mask, c_prime=None) -> Dict[str, InterfaceSignature]:
        return {k: g.analyze_with_label(mask, c_prime) for k, g in self._gauges.items()}


@dataclass
class InterfaceZPulse:
    source: str = "microlocal"
    support: float = 0.0
    interface_cells: float = 0.0
    band_energy: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    scale: Optional[ZScale] = ZScale.ONE
    drift: float = 0.0
    z_bias: float = 0.0
    quality_hint: Optional[float] = None
    standard_error: Optional[float] = None
    elliptic: Optional[EllipticTelemetry] = None

    def total_energy(self) -> float:
        return sum(self.band_energy)

    def density_fluctuation(self) -> float:
        return ZPulse.density_fluctuation_for(self.band_energy)

    def is_empty(self) -> bool:
        return self.support <= EPS and self.total_energy() <= EPS

    def _weight(self) -> float:
        return max(self.support, self.total_energy(), EPS)

    @staticmethod
    def aggregate(pulses: Sequence["InterfaceZPulse"]) -> "InterfaceZPulse":
        """Supports, cells and bands add; drift, bias and scale are weighted by ``max(support, energy)``."""
        if not pulses:
            return InterfaceZPulse()
        w = [p._weight() for p in pulses]
        total = sum(w)
        scale = ZScale.weighted_average((p.scale, wi) for p, wi in zip(pulses, w) if p.scale is not None) \
            or next((p.scale for p in reversed(pulses) if p.scale is not None), None) or ZScale.ONE
        acc = EllipticAccumulator()
        for p, wi in zip(pulses, w):
            if p.elliptic is not None:
                acc.accumulate(p.elliptic, wi)
        return InterfaceZPulse("microlocal", sum(p.support for p in pulses), sum(p.interface_cells for p in pulses),
                               tuple(sum(p.band_energy[i] for p in pulses) for i in range(3)), scale,
                               sum(p.drift * wi for p, wi in zip(pulses, w)) / total, sum(p.z_bias * wi for p, wi in zip(pulses, w)) / total,
                               elliptic=acc.finish())

    @staticmethod
    def lerp(current: "InterfaceZPulse", nxt: "InterfaceZPulse", alpha: float) -> "InterfaceZPulse":
        t = min(max(alpha, 0.0), 1.0)
        mix = lambda a, b: a + (b - a) * t                             # noqa: E731
        scale = ZScale.lerp(current.scale, nxt.scale, t) if current.scale and nxt.scale else (current.scale or nxt.scale)
        return InterfaceZPulse(nxt.source, mix(current.support, nxt.support), mix(current.interface_cells, nxt.interface_cells),
                               tuple(mix(a, b) for a, b in zip(current.band_energy, nxt.band_energy)), scale, mix(current.drift, nxt.drift),
                               mix(current.z_bias, nxt.z_bias), nxt.quality_hint if nxt.quality_hint is not None else current.quality_hint,
                               nxt.standard_error if nxt.standard_error is not None else current.standard_error,
                               current.elliptic.lerp(nxt.elliptic, t) if current.elliptic and nxt.elliptic else (current.elliptic or nxt.elliptic))

    def scaled(self, gain: float) -> "InterfaceZPulse":
        g = max(gain, 0.0)
        return replace(self, support=self.support * g, interface_cells=self.interface_cells * g,
                       band_energy=tuple(b * g for b in self.band_energy), drift=self.drift * g, z_bias=self.z_bias * g)

    def into_softlogic_feedback(self, psi_total: float = 0.0, weighted_loss: float = 0.0) -> SoftlogicZFeedback:
        return SoftlogicZFeedback(psi_total, weighted_loss, tuple(self.band_energy), self.drift, self.z_bias, self.scale,
                                  elliptic=None if self.elliptic is None else self.elliptic.as_dict())


class InterfaceZLift:
    """Turns a signature into a pulse: the mean variation is the "here" band, the support-weighted mean orientation along
    the first axis splits it into above / beneath, and its Leech-enriched magnitude (times the bias gain) is the bias."""

    def __init__(self, weights: Sequence[float], projector: LeechProjector, bias_gain: float = 1.0, elliptic: Optional[EllipticWarp] = None):
        if not len(weights):
            raise ValueError("at least one weight expected")
        norm = max(sum(weights), EPS)
        self.weights, self.projector, self._bias_gain = [w / norm for w in weights], projector, max(bias_gain, 0.0)
        self.elliptic = elliptic

    def with_elliptic_warp(self, warp: EllipticWarp) -> "InterfaceZLift":
        self.elliptic = warp
        return self

    def set_elliptic_warp(self, warp: Optional[EllipticWarp]) -> None:
        self.elliptic = warp

    def elliptic_warp(self) -> Optional[EllipticWarp]:
        return self.elliptic

    def with_bias_gain(self, gain: float) -> "InterfaceZLift":
        self._bias_gain = max(gain, 0.0)
        return self

    def set_bias_gain(self, gain: float) -> None:
        if gain > 0.0:
            self._bias_gain = gain

    def bias_gain(self) -> float:
        return self._bias_gain

    def clone(self) -> "InterfaceZLift":
        out = InterfaceZLift([1.0], self.projector, self._bias_gain, None if self.elliptic is None else self.elliptic.clone())
        out.weights = list(self.weights)
        return out

    def project(self, signature: InterfaceSignature) -> InterfaceZPulse:
        r = signature.r_machine
        support = float(r.sum())
        here = max(float(signature.raw_density.mean()) if signature.raw_density.numel() else 0.0, 0.0)
        above = beneath = bias = 0.0
        sample = None
        if signature.orientation is not None:
            o = signature.orientation
            mean = [(float((o[a] * r).sum()) / support if support > 0.0 else 0.0) for a in range(o.shape[0])]
            sample = self.elliptic.map_orientation(mean) if self.elliptic is not None else None
            if sample is not None:
                above, beneath, bias = self._elliptic_split(sample, here)
            else:
                primary = mean[0] * self.weights[0]
                bias = self.projector.enrich(abs(primary)) * math.copysign(1.0, primary) * self._bias_gain if primary != 0.0 else 0.0
                above, beneath = max(primary, 0.0) * here, max(-primary, 0.0) * here
        band = (max(above, 0.0), here, max(beneath, 0.0))
        drift = (band[0] - band[2]) / max(support, 1e-6) if support > 0.0 else 0.0
        return InterfaceZPulse("microlocal", support, float((r > 0.5).sum()), band, ZScale.new(signature.physical_radius), drift, bias,
                               elliptic=sample)

    def _elliptic_split(self, s: EllipticTelemetry, here: float):
        """Leading / trailing shares of the "here" energy and the bias on a curved chart: the distance from the pole sets
        the base split, the sheet position, homology phase, spin, rotor focus against lateral flux, noise and resonance
        heat tilt it, and the sector parity picks which side the heat favours (microlocal.rs:487-545)."""
        normalized, spin = s.clamped_radius(), min(max(s.spin_alignment, -1.0), 1.0)
        leading, trailing = max(1.0 - normalized, 0.0), max(normalized, 0.0)
        rotor_focus = math.sqrt(abs(s.rotor_field[2]) + 1e-3)
        lateral = (abs(s.rotor_field[0]) + abs(s.rotor_field[1])) * 0.5
        gate = min(max(1.0 - s.noise_density, 0.05), 1.0)
        sector_bias = 1.0 + (s.topological_sector & 0x7) * 0.05
        phase = (s.homology_index & 0xFF) / 255.0
        leading *= max(0.55 + 0.45 * s.sheet_position + phase * 0.2, 1e-3)
        trailing *= max(0.55 + 0.45 * (1.0 - s.sheet_position) + (1.0 - phase) * 0.2, 1e-3)
        leading *= max(0.5 * (1.0 + spin), 1e-3) * (1.0 + rotor_focus * 0.5) * gate
        trailing *= max(0.5 * (1.0 - spin), 1e-3) * (1.0 + lateral * 0.5) * (1.0 - gate * 0.35)
        even = s.topological_sector & 1 == 0
        leading *= 1.0 + s.resonance_heat * (1.0 if even else 0.25)
        trailing *= 1.0 + s.resonance_heat * (0.25 if even else 1.0)
        leading *= sector_bias
        trailing *= max(2.0 - sector_bias, 0.25)
        total = max(leading + trailing, 1e-5)
        bias = self.projector.enrich(abs(s.normal_bias)) * (math.copysign(1.0, s.normal_bias) if s.normal_bias != 0.0 else 0.0) * self._bias_gain
        bias *= (1.0 + spin * 0.25) * (1.0 + min(max(s.flow_vector[2], -1.0), 1.0) * 0.5) * (1.0 - s.noise_density * 0.5)
        bias += (1.0 if even else -1.0) * s.resonance_heat * 0.1
        return here * leading / total, here * trailing / total, bias


@dataclass
class MicrolocalFeedback:
    threshold_scale: Optional[float] = None
    bias_gain: Optional[float] = None
    smoothing: Optional[float] = None
    tempo_hint: Optional[float] = None
    stderr_hint: Optional[float] = None
    elliptic_radius: Optional[float] = None
    elliptic_sheet_count: Optional[int] = None
    elliptic_spin_harmonics: Optional[int] = None

    def merge(self, other: "MicrolocalFeedback") -> "MicrolocalFeedback":
        """Threshold scales multiply; for everything else the other side wins when it has a value."""
        a, b = self.threshold_scale, other.threshold_scale
        pick = lambda x, y: y if y is not None else x                      # noqa: E731
        return MicrolocalFeedback(max(a * b, 0.0) if a is not None and b is not None else pick(a, b), pick(self.bias_gain, other.bias_gain),
                                  pick(self.smoothing, other.smoothing), pick(self.tempo_hint, other.tempo_hint), pick(self.stderr_hint, other.stderr_hint),
                                  pick(self.elliptic_radius, other.elliptic_radius), pick(self.elliptic_sheet_count, other.elliptic_sheet_count),
                                  pick(self.elliptic_spin_harmonics, other.elliptic_spin_harmonics))

    def with_threshold_scale(self, scale: float) -> "MicrolocalFeedback":
        return replace(self, threshold_scale=(self.threshold_scale or 1.0) * scale) if scale > 0.0 else self

    def with_bias_gain(self, gain: float) -> "MicrolocalFeedback":
        return replace(self, bias_gain=gain) if gain > 0.0 else self

    def with_smoothing(self, smoothing: float) -> "MicrolocalFeedback":
        return replace(self, smoothing=min(max(smoothing, 0.0), 1.0))

    def with_tempo_hint(self, tempo: float) -> "MicrolocalFeedback":
        return replace(self, tempo_hint=tempo) if tempo >= 0.0 else self

    def with_stderr_hint(self, stderr: float) -> "MicrolocalFeedback":
        return replace(self, stderr_hint=stderr) if stderr >= 0.0 else self

    def with_elliptic_radius(self, radius: float) -> "MicrolocalFeedback":
        return replace(self, elliptic_radius=radius) if math.isfinite(radius) and radius > 0.0 else self

    def with_elliptic_sheet_count(self, sheets: int) -> "MicrolocalFeedback":
        return replace(self, elliptic_sheet_count=sheets) if sheets > 0 else self

    def with_elliptic_spin_harmonics(self, harmonics: int) -> "MicrolocalFeedback":
        return replace(self, elliptic_spin_harmonics=harmonics) if harmonics > 0 else self


# ---- quality policies -------------------------------------------------------------------------------------------------------
class ZSourcePolicy:
    def quality(self, pulse: InterfaceZPulse) -> float:
        raise NotImplementedError

    def late_fuse(self, fused: InterfaceZPulse, pulses: Sequence[InterfaceZPulse], qualities: Sequence[float]) -> None:
        return None


class DefaultZSourcePolicy(ZSourcePolicy):
    def quality(self, pulse):
        return 0.0 if pulse.is_empty() else min(max(pulse.support / max(pulse.total_energy(), 1e-6), 0.0), 1.0)


class FixedPolicy(ZSourcePolicy):
    def __init__(self, value: float):
        self.value = value

    def quality(self, pulse):
        return min(max(self.value, 0.0), 1.0)


class CompositePolicy(ZSourcePolicy):
    def __init__(self, default: ZSourcePolicy):
        self.default, self.overrides = default, {}

    def with_source(self, source: str, policy: ZSourcePolicy) -> "CompositePolicy":
        self.overrides[source_label(source)] = policy
        return self

    def quality(self, pulse):
        return self.overrides.get(pulse.source, self.default).quality(pulse)

    def late_fuse(self, fused, pulses, qualities):
        self.default.late_fuse(fused, pulses, qualities)
        for source, policy in self.overrides.items():
            if any(p.source == source for p in pulses):
                policy.late_fuse(fused, pulses, qualities)


class BandPolicy:
    """A pulse whose band shares fall below the minimum shares is discounted in proportion to the shortfall."""

    def __init__(self, min_quality: Sequence[float], hysteresis: float = 0.0):
        self.min_quality, self.hysteresis = [min(max(v, 0.0), 1.0) for v in min_quality], max(hysteresis, 0.0)

    def with_hysteresis(self, hysteresis: float) -> "BandPolicy":
        self.hysteresis = max(hysteresis, 0.0)
        return self

    @classmethod
    def positive_curvature(cls, radius: float) -> "BandPolicy":
        polar = math.tanh(1.0 / max(radius, 1e-6))
        leading = min(max(0.2 + 0.15 * polar, 0.1), 0.45)
        return cls([leading, min(max(0.5 + 0.25 * polar, 0.35), 0.9), leading])

    def project_quality(self, pulse: InterfaceZPulse) -> float:
        total, scale = max(pulse.total_energy(), 1e-6), 1.0
        for band, threshold in zip(pulse.band_energy, self.min_quality):
            ratio = band / total
            if ratio + self.hysteresis < threshold:
                scale *= 0.0 if threshold <= EPS else min(max(ratio / threshold, 0.0), 1.0)
        return min(max(scale, 0.0), 1.0)


class BudgetPolicy:
    def __init__(self, z_max: float):
        self.z_max = max(abs(z_max), 1e-6)

    def apply(self, fused: InterfaceZPulse) -> float:
        """Scales bias, the outer bands and the support so that ``|z_bias| <= z_max``; returns the scale."""
        if abs(fused.z_bias) <= self.z_max:
            return 1.0
        s = self.z_max / abs(fused.z_bias)
        fused.z_bias *= s
        fused.band_energy = (fused.band_energy[0] * s, fused.band_energy[1], fused.band_energy[2] * s)
        fused.support *= s
        return s


class _QueueEmitter(ZEmitter):
    def __init__(self):
        self.queue: deque = deque()

    def name(self) -> str:
        return "microlocal"

    def tick(self, now: int) -> Optional[ZPulse]:
        return self.queue.popleft() if self.queue else None


@dataclass
class InterfaceZFused:
    pulse: ZPulse
    z: float
    support: float
    attributions: List[Tuple[str, float]]
    events: List[str]


@dataclass
class InterfaceZReport:
    gauge_ids: List[Optional[str]]
    signatures: List[InterfaceSignature]
    lift: InterfaceZLift
    pulses: List[InterfaceZPulse]
    qualities: List[float]
    fused_pulse: InterfaceZPulse
    fused_z: InterfaceZFused
    feedback: SoftlogicZFeedback
    budget_scale: float

    def has_interface(self) -> bool:
        return self.fused_pulse.support > 0.0

    def gauge_id(self, index: int) -> Optional[str]:
        return self.gauge_ids[index] if 0 <= index < len(self.gauge_ids) else None

    def signature_for(self, gauge_id: str) -> Optional[InterfaceSignature]:
        return next((s for g, s in zip(self.gauge_ids, self.signatures) if g == gauge_id), None)


class InterfaceZConductor:
    """Every gauge analyses the mask; the lift turns each signature into a pulse; a quality policy (and an optional band
    policy) weights them; the weighted aggregate is smoothed against the previous step and clamped by the budget; the raw
    pulses go through a `ZConductor` for the control value ``z``; the fused pulse becomes the soft-logic feedback."""

    def __init__(self, gauges, lift: InterfaceZLift):
        if isinstance(gauges, MicrolocalGaugeBank):
            slots = [(k, g) for k, g in gauges.items()]
        else:
            slots = [(None, g) for g in gauges]
        if not slots:
            raise ValueError("at least one gauge must be supplied")
        self.slots, self._lift = slots, lift
        self.conductor, self.clock, self.smoothing = ZConductor(), 0, 0.0
        self.policy: ZSourcePolicy = DefaultZSourcePolicy()
        self.band_policy: Optional[BandPolicy] = None
        self.budget_policy: Optional[BudgetPolicy] = None
        self.previous: Optional[InterfaceZPulse] = None
        self.emitter = _QueueEmitter()
        self.default_tempo_hint: Optional[float] = None
        self.default_stderr_hint: Optional[float] = None

    from_bank = classmethod(lambda cls, bank, lift: cls(bank, lift))

    def lift(self) -> InterfaceZLift:
        return self._lift.clone()

    def with_smoothing(self, smoothing: float) -> "InterfaceZConductor":
        self.smoothing = min(max(smoothing, 0.0), 1.0)
        return self

    def with_policy(self, policy: ZSourcePolicy) -> "InterfaceZConductor":
        self.policy = policy
        return self

    def with_band_policy(self, policy: BandPolicy) -> "InterfaceZConductor":
        self.band_policy = policy
        return self

    def with_budget_policy(self, policy: BudgetPolicy) -> "InterfaceZConductor":
        self.budget_policy = policy
        return self

    def reinforce_positive_curvature(self, radius: float) -> "InterfaceZConductor":
        self._lift.set_elliptic_warp(EllipticWarp(radius))
        self.band_policy = BandPolicy.positive_curvature(radius).with_hysteresis(0.05)
        return self

    def gauge_thresholds(self) -> List[float]:
        return [g.threshold() for _, g in self.slots]

    def bias_gain(self) -> float:
        return self._lift.bias_gain()

    def apply_feedback(self, feedback: MicrolocalFeedback) -> None:
        if feedback.threshold_scale is not None and feedback.threshold_scale > 0.0:
            for _, g in self.slots:
                g.scale_threshold(feedback.threshold_scale)
        if feedback.bias_gain is not None:
            self._lift.set_bias_gain(feedback.bias_gain)
        if feedback.smoothing is not None:
            self.smoothing = min(max(feedback.smoothing, 0.0), 1.0)
        if feedback.tempo_hint is not None:
            self.default_tempo_hint = max(feedback.tempo_hint, 0.0)
        if feedback.stderr_hint is not None:
            self.default_stderr_hint = max(feedback.stderr_hint, 0.0)
        if feedback.elliptic_radius is not None or feedback.elliptic_sheet_count is not None or feedback.elliptic_spin_harmonics is not None:
            cur = self._lift.elliptic_warp()
            r = feedback.elliptic_radius
            if r is not None and math.isfinite(r) and r > 0.0:
                warp = EllipticWarp(r, cur.sheet_count() if cur else 2, cur.spin_harmonics() if cur else 1)
            else:
                warp = cur.clone() if cur else None
            if warp is not None:
                warp.configure(feedback.elliptic_sheet_count, feedback.elliptic_spin_harmonics)
                self._lift.set_elliptic_warp(warp)

    def last_fused_pulse(self) -> InterfaceZPulse:
        return replace(self.previous) if self.previous is not None else InterfaceZPulse()

    def step(self, mask, c_prime=None, tempo_hint: Optional[float] = None, stderr_hint: Optional[float] = None) -> InterfaceZReport:
        stderr_base = stderr_hint if stderr_hint is not None else self.default_stderr_hint
        stderr_base = None if stderr_base is None else max(stderr_base, 0.0)
        ids, signatures, pulses = [], [], []
        for gid, gauge in self.slots:
            sig = gauge.analyze_with_label(mask, c_prime)
            pulse = self._lift.project(sig)
            pulse.standard_error = stderr_base
            ids.append(gid)
            signatures.append(sig)
            pulses.append(pulse)
        qualities = []
        for p in pulses:
            q = min(max(self.policy.quality(p), 0.0), 1.0)
            qualities.append(q * self.band_policy.project_quality(p) if self.band_policy is not None else q)
        fused = InterfaceZPulse.aggregate([p.scaled(q) for p, q in zip(pulses, qualities)])
        events: List[str] = []
        if self.previous is not None and self.smoothing > 0.0:
            fused = InterfaceZPulse.lerp(self.previous, fused, self.smoothing)
            events.append("smoothing.applied")
        if fused.elliptic is not None:
            events.extend(fused.elliptic.event_tags())
        budget_scale = self.budget_policy.apply(fused) if self.budget_policy is not None else 1.0
        self.policy.late_fuse(fused, pulses, qualities)
        now, self.clock = self.clock, self.clock + 1
        if fused.standard_error is None:
            fused.standard_error = stderr_base
        tempo = tempo_hint if tempo_hint is not None else (self.default_tempo_hint if self.default_tempo_hint is not None else fused.total_energy())
        for p, q in zip(pulses, qualities):
            self.emitter.queue.append(ZPulse(p.source, now, tempo, p.band_energy, ZPulse.density_fluctuation_for(p.band_energy), p.drift, p.z_bias,
                                             ZSupport.from_band_energy(p.band_energy), p.scale, q,
                                             p.standard_error if p.standard_error is not None else (stderr_base or 0.0), 0.0))
        registry = ZRegistry()
        registry.register(self.emitter)
        z = self.conductor.step_from_registry(registry, now)
        events.extend(z.events)
        feedback = fused.into_softlogic_feedback()
        feedback.set_events(events)
        feedback.set_attributions(z.attributions)
        self.previous = replace(fused)
        zp = ZPulse(fused.source, now, tempo, fused.band_energy, ZPulse.density_fluctuation_for(fused.band_energy), fused.drift, fused.z_bias,
                    ZSupport.from_band_energy(fused.band_energy), fused.scale, sum(qualities) / len(qualities) if qualities else 0.0,
                    fused.standard_error or 0.0, 0.0)
        report = InterfaceZReport(ids, signatures, self._lift.clone(), pulses, qualities, replace(fused),
                                  InterfaceZFused(zp, z.z, z.support, list(z.attributions), list(events)), feedback, budget_scale)
        m = torch.as_tensor(mask)
        observability.emit_tensor_op("microlocal_conductor_step", tuple(m.shape), (len(pulses), 1))
        observability.emit_tensor_op_meta("microlocal_conductor_step", lambda: {
            "backend": "torch", "kind": "microlocal_conductor_step", "clock": now, "mask_ndim": m.dim(), "mask_len": m.numel(),
            "has_label": c_prime is not None, "gauges": len(self.slots), "smoothing": self.smoothing, "has_band_policy": self.band_policy is not None,
            "has_budget_policy": self.budget_policy is not None, "budget_scale": budget_scale, "fused_support": fused.support,
            "fused_z_bias": fused.z_bias, "z": z.z, "events": len(events), "quality_mean": sum(qualities) / len(qualities)})
        return report
