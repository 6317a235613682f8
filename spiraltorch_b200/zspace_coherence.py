"""Coherence-distribution contract: summary, witness, control, classification and the Z-space partial
projection of a channel-weight distribution.

Parity: crates/st-core/src/inference/zspace_coherence.rs — `summarize_zspace_coherence_distribution`
(:423-500), distribution witness (:503-587), `derive_zspace_coherence_control` (:589-702),
`is_zspace_coherence_swap_invariant` (:704-724), `classify_zspace_coherence` (:727-790) and
`project_zspace_coherence` (:1114-1290).  Everything is scalar bookkeeping over at most 4096 channel
weights, done in Python floats (IEEE double, as the reference does).

Formulas (``p = w / sum w`` over N channels):
  ``H = -sum p ln p``; ``H_norm = H / ln N`` (0 when N = 1); ``C = (sum p^2 - 1/N) / (1 - 1/N)`` (1 when N = 1);
  ``N_eff = min(exp H, N)``; spectral radius = C, spectral entropy = H_norm, spectral pressure = energy_ratio (1 - H_norm).
Partial: ``speed = tanh(g_s C)``, ``memory = tanh(z_bias)``, ``stability = tanh(g_st (1 - 2 H_norm))``,
``frac = tanh(g_f order)``, ``drs = tanh(g_d (energy_ratio - 0.5))`` plus the ``coherence_*`` metrics.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional, Sequence

PROJECTION_KIND = "spiraltorch.zspace_coherence_projection"
PROJECTION_CONTRACT_VERSION = "spiraltorch.zspace_coherence_projection.v2"
WITNESS_KIND = "spiraltorch.zspace_coherence_distribution_witness"
WITNESS_CONTRACT_VERSION = "spiraltorch.zspace_coherence_distribution_witness.v1"
WITNESS_FORMULA = ("normalized_weights are the complete simplex witness;all distribution summaries and controls must be "
                   "re-derived by st-core")
CLASSIFICATION_KIND = "spiraltorch.zspace_coherence_classification"
CLASSIFICATION_CONTRACT_VERSION = "spiraltorch.zspace_coherence_classification.v1"
CONTROL_KIND = "spiraltorch.zspace_coherence_control"
CONTROL_CONTRACT_VERSION = "spiraltorch.zspace_coherence_control.v1"
SEMANTIC_OWNER = "st-core::inference::zspace_coherence"
SEMANTIC_BACKEND = "rust"        # the wire value consumers of the contract compare against
MAX_CHANNELS = 4096
PARTIAL_METRICS = (
    "coherence_mean", "coherence_entropy", "coherence_energy_ratio", "coherence_z_bias", "coherence_fractional_order",
    "coherence_channels", "coherence_preserved", "coherence_discarded", "coherence_dominant", "coherence_peak",
    "coherence_weight_mass", "coherence_weight_entropy", "coherence_normalized_entropy", "coherence_entropy_residual",
    "coherence_concentration", "coherence_effective_channels", "coherence_response_peak", "coherence_response_mean",
    "coherence_strength", "coherence_prosody", "coherence_articulation", "coherence_timbre_spread")
_TOL_FLOOR = 1.0e-6
_F32_EPS = 1.1920929e-07
_F32_MIN_POSITIVE = 1.17549435e-38

LABELS = ("background", "symmetric_pulse", "cascade_imbalance", "diffuse_drift")


class CoherenceProjectionError(ValueError):
    """Invalid evidence for the coherence contract; ``code`` names the violated rule."""

    def __init__(self, code: str, message: str):
        super().__init__(message)
        self.code = code


def canonical_metric_name(name: str) -> Optional[str]:
    n = name.lower()
    return n if n in PARTIAL_METRICS else None


def _scalar(name: str, v: float) -> None:
    if not math.isfinite(v):
        raise CoherenceProjectionError("non_finite_scalar", f"Z-space coherence field '{name}' must be finite")


def _range(name: str, v: float, lo: float, hi: float) -> None:
    _scalar(name, v)
    if not lo <= v <= hi:
        raise CoherenceProjectionError("scalar_out_of_range",
                                       f"Z-space coherence field '{name}' must lie in [{lo}, {hi}], received {v}")


def _acc_tol(channels: int, scale: float) -> float:
    return max(channels * _F32_EPS * 4.0 * max(scale, 1.0), _TOL_FLOOR)


def _near(v: float, t: float) -> bool:
    return abs(v - t) <= _F32_EPS * max(abs(v), abs(t), _F32_MIN_POSITIVE)


@dataclass(frozen=True)
class DistributionSummary:
    channels: int
    weight_mass: float
    weight_entropy: float
    normalized_entropy: float
    concentration: float
    effective_channels: float


def summarize_distribution(weights: Sequence[float]) -> DistributionSummary:
    w = [float(x) for x in weights]
    if not w:
        raise CoherenceProjectionError("empty_channels", "Z-space coherence projection requires channel evidence")
    if len(w) > MAX_CHANNELS:
        raise CoherenceProjectionError("channel_limit", f"Z-space coherence channel count {len(w)} exceeds limit {MAX_CHANNELS}")
    for i, x in enumerate(w):
        if not math.isfinite(x):
            raise CoherenceProjectionError("non_finite_vector", f"Z-space coherence field 'normalized_weights' entry {i} must be finite")
        if x < 0:
            raise CoherenceProjectionError("negative_weight", f"normalized coherence weight {i} must be non-negative")
        if x > 1:
            raise CoherenceProjectionError("weight_above_one", f"normalized coherence weight {i} must not exceed one")
    mass = sum(w)
    if abs(mass - 1.0) > _acc_tol(len(w), 1.0):
        raise CoherenceProjectionError("invalid_weight_mass", f"normalized coherence weights must sum to one, received {mass}")
    h = sq = 0.0
    for x in w:
        p = x / mass
        if p > 0:
            h -= p * math.log(p)
        sq += p * p
    n = len(w)
    hmax = math.log(n) if n > 1 else 0.0
    hn = min(max(h / hmax, 0.0), 1.0) if hmax > 0 else 0.0
    conc = min(max((sq - 1.0 / n) / (1.0 - 1.0 / n), 0.0), 1.0) if n > 1 else 1.0
    return DistributionSummary(n, mass, h, hn, conc, min(math.exp(h), float(n)))


@dataclass
class DistributionWitness:
    normalized_weights: List[float]
    kind: str = WITNESS_KIND
    contract_version: str = WITNESS_CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND
    witness_formula: str = WITNESS_FORMULA

    def as_dict(self) -> dict:
        return asdict(self)


def build_distribution_witness(weights: Sequence[float]) -> DistributionWitness:
    summarize_distribution(weights)
    return DistributionWitness([float(x) for x in weights])


def _peak(v: Sequence[float]) -> float:
    return max(v) if len(v) else 0.0


def _check_observation(weights, dist: DistributionSummary, preserved, discarded, dominant) -> None:
    seen = sum(1 for x in weights if x > 0)
    for name, got, want in (("preserved_channels", preserved, seen), ("discarded_channels", discarded, dist.channels - seen)):
        if got is not None and got != want:
            raise CoherenceProjectionError("inconsistent_channel_support",
                                           f"Z-space coherence field '{name}' reports {got} supported channels, observed {want}")
    if dominant is not None:
        if dominant >= dist.channels:
            raise CoherenceProjectionError("dominant_out_of_range",
                                           f"dominant coherence channel {dominant} is outside {dist.channels} channels")
        dw, pk = weights[dominant], _peak(weights)
        if pk - dw > _acc_tol(dist.channels, max(abs(dw), abs(pk))):
            raise CoherenceProjectionError("inconsistent_dominant_channel",
                                           f"dominant coherence channel {dominant} has normalized weight {dw}, below observed peak {pk}")


def validate_distribution_witness(witness: DistributionWitness) -> DistributionSummary:
    for name, want in (("kind", WITNESS_KIND), ("contract_version", WITNESS_CONTRACT_VERSION), ("semantic_owner", SEMANTIC_OWNER),
                       ("semantic_backend", SEMANTIC_BACKEND), ("witness_formula", WITNESS_FORMULA)):
        got = getattr(witness, name)
        if got != want:
            raise CoherenceProjectionError("invalid_witness_contract",
                                           f"Z-space coherence distribution witness field '{name}' must be '{want}', received '{got}'")
    return summarize_distribution(witness.normalized_weights)


def validate_distribution_observation(witness: DistributionWitness, preserved_channels: int,
                                      dominant_channel: Optional[int]) -> DistributionSummary:
    dist = validate_distribution_witness(witness)
    _check_observation(witness.normalized_weights, dist, preserved_channels, None, dominant_channel)
    return dist


@dataclass(frozen=True)
class ControlPayload:
    channels: int
    raw_mean_coherence: float
    raw_coherence_entropy: float
    spectral_radius: float
    spectral_entropy: float
    spectral_pressure: float
    effective_channels: float
    energy_ratio: float
    kind: str = CONTROL_KIND
    contract_version: str = CONTROL_CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND


def derive_control(dist: DistributionSummary, energy_ratio: float, raw_mean_coherence: float) -> ControlPayload:
    if dist.channels == 0:
        raise CoherenceProjectionError("empty_channels", "Z-space coherence projection requires channel evidence")
    if dist.channels > MAX_CHANNELS:
        raise CoherenceProjectionError("channel_limit", f"Z-space coherence channel count {dist.channels} exceeds limit {MAX_CHANNELS}")
    _range("energy_ratio", energy_ratio, 0.0, 1.0)
    _range("mean_coherence", raw_mean_coherence, 0.0, 1.0)
    _range("normalized_entropy", dist.normalized_entropy, 0.0, 1.0)
    _range("concentration", dist.concentration, 0.0, 1.0)
    _range("effective_channels", dist.effective_channels, 1.0, float(dist.channels))
    _scalar("weight_mass", dist.weight_mass)
    _scalar("weight_entropy", dist.weight_entropy)
    if abs(dist.weight_mass - 1.0) > _acc_tol(dist.channels, 1.0):
        raise CoherenceProjectionError("invalid_weight_mass", f"normalized coherence weights must sum to one, received {dist.weight_mass}")
    hmax = math.log(dist.channels) if dist.channels > 1 else 0.0
    tol = _acc_tol(dist.channels, hmax)
    if dist.weight_entropy < 0 or dist.weight_entropy > hmax + tol:
        raise CoherenceProjectionError("scalar_out_of_range", f"Z-space coherence field 'weight_entropy' must lie in [0, {hmax}]")
    want_hn = min(max(dist.weight_entropy / hmax, 0.0), 1.0) if hmax > 0 else 0.0
    if abs(dist.normalized_entropy - want_hn) > tol:
        raise CoherenceProjectionError("inconsistent_distribution_metric",
                                       f"Z-space coherence distribution metric 'normalized_entropy' is inconsistent: received "
                                       f"{dist.normalized_entropy}, expected {want_hn}")
    want_eff = min(math.exp(dist.weight_entropy), float(dist.channels))
    if abs(dist.effective_channels - want_eff) > tol:
        raise CoherenceProjectionError("inconsistent_distribution_metric",
                                       f"Z-space coherence distribution metric 'effective_channels' is inconsistent: received "
                                       f"{dist.effective_channels}, expected {want_eff}")
    return ControlPayload(dist.channels, raw_mean_coherence, dist.weight_entropy, dist.concentration, dist.normalized_entropy,
                          energy_ratio * (1.0 - dist.normalized_entropy), dist.effective_channels, energy_ratio)


def is_swap_invariant(arrangement: Sequence[float]) -> bool:
    """All entries equal up to 1e-4 of the largest magnitude (floor 1e-6); empty or non-finite input is not."""
    a = [float(x) for x in arrangement]
    if not a or not all(math.isfinite(x) for x in a):
        return False
    lo, hi = min(a), max(a)
    return hi - lo <= max(max(abs(lo), abs(hi)) * 1.0e-4, _TOL_FLOOR)


@dataclass(frozen=True)
class ClassificationPolicy:
    background_energy_ratio_max: float = 1.0e-5
    cascade_energy_ratio_min: float = 0.7


@dataclass(frozen=True)
class ClassificationPayload:
    label: str
    reason: str
    energy_ratio: float
    swap_invariant: bool
    policy: ClassificationPolicy
    kind: str = CLASSIFICATION_KIND
    contract_version: str = CLASSIFICATION_CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND


def classify(energy_ratio: float, swap_invariant: bool, policy: Optional[ClassificationPolicy] = None) -> ClassificationPayload:
    """Background when the dominant channel carries (almost) no energy, symmetric pulse when all channels weigh the
    same, cascade imbalance at or above the cascade ratio, diffuse drift otherwise.  Threshold comparisons tolerate
    one relative float32 epsilon."""
    policy = policy or ClassificationPolicy()
    _range("energy_ratio", energy_ratio, 0.0, 1.0)
    _range("background_energy_ratio_max", policy.background_energy_ratio_max, 0.0, 1.0)
    _range("cascade_energy_ratio_min", policy.cascade_energy_ratio_min, 0.0, 1.0)
    if policy.background_energy_ratio_max > policy.cascade_energy_ratio_min:
        raise CoherenceProjectionError("invalid_classification_policy",
                                       f"Z-space coherence background energy-ratio maximum {policy.background_energy_ratio_max} "
                                       f"must not exceed cascade energy-ratio minimum {policy.cascade_energy_ratio_min}")
    if energy_ratio <= policy.background_energy_ratio_max or _near(energy_ratio, policy.background_energy_ratio_max):
        label, reason = "background", "energy_ratio_at_or_below_background_max"
    elif swap_invariant:
        label, reason = "symmetric_pulse", "swap_invariant"
    elif energy_ratio >= policy.cascade_energy_ratio_min or _near(energy_ratio, policy.cascade_energy_ratio_min):
        label, reason = "cascade_imbalance", "dominant_energy_ratio_at_or_above_cascade_min"
    else:
        label, reason = "diffuse_drift", "asymmetric_energy_below_cascade_ratio"
    return ClassificationPayload(label, reason, energy_ratio, swap_invariant, policy)


@dataclass
class DiagnosticsInput:
    mean_coherence: float
    coherence_entropy: float
    energy_ratio: float
    z_bias: float
    fractional_order: float
    normalized_weights: List[float] = field(default_factory=list)
    preserved_channels: Optional[int] = None
    discarded_channels: Optional[int] = None
    dominant_channel: Optional[int] = None


@dataclass
class ContourInput:
    coherence_strength: float
    prosody_index: float
    articulation_bias: float
    timbre_spread: Optional[float] = None


@dataclass
class ProjectionConfig:
    speed_gain: float = 1.0
    stability_gain: float = 1.0
    frac_gain: float = 1.0
    drs_gain: float = 1.0


@dataclass
class ProjectionDerived:
    channels: int
    distribution_source: str
    weight_mass: float
    weight_entropy: float
    normalized_entropy: float
    concentration: float
    effective_channels: float
    response_peak: float
    response_mean: float


@dataclass
class ProjectionPayload:
    diagnostics: DiagnosticsInput
    coherence: List[float]
    contour: Optional[ContourInput]
    config: ProjectionConfig
    derived: ProjectionDerived
    classification: Optional[ClassificationPayload]
    control: Optional[ControlPayload]
    partial: Dict[str, float]
    kind: str = PROJECTION_KIND
    contract_version: str = PROJECTION_CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND

    def as_dict(self) -> dict:
        return asdict(self)


def _stable_mean(values: Sequence[float]) -> float:
    """Mean with the values pre-scaled by the largest magnitude and a Neumaier-compensated sum."""
    scale = max((abs(v) for v in values), default=0.0)
    if scale == 0.0:
        return 0.0
    s = c = 0.0
    for v in values:
        v = v / scale
        t = s + v
        c += (s - t) + v if abs(s) >= abs(v) else (v - t) + s
        s = t
    return scale * min(max((s + c) / len(values), -1.0), 1.0)


def _channel_count(d: DiagnosticsInput, coherence: Sequence[float]) -> int:
    both = (d.preserved_channels + d.discarded_channels) if (d.preserved_channels is not None and d.discarded_channels is not None) else 0
    return max(both, d.preserved_channels or 0, d.discarded_channels or 0, len(d.normalized_weights), len(coherence))


def _validate(d: DiagnosticsInput, coherence, contour, config) -> Optional[DistributionSummary]:
    _range("mean_coherence", d.mean_coherence, 0.0, 1.0)
    _range("coherence_entropy", d.coherence_entropy, 0.0, 1.7976931348623157e308)
    _range("energy_ratio", d.energy_ratio, 0.0, 1.0)
    _scalar("z_bias", d.z_bias)
    _range("fractional_order", d.fractional_order, 0.0, 1.0)
    dist = summarize_distribution(d.normalized_weights) if d.normalized_weights else None
    for i, v in enumerate(coherence):
        if not math.isfinite(v):
            raise CoherenceProjectionError("non_finite_vector", f"Z-space coherence field 'coherence' entry {i} must be finite")
    for cnt in (len(d.normalized_weights), len(coherence), d.preserved_channels or 0, d.discarded_channels or 0):
        if cnt > MAX_CHANNELS:
            raise CoherenceProjectionError("channel_limit", f"Z-space coherence channel count {cnt} exceeds limit {MAX_CHANNELS}")
    for name in ("speed_gain", "stability_gain", "frac_gain", "drs_gain"):
        g = getattr(config, name)
        if not (math.isfinite(g) and g >= 0):
            raise CoherenceProjectionError("invalid_gain", f"Z-space coherence gain '{name}' must be finite and non-negative")
    if contour is not None:
        _range("coherence_strength", contour.coherence_strength, 0.0, 1.0)
        _range("prosody_index", contour.prosody_index, 0.0, 1.0)
        _range("articulation_bias", contour.articulation_bias, 0.0, 4.0)
        if contour.timbre_spread is not None:
            _range("timbre_spread", contour.timbre_spread, 0.0, 1.7976931348623157e308)
    wc, rc = len(d.normalized_weights), len(coherence)
    if wc and rc and wc != rc:
        raise CoherenceProjectionError("channel_count_mismatch", f"Z-space coherence field 'coherence' describes {rc} channels, expected {wc}")
    vec = max(wc, rc)
    complete = d.preserved_channels is not None and d.discarded_channels is not None
    if complete and vec and d.preserved_channels + d.discarded_channels != vec:
        raise CoherenceProjectionError("channel_count_mismatch",
                                       f"Z-space coherence field 'preserved_channels+discarded_channels' describes "
                                       f"{d.preserved_channels + d.discarded_channels} channels, expected {vec}")
    for name in ("preserved_channels", "discarded_channels"):
        c = getattr(d, name)
        if c is not None and vec and c > vec:
            raise CoherenceProjectionError("channel_count_mismatch", f"Z-space coherence field '{name}' describes {c} channels, expected {vec}")
    channels = _channel_count(d, coherence)
    if channels == 0:
        raise CoherenceProjectionError("empty_channels", "Z-space coherence projection requires channel evidence")
    if channels > MAX_CHANNELS:
        raise CoherenceProjectionError("channel_limit", f"Z-space coherence channel count {channels} exceeds limit {MAX_CHANNELS}")
    hmax = math.log(channels) if channels > 1 else 0.0
    if d.coherence_entropy > hmax + _acc_tol(channels, hmax):
        raise CoherenceProjectionError("entropy_above_maximum", f"coherence entropy {d.coherence_entropy} exceeds ln({channels})={hmax}")
    if d.dominant_channel is not None and d.dominant_channel >= channels:
        raise CoherenceProjectionError("dominant_out_of_range", f"dominant coherence channel {d.dominant_channel} is outside {channels} channels")
    if dist is not None:
        tol = _acc_tol(dist.channels, max(abs(d.coherence_entropy), abs(dist.weight_entropy)))
        if abs(d.coherence_entropy - dist.weight_entropy) > tol:
            raise CoherenceProjectionError("inconsistent_distribution_metric",
                                           f"Z-space coherence distribution metric 'coherence_entropy' is inconsistent: received "
                                           f"{d.coherence_entropy}, expected {dist.weight_entropy}")
        _check_observation(d.normalized_weights, dist, d.preserved_channels, d.discarded_channels, d.dominant_channel)
    if coherence:
        m = _stable_mean(coherence)
        if abs(d.mean_coherence - m) > _acc_tol(len(coherence), max(abs(d.mean_coherence), abs(m))):
            raise CoherenceProjectionError("inconsistent_distribution_metric",
                                           f"Z-space coherence distribution metric 'mean_coherence' is inconsistent: received "
                                           f"{d.mean_coherence}, expected {m}")
    return dist


def project(diagnostics: DiagnosticsInput, coherence: Sequence[float] = (), contour: Optional[ContourInput] = None,
            config: Optional[ProjectionConfig] = None, classification_policy: Optional[ClassificationPolicy] = None) -> ProjectionPayload:
    """Validates the evidence against itself (entropy, support counts, dominant channel and mean must agree with the
    normalized weights) and derives the Z-space partial.  Without normalized weights the diagnostic entropy alone
    drives the distribution controls and no classification / control payload is produced."""
    d, coherence = diagnostics, [float(v) for v in coherence]
    config = config or ProjectionConfig()
    dist = _validate(d, coherence, contour, config)
    channels = _channel_count(d, coherence)
    rmean = _stable_mean(coherence) if coherence else 0.0
    if dist is None:
        hmax = math.log(channels) if channels > 1 else 0.0
        hn = min(max(d.coherence_entropy / hmax, 0.0), 1.0) if hmax > 0 else 0.0
        derived = ProjectionDerived(channels, "diagnostic_entropy", 0.0, d.coherence_entropy, hn, 1.0 - hn,
                                    min(math.exp(d.coherence_entropy), float(channels)), _peak(coherence), rmean)
    else:
        derived = ProjectionDerived(channels, "normalized_weights", dist.weight_mass, dist.weight_entropy, dist.normalized_entropy,
                                    dist.concentration, dist.effective_channels, _peak(coherence), rmean)
    if d.normalized_weights:
        seen = sum(1 for x in d.normalized_weights if x > 0)
    elif coherence:
        seen = sum(1 for x in coherence if x > 0)
    else:
        seen = channels
    if d.preserved_channels is not None:
        preserved = d.preserved_channels
    elif d.discarded_channels is not None:
        preserved = max(channels - d.discarded_channels, 0)
    else:
        preserved = seen
    discarded = d.discarded_channels if d.discarded_channels is not None else max(channels - preserved, 0)
    partial = {
        "speed": math.tanh(config.speed_gain * derived.concentration),
        "memory": math.tanh(d.z_bias),
        "stability": math.tanh(config.stability_gain * (1.0 - 2.0 * derived.normalized_entropy)),
        "frac": math.tanh(config.frac_gain * d.fractional_order),
        "drs": math.tanh(config.drs_gain * (d.energy_ratio - 0.5)),
        "coherence_mean": d.mean_coherence, "coherence_entropy": d.coherence_entropy,
        "coherence_energy_ratio": d.energy_ratio, "coherence_z_bias": d.z_bias,
        "coherence_fractional_order": d.fractional_order, "coherence_channels": float(channels),
        "coherence_preserved": float(preserved), "coherence_discarded": float(discarded),
        "coherence_peak": _peak(d.normalized_weights), "coherence_weight_mass": derived.weight_mass,
        "coherence_weight_entropy": derived.weight_entropy, "coherence_normalized_entropy": derived.normalized_entropy,
        "coherence_entropy_residual": d.coherence_entropy - derived.weight_entropy,
        "coherence_concentration": derived.concentration, "coherence_effective_channels": derived.effective_channels,
        "coherence_response_peak": derived.response_peak, "coherence_response_mean": derived.response_mean,
    }
    if d.dominant_channel is not None:
        partial["coherence_dominant"] = float(d.dominant_channel)
    if contour is not None:
        partial["coherence_strength"] = contour.coherence_strength
        partial["coherence_prosody"] = contour.prosody_index
        partial["coherence_articulation"] = contour.articulation_bias
        if contour.timbre_spread is not None:
            partial["coherence_timbre_spread"] = contour.timbre_spread
    for k, v in partial.items():
        if not math.isfinite(v):
            raise CoherenceProjectionError("non_finite_derived", f"derived Z-space coherence metric '{k}' is not finite")
    partial = dict(sorted(partial.items()))
    classification = control = None
    if dist is not None:
        classification = classify(d.energy_ratio, is_swap_invariant(d.normalized_weights), classification_policy)
        control = derive_control(dist, d.energy_ratio, d.mean_coherence)
    return ProjectionPayload(d, coherence, contour, config, derived, classification, control, partial)
