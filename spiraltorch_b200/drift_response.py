"""Drift-response linguistics: how risky it is for a word's meaning to drift, per interpretive frame.

Parity: crates/spiral-safety/src/drift_response.rs:31-660 (`FrameState`, `WordState`,
`analyse_word_with_options`, `trainer_penalty_with`, `frame_summary`).

Each frame mixes a "denotative" and a "connotative" reading with weight `phi`; the hazard of a
frame is `c * exp(beta * H * phi * timing) * max(0, lambda*b*s - a)`, the safe radius is the smaller
of a comprehension limit `(1-tau)/kappa` and a risk limit `rho/(b*s)`.  The penalty returned by
`trainer_penalty` is a scalar a trainer adds to its loss.  Host-side scalar arithmetic only.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional


@dataclass(frozen=True)
class FrameThreshold:
    tau: float
    rho: float
    hazard: float = 1.0


@dataclass
class DirectionalAxis:
    value_components: List[float] = field(default_factory=list)
    risk_components: List[float] = field(default_factory=list)
    kappa_components: List[float] = field(default_factory=list)
    value_curvature_components: List[float] = field(default_factory=list)
    risk_curvature_components: List[float] = field(default_factory=list)
    kappa_slope_components: List[float] = field(default_factory=list)


@dataclass
class FrameState:
    phi: float = 0.0
    c: float = 0.0
    s: float = 0.0
    a_den: float = 0.0
    a_con: float = 0.0
    b_den: float = 0.0
    b_con: float = 0.0
    kappa: float = 0.0
    timing_scale: float = 1.0
    curvature_a_den: float = 0.0
    curvature_a_con: float = 0.0
    curvature_b_den: float = 0.0
    curvature_b_con: float = 0.0
    kappa_slope: float = 0.0
    directional_axes: Dict[str, DirectionalAxis] = field(default_factory=dict)

    def _mix(self, den: float, con: float) -> float:
        return (1.0 - self.phi) * den + self.phi * con

    def mix_a(self) -> float:
        return self._mix(self.a_den, self.a_con)

    def mix_b(self) -> float:
        return self._mix(self.b_den, self.b_con)

    def mix_curvature_a(self) -> float:
        return self._mix(self.curvature_a_den, self.curvature_a_con)

    def mix_curvature_b(self) -> float:
        return self._mix(self.curvature_b_den, self.curvature_b_con)


@dataclass
class WordState:
    name: str
    definition_entropy: float
    frames: Dict[str, FrameState] = field(default_factory=dict)
    timing_signal: float = 0.0
    base_lambda: float = 1.0
    beta: float = 1.0

    def with_frame(self, name: str, frame: FrameState) -> "WordState":
        self.frames[name] = frame
        return self


@dataclass
class FrameSignature:
    value_slope: float
    risk_slope: float
    net_slope: float
    value_curvature: float
    risk_curvature: float
    net_curvature: float
    hazard_multiplier: float
    timing_elasticity: float
    safe_radius: Optional[float]
    kappa_slope: float
    tipping_radius: Optional[float]


@dataclass
class DirectionalSignature(FrameSignature):
    hazard_base: float = 0.0
    hazard: float = 0.0


@dataclass
class DirectionQuery:
    axis: str
    weights: List[float]
    label: Optional[str] = None


@dataclass
class AnalysisOptions:
    hazard_cut: Optional[float] = None
    min_radius: float = 0.2
    direction_queries: Dict[str, List[DirectionQuery]] = field(default_factory=dict)


@dataclass
class DrlMetrics:
    word: WordState
    existence_load: float
    frame_hazards: Dict[str, float]
    safe_radii: Dict[str, float]
    chi: int
    strict_mode: bool
    frame_signatures: Dict[str, FrameSignature]
    direction_signatures: Dict[str, Dict[str, DirectionalSignature]] = field(default_factory=dict)


DrsMetrics = DrlMetrics


def default_thresholds() -> Dict[str, FrameThreshold]:
    return {"Physical": FrameThreshold(0.05, 0.1, 0.8), "Normative": FrameThreshold(0.1, 0.08, 0.9),
            "Social": FrameThreshold(0.15, 0.06, 0.7), "Protocol": FrameThreshold(0.02, 0.05, 0.95),
            "MetaLanguage": FrameThreshold(0.08, 0.07, 0.75), "Mythic": FrameThreshold(0.2, 0.05, 0.6)}


def _hazard_multiplier(word: WordState, frame: FrameState) -> float:
    timing = max(word.timing_signal * frame.timing_scale, 0.0)
    if timing == 0.0 or word.definition_entropy == 0.0 or frame.phi == 0.0:
        return 1.0
    return math.exp(min(max(word.beta * word.definition_entropy * frame.phi * timing, -30.0), 30.0))


def _timing_elasticity(word: WordState, frame: FrameState, multiplier: float) -> float:
    return multiplier * word.beta * word.definition_entropy * frame.phi * frame.timing_scale


def _tipping_radius(net_slope: float, net_curvature: float) -> Optional[float]:
    if abs(net_curvature) < 1e-9:
        return None
    t = -net_slope / net_curvature
    return t if t > 0.0 else None


def _hazard_base(word: WordState, frame: FrameState) -> float:
    return max(0.0, -(frame.mix_a() - word.base_lambda * frame.mix_b() * frame.s))


def frame_hazard(word: WordState, frame: FrameState) -> float:
    base = _hazard_base(word, frame)
    return 0.0 if base == 0.0 else frame.c * _hazard_multiplier(word, frame) * base


def existence_load(word: WordState) -> float:
    return sum(f.c * _hazard_base(word, f) * (1.0 + word.beta * word.definition_entropy * f.phi)
               for f in word.frames.values())


def _radius(tau: float, rho: float, kappa: float, risk: float) -> float:
    return min((1.0 - tau) / max(kappa, 1e-6), rho / max(risk, 1e-9))


def safe_radius(word: WordState, thresholds: Dict[str, FrameThreshold]) -> Dict[str, float]:
    return {n: _radius(thresholds[n].tau, thresholds[n].rho, f.kappa, f.mix_b() * f.s)
            for n, f in sorted(word.frames.items()) if n in thresholds}


def _dot(components: List[float], weights: List[float]) -> Optional[float]:
    if not components or len(components) != len(weights):
        return None
    return sum(c * w for c, w in zip(components, weights))


def _or(value: Optional[float], default: float) -> float:
    return default if value is None else value


def _directional_signature(word: WordState, frame: FrameState, axis: DirectionalAxis, weights: List[float],
                           threshold: Optional[FrameThreshold]) -> DirectionalSignature:
    value_slope = _or(_dot(axis.value_components, weights), frame.mix_a())
    risk_linear = _or(_dot(axis.risk_components, weights), frame.mix_b())
    risk_slope = word.base_lambda * risk_linear * frame.s
    value_curv = _or(_dot(axis.value_curvature_components, weights), frame.mix_curvature_a())
    risk_curv = word.base_lambda * _or(_dot(axis.risk_curvature_components, weights), frame.mix_curvature_b()) * frame.s
    mult = _hazard_multiplier(word, frame)
    base = max(0.0, risk_slope - value_slope)
    kappa = _or(_dot(axis.kappa_components, weights), frame.kappa)
    radius = None if threshold is None else _radius(threshold.tau, threshold.rho, kappa, abs(risk_linear) * frame.s)
    net_slope, net_curv = value_slope - risk_slope, value_curv - risk_curv
    return DirectionalSignature(value_slope, risk_slope, net_slope, value_curv, risk_curv, net_curv, mult,
                                _timing_elasticity(word, frame, mult), radius,
                                _or(_dot(axis.kappa_slope_components, weights), frame.kappa_slope),
                                _tipping_radius(net_slope, net_curv), hazard_base=base, hazard=frame.c * mult * base)


def analyse_word(word: WordState, thresholds: Optional[Dict[str, FrameThreshold]] = None,
                 options: Optional[AnalysisOptions] = None) -> DrlMetrics:
    """Hazards, safe radii, slope/curvature signatures and the strict-mode flag for one word."""
    thresholds = default_thresholds() if thresholds is None else thresholds
    options = options or AnalysisOptions()
    hazards, sigs = {}, {}
    for name, f in sorted(word.frames.items()):
        hazards[name] = frame_hazard(word, f)
        vs, rs = f.mix_a(), word.base_lambda * f.mix_b() * f.s
        vc, rc = f.mix_curvature_a(), word.base_lambda * f.mix_curvature_b() * f.s
        mult = _hazard_multiplier(word, f)
        sigs[name] = FrameSignature(vs, rs, vs - rs, vc, rc, vc - rc, mult, _timing_elasticity(word, f, mult), None,
                                    f.kappa_slope, _tipping_radius(vs - rs, vc - rc))
    radii = safe_radius(word, thresholds)
    for name, r in radii.items():
        sigs[name].safe_radius = r
    chi = sum(1 for n, h in hazards.items()
              if n in thresholds and h >= (thresholds[n].hazard if options.hazard_cut is None else options.hazard_cut))
    load = existence_load(word)
    strict = chi >= 4 or min(radii.values(), default=math.inf) <= options.min_radius or load >= 1.0
    directions: Dict[str, Dict[str, DirectionalSignature]] = {}
    for fname, queries in sorted(options.direction_queries.items()):
        f = word.frames.get(fname)
        if f is None or not f.directional_axes:
            continue
        got = {q.label or q.axis: _directional_signature(word, f, f.directional_axes[q.axis], q.weights, thresholds.get(fname))
               for q in queries if q.axis in f.directional_axes}
        if got:
            directions[fname] = got
    return DrlMetrics(word, load, hazards, radii, chi, strict, sigs, directions)


def analyse_word_with(word: WordState, thresholds: Dict[str, FrameThreshold], hazard_cut: Optional[float],
                      min_radius: float) -> DrlMetrics:
    return analyse_word(word, thresholds, AnalysisOptions(hazard_cut, min_radius))


analyse_word_with_options = analyse_word


def _shortfall(value: Optional[float], min_radius: float) -> float:
    if value is None or value >= min_radius:
        return 0.0
    return (min_radius - value) / max(min_radius, 1e-6)


def trainer_penalty(metrics: DrlMetrics, min_radius: float = 0.2) -> float:
    """Existence load + hazard count + shortfalls of the smallest safe / tipping radii below
    `min_radius` (frames, then queried directions); x1.25 in strict mode."""
    p = metrics.existence_load + float(metrics.chi)
    p += _shortfall(min(metrics.safe_radii.values(), default=None), min_radius)
    tips = [s.tipping_radius for s in metrics.frame_signatures.values() if s.tipping_radius and s.tipping_radius > 0]
    p += _shortfall(min(tips, default=None), min_radius)
    dirs = [s for m in metrics.direction_signatures.values() for s in m.values()]
    p += _shortfall(min((s.safe_radius for s in dirs if s.safe_radius is not None), default=None), min_radius)
    p += _shortfall(min((s.tipping_radius for s in dirs if s.tipping_radius and s.tipping_radius > 0), default=None),
                    min_radius)
    return p * 1.25 if metrics.strict_mode else p


trainer_penalty_with = trainer_penalty


def aggregate_penalty(metrics: Iterable[DrlMetrics], min_radius: float = 0.2) -> float:
    return sum(trainer_penalty(m, min_radius) for m in metrics)


aggregate_penalty_with = aggregate_penalty


def frame_summary(metrics: DrlMetrics) -> Dict[str, float]:
    """Hazard per unit of safe radius for every frame (plain hazard where no radius is known)."""
    return {n: (h / max(metrics.safe_radii[n], 1e-6) if n in metrics.safe_radii else h)
            for n, h in metrics.frame_hazards.items()}
