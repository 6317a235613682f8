"""Z-space meta-optimizer: an Adam walk of a small control vector ``z`` driven by observed training metrics, a
fractional spectral regulariser on ``z`` and topos telemetry that scales the learning rate, clips and biases the
gradient; every step returns a report that can be turned into a learning-rate control for the parameter optimizers.

Parity: crates/st-core/src/runtime/zspace_optimizer.rs — config / state / observation (:83-245), checkpoints and
restore (:783-820, 1810-1842), `transition_zspace_meta_optimizer` (:821-1059), fractional regulariser (:1843-1961),
topos control (:1963-2140), gradient projection / RMS / objective (:2142-2245), parameter control (:1081-1243); the
gradient bias basis / amplitude / clip threshold come from crates/st-tensor/src/pure/topos.rs:609-657.

Rules (all in float64; the vector has at most 4096 entries, so this is host arithmetic by design):
  objective  ``J = sum_i lambda_i tanh(metric_i) + gain tanh(topos pressure) + lambda_frac_eff R_alpha(z)``
  regulariser ``R_alpha(z) = mean_k ((k / k_max)^(2 alpha) |DFT(z)_k|^2)`` over the one-sided spectrum
  gradient   ``g = clip_rms(bias_rms(project(tanh(g_observed)) + lambda_frac_eff normalised(dR/dz)))``
  update     ``z <- z - lr_eff m_hat / (sqrt(v_hat) + eps)``
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch

CONTRACT_VERSION = "spiraltorch.zspace_meta_optimizer.v2"
KIND = "spiraltorch.zspace_meta_optimizer"
SEMANTIC_OWNER = "st-core::runtime::zspace_optimizer"
SEMANTIC_BACKEND = "rust"             # wire value consumers compare against
PARAMETER_CONTROL_KIND = "spiraltorch.zspace_parameter_control"
PARAMETER_CONTROL_CONTRACT_VERSION = "spiraltorch.zspace_parameter_control.v1"
MAX_DIMENSION = 4096
MAX_SAFE_STEP = 9_007_199_254_740_991
MIN_LR_SCALE, MAX_LR_SCALE = 0.1, 1.25
_TOL = 128.0 * 2.220446049250313e-16
_TOPOS_KEYS = ("closure_pressure", "depth_pressure", "volume_pressure", "guard_strength", "training_hints.step_damping", "step_damping",
               "sampling_focus", "openness", "exploration_hint", "training_hints.learning_rate_scale", "learning_rate_scale",
               "training_hints.clip_scale", "clip_scale", "training_hints.regularization_scale", "regularization_scale",
               "training_hints.gradient_bias_scale", "gradient_bias_scale")


class ZSpaceMetaOptimizerError(ValueError):
    def __init__(self, code: str, message: str):
        super().__init__(message)
        self.code = code


def _finite(name: str, v: float) -> float:
    if not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ZSpaceMetaOptimizerError("non_finite", f"'{name}' must be finite, got {v}")
    return float(v)


def _positive(name: str, v: float) -> float:
    if _finite(name, v) <= 0:
        raise ZSpaceMetaOptimizerError("non_positive", f"'{name}' must be positive, got {v}")
    return float(v)


def _non_negative(name: str, v: float) -> float:
    if _finite(name, v) < 0:
        raise ZSpaceMetaOptimizerError("negative", f"'{name}' must be non-negative, got {v}")
    return float(v)


def _vector(name: str, values) -> List[float]:
    out = [float(v) for v in values]
    for i, v in enumerate(out):
        if not math.isfinite(v):
            raise ZSpaceMetaOptimizerError("non_finite", f"'{name}[{i}]' must be finite, got {v}")
    return out


@dataclass
class Weights:
    speed: float = 0.5
    memory: float = 0.3
    stability: float = 0.2
    fractional: float = 0.1
    drift_response: float = 0.0


@dataclass
class Config:
    dimension: int = 4
    fractional_order: float = 0.35
    weights: Weights = field(default_factory=Weights)
    learning_rate: float = 1.0e-2
    first_moment_decay: float = 0.9
    second_moment_decay: float = 0.999
    epsilon: float = 1.0e-8
    topos_control_gain: float = 0.0
    gradient_projection: str = "tile_or_truncate"          # or "exact"

    def validate(self) -> None:
        if self.dimension <= 0:
            raise ZSpaceMetaOptimizerError("invalid_dimension", f"dimension must be positive, got {self.dimension}")
        if self.dimension > MAX_DIMENSION:
            raise ZSpaceMetaOptimizerError("dimension_limit", f"dimension {self.dimension} exceeds {MAX_DIMENSION}")
        _positive("config.fractional_order", self.fractional_order)
        for k, v in asdict(self.weights).items():
            _non_negative(f"config.weights.{k}", v)
        _positive("config.learning_rate", self.learning_rate)
        for name in ("first_moment_decay", "second_moment_decay"):
            v = _finite(f"config.{name}", getattr(self, name))
            if not 0.0 <= v < 1.0:
                raise ZSpaceMetaOptimizerError("invalid_decay", f"'config.{name}' must lie in [0, 1), got {v}")
        _positive("config.epsilon", self.epsilon)
        _non_negative("config.topos_control_gain", self.topos_control_gain)
        if self.gradient_projection not in ("tile_or_truncate", "exact"):
            raise ZSpaceMetaOptimizerError("invalid_projection", f"unknown gradient projection '{self.gradient_projection}'")

    @classmethod
    def from_dict(cls, d: dict) -> "Config":
        alias = {"alpha": "fractional_order", "lr": "learning_rate", "beta1": "first_moment_decay", "beta2": "second_moment_decay",
                 "eps": "epsilon"}
        d = {alias.get(k, k): v for k, v in d.items()}
        known = set(cls.__dataclass_fields__)
        extra = set(d) - known
        if extra:
            raise ZSpaceMetaOptimizerError("unknown_field", f"unknown config field(s): {sorted(extra)}")
        if isinstance(d.get("weights"), dict):
            w = {("drift_response" if k == "drs" else k): v for k, v in d["weights"].items()}
            d = {**d, "weights": Weights(**w)}
        return cls(**d)


@dataclass
class State:
    z: List[float] = field(default_factory=list)
    first_moment: List[float] = field(default_factory=list)
    second_moment: List[float] = field(default_factory=list)
    step: int = 0

    @classmethod
    def zeros(cls, dimension: int) -> "State":
        return cls([0.0] * dimension, [0.0] * dimension, [0.0] * dimension, 0)

    def validate_values(self) -> None:
        self.z, self.first_moment = _vector("state.z", self.z), _vector("state.first_moment", self.first_moment)
        self.second_moment = _vector("state.second_moment", self.second_moment)
        for i, v in enumerate(self.second_moment):
            if v < 0:
                raise ZSpaceMetaOptimizerError("negative_second_moment", f"second moment {i} is negative ({v})")
        if not 0 <= self.step <= MAX_SAFE_STEP:
            raise ZSpaceMetaOptimizerError("step_limit", f"step {self.step} outside [0, {MAX_SAFE_STEP}]")

    def validate(self, dimension: int) -> None:
        for name in ("z", "first_moment", "second_moment"):
            if len(getattr(self, name)) != dimension:
                raise ZSpaceMetaOptimizerError("state_length", f"'state.{name}' has {len(getattr(self, name))} entries, expected {dimension}")
        self.validate_values()


@dataclass
class Observation:
    speed: float = 0.0
    memory: float = 0.0
    stability: float = 0.0
    drift_response: float = 0.0
    gradient: List[float] = field(default_factory=list)
    telemetry: Dict[str, float] = field(default_factory=dict)

    def validate(self) -> None:
        for name in ("speed", "memory", "stability", "drift_response"):
            _finite(f"observation.{name}", getattr(self, name))
        self.gradient = _vector("observation.gradient", self.gradient)
        for k, v in self.telemetry.items():
            _finite(f"observation.telemetry.{k}", v)


def checkpoint(config: Config, state: State) -> dict:
    return {"contract_version": CONTRACT_VERSION, "kind": KIND, "semantic_owner": SEMANTIC_OWNER, "semantic_backend": SEMANTIC_BACKEND,
            "config": asdict(config), "state": asdict(state)}


def initialize(config: Config) -> dict:
    config.validate()
    return checkpoint(config, State.zeros(config.dimension))


def restore(config: Config, state: State, strict: bool = True) -> dict:
    """Non-strict restore pads with zeros or truncates to the configured dimension, but never accepts invalid values,
    not even in a tail it would discard."""
    config.validate()
    state.validate_values()
    n = config.dimension
    out = {}
    for name in ("z", "first_moment", "second_moment"):
        v = list(getattr(state, name))
        if strict and len(v) != n:
            raise ZSpaceMetaOptimizerError("state_length", f"'state.{name}' has {len(v)} entries, expected {n}")
        out[name] = (v + [0.0] * n)[:n]
    new = State(out["z"], out["first_moment"], out["second_moment"], state.step)
    new.validate(n)
    return checkpoint(config, new)


# ---- fractional regulariser ---------------------------------------------------------------------------------------------
def fractional_regularizer(z, order: float) -> dict:
    """Energy ``R_alpha(z)`` and its gradient (raw, and divided by ``max(1, max |raw|)``).  The gradient is evaluated
    with a second forward DFT of the weighted conjugate spectrum, ``dR/dz_j = (2 / bins) Re DFT(w conj(Z))_j``."""
    z = _vector("state.z", z)
    _positive("config.fractional_order", order)
    n = len(z)
    if n == 0:
        raise ZSpaceMetaOptimizerError("invalid_dimension", "fractional regulariser needs a non-empty signal")
    if n > MAX_DIMENSION:
        raise ZSpaceMetaOptimizerError("dimension_limit", f"signal length {n} exceeds {MAX_DIMENSION}")
    bins = n // 2 + 1
    if n <= 1 or bins <= 1:
        return {"order": order, "signal_length": n, "spectral_bins": bins, "energy": 0.0, "raw_gradient": [0.0] * n,
                "gradient_normalization_scale": 1.0, "normalized_gradient": [0.0] * n}
    spec = torch.fft.fft(torch.tensor(z, dtype=torch.float64))
    k = torch.arange(bins, dtype=torch.float64)
    w = (k / (bins - 1)) ** (2.0 * order)
    one_sided = spec[:bins]
    energy = float((w * (one_sided.real ** 2 + one_sided.imag ** 2)).sum() / bins)
    gspec = torch.zeros(n, dtype=torch.complex128)
    gspec[:bins] = torch.complex(w * one_sided.real, -w * one_sided.imag)
    raw = (torch.fft.fft(gspec).real * (2.0 / bins)).tolist()
    scale = max([1.0] + [abs(v) for v in raw])
    if not math.isfinite(energy) or not all(math.isfinite(v) for v in raw):
        raise ZSpaceMetaOptimizerError("non_finite_derived", "fractional regulariser overflowed")
    return {"order": order, "signal_length": n, "spectral_bins": bins, "energy": energy, "raw_gradient": raw,
            "gradient_normalization_scale": scale, "normalized_gradient": [v / scale for v in raw]}


# ---- topos control ------------------------------------------------------------------------------------------------------
def _cl(v, lo, hi):
    return min(max(v, lo), hi)


def gradient_bias_basis(closure, volume, depth, guard, damping, focus, lr_hint, reg_scale, openness, exploration) -> List[float]:
    return [closure - 0.5, volume - 0.5, depth - 0.5, guard - 0.5, damping - 0.5, focus - 0.5, 1.0 - lr_hint, reg_scale - 1.0,
            0.5 - openness, 0.5 - exploration]


def gradient_clip_threshold(biased_rms: float, clip_scale: float) -> Optional[float]:
    """``rms / (1 - clip_scale)``; a scale of one disables clipping."""
    return biased_rms / (1.0 - clip_scale) if clip_scale < 1.0 else None


def resolve_topos_control(config: Config, telemetry: Dict[str, float], fractional_weight: float) -> dict:
    """Reads ``topos.*`` telemetry.  Without any such key, or with zero gain, every scale is neutral.  Otherwise each
    scale is ``1 + gain (hint - 1)`` clamped to its window: learning rate [0.1, 1.25], clip [0.25, 1], regularisation
    [0.25, 4]; the gradient-bias scale is ``gain * clamp(hint, 0, 0.35)``."""
    get = lambda k: telemetry.get(f"topos.{k}")                                         # noqa: E731
    unit = lambda k: None if get(k) is None else _cl(get(k), 0.0, 1.0)                  # noqa: E731
    first = lambda *ks: next((get(k) for k in ks if get(k) is not None), None)          # noqa: E731
    present = any(get(k) is not None for k in _TOPOS_KEYS)
    gain = config.topos_control_gain
    closure, depth, volume = unit("closure_pressure") or 0.0, unit("depth_pressure") or 0.0, unit("volume_pressure") or 0.0
    guard = unit("guard_strength") if unit("guard_strength") is not None else closure
    d = first("training_hints.step_damping", "step_damping")
    damping = _cl(d, 0.0, 1.0) if d is not None else closure * guard
    focus = unit("sampling_focus") if unit("sampling_focus") is not None else guard
    openness = unit("openness") if unit("openness") is not None else _cl(1.0 - closure, 0.0, 1.0)
    exploration = unit("exploration_hint") or 0.0
    raw_lr = first("training_hints.learning_rate_scale", "learning_rate_scale")
    raw_clip = first("training_hints.clip_scale", "clip_scale")
    raw_reg = first("training_hints.regularization_scale", "regularization_scale")
    raw_bias = first("training_hints.gradient_bias_scale", "gradient_bias_scale")
    pressure = max(closure, depth, volume, guard, damping, focus) if present else 0.0
    active = present and gain > 0.0
    blend = lambda hint, lo, hi: _cl(1.0 + gain * (hint - 1.0), lo, hi)               # noqa: E731
    lr_hint = _cl(1.0 if raw_lr is None else raw_lr, 0.1, 1.25)
    lr_scale = blend(lr_hint, 0.1, 1.25) if active else 1.0
    clip_hint = _cl(1.0 if raw_clip is None else raw_clip, 0.25, 1.0)
    clip_scale = blend(clip_hint, 0.25, 1.0) if active else 1.0
    reg_hint = _cl(1.0 if raw_reg is None else raw_reg, 0.25, 4.0)
    reg_scale = blend(reg_hint, 0.25, 4.0) if active else 1.0
    bias_scale = _cl(0.05 if raw_bias is None else raw_bias, 0.0, 0.35) * gain if active else 0.0
    return {"present": present, "active": active, "closure_pressure": closure, "depth_pressure": depth, "volume_pressure": volume,
            "guard_strength": guard, "step_damping": damping, "sampling_focus": focus, "openness": openness,
            "exploration_hint": exploration, "pressure": pressure, "learning_rate_hint": lr_hint, "learning_rate_scale": lr_scale,
            "effective_learning_rate": _positive("topos.effective_learning_rate", config.learning_rate * lr_scale),
            "clip_hint": clip_hint, "clip_scale": clip_scale, "regularization_hint": reg_hint, "regularization_scale": reg_scale,
            "effective_fractional_weight": fractional_weight * reg_scale, "gradient_bias_scale": bias_scale,
            "gradient_bias_basis": gradient_bias_basis(closure, volume, depth, guard, damping, focus, lr_hint, reg_scale, openness, exploration),
            "raw_gradient_rms": 0.0, "gradient_bias_amplitude": 0.0, "gradient_bias": [0.0] * config.dimension,
            "biased_gradient_rms": 0.0, "gradient_clip_threshold": None}


def project_observed_gradient(gradient: List[float], dimension: int, projection: str) -> List[float]:
    """``tanh`` of the observed gradient, tiled or truncated to ``dimension`` (``exact`` demands equal length)."""
    if projection == "exact" and len(gradient) != dimension:
        raise ZSpaceMetaOptimizerError("gradient_length", f"gradient has {len(gradient)} entries, expected {dimension}")
    if not gradient:
        return [0.0] * dimension
    return [math.tanh(gradient[i % len(gradient)]) for i in range(dimension)]


def _rms(v: List[float]) -> float:
    return math.sqrt(sum(x * x for x in v) / len(v)) if v else 0.0


def _bias_correction(decay: float, step: int) -> float:
    return 1.0 if decay == 0.0 else -math.expm1(math.log(decay) * step)


def transition(config: Config, state: State, observation: Observation) -> dict:
    """One validated step; returns the full report (``state_after`` inside).  Nothing is mutated."""
    config.validate()
    state.validate(config.dimension)
    observation.validate()
    n = config.dimension
    frac = fractional_regularizer(state.z, config.fractional_order)
    topos = resolve_topos_control(config, observation.telemetry, config.weights.fractional)
    projected = project_observed_gradient(observation.gradient, n, config.gradient_projection)
    regularized = [p + topos["effective_fractional_weight"] * g for p, g in zip(projected, frac["normalized_gradient"])]
    raw_rms = _rms(regularized)
    amp = raw_rms * topos["gradient_bias_scale"]
    basis = topos["gradient_bias_basis"]
    bias = [amp * basis[i % len(basis)] for i in range(n)]
    before_clip = [r + b for r, b in zip(regularized, bias)]
    biased_rms = _rms(before_clip)
    threshold = gradient_clip_threshold(biased_rms, topos["clip_scale"])
    applied = before_clip if threshold is None else [_cl(v, -threshold, threshold) for v in before_clip]
    clipped = sum(1 for a, b in zip(applied, before_clip) if a != b)
    topos.update(raw_gradient_rms=raw_rms, gradient_bias_amplitude=amp, gradient_bias=bias, biased_gradient_rms=biased_rms,
                 gradient_clip_threshold=threshold)
    step = state.step + 1
    if step > MAX_SAFE_STEP:
        raise ZSpaceMetaOptimizerError("step_limit", f"step {step} exceeds {MAX_SAFE_STEP}")
    b1, b2 = config.first_moment_decay, config.second_moment_decay
    c1, c2 = _bias_correction(b1, step), _bias_correction(b2, step)
    lr = topos["effective_learning_rate"]
    m = [b1 * mi + (1.0 - b1) * g for mi, g in zip(state.first_moment, applied)]
    v = [b2 * vi + (1.0 - b2) * g * g for vi, g in zip(state.second_moment, applied)]
    delta = [-(lr * (mi / c1)) / (math.sqrt(vi / c2) + config.epsilon) for mi, vi in zip(m, v)]
    z = [zi + d for zi, d in zip(state.z, delta)]
    after = State(z, m, v, step)
    after.validate(n)
    for i in range(n):                                              # the reported delta must reproduce the state change
        scale = max(abs(state.z[i]), abs(z[i]), abs(delta[i]), 1.0)
        if abs((z[i] - state.z[i]) - delta[i]) > _TOL * scale:
            raise ZSpaceMetaOptimizerError("invariant_violation", f"parameter delta {i} does not reproduce the state change")
    w = config.weights
    terms = {"speed_term": w.speed * math.tanh(observation.speed), "memory_term": w.memory * math.tanh(observation.memory),
             "stability_term": w.stability * math.tanh(observation.stability),
             "drift_response_term": w.drift_response * math.tanh(observation.drift_response),
             "topos_term": config.topos_control_gain * math.tanh(topos["pressure"])}
    penalty = sum(terms.values())
    frac_term = topos["effective_fractional_weight"] * frac["energy"]
    objective = {**terms, "fractional_term": frac_term, "observed_resource_penalty": penalty, "objective_before": penalty + frac_term}
    return {"contract_version": CONTRACT_VERSION, "kind": KIND, "semantic_owner": SEMANTIC_OWNER, "semantic_backend": SEMANTIC_BACKEND,
            "transition_validated": True, "config": asdict(config), "observation": asdict(observation), "objective": objective,
            "fractional_regularizer": frac, "topos_control": topos,
            "gradient": {"source_dimension": len(observation.gradient), "target_dimension": n, "projection": config.gradient_projection,
                         "observed": list(observation.gradient), "projected_normalized": projected, "before_clip": before_clip,
                         "applied": applied, "clipped_values": clipped},
            "adam": {"step": step, "first_moment_bias_correction": c1, "second_moment_bias_correction": c2,
                     "effective_learning_rate": lr, "parameter_delta": delta},
            "state_before": asdict(state), "state_after": asdict(after)}


@dataclass(frozen=True)
class ParameterControl:
    source_step: int
    absolute_learning_rate_scale: float
    source_learning_rate: float
    source_effective_learning_rate: float
    kind: str = PARAMETER_CONTROL_KIND
    contract_version: str = PARAMETER_CONTROL_CONTRACT_VERSION
    source_contract_version: str = CONTRACT_VERSION


def parameter_control_from_report(report: dict) -> ParameterControl:
    """The learning-rate scale a report grants to the parameter optimizers — accepted only when the report carries this
    contract's identity, was validated, and its scale, effective learning rates and step counters re-derive from its
    own config and telemetry."""
    for key, want in (("contract_version", CONTRACT_VERSION), ("kind", KIND), ("semantic_owner", SEMANTIC_OWNER),
                      ("semantic_backend", SEMANTIC_BACKEND)):
        if report.get(key) != want:
            raise ZSpaceMetaOptimizerError("contract_field", f"report.{key} must be '{want}', got {report.get(key)!r}")
    if report.get("transition_validated") is not True:
        raise ZSpaceMetaOptimizerError("unvalidated_transition", "the report does not come from a validated transition")
    try:
        config = Config.from_dict(report["config"])
        obs = Observation(**report["observation"])
        scale = float(report["topos_control"]["learning_rate_scale"])
        topos_lr, adam_lr = float(report["topos_control"]["effective_learning_rate"]), float(report["adam"]["effective_learning_rate"])
        before, after, adam_step = int(report["state_before"]["step"]), int(report["state_after"]["step"]), int(report["adam"]["step"])
    except (KeyError, TypeError, ValueError) as exc:
        raise ZSpaceMetaOptimizerError("malformed_report", f"malformed report: {exc}") from exc
    config.validate()
    obs.validate()
    canonical = resolve_topos_control(config, obs.telemetry, config.weights.fractional)["learning_rate_scale"]

    def same(name, actual, expected):
        if not math.isfinite(actual) or abs(actual - expected) > _TOL * max(abs(actual), abs(expected), 1.0):
            raise ZSpaceMetaOptimizerError("invariant_violation", f"'{name}' is {actual}, expected {expected}")
    same("topos_control.learning_rate_scale", scale, canonical)
    if not MIN_LR_SCALE <= scale <= MAX_LR_SCALE:
        raise ZSpaceMetaOptimizerError("scale_out_of_range", f"learning-rate scale {scale} outside [{MIN_LR_SCALE}, {MAX_LR_SCALE}]")
    if before + 1 != after or after != adam_step:
        raise ZSpaceMetaOptimizerError("inconsistent_step", f"steps before={before} after={after} adam={adam_step} do not line up")
    if after > MAX_SAFE_STEP:
        raise ZSpaceMetaOptimizerError("step_limit", f"step {after} exceeds {MAX_SAFE_STEP}")
    expected = config.learning_rate * scale
    same("topos_control.effective_learning_rate", topos_lr, expected)
    same("adam.effective_learning_rate", adam_lr, expected)
    return ParameterControl(after, scale, config.learning_rate, expected)


class ZSpaceMetaOptimizer:
    def __init__(self, config: Optional[Config] = None):
        self.config = config or Config()
        self.config.validate()
        self.state = State.zeros(self.config.dimension)
        self.last_report: Optional[dict] = None

    @classmethod
    def from_checkpoint(cls, ck: dict, strict: bool = True) -> "ZSpaceMetaOptimizer":
        for key, want in (("contract_version", CONTRACT_VERSION), ("kind", KIND)):
            if ck.get(key) != want:
                raise ZSpaceMetaOptimizerError("contract_field", f"checkpoint.{key} must be '{want}', got {ck.get(key)!r}")
        config = Config.from_dict(ck["config"])
        restored = restore(config, State(**ck["state"]), strict)
        opt = cls(config)
        opt.state = State(**restored["state"])
        return opt

    def checkpoint(self) -> dict:
        return checkpoint(self.config, self.state)

    def reset(self) -> None:
        self.state, self.last_report = State.zeros(self.config.dimension), None

    def try_step(self, observation: Observation) -> dict:
        """Commits the new state only after the whole transition validated."""
        report = transition(self.config, self.state, observation)
        self.state = State(**report["state_after"])
        self.last_report = report
        return report

    def parameter_control(self) -> Optional[ParameterControl]:
        return None if self.last_report is None else parameter_control_from_report(self.last_report)
