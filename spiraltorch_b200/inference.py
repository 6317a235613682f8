"""Inference-side controllers: concept diffusion on a tag graph and free-energy scoring of
band energies.

Parity: crates/st-core/src/inference/concept_diffusion.rs:27-1000 (`ConceptDiffusionConfig`,
`blend_concept_diffusion_observation`, `apply_concept_diffusion` and its invariants),
crates/st-core/src/heur/free_energy.rs:38-800 (`BandEnergy`, `BandPrior`, `evaluate_free_energy`,
`score_with_free_energy`).

A diffusion step is `p <- p - dt * (deg * p - C p)` on the conductance graph `C = affinity * tensor`,
run as CFL-limited sub-steps; each sub-step is one matrix-vector product in float64 on the state's
device, so a graph of a few thousand concept tags steps on the GPU without a host loop over edges.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

_TOL = 1e-12


class ConceptDiffusionError(ValueError):
    pass


def concept_probability_sum_tolerance(n: int) -> float:
    return 1e-9 * max(1.0, math.sqrt(max(n, 1)))


@dataclass(frozen=True)
class ConceptDiffusionConfig:
    timestep: float = 1e-2
    cfl_limit: float = 0.9
    max_substeps: int = 4096
    symmetry_tolerance: float = 1e-10

    def __post_init__(self):
        self.validate()

    def validate(self) -> None:
        if not math.isfinite(self.timestep) or self.timestep < 0:
            raise ConceptDiffusionError(f"timestep must be finite and >= 0, got {self.timestep}")
        if not math.isfinite(self.cfl_limit) or not 0 < self.cfl_limit <= 1:
            raise ConceptDiffusionError(f"cfl_limit must lie in (0, 1], got {self.cfl_limit}")
        if self.max_substeps <= 0:
            raise ConceptDiffusionError("max_substeps must be positive")
        if not math.isfinite(self.symmetry_tolerance) or self.symmetry_tolerance < 0:
            raise ConceptDiffusionError("symmetry_tolerance must be finite and >= 0")


@dataclass
class ConceptDiffusionObservation:
    probabilities: Sequence[float]
    weight: float


@dataclass
class ConceptDiffusionEffects:
    observation_provided: bool
    observation_applied: bool
    observation_weight: float
    z_bias_applied: bool
    diffusion_applied: bool
    edge_count: int
    substeps: int
    substep_timestep: float
    max_degree: float
    entropy_before: float
    entropy_after_observation: float
    entropy_after_bias: float
    entropy_after_diffusion: float
    dirichlet_energy_before: float
    dirichlet_energy_after: float
    total_variation: float


@dataclass
class ConceptDiffusionPayload:
    tags: List[str]
    previous_state: torch.Tensor
    state_after_observation: torch.Tensor
    state_after_bias: torch.Tensor
    next_state: torch.Tensor
    input_probability_sum: float
    output_probability_sum: float
    conductivity_source: str
    effects: ConceptDiffusionEffects
    config: ConceptDiffusionConfig
    kind: str = "spiraltorch.zspace_concept_diffusion"
    contract_version: str = "v1"


def _distribution(name: str, values, n: Optional[int] = None, device=None) -> tuple:
    p = torch.as_tensor(values, dtype=torch.float64, device=device).flatten()
    if p.numel() == 0:
        raise ConceptDiffusionError(f"{name} must not be empty")
    if n is not None and p.numel() != n:
        raise ConceptDiffusionError(f"{name} has {p.numel()} entries, expected {n}")
    if not bool(torch.isfinite(p).all()):
        raise ConceptDiffusionError(f"{name} contains a non-finite value")
    if bool((p < 0).any()):
        raise ConceptDiffusionError(f"{name} contains a negative value")
    s = float(p.sum())
    if abs(s - 1.0) > concept_probability_sum_tolerance(p.numel()):
        raise ConceptDiffusionError(f"{name} sums to {s}, expected 1")
    return p / s, s


def _matrix(name: str, m, n: int, tol: float, device) -> torch.Tensor:
    a = torch.as_tensor(m, dtype=torch.float64, device=device)
    if a.shape != (n, n):
        raise ConceptDiffusionError(f"{name} has shape {tuple(a.shape)}, expected ({n}, {n})")
    if not bool(torch.isfinite(a).all()):
        raise ConceptDiffusionError(f"{name} contains a non-finite value")
    if bool((a < 0).any()):
        raise ConceptDiffusionError(f"{name} contains a negative value")
    if float((a - a.T).abs().max()) > tol * (1.0 + float(a.abs().max())):
        raise ConceptDiffusionError(f"{name} is not symmetric")
    return a


def _entropy(p: torch.Tensor) -> float:
    q = p[p > 0]
    return float(-(q * torch.log(q)).sum())


def _dirichlet(p: torch.Tensor, c: torch.Tensor) -> float:
    d = p[:, None] - p[None, :]
    return float(0.5 * (c * d * d).sum())


def blend_concept_diffusion_observation(state, observation: ConceptDiffusionObservation) -> torch.Tensor:
    """`(1 - w) * state + w * observed`, renormalised; `w` must lie in [0, 1]."""
    p, _ = _distribution("state", state)
    o, _ = _distribution("observation_probability", observation.probabilities, p.numel(), p.device)
    w = observation.weight
    if not math.isfinite(w) or not 0 <= w <= 1:
        raise ConceptDiffusionError(f"observation_weight must lie in [0, 1], got {w}")
    b = (1 - w) * p + w * o
    return b / b.sum()


def apply_concept_diffusion(tags: Sequence[str], state, affinity, diffusion_tensor=None, z_bias=None,
                            observation: Optional[ConceptDiffusionObservation] = None,
                            config: Optional[ConceptDiffusionConfig] = None) -> ConceptDiffusionPayload:
    """One step: optional observation blend -> exponential Z-bias tilt -> graph heat flow.

    Raises when an invariant breaks: entropy must not drop and Dirichlet energy must not rise across
    the heat flow, and the CFL sub-step count `ceil(dt * max_degree / cfl_limit)` must fit the budget.
    """
    config = config or ConceptDiffusionConfig()
    device = state.device if isinstance(state, torch.Tensor) else None
    p0, in_sum = _distribution("state", state, None, device)
    n = p0.numel()
    tags = list(tags)
    if len(tags) != n:
        raise ConceptDiffusionError(f"tags has {len(tags)} entries, expected {n}")
    if len(set(tags)) != n or any(not t for t in tags):
        raise ConceptDiffusionError("tags must be unique and non-empty")
    aff = _matrix("affinity", affinity, n, config.symmetry_tolerance, p0.device)
    if diffusion_tensor is None:
        cond, source = torch.ones(n, n, dtype=torch.float64, device=p0.device), "uniform"
    else:
        cond, source = _matrix("diffusion_tensor", diffusion_tensor, n, config.symmetry_tolerance, p0.device), "request"
    zb = torch.zeros(n, dtype=torch.float64, device=p0.device) if z_bias is None or len(z_bias) == 0 else \
        torch.as_tensor(z_bias, dtype=torch.float64, device=p0.device).flatten()
    if zb.numel() != n:
        raise ConceptDiffusionError(f"z_bias has {zb.numel()} entries, expected {n}")
    if not bool(torch.isfinite(zb).all()):
        raise ConceptDiffusionError("z_bias contains a non-finite value")

    h0 = _entropy(p0)
    p1 = blend_concept_diffusion_observation(p0, observation) if observation is not None else p0.clone()
    w = observation.weight if observation is not None else 0.0
    h1 = _entropy(p1)

    tilt = config.timestep > 0 and bool((zb != 0).any())
    if tilt:
        e = config.timestep * zb
        p2 = p1 * torch.exp(e - e[p1 > 0].max())
        p2 = p2 / p2.sum()
    else:
        p2 = p1.clone()
    h2 = _entropy(p2)

    c = aff * cond
    c = c - torch.diag(torch.diag(c))
    deg = c.sum(1)
    edges, max_deg = int((torch.triu(c, 1) > 0).sum()), float(deg.max())
    e_before = _dirichlet(p2, c)
    p3, substeps, sub_dt, e_after = p2.clone(), 0, 0.0, e_before
    if config.timestep > 0 and edges > 0 and max_deg > 0:
        need = max(math.ceil(config.timestep * max_deg / config.cfl_limit), 1)
        if need > config.max_substeps:
            raise ConceptDiffusionError(f"step budget exceeded: at least {need} sub-steps needed, maximum {config.max_substeps}")
        substeps, sub_dt = need, config.timestep / need
        keep = (1.0 - sub_dt * deg).clamp(min=0.0)
        for _ in range(substeps):
            p3 = keep * p3 + sub_dt * (c @ p3)
            p3 = p3 / p3.sum()
        e_after = _dirichlet(p3, c)
    h3 = _entropy(p3)
    if h3 + _TOL * (1 + abs(h2)) < h2:
        raise ConceptDiffusionError(f"entropy decreased across diffusion: {h2} -> {h3}")
    if e_after > e_before + _TOL * (1 + abs(e_before)):
        raise ConceptDiffusionError(f"Dirichlet energy increased across diffusion: {e_before} -> {e_after}")
    eff = ConceptDiffusionEffects(observation is not None, observation is not None and w > 0, w, tilt, substeps > 0, edges,
                                  substeps, sub_dt, max_deg, h0, h1, h2, h3, e_before, e_after,
                                  float(0.5 * (p0 - p3).abs().sum()))
    return ConceptDiffusionPayload(tags, p0, p1, p2, p3, in_sum, float(p3.sum()), source, eff, config)


@dataclass
class FisherRaoComparison:
    distance: float
    bhattacharyya: float
    hellinger: float


def compare_fisher_rao(p, q) -> FisherRaoComparison:
    """Fisher-Rao geodesic distance `2 acos(sum sqrt(p q))` with its Bhattacharyya / Hellinger companions."""
    a, _ = _distribution("left", p)
    b, _ = _distribution("right", q, a.numel(), a.device)
    bc = float(torch.sqrt(a * b).sum().clamp(0.0, 1.0))
    return FisherRaoComparison(2.0 * math.acos(bc), bc, math.sqrt(max(0.0, 1.0 - bc)))


# ----------------------------------------------------------------------------------------------
# Free energy of a candidate step
# ----------------------------------------------------------------------------------------------
class FreeEnergyError(ValueError):
    pass


@dataclass
class BandEnergy:
    above: float = 0.0
    here: float = 0.0
    beneath: float = 0.0

    def l1(self) -> float:
        return abs(self.above) + abs(self.here) + abs(self.beneath)

    def probabilities(self) -> list:
        v = [self.above, self.here, self.beneath]
        if any(not math.isfinite(x) or x < 0 for x in v):
            raise FreeEnergyError("band energies must be finite and non-negative")
        t = sum(v)
        return [1 / 3] * 3 if t <= 0 else [x / t for x in v]

    def norm(self) -> "BandEnergy":
        return BandEnergy(*self.probabilities())


@dataclass
class FreeEnergyConfig:
    loss_scale: float = 1.0
    step_time_scale_ms: float = 10.0
    memory_scale_mb: float = 1024.0
    retry_scale: float = 1.0
    observation_entropy_scale: float = 1.0
    loss_weight: float = 1.0
    speed_weight: float = 0.5
    memory_weight: float = 0.3
    retry_weight: float = 0.2
    uncertainty_weight: float = 0.0
    external_penalty_weight: float = 1.0
    temperature: float = 0.1
    prior: tuple = (1 / 3, 1 / 3, 1 / 3)
    band_potentials: tuple = (-0.1, 0.0, 0.3)

    def validate(self) -> None:
        for name in ("loss_scale", "step_time_scale_ms", "memory_scale_mb", "retry_scale", "observation_entropy_scale"):
            v = getattr(self, name)
            if not math.isfinite(v) or v <= 0:
                raise FreeEnergyError(f"{name} must be finite and > 0, got {v}")
        for name in ("loss_weight", "speed_weight", "memory_weight", "retry_weight", "uncertainty_weight",
                     "external_penalty_weight", "temperature"):
            v = getattr(self, name)
            if not math.isfinite(v) or v < 0:
                raise FreeEnergyError(f"{name} must be finite and >= 0, got {v}")
        if len(self.prior) != 3 or any(not math.isfinite(x) or x <= 0 for x in self.prior):
            raise FreeEnergyError("prior must hold three positive values")
        if len(self.band_potentials) != 3 or any(not math.isfinite(x) for x in self.band_potentials):
            raise FreeEnergyError("band potentials must hold three finite values")


@dataclass
class FreeEnergyObservation:
    reference_loss: float = 0.0
    candidate_loss: float = 0.0
    step_time_ms: float = 0.0
    memory_mb: float = 0.0
    retry_rate: float = 0.0
    observation_entropy: float = 0.0
    external_penalty: float = 0.0
    band: BandEnergy = field(default_factory=BandEnergy)


@dataclass
class FreeEnergyReport:
    free_energy: float
    utility: float
    acceptance_probability: float
    components: dict
    distribution: dict
    normalized: dict
    formula: str = "F = E_observed + (E_q[V] - E_prior[V]) + T * KL(q || prior)"
    acceptance_rule: str = "sigmoid(-F)"


def evaluate_free_energy(obs: FreeEnergyObservation, config: Optional[FreeEnergyConfig] = None) -> FreeEnergyReport:
    cfg = config or FreeEnergyConfig()
    cfg.validate()
    for name in ("reference_loss", "candidate_loss"):
        if not math.isfinite(getattr(obs, name)):
            raise FreeEnergyError(f"{name} must be finite")
    for name in ("step_time_ms", "memory_mb", "retry_rate", "observation_entropy", "external_penalty"):
        v = getattr(obs, name)
        if not math.isfinite(v) or v < 0:
            raise FreeEnergyError(f"{name} must be finite and >= 0, got {v}")
    tot = sum(cfg.prior)
    prior = [x / tot for x in cfg.prior]
    zero = obs.band.l1() <= 1.1920929e-07
    q = prior if zero else obs.band.probabilities()
    norm = {"loss_delta": (obs.candidate_loss - obs.reference_loss) / cfg.loss_scale,
            "step_time": obs.step_time_ms / cfg.step_time_scale_ms, "memory": obs.memory_mb / cfg.memory_scale_mb,
            "retry": obs.retry_rate / cfg.retry_scale,
            "observation_entropy": obs.observation_entropy / cfg.observation_entropy_scale,
            "external_penalty": obs.external_penalty}
    comp = {"loss": cfg.loss_weight * norm["loss_delta"], "speed": cfg.speed_weight * norm["step_time"],
            "memory": cfg.memory_weight * norm["memory"], "retry": cfg.retry_weight * norm["retry"],
            "uncertainty": cfg.uncertainty_weight * norm["observation_entropy"],
            "external_penalty": cfg.external_penalty_weight * norm["external_penalty"]}
    comp["observed_energy"] = sum(comp.values())
    comp["band_potential_expectation"] = sum(a * b for a, b in zip(q, cfg.band_potentials))
    comp["prior_band_potential"] = sum(a * b for a, b in zip(prior, cfg.band_potentials))
    comp["band_potential"] = comp["band_potential_expectation"] - comp["prior_band_potential"]
    ent = -sum(x * math.log(x) for x in q if x > 0)
    cross = -sum(x * math.log(p) for x, p in zip(q, prior) if x > 0)
    kl = cross - ent
    if kl < -1e-12:
        raise FreeEnergyError(f"distribution.kl_divergence is negative: {kl}")
    kl = max(kl, 0.0)
    comp["relative_entropy"] = cfg.temperature * kl
    f = comp["observed_energy"] + comp["band_potential"] + comp["relative_entropy"]
    if not math.isfinite(f):
        raise FreeEnergyError("free energy is not finite")
    accept = 1 / (1 + math.exp(f)) if f < 0 else math.exp(-f) / (1 + math.exp(-f))
    dist = {"status": "prior_zero_mass" if zero else "normalized", "raw_total": obs.band.l1(), "above": q[0], "here": q[1],
            "beneath": q[2], "entropy": ent, "normalized_entropy": ent / math.log(3), "cross_entropy": cross,
            "kl_divergence": kl, "dominant_band": ("above", "here", "beneath")[max(range(3), key=lambda i: (q[i], -i))]}
    return FreeEnergyReport(f, -f, accept, comp, dist, norm)


def score_with_free_energy(loss_before: float, loss_after: float, step_ms: float, mem_mb: float, retry: float,
                           band: BandEnergy, entropy: float, beta: float) -> float:
    """Scalar utility of a candidate for the heuristics chooser: higher is better; `-inf` on invalid
    input.  Uses unit resource scales, weights `(1, 0.0025, 0.001, 0.5, beta, 0)`, temperature 0 and an
    uncentred band potential."""
    try:
        if not math.isfinite(beta) or beta < 0:
            raise FreeEnergyError("beta must be >= 0")
        cfg = FreeEnergyConfig(step_time_scale_ms=1.0, memory_scale_mb=1.0, retry_scale=1.0, loss_weight=1.0,
                               speed_weight=0.0025, memory_weight=0.001, retry_weight=0.5, uncertainty_weight=beta,
                               external_penalty_weight=0.0, temperature=0.0)
        r = evaluate_free_energy(FreeEnergyObservation(loss_before, loss_after, step_ms, mem_mb, retry, entropy, 0.0, band), cfg)
        return r.utility - r.components["prior_band_potential"]
    except FreeEnergyError:
        return -math.inf


# ----------------------------------------------------------------------------------------------
# Z-space generation control (crates/st-core/src/inference/generation_control.rs:88-700)
# ----------------------------------------------------------------------------------------------
class ZSpaceGenerationControlError(ValueError):
    pass


_LOG_FLOOR, _ADJ_MIN, _ADJ_MAX = 1e-12, 0.25, 4.0


@dataclass
class ZSpaceSoftmaxConfig:
    """Softmax at scale `sqrt(-curvature) / T`; with an entropy target, `T` is multiplied once by
    `clamp(1 + gain * (target - H), 0.25, 4)` and clamped to `[min_temperature, max_temperature]`."""
    curvature: float
    temperature: float
    min_temperature: Optional[float] = None
    max_temperature: Optional[float] = None
    entropy_target: Optional[float] = None
    entropy_tolerance: float = 1e-4
    entropy_gain: float = 0.5

    def __post_init__(self):
        if not math.isfinite(self.curvature) or self.curvature >= 0:
            raise ZSpaceGenerationControlError("curvature must be finite and negative")
        if not math.isfinite(self.temperature) or self.temperature <= 0:
            raise ZSpaceGenerationControlError("temperature must be finite and positive")
        if self.min_temperature is None:
            self.min_temperature = max(self.temperature * 0.1, 1e-3)
        if self.max_temperature is None:
            self.max_temperature = self.temperature * 10.0
        if not 0 < self.min_temperature <= self.max_temperature:
            raise ZSpaceGenerationControlError("temperature bounds must satisfy 0 < min <= max")
        if self.entropy_target is not None and (not math.isfinite(self.entropy_target) or self.entropy_target < 0):
            raise ZSpaceGenerationControlError("entropy_target must be finite and >= 0")
        if self.entropy_tolerance < 0 or self.entropy_gain < 0:
            raise ZSpaceGenerationControlError("entropy tolerance and gain must be >= 0")

    def fixed_temperature(self) -> float:
        return min(max(self.temperature, self.min_temperature), self.max_temperature)

    def curvature_scale(self) -> float:
        return math.sqrt(-self.curvature)


@dataclass
class ZSpaceSoftmaxProjection:
    probabilities: torch.Tensor
    base_probabilities: torch.Tensor
    entropy: float
    base_entropy: float
    effective_temperature: float
    base_temperature: float
    adaptive_temperature: bool
    temperature_gradient_active: bool
    scale: float
    base_scale: float


def zspace_entropy(p: torch.Tensor) -> float:
    p = torch.as_tensor(p, dtype=torch.float64)
    if not bool(torch.isfinite(p).all()) or bool(((p < 0) | (p > 1)).any()):
        raise ZSpaceGenerationControlError("probability must lie in [0, 1]")
    return float(-(p * torch.log(p.clamp(min=_LOG_FLOOR))).sum())


def project_zspace_softmax(logits, config: ZSpaceSoftmaxConfig) -> ZSpaceSoftmaxProjection:
    x = torch.as_tensor(logits, dtype=torch.float64)
    if not bool(torch.isfinite(x).all()):
        raise ZSpaceGenerationControlError("logit must be finite")
    t0 = config.fixed_temperature()
    s0 = config.curvature_scale() / t0
    base = torch.softmax(x * s0, -1)
    h0 = zspace_entropy(base) if x.numel() else 0.0
    t, adaptive, grad_active = t0, False, False
    if config.entropy_target is not None:
        delta = config.entropy_target - h0
        if abs(delta) > config.entropy_tolerance:
            raw_adj = 1.0 + config.entropy_gain * delta
            raw_t = t0 * min(max(raw_adj, _ADJ_MIN), _ADJ_MAX)
            t = min(max(raw_t, config.min_temperature), config.max_temperature)
            adaptive = True
            grad_active = (config.entropy_gain > 0 and _ADJ_MIN < raw_adj < _ADJ_MAX
                           and config.min_temperature < raw_t < config.max_temperature)
    s = config.curvature_scale() / t
    p = torch.softmax(x * s, -1) if adaptive else base.clone()
    return ZSpaceSoftmaxProjection(p, base, zspace_entropy(p) if adaptive and x.numel() else h0, h0, t, t0, adaptive,
                                   grad_active, s, s0)


@dataclass
class ZSpaceGenerationControlConfig:
    curvature: float = -0.04
    temperature: float = 1.0
    entropy_target: Optional[float] = None
    entropy_tolerance: float = 1e-4
    entropy_gain: float = 0.5
    min_temperature: Optional[float] = None
    max_temperature: Optional[float] = None
    repression_window: int = 32
    repression_strength: float = 1.0
    last_token_repression: float = 0.5
    ngram_size: int = 0
    ngram_window: int = 0
    ngram_repression_strength: float = 0.0
    ngram_decay: float = 1.0

    def softmax_config(self) -> ZSpaceSoftmaxConfig:
        for name in ("repression_strength", "last_token_repression", "ngram_repression_strength"):
            v = getattr(self, name)
            if not math.isfinite(v) or v < 0:
                raise ZSpaceGenerationControlError(f"{name} must be finite and >= 0")
        if not math.isfinite(self.ngram_decay) or not 0 < self.ngram_decay <= 1:
            raise ZSpaceGenerationControlError("ngram_decay must lie in (0, 1]")
        return ZSpaceSoftmaxConfig(self.curvature, self.temperature, self.min_temperature, self.max_temperature,
                                   self.entropy_target, self.entropy_tolerance, self.entropy_gain)


@dataclass
class ZSpaceGenerationControlPayload:
    token_ids: list
    adjusted_logits: torch.Tensor
    probabilities: torch.Tensor
    log_probabilities: torch.Tensor
    repression_penalties: torch.Tensor
    ngram_repression_penalties: torch.Tensor
    projection: ZSpaceSoftmaxProjection
    before_top_token: Optional[int]
    after_top_token: Optional[int]
    top_changed: bool
    repressed_token_count: int
    ngram_repressed_token_count: int
    max_repression: float
    kind: str = "spiraltorch.zspace_generation_control"
    contract_version: str = "v1"


def _ngram_continuations(history: Sequence[int], n: int, decay: float) -> dict:
    """token -> sum of decay^distance over earlier occurrences of the current (n-1)-prefix followed by it."""
    if n <= 1 or len(history) < n:
        return {}
    k = n - 1
    prefix, latest = list(history[-k:]), len(history) - n
    out: dict = {}
    for start in range(latest + 1):
        if list(history[start:start + k]) == prefix:
            tok = history[start + k]
            out[tok] = out.get(tok, 0.0) + decay ** (latest - start)
    return out


def apply_zspace_generation_control(logits, token_ids: Sequence[int], recent_tokens: Sequence[int],
                                    config: Optional[ZSpaceGenerationControlConfig] = None) -> ZSpaceGenerationControlPayload:
    """Repetition / n-gram repression of candidate logits followed by the Z-space softmax.

    A candidate's logit drops by `repression_strength * count(token in the last repression_window)`,
    by `last_token_repression` if it repeats the last token, and by `ngram_repression_strength` times
    the decayed count of times it already completed the current (n-1)-gram."""
    cfg = config or ZSpaceGenerationControlConfig()
    x = torch.as_tensor(logits, dtype=torch.float64)
    ids = [int(t) for t in token_ids]
    if x.numel() != len(ids):
        raise ZSpaceGenerationControlError(f"candidate length mismatch: {x.numel()} logits, {len(ids)} token ids")
    if not bool(torch.isfinite(x).all()):
        raise ZSpaceGenerationControlError("logit must be finite")
    soft = cfg.softmax_config()
    recent = [int(t) for t in recent_tokens]
    hist = recent[max(0, len(recent) - cfg.repression_window):] if cfg.repression_window > 0 else []
    counts: dict = {}
    for t in hist:
        counts[t] = counts.get(t, 0) + 1
    last = hist[-1] if hist else None
    win = cfg.ngram_window or cfg.repression_window
    cont = _ngram_continuations(recent[max(0, len(recent) - win):], cfg.ngram_size, cfg.ngram_decay) \
        if cfg.ngram_repression_strength > 0 else {}
    ngram = torch.tensor([cfg.ngram_repression_strength * cont.get(t, 0.0) for t in ids], dtype=torch.float64)
    pen = torch.tensor([cfg.repression_strength * counts.get(t, 0) + (cfg.last_token_repression if t == last else 0.0)
                        for t in ids], dtype=torch.float64) + ngram
    adj = x.cpu() - pen
    proj = project_zspace_softmax(adj, soft)
    before = ids[int(x.argmax())] if ids else None
    after = ids[int(adj.argmax())] if ids else None
    return ZSpaceGenerationControlPayload(ids, adj, proj.probabilities, torch.log(proj.probabilities.clamp(min=_LOG_FLOOR)),
                                          pen, ngram, proj, before, after, before != after, int((pen > 0).sum()),
                                          int((ngram > 0).sum()), float(pen.max()) if ids else 0.0)
