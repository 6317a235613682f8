"""Two Schrödinger evolutions used as tensor clients.

* Real-time **stochastic** evolution of real-valued rows: every row is the real quadrature of a complex wavefunction;
  one step is a Strang split between a diagonal learned Hamiltonian (phase = potential dt + noise sqrt(dt) xi, the
  Stratonovich phase diffusion driven by supplied standard-normal samples) and Hermitian hopping between the disjoint
  feature pairs (0,1), (2,3), ..., followed by the uniform no-jump attenuation exp(-loss dt / 2).  The real quadrature is
  returned for the network, the imaginary quadrature and the phases stay available, and the backward pass is the
  analytic one.  crates/st-core/src/dynamics/stochastic_schrodinger.rs (`StochasticSchrodingerConfig` :142-240, the
  pair evolution :367-409, `apply_stochastic_schrodinger_step` :582-664, `backward_stochastic_schrodinger_step` :666-724).
* **Imaginary-time** evolution of a positive amplitude on a weighted undirected graph: H = Laplacian + diagonal potential,
  exp(-tau H) by positivity-preserving Euler sub-steps under a CFL limit, carried in the log domain and renormalised
  in L2 after each sub-step; reports the Rayleigh energy before and after (it must not rise), the eigen-residual, the
  Born probabilities and their entropy.  crates/st-core/src/inference/imaginary_time_schrodinger.rs (config :165-235,
  edge validation :319-364, `apply_imaginary_time_schrodinger` :521-735).

Both are whole-tensor programs: the stochastic step is a handful of element-wise operations on [rows, features]
(usable on the GPU inside a training graph through :class:`StochasticSchrodingerFunction`), the imaginary-time sub-step
one scatter log-sum-exp over the directed edge list.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


class SchrodingerError(ValueError):
    pass


def _finite(name: str, v: float) -> float:
    if not math.isfinite(v):
        raise SchrodingerError(f"{name} must be finite, received {v}")
    return v


# ---------------------------------------------------------------------------------------------------------------
# real-time stochastic evolution
# ---------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class StochasticSchrodingerConfig:
    loss_rate: float = 0.0
    noise_scale: float = 0.0
    time_step: float = 0.1
    hopping_rate: float = 1.0

    def __post_init__(self):
        for name in ("time_step", "loss_rate", "noise_scale"):
            v = getattr(self, name)
            if not (math.isfinite(v) and v >= 0.0):
                raise SchrodingerError(f"{name} must be finite and non-negative, received {v}")
        _finite("hopping_rate", self.hopping_rate)
        for name in ("hopping_angle", "noise_step_scale", "ensemble_dephasing_rate", "damping_factor"):
            _finite(name, getattr(self, name))

    def with_time_step(self, dt: float) -> "StochasticSchrodingerConfig":
        return StochasticSchrodingerConfig(self.loss_rate, self.noise_scale, dt, self.hopping_rate)

    def with_hopping_rate(self, rate: float) -> "StochasticSchrodingerConfig":
        return StochasticSchrodingerConfig(self.loss_rate, self.noise_scale, self.time_step, rate)

    @property
    def decoherence_rate(self) -> float:
        return self.loss_rate

    @property
    def hopping_angle(self) -> float:
        return self.hopping_rate * self.time_step

    @property
    def noise_step_scale(self) -> float:
        return self.noise_scale * math.sqrt(self.time_step)

    @property
    def damping_factor(self) -> float:
        return math.exp(-0.5 * self.loss_rate * self.time_step)

    @property
    def ensemble_dephasing_rate(self) -> float:
        """The off-diagonal dephasing rate of the noise ensemble: the squared phase-noise scale (distinct from the loss)."""
        return self.noise_scale * self.noise_scale


def _partner(features: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Index of every feature's hopping partner and a mask of the features that have one (an odd last feature has none)."""
    idx = torch.arange(features, device=device)
    p = idx ^ 1
    has = p < features
    return torch.where(has, p, idx), has


@dataclass
class StochasticSchrodingerStep:
    output_real: torch.Tensor
    output_imaginary: torch.Tensor
    phase: torch.Tensor
    config: StochasticSchrodingerConfig

    def norm_ratio(self, inputs: torch.Tensor) -> torch.Tensor:
        """|psi_out|^2 / |psi_in|^2 per row: exp(-loss dt) for the unitary part plus the uniform attenuation."""
        out = (self.output_real ** 2 + self.output_imaginary ** 2).sum(-1)
        return out / (inputs ** 2).sum(-1).clamp_min(1e-30)


def apply_stochastic_schrodinger_step(inputs: torch.Tensor, potential: torch.Tensor, standard_normal: torch.Tensor,
                                      config: StochasticSchrodingerConfig) -> StochasticSchrodingerStep:
    if inputs.dim() != 2 or potential.shape != (inputs.shape[1],) or standard_normal.shape != inputs.shape:
        raise SchrodingerError(f"shapes: input {tuple(inputs.shape)}, potential {tuple(potential.shape)}, noise {tuple(standard_normal.shape)}")
    if not (bool(torch.isfinite(inputs).all()) and bool(torch.isfinite(potential).all()) and bool(torch.isfinite(standard_normal).all())):
        raise SchrodingerError("inputs, potential and noise must be finite")
    phase = potential * config.time_step + standard_normal * config.noise_step_scale
    partner, has = _partner(inputs.shape[1], inputs.device)
    c, s, d = math.cos(config.hopping_angle), math.sin(config.hopping_angle), config.damping_factor
    mean = 0.5 * phase + 0.5 * phase[:, partner]
    xp = inputs[:, partner]
    real = torch.where(has, d * (c * inputs * phase.cos() - s * xp * mean.sin()), d * inputs * phase.cos())
    imag = torch.where(has, d * (-c * inputs * phase.sin() - s * xp * mean.cos()), -d * inputs * phase.sin())
    return StochasticSchrodingerStep(real, imag, phase, config)


def backward_stochastic_schrodinger_step(inputs: torch.Tensor, phase: torch.Tensor, grad_output: torch.Tensor,
                                         config: StochasticSchrodingerConfig) -> Tuple[torch.Tensor, torch.Tensor]:
    """(grad of the input, grad of the potential) for a gradient arriving on the real quadrature."""
    partner, has = _partner(inputs.shape[1], inputs.device)
    c, s, d = math.cos(config.hopping_angle), math.sin(config.hopping_angle), config.damping_factor
    mean = 0.5 * phase + 0.5 * phase[:, partner]
    xp, gp = inputs[:, partner], grad_output[:, partner]
    g_amp = torch.where(has, d * (grad_output * c * phase.cos() - gp * s * mean.sin()), d * grad_output * phase.cos())
    g_phase = torch.where(has, d * (grad_output * (-c * inputs * phase.sin() - 0.5 * s * xp * mean.cos()) - 0.5 * gp * s * inputs * mean.cos()),
                          -d * grad_output * inputs * phase.sin())
    return g_amp, (g_phase * config.time_step).sum(0)


class StochasticSchrodingerFunction(torch.autograd.Function):
    """`y = Re psi(t + dt)` with the analytic backward; ``noise`` is data (no gradient)."""

    @staticmethod
    def forward(ctx, inputs, potential, noise, config):
        step = apply_stochastic_schrodinger_step(inputs, potential, noise, config)
        ctx.save_for_backward(inputs, step.phase)
        ctx.config = config
        return step.output_real

    @staticmethod
    def backward(ctx, grad_output):
        inputs, phase = ctx.saved_tensors
        g_in, g_pot = backward_stochastic_schrodinger_step(inputs, phase, grad_output, ctx.config)
        return g_in, g_pot, None, None


# ---------------------------------------------------------------------------------------------------------------
# imaginary-time evolution on a graph
# ---------------------------------------------------------------------------------------------------------------
_TOL = 1.0e-10
_MAX_CFL = 1.0 - 2.220446049250313e-16


@dataclass(frozen=True)
class ImaginaryTimeSchrodingerConfig:
    imaginary_time: float = 1.0
    cfl_limit: float = 0.9
    max_substeps: int = 16_384

    def __post_init__(self):
        if not (math.isfinite(self.imaginary_time) and self.imaginary_time >= 0.0):
            raise SchrodingerError(f"imaginary_time must be finite and non-negative, received {self.imaginary_time}")
        if not (math.isfinite(self.cfl_limit) and 0.0 < self.cfl_limit <= _MAX_CFL):
            raise SchrodingerError(f"cfl_limit must lie in (0, 1), received {self.cfl_limit}")
        if self.max_substeps <= 0:
            raise SchrodingerError("max_substeps must be positive")


@dataclass
class ImaginaryTimeSchrodingerEffects:
    evolution_applied: bool
    edge_count: int
    substeps: int
    substep_imaginary_time: float
    potential_shift: float
    max_degree: float
    spectral_upper_bound: float
    initial_rayleigh_energy: float
    final_rayleigh_energy: float
    rayleigh_energy_drop: float
    energy_tolerance: float
    initial_l2_norm: float
    final_l2_norm: float
    initial_residual_l2: float
    final_residual_l2: float
    accumulated_log_norm: float
    probability_entropy: float


@dataclass
class ImaginaryTimeSchrodingerPayload:
    tags: List[str]
    potential: torch.Tensor
    shifted_potential: torch.Tensor
    edges: List[Tuple[int, int, float]]
    initial_amplitude: torch.Tensor
    final_amplitude: torch.Tensor
    probability: torch.Tensor
    log_amplitude_boost: torch.Tensor
    probability_sum: float
    effects: ImaginaryTimeSchrodingerEffects
    config: ImaginaryTimeSchrodingerConfig


def _check_edges(edges: Sequence[Tuple[int, int, float]], n: int):
    seen = set()
    for k, (a, b, w) in enumerate(edges):
        if not (0 <= a < n and 0 <= b < n):
            raise SchrodingerError(f"edge {k} endpoint out of range for dimension {n}")
        if a == b:
            raise SchrodingerError(f"edge {k} is a self edge")
        if a > b:
            raise SchrodingerError(f"edge {k} must be given as (left < right), received ({a}, {b})")
        if not (math.isfinite(w) and w > 0.0):
            raise SchrodingerError(f"edge_weight must be positive, received {w}")
        if (a, b) in seen:
            raise SchrodingerError(f"duplicate edge ({a}, {b})")
        seen.add((a, b))


def apply_imaginary_time_schrodinger(potential, edges: Sequence[Tuple[int, int, float]], config: Optional[ImaginaryTimeSchrodingerConfig] = None,
                                     initial_amplitude=None, tags: Optional[Sequence[str]] = None, device=None) -> ImaginaryTimeSchrodingerPayload:
    config = config or ImaginaryTimeSchrodingerConfig()
    v = torch.as_tensor(potential, dtype=torch.float64, device=device).flatten()
    n = v.numel()
    if n == 0:
        raise SchrodingerError("empty state")
    if tags is not None and len(tags) != n:
        raise SchrodingerError(f"tags: expected {n}, got {len(tags)}")
    if not bool(torch.isfinite(v).all()):
        raise SchrodingerError("potential must be finite")
    edges = [(int(a), int(b), float(w)) for a, b, w in edges]
    _check_edges(edges, n)
    dev = v.device
    # directed edge list (both directions): row = receiving node
    if edges:
        e = torch.tensor([(a, b) for a, b, _ in edges], dtype=torch.int64, device=dev)
        w1 = torch.tensor([w for _, _, w in edges], dtype=torch.float64, device=dev)
        rows, cols, w = torch.cat([e[:, 0], e[:, 1]]), torch.cat([e[:, 1], e[:, 0]]), torch.cat([w1, w1])
    else:
        rows = cols = torch.zeros(0, dtype=torch.int64, device=dev)
        w = torch.zeros(0, dtype=torch.float64, device=dev)
    degree = torch.zeros(n, dtype=torch.float64, device=dev).index_add(0, rows, w)
    shift = float(v.min())
    vs = v - shift
    if initial_amplitude is None or (hasattr(initial_amplitude, "__len__") and len(initial_amplitude) == 0):
        amp0 = torch.ones(n, dtype=torch.float64, device=dev)
    else:
        amp0 = torch.as_tensor(initial_amplitude, dtype=torch.float64, device=dev).flatten()
        if amp0.numel() != n:
            raise SchrodingerError(f"initial_amplitude: expected {n}, got {amp0.numel()}")
    if not bool((torch.isfinite(amp0) & (amp0 > 0.0)).all()):
        raise SchrodingerError("initial_amplitude must be positive")

    def normalise(log_a: torch.Tensor):
        log_norm = 0.5 * torch.logsumexp(2.0 * log_a, 0)
        return log_a - log_norm, float(log_norm)

    def h_apply(a: torch.Tensor) -> torch.Tensor:
        return vs * a + degree * a - torch.zeros_like(a).index_add(0, rows, w * a[cols])

    def rayleigh(a: torch.Tensor) -> float:
        return float((a * h_apply(a)).sum())

    def residual(a: torch.Tensor, energy: float) -> float:
        return float((h_apply(a) - energy * a).norm())

    log_a, _ = normalise(amp0.log())
    a0 = log_a.exp()
    bound = float((2.0 * degree + vs).max())
    need = 0 if config.imaginary_time == 0.0 or bound == 0.0 else max(math.ceil(config.imaginary_time * bound / config.cfl_limit), 1)
    if need > config.max_substeps:
        raise SchrodingerError(f"step budget exceeded: at least {need} sub-steps needed, maximum {config.max_substeps}")
    dt = config.imaginary_time / need if need else 0.0
    e0 = rayleigh(a0)
    r0 = residual(a0, e0)
    acc = 0.0
    if need:
        self_coeff = 1.0 - dt * (degree + vs)
        if not bool((self_coeff > 0.0).all()):
            raise SchrodingerError("self_coefficient must be positive")
        log_self, log_edge = self_coeff.log(), (dt * w).log()
        for _ in range(need):
            terms_self = log_self + log_a
            terms_edge = log_edge + log_a[cols]
            top = terms_self.clone().scatter_reduce(0, rows, terms_edge, reduce="amax", include_self=True)
            total = (terms_self - top).exp().index_add(0, rows, (terms_edge - top[rows]).exp())
            log_a, ln = normalise(top + total.log())
            acc += ln
    a1 = log_a.exp()
    e1 = rayleigh(a1)
    tol_e = _TOL * (1.0 + abs(e0))
    if e1 > e0 + tol_e:
        raise SchrodingerError(f"Rayleigh energy increased: {e0} -> {e1}")
    prob = torch.softmax(2.0 * log_a, 0)
    ent = float(-(prob * prob.clamp_min(1e-300).log()).sum())
    eff = ImaginaryTimeSchrodingerEffects(need > 0, len(edges), need, dt, shift, float(degree.max()) if n else 0.0, bound, e0, e1, max(e0 - e1, 0.0),
                                          tol_e, float(a0.norm()), float(a1.norm()), r0, residual(a1, e1), acc, ent)
    return ImaginaryTimeSchrodingerPayload(list(tags) if tags is not None else [str(i) for i in range(n)], v, vs, edges, a0, a1, prob,
                                           log_a - log_a.max(), float(prob.sum()), eff, config)
