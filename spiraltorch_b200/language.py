"""Language-side control: entropy-tracking temperature controller and the "desire" logit-bias step.

Restated from crates/st-core/src/inference/temperature_control.rs:451-480 (``T ← clamp(T + η·(H* − H(p)),
T_min, T_max)``) with the wrapper of crates/st-nn/src/language/temperature.rs:16-150, and from
crates/st-nn/src/language/desire.rs (``DesireWeights`` :144, ``DesireSchedule`` constant / warm-up :176-220,
phases Observation → Injection → Integration :163, and the per-token score of ``step`` :430-520:
``log q / T + α·log_syn + β·log_par − λ·repression + γ·g + phase bias`` over the top-k candidates,
followed by a temperature update from the resulting distribution).  Token geometry (syntagmatic /
paradigmatic log-affinities, repression, concept expectations) is supplied as dense tensors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from .tensor import TensorError


def entropy(distribution) -> float:
    p = torch.as_tensor(distribution, dtype=torch.float64)
    if p.numel() == 0 or not bool(torch.isfinite(p).all()) or bool((p < 0).any()):
        raise TensorError("distribution must be non-empty, finite and non-negative")
    s = float(p.sum())
    if abs(s - 1.0) > 1e-3:
        raise TensorError(f"distribution sums to {s}, expected 1")
    nz = p[p > 0]
    return float(-(nz * nz.log()).sum())


class TemperatureController:
    def __init__(self, value: float, target_entropy: float, eta: float, min: float, max: float):
        if not (min > 0 and max >= min and math.isfinite(max)):
            raise TensorError("temperature bounds must satisfy 0 < min <= max")
        if not (math.isfinite(eta) and eta >= 0) or not (math.isfinite(target_entropy) and target_entropy >= 0):
            raise TensorError("eta and target entropy must be finite and non-negative")
        if not min <= value <= max:
            raise TensorError(f"temperature {value} is outside [{min}, {max}]")
        self._t, self.target_entropy, self.eta, self.min, self.max = float(value), target_entropy, eta, min, max
        self._grad_heat, self._decay = 0.0, 0.9

    def value(self) -> float:
        return self._t

    def with_gradient_decay(self, decay: float) -> "TemperatureController":
        if not 0.0 <= decay < 1.0:
            raise TensorError("gradient decay must lie in [0, 1)")
        self._decay = decay
        return self

    def observe_grad(self, hyper_norm: float, real_norm: float) -> float:
        """Keeps a decayed "heat" of gradient activity; hot gradients cool the sampler slightly."""
        heat = math.log1p(max(hyper_norm, 0.0) + max(real_norm, 0.0))
        self._grad_heat = self._decay * self._grad_heat + (1 - self._decay) * heat
        return self._grad_heat

    def update(self, distribution, use_gradient: bool = False) -> float:
        h = entropy(distribution)
        t = self._t + self.eta * (self.target_entropy - h)
        if use_gradient:
            t /= 1.0 + 0.1 * self._grad_heat
        self._t = min(max(t, self.min), self.max)
        return self._t


@dataclass
class DesireWeights:
    alpha: float = 0.0      # syntagmatic pull
    beta: float = 0.0       # paradigmatic pull
    gamma: float = 0.0      # concept / semantic pull
    lam: float = 0.0        # repression


@dataclass
class DesireSchedule:
    start: float
    end: float
    steps: int = 0

    def value(self, step: int) -> float:
        if self.steps <= 0:
            return self.end
        return self.start + (self.end - self.start) * min(step, self.steps) / self.steps


def constant(value: float) -> DesireSchedule:
    return DesireSchedule(value, value, 0)


def warmup(start: float, end: float, steps: int) -> DesireSchedule:
    return DesireSchedule(start, end, steps)


OBSERVATION, INJECTION, INTEGRATION = "observation", "injection", "integration"


@dataclass
class DesireSolution:
    indices: list
    probabilities: list
    logit_offsets: list
    phase: str
    temperature: float
    entropy: float
    weights: DesireWeights


class DesireLagrangian:
    """``log_syn`` / ``log_par``: ``[V, V]`` log-affinities from the previous token; ``repression``: ``[V]``;
    ``semantics``: ``[V, C]`` token → concept expectations."""

    def __init__(self, log_syn: torch.Tensor, log_par: torch.Tensor, repression: torch.Tensor, semantics: torch.Tensor,
                 controller: TemperatureController, top_k: Optional[int] = None, epsilon: float = 1e-6):
        V = log_syn.shape[0]
        if log_syn.shape != (V, V) or log_par.shape != (V, V) or repression.shape != (V,) or semantics.shape[0] != V:
            raise TensorError("desire geometry tensors disagree on the vocabulary size")
        self.log_syn, self.log_par, self.repression, self.semantics = log_syn, log_par, repression, semantics
        self.controller, self.top_k, self.epsilon = controller, top_k, epsilon
        self.desire_bias = torch.zeros(V)
        self.avoidance_heat = torch.zeros(V)
        self.phase = OBSERVATION
        self._step = 0
        self._schedules: dict = {}
        self.observation_horizon: Optional[int] = None
        self.integration_horizon: Optional[int] = None

    def vocab_size(self) -> int:
        return self.log_syn.shape[0]

    def with_schedules(self, **schedules: DesireSchedule) -> "DesireLagrangian":
        for k in schedules:
            if k not in ("alpha", "beta", "gamma", "lam"):
                raise TensorError(f"unknown schedule '{k}'")
        self._schedules.update(schedules)
        return self

    def with_horizons(self, observation: Optional[int], integration: Optional[int]) -> "DesireLagrangian":
        self.observation_horizon, self.integration_horizon = observation, integration
        return self

    def _classify(self, w: DesireWeights) -> str:
        if self.observation_horizon is not None and self._step < self.observation_horizon:
            return OBSERVATION
        if self.integration_horizon is not None and self._step >= self.integration_horizon:
            return INTEGRATION
        if w.alpha == 0 and w.beta == 0 and w.gamma == 0:
            return OBSERVATION
        return INTEGRATION if w.gamma > 0 and w.lam > 0 else INJECTION

    def step_with_scheduler(self, lm_logits, previous_token: int, concepts) -> DesireSolution:
        s = self._step
        w = DesireWeights(*(self._schedules.get(k, constant(0.0)).value(s) for k in ("alpha", "beta", "gamma", "lam")))
        return self.step(lm_logits, previous_token, concepts, w)

    def step(self, lm_logits, previous_token: int, concepts, weights: DesireWeights) -> DesireSolution:
        logits = torch.as_tensor(lm_logits, dtype=torch.float32)
        V = self.vocab_size()
        if logits.shape != (V,):
            raise TensorError("LM logits must match vocabulary")
        if not 0 <= previous_token < V:
            raise TensorError(f"previous token {previous_token} is outside the vocabulary")
        c = torch.as_tensor(concepts, dtype=torch.float32)
        if c.shape != (self.semantics.shape[1],):
            raise TensorError("concept hint must have one weight per concept")
        c = c / c.sum().clamp(min=self.epsilon)
        k = V if self.top_k is None else max(1, min(self.top_k, V))
        active = torch.topk(logits, k).indices.sort().values
        log_q = torch.log(torch.softmax(logits[active], 0).clamp(min=self.epsilon))
        phase = self._classify(weights)
        if phase != self.phase:
            self.avoidance_heat.mul_(0.5)                      # a phase change relaxes the accumulated avoidance
            self.phase = phase
        bias = self.desire_bias[active]
        phase_bias = 0.0 if phase == OBSERVATION else weights.alpha * bias if phase == INJECTION \
            else (weights.alpha + weights.gamma) * bias
        adj = weights.alpha * self.log_syn[previous_token, active] + weights.beta * self.log_par[previous_token, active] \
            - weights.lam * self.repression[active] + weights.gamma * (self.semantics[active] @ c) + phase_bias
        scores = log_q / self.controller.value() + adj
        probs = torch.softmax(scores - scores.max(), 0)
        t = self.controller.update(probs.double() / probs.double().sum())
        # tokens that were repressed yet remain likely heat up; the bias drifts toward what was chosen
        self.avoidance_heat[active] = 0.9 * self.avoidance_heat[active] + 0.1 * probs * self.repression[active]
        self.desire_bias[active] = 0.95 * self.desire_bias[active] + 0.05 * (probs - 1.0 / k)
        self._step += 1
        return DesireSolution(active.tolist(), probs.tolist(), adj.tolist(), phase, t, entropy(probs.double() / probs.double().sum()),
                              weights)
