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
    hypergrad_penalty: float = 0.0      # lambda-weighted probability mass that stayed on repressed tokens


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
        penalty = float(weights.lam * (probs * self.repression[active].clamp(min=0)).sum())
        return DesireSolution(active.tolist(), probs.tolist(), adj.tolist(), phase, t, entropy(probs.double() / probs.double().sum()),
                              weights, penalty)


# ----------------------------------------------------------------------------------------------
# Semantic bridge + entropic Gromov-Wasserstein alignment
# ----------------------------------------------------------------------------------------------
class SemanticBridge:
    """Token -> concept coupling kept as a dense ``[V, C]`` log-probability tensor.

    Parity: crates/st-nn/src/language/geometry.rs:418-760 (`log_pi`, `expectation`,
    `infer_from_window`, marginals, anchors).  The reference stores sparse rows and scans them per
    query; dense rows turn every query into one gather + reduction on the tensor's device.
    """

    def __init__(self, log_pi: torch.Tensor, row_marginal: torch.Tensor, col_marginal: torch.Tensor,
                 anchors=(), epsilon: float = 1e-6):
        if log_pi.dim() != 2 or row_marginal.shape != (log_pi.shape[0],) or col_marginal.shape != (log_pi.shape[1],):
            raise TensorError("semantic bridge marginals must match the coupling's shape")
        if not epsilon > 0:
            raise TensorError("semantic bridge epsilon must be positive")
        self.log_pi_matrix, self.row_sums, self.col_sums = log_pi.float(), row_marginal.float(), col_marginal.float()
        self._anchors = {(int(i), int(j)) for i, j in anchors}
        self.log_epsilon = math.log(epsilon)

    @classmethod
    def from_dense(cls, pi, anchors=(), epsilon: float = 1e-6) -> "SemanticBridge":
        pi = torch.as_tensor(pi, dtype=torch.float32)
        if pi.dim() != 2 or pi.numel() == 0 or not bool(torch.isfinite(pi).all()) or bool((pi < 0).any()):
            raise TensorError("coupling must be a non-empty, finite, non-negative matrix")
        rows, cols = pi.sum(1), pi.sum(0)
        return cls(torch.log(pi.clamp(min=epsilon)), rows / rows.sum().clamp(min=1e-30), cols / cols.sum().clamp(min=1e-30),
                   anchors, epsilon)

    def vocab_size(self) -> int:
        return self.log_pi_matrix.shape[0]

    def concept_count(self) -> int:
        return self.log_pi_matrix.shape[1]

    def log_pi(self, token: int, concept: int) -> float:
        if 0 <= token < self.vocab_size() and 0 <= concept < self.concept_count():
            return float(self.log_pi_matrix[token, concept])
        return self.log_epsilon

    def anchors(self) -> set:
        return set(self._anchors)

    def row_marginal(self) -> torch.Tensor:
        return self.row_sums

    def col_marginal(self) -> torch.Tensor:
        return self.col_sums

    def expectation(self, token: int, concept_dist) -> float:
        """Concept-weighted mean log-probability of `token`, floored at log(epsilon)."""
        w = torch.as_tensor(concept_dist, dtype=torch.float32, device=self.log_pi_matrix.device).clamp(min=0.0)
        w = torch.where(w > 1.1920929e-07, w, torch.zeros_like(w))
        tot = float(w.sum())
        if tot <= 1.1920929e-07 or not 0 <= token < self.vocab_size():
            return self.log_epsilon
        return max(float((w * self.log_pi_matrix[token, :w.numel()]).sum()) / tot, self.log_epsilon)

    def expectations(self, concept_dist) -> torch.Tensor:
        """`expectation` for every token at once: one matrix-vector product."""
        w = torch.as_tensor(concept_dist, dtype=torch.float32, device=self.log_pi_matrix.device).clamp(min=0.0)
        tot = w.sum()
        if float(tot) <= 1.1920929e-07:
            return torch.full((self.vocab_size(),), self.log_epsilon, device=w.device)
        return (self.log_pi_matrix @ (w / tot)).clamp(min=self.log_epsilon)

    def infer_from_window(self, window, smoothing: float = 0.0) -> torch.Tensor:
        """Concept distribution implied by weighted tokens `[(token, weight), ...]`; uniform when the
        window carries no mass."""
        C = self.concept_count()
        keep = [(t, w) for t, w in window if 0 <= t < self.vocab_size() and w > 0]
        acc = torch.full((C,), float(smoothing), device=self.log_pi_matrix.device)
        if keep:
            idx = torch.tensor([t for t, _ in keep], device=acc.device)
            wts = torch.tensor([w for _, w in keep], dtype=torch.float32, device=acc.device)
            acc = acc + wts @ torch.exp(self.log_pi_matrix[idx])
        tot = float(acc.sum())
        if tot <= 1.1920929e-07:
            return torch.full((C,), 1.0 / C, device=acc.device)
        return (acc / tot).clamp(min=1.1920929e-07)


def _gw_marginal(label: str, w) -> torch.Tensor:
    w = torch.as_tensor(w, dtype=torch.float32)
    if w.numel() == 0:
        raise TensorError("marginals cannot be empty")
    if not bool(torch.isfinite(w).all()) or bool((w < 0).any()):
        raise TensorError("marginals must be finite and non-negative")
    if float(w.sum()) <= 1.1920929e-07:
        raise TensorError("marginal sum must be positive")
    return w / w.sum()


class EntropicGwSolver:
    """Entropic Gromov-Wasserstein alignment of a symbol metric space to a concept metric space.

    Parity: crates/st-nn/src/language/gw.rs:96-330 (`solve`, Sinkhorn inner loop, anchor boost, the
    cooperative `propose` / `observe` self-tuning).  The reference evaluates the quadratic cost
    `sum_{i',j'} (Ds[i,i'] - Dz[j,j'])^2 pi[i',j']` with four nested loops; expanding the square gives
    `(Ds^2 a)[i] + (Dz^2 b)[j] - 2 (Ds pi Dz^T)[i,j]`, i.e. two GEMMs per outer iteration, and the
    Sinkhorn updates are matrix-vector products — everything stays on the inputs' device.
    """

    def __init__(self, epsilon: float = 0.5, anchor_strength: float = 3.0, max_iter: int = 25, sinkhorn_iter: int = 40):
        self.epsilon, self.anchor_strength, self.max_iter, self.sinkhorn_iter = epsilon, anchor_strength, max_iter, sinkhorn_iter

    def solve(self, symbol_distances, concept_distances, symbol_marginal, concept_marginal, anchors=()) -> SemanticBridge:
        ds = torch.as_tensor(symbol_distances, dtype=torch.float32)
        dz = torch.as_tensor(concept_distances, dtype=torch.float32).to(ds.device)
        if ds.dim() != 2 or ds.shape[0] != ds.shape[1] or dz.dim() != 2 or dz.shape[0] != dz.shape[1]:
            raise TensorError("distance matrices must be square")
        n, m = ds.shape[0], dz.shape[0]
        a, b = _gw_marginal("gw_symbol_marginal", symbol_marginal).to(ds.device), _gw_marginal("gw_concept_marginal", concept_marginal).to(ds.device)
        if a.numel() != n:
            raise TensorError("symbol marginal must match symbol distance matrix")
        if b.numel() != m:
            raise TensorError("concept marginal must match concept distance matrix")
        boost = torch.ones(n, m, device=ds.device)
        anchors = [(int(i), int(j)) for i, j in anchors if 0 <= i < n and 0 <= j < m]
        if anchors:
            ij = torch.tensor(anchors, device=ds.device)
            boost[ij[:, 0], ij[:, 1]] = math.exp(self.anchor_strength / self.epsilon)
        pi = a[:, None] * b[None, :]
        ds2, dz2 = ds * ds, dz * dz
        for _ in range(self.max_iter):
            cost = (ds2 @ pi.sum(1))[:, None] + (dz2 @ pi.sum(0))[None, :] - 2.0 * (ds @ pi @ dz.T)
            kern = (torch.exp(-cost / self.epsilon) * boost).clamp(min=1e-12)
            u, v = torch.ones(n, device=ds.device), torch.ones(m, device=ds.device)
            for _ in range(self.sinkhorn_iter):
                kv = kern @ v
                u = torch.where(kv > 0, a / kv, u)
                ku = kern.T @ u
                v = torch.where(ku > 0, b / ku, v)
            pi = kern * u[:, None] * v[None, :]
        return SemanticBridge.from_dense(pi.clamp(min=0.0), anchors, epsilon=1e-6) if float(pi.sum()) > 0 else \
            SemanticBridge.from_dense(a[:, None] * b[None, :], anchors)

    # cooperative self-tuning -------------------------------------------------------------------
    def propose(self) -> tuple:
        """(z_bias, weight) offered to a cooperative controller."""
        return math.tanh(self.anchor_strength - self.epsilon), max(self.anchor_strength + self.epsilon, 1e-3)

    def observe(self, team_reward: float, credit: float) -> None:
        c, r = math.tanh(credit), math.tanh(team_reward)
        cl = lambda x, lo, hi: min(max(x, lo), hi)
        if c >= 0:
            self.anchor_strength = cl(self.anchor_strength * (1 + 0.12 * c), 0.5, 24.0)
            self.epsilon = cl(self.epsilon * (1 - 0.04 * c), 1e-3, 8.0)
        else:
            self.anchor_strength = cl(self.anchor_strength * (1 - 0.05 * -c), 0.5, 24.0)
            self.epsilon = cl(self.epsilon * (1 + 0.1 * -c), 1e-3, 8.0)
        self.epsilon = cl(self.epsilon * (1 - 0.03 * r), 1e-3, 8.0)


# ---- concept hints, narrative hints and the Maxwell -> desire bridge --------------------------------------------------
class ConceptHint:
    """Either a concept distribution or a weighted token window (crates/st-nn/src/language/geometry.rs:752-870).
    ``as_distribution`` resolves both against a semantic bridge: a distribution is padded with 1e-6 to the concept
    count, clipped at zero and normalised (floor: float32 epsilon; uniform when it carries no mass); a window is
    pushed through the bridge's window inference."""

    def __init__(self, distribution=None, window=None):
        if (distribution is None) == (window is None):
            raise TensorError("a concept hint is either a distribution or a window")
        self.distribution = None if distribution is None else [float(v) for v in distribution]
        self.window = None if window is None else [(int(t), float(w)) for t, w in window]

    @classmethod
    def from_distribution(cls, dist) -> "ConceptHint":
        return cls(distribution=dist)

    @classmethod
    def from_window(cls, window) -> "ConceptHint":
        return cls(window=window)

    def as_distribution(self, bridge: SemanticBridge) -> list:
        c = bridge.concept_count()
        if self.window is not None:
            return [float(v) for v in bridge.infer_from_window(self.window, 1e-6).tolist()]
        if not self.distribution:
            return [1.0 / c] * c
        buf = [1e-6] * c
        for i, v in enumerate(self.distribution[:c]):
            buf[i] = v
        buf = [max(v, 0.0) if math.isfinite(v) else 0.0 for v in buf]
        s = sum(buf)
        if s <= 1.1920929e-07:
            return [1.0 / c] * c
        return [max(v / s, 1.1920929e-07) for v in buf]

    def snapshot(self, max_len: int = 256) -> dict:
        n = max(int(max_len), 1)
        if self.window is not None:
            return {"window": [[t, w] for t, w in self.window[:n]]}
        return {"distribution": self.distribution[:n]}


@dataclass
class NarrativeSummary:
    channel: str
    dominant_tag: Optional[str]
    tags: list
    intensity: float
    amplitude: float
    phase: float
    coherence: float
    decoherence: float
    emphasis: float

    def describe(self) -> str:
        what = f"tag `{self.dominant_tag}`" if self.dominant_tag is not None else "neutral"
        return (f"[{self.channel}] {what} emphasis {self.emphasis:.3f} (amp {self.amplitude:.3f}, coh {self.coherence:.2f}, "
                f"deco {self.decoherence:.2f})")

    __str__ = describe

    def as_dict(self) -> dict:
        return dict(self.__dict__)


class NarrativeHint:
    """Tags attached to a Maxwell channel with a small "quantum" state (crates/st-nn/src/language/maxwell.rs:15-170):
    the collapsed tag is the one maximising ``|amplitude| * coherence * (1 - decoherence) * max(|sin(phase + i * phi)|
    + 0.5, 1e-3)`` over tag positions ``i`` (phi = 1.618034); emphasis is the first three factors."""

    def __init__(self, channel: str, tags, intensity: float):
        self.channel, self.tags, self.intensity = str(channel), list(tags), float(intensity)
        self.amplitude, self.phase, self.coherence, self.decoherence = float(intensity), 0.0, 1.0, 0.0
        self.collapsed_tag: Optional[str] = None
        self._recompute()

    def _recompute(self) -> None:
        if not self.tags:
            self.collapsed_tag = None
            return
        base = max(1.0 - self.decoherence, 0.0)
        best, best_w = self.tags[0], -math.inf
        for i, tag in enumerate(self.tags):
            w = abs(self.amplitude) * self.coherence * base * max(abs(math.sin(self.phase + i * 1.618034)) + 0.5, 1e-3)
            if w > best_w:
                best, best_w = tag, w
        self.collapsed_tag = best

    def with_quantum_state(self, amplitude: float, phase: float, coherence: float, decoherence: float) -> "NarrativeHint":
        self.amplitude, self.phase = float(amplitude), float(phase)
        self.coherence, self.decoherence = min(max(coherence, 0.0), 1.0), min(max(decoherence, 0.0), 1.0)
        self._recompute()
        return self

    def collapse(self) -> "NarrativeHint":
        self._recompute()
        return self

    def dominant_tag(self) -> Optional[str]:
        return self.collapsed_tag if self.collapsed_tag is not None else (self.tags[0] if self.tags else None)

    def quantum_emphasis(self) -> float:
        a = abs(self.amplitude)
        return 0.0 if a <= 1.1920929e-07 else a * self.coherence * (1.0 - self.decoherence)

    def summary(self) -> NarrativeSummary:
        return NarrativeSummary(self.channel, self.dominant_tag(), list(self.tags), self.intensity, self.amplitude, self.phase,
                                self.coherence, self.decoherence, self.quantum_emphasis())


def _clean_tags(tags) -> list:
    out = []
    for t in tags or ():
        t = str(t).strip()
        if not t:
            raise TensorError("invalid value: narrative tag cannot be empty")
        out.append(t)
    return sorted(set(out))


class MaxwellDesireBridge:
    """Maps a Maxwell Z pulse on a named channel to a concept window (each registered ``(token, weight)`` becomes
    ``(weight + smoothing) * max(|z|, magnitude_floor)``) and, when the channel has tags, a narrative hint of
    intensity ``magnitude * gain`` (crates/st-nn/src/language/maxwell.rs:196-460)."""

    def __init__(self, smoothing: float = 1e-4, magnitude_floor: float = 0.0):
        self.smoothing, self.magnitude_floor = max(float(smoothing), 0.0), max(float(magnitude_floor), 0.0)
        self._channels: dict = {}

    def with_smoothing(self, s: float) -> "MaxwellDesireBridge":
        self.smoothing = max(float(s), 0.0)
        return self

    def with_magnitude_floor(self, f: float) -> "MaxwellDesireBridge":
        self.magnitude_floor = max(float(f), 0.0)
        return self

    def __len__(self) -> int:
        return len(self._channels)

    def is_empty(self) -> bool:
        return not self._channels

    def contains(self, channel: str) -> bool:
        return channel in self._channels

    def channel_names(self) -> list:
        return list(self._channels)

    def register_channel(self, channel: str, window, tags=(), gain: float = 1.0) -> None:
        if not str(channel).strip():
            raise TensorError("invalid value: channel name cannot be empty")
        window = list(window)
        if not window:
            raise TensorError("invalid value: Maxwell concept window cannot be empty")
        clean = []
        for tok, w in window:
            if not math.isfinite(w):
                raise TensorError("invalid value: window weight must be finite")
            if w < 0:
                raise TensorError("invalid value: window weight must be non-negative")
            clean.append((int(tok), float(w)))
        self._channels[str(channel)] = {"window": clean, "tags": _clean_tags(tags), "gain": max(float(gain), 0.0)}

    register_channel_with_narrative = register_channel

    def with_channel(self, channel: str, window, tags=()) -> "MaxwellDesireBridge":
        self.register_channel(channel, window, tags)
        return self

    with_channel_and_narrative = with_channel

    def _program(self, channel: str) -> dict:
        if channel not in self._channels:
            raise TensorError("invalid value: channel is not registered")
        return self._channels[channel]

    def set_narrative_tags(self, channel: str, tags) -> None:
        self._program(channel)["tags"] = _clean_tags(tags)

    def set_narrative_gain(self, channel: str, gain: float) -> None:
        self._program(channel)["gain"] = max(float(gain), 0.0)

    def narrative_tags(self, channel: str) -> Optional[list]:
        p = self._channels.get(channel)
        return None if p is None else list(p["tags"])

    def narrative_gain(self, channel: str) -> Optional[float]:
        p = self._channels.get(channel)
        return None if p is None else p["gain"]

    def hint_for(self, channel: str, pulse) -> Optional[ConceptHint]:
        p = self._channels.get(channel)
        if p is None or not p["window"]:
            return None
        mag = max(float(pulse.magnitude()), self.magnitude_floor)
        if mag <= 1.1920929e-07 and self.smoothing <= 1.1920929e-07:
            return None
        scaled = [(t, (max(w, 0.0) + self.smoothing) * mag) for t, w in p["window"]]
        scaled = [(t, v) for t, v in scaled if v > 1.1920929e-07]
        return ConceptHint.from_window(scaled) if scaled else None

    def narrative_for(self, channel: str, pulse) -> Optional[NarrativeHint]:
        p = self._channels.get(channel)
        if p is None or not p["tags"]:
            return None
        mag = max(float(pulse.magnitude()), self.magnitude_floor)
        intensity = mag * p["gain"]
        if mag <= 1.1920929e-07 or intensity <= 1.1920929e-07:
            return None
        above, here, beneath = pulse.band_energy
        coherence = min(max((above + beneath) / (above + here + beneath + 1e-6), 0.0), 1.0)
        se = abs(pulse.standard_error)
        phase = math.atan(pulse.z_score) * max(len(p["tags"]), 1)
        return NarrativeHint(channel, p["tags"], intensity).with_quantum_state(intensity, phase, coherence, min(se / (se + 1.0), 1.0)).collapse()

    def emit(self, channel: str, pulse):
        hint = self.hint_for(channel, pulse)
        return None if hint is None else (hint, self.narrative_for(channel, pulse))
