"""The "sync theorems" bridge between a structural Bures gap and an observation-side e-process.

Each sample carries a running log e-value; one step adds the expected increment 2 cos^2(phi) Delta_B^2 - epsilon, the
structure gate opens where Delta_B^2 >= tau_B (after an optional slew lag), the observation gate where the log e-value
reaches ln(1 / alpha), and the pair of gates gives an I x K label: critical (both open), safe (both closed and the
anytime confidence 1 - exp(-log e) at least 1 - alpha) or abstain.  A family of pairs is folded into one signal by
averaging the log e-values and combining the structure gates under an any / all / majority policy.

Reference parity: crates/st-core/src/theory/sync_bridge.rs (`SyncConfig` :54-149, `SyncStep` :185-204,
`FamilyStructurePolicy` / `FamilyAggregation` :207-252, `SyncTheoremTrainer` :255-557, telemetry :559-690).  The state
and every step are tensors, so a batch of any size advances in a handful of element-wise operations, and
:meth:`SyncTheoremTrainer.run` replaces the reference's step-per-sample loop for a trajectory with one cumulative sum.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch

from . import observability as _obs

CRITICAL, SAFE, ABSTAIN = 0, 1, 2
LABEL_NAMES = ("critical", "safe", "abstain")
FAMILY_POLICIES = ("any", "all", "majority")
_Arr = Union[torch.Tensor, Sequence[float]]


class SyncError(ValueError):
    pass


class SyncConfig:
    def __init__(self, alpha: float, tau_b: float, epsilon_max: float, cos_phi_min: float, slew_steps: int = 0):
        if not 0.0 <= alpha < 1.0:
            raise SyncError(f"alpha must be in (0, 1), received {alpha}")
        if not (math.isfinite(tau_b) and tau_b > 0.0):
            raise SyncError(f"tau_b must be positive, received {tau_b}")
        if epsilon_max < 0.0 or not math.isfinite(epsilon_max):
            raise SyncError(f"epsilon_max must be non-negative, received {epsilon_max}")
        if not (math.isfinite(cos_phi_min) and 0.0 < cos_phi_min <= 1.0):
            raise SyncError(f"cos_phi_min must lie in (0, 1], received {cos_phi_min}")
        self.alpha, self.tau_b, self.epsilon_max, self.cos_phi_min = float(alpha), float(tau_b), float(epsilon_max), float(cos_phi_min)
        self.slew_steps = int(slew_steps)
        self.azuma_c: Optional[float] = None

    def with_azuma_c(self, azuma_c: float) -> "SyncConfig":
        if not (math.isfinite(azuma_c) and azuma_c > 0.0):
            raise SyncError(f"azuma coefficient must be positive, received {azuma_c}")
        self.azuma_c = float(azuma_c)
        return self

    def threshold(self) -> float:
        """ln(1 / alpha): the level at which the e-process rejects at size alpha."""
        return math.log(1.0 / self.alpha) if self.alpha > 0.0 else math.inf

    def hitting_time_bound(self) -> float:
        """Steps until the observation gate opens at the worst admissible drift 2 tau_B cos^2 - epsilon_max."""
        denom = 2.0 * self.tau_b * self.cos_phi_min - self.epsilon_max
        if denom <= 0.0:
            raise SyncError(f"expected positive observation drift, denominator = {denom}")
        return self.threshold() / denom

    def hitting_time_tail(self, delta: float) -> Optional[float]:
        """Azuma-Hoeffding bound exp(-c delta^2) on overshooting the hitting-time bound by ``delta`` (None without c)."""
        if self.azuma_c is None:
            return None
        return 1.0 if delta <= 0.0 else math.exp(-self.azuma_c * delta * delta)


@dataclass
class SyncStep:
    log_e: torch.Tensor
    structure_gate: torch.Tensor          # bool
    observation_gate: torch.Tensor        # bool
    labels: torch.Tensor                  # int8: CRITICAL / SAFE / ABSTAIN
    hitting_time_bound: float
    increment: torch.Tensor
    confidence: torch.Tensor
    effective_delta_b_sq: torch.Tensor

    def label_names(self) -> List[str]:
        return [LABEL_NAMES[int(v)] for v in self.labels.tolist()]


@dataclass
class FamilyAggregation:
    log_e_family: float
    confidence: float
    structure_gate: bool
    observation_gate: bool
    label: str
    pair_count: int
    dominant_pair: Optional[int]
    dominant_log_e: Optional[float]


def _label(structure: torch.Tensor, observation: torch.Tensor, confidence: torch.Tensor, alpha: float) -> torch.Tensor:
    safe = ~structure & ~observation & (confidence >= 1.0 - alpha)
    return torch.where(structure & observation, CRITICAL, torch.where(safe, SAFE, ABSTAIN)).to(torch.int8)


class SyncTheoremTrainer:
    def __init__(self, config: SyncConfig):
        self.config = config
        self._log_e: Optional[torch.Tensor] = None
        self.log_e_mean = 0.0
        self.iteration = 0

    def reset(self) -> None:
        self._log_e, self.log_e_mean, self.iteration = None, 0.0, 0

    def set_log_e(self, log_e: _Arr) -> None:
        self._log_e = torch.as_tensor(log_e, dtype=torch.float32).clone()
        self.log_e_mean = float(self._log_e.mean()) if self._log_e.numel() else 0.0

    def log_e(self) -> torch.Tensor:
        return self._log_e if self._log_e is not None else torch.zeros(0)

    def threshold(self) -> float:
        return self.config.threshold()

    def _vec(self, name: str, values: Optional[_Arr], like: torch.Tensor, fallback: float) -> torch.Tensor:
        if values is None:
            return torch.full_like(like, fallback)
        v = torch.as_tensor(values, dtype=torch.float32, device=like.device)
        if v.shape != like.shape:
            raise SyncError(f"length mismatch for {name}: expected {like.numel()}, got {v.numel()}")
        return v

    def expected_increment_profile(self, delta_b_sq: _Arr, epsilon: _Arr, cos_sq_phi: Optional[_Arr] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(increment, misalignment-adjusted gap): 2 cos^2(phi) Delta_B^2 - epsilon and cos^2(phi) Delta_B^2."""
        d = torch.as_tensor(delta_b_sq, dtype=torch.float32)
        eps = self._vec("epsilon", epsilon, d, 0.0)
        cos = self._vec("cos_sq_phi", cos_sq_phi, d, self.config.cos_phi_min)
        eff = d * cos
        return 2.0 * eff - eps, eff

    def expected_increment(self, delta_b_sq: _Arr, epsilon: _Arr, cos_sq_phi: Optional[_Arr] = None) -> torch.Tensor:
        return self.expected_increment_profile(delta_b_sq, epsilon, cos_sq_phi)[0]

    def step(self, delta_b_sq: _Arr, epsilon: Optional[_Arr] = None, cos_sq_phi: Optional[_Arr] = None) -> SyncStep:
        cfg = self.config
        d = torch.as_tensor(delta_b_sq, dtype=torch.float32).flatten()
        bound = cfg.hitting_time_bound()
        if d.numel() == 0:
            z = torch.zeros(0)
            step = SyncStep(z, z.bool(), z.bool(), z.to(torch.int8), bound, z, z, z)
            self._emit_step(step)
            return step
        eps = self._vec("epsilon", epsilon, d, cfg.epsilon_max)
        inc, eff = self.expected_increment_profile(d, eps, self._vec("cos_sq_phi", cos_sq_phi, d, cfg.cos_phi_min))
        if self._log_e is None or self._log_e.shape != d.shape or self._log_e.device != d.device:
            self._log_e = torch.zeros_like(d)
        self._log_e = self._log_e + inc
        self.iteration += 1
        structure = d >= cfg.tau_b
        if cfg.slew_steps > 0 and self.iteration <= cfg.slew_steps:
            structure = torch.zeros_like(structure)
        log_e = self._log_e.clone()
        observation = log_e >= self.threshold()
        confidence = 1.0 - torch.exp(-log_e)
        self.log_e_mean = float(log_e.mean())
        step = SyncStep(log_e, structure, observation, _label(structure, observation, confidence, cfg.alpha), bound, inc, confidence, eff)
        self._emit_step(step)
        return step

    def run(self, delta_b_sq: _Arr, epsilon: Optional[_Arr] = None, cos_sq_phi: Optional[_Arr] = None) -> Tuple[torch.Tensor, Optional[int]]:
        """One sample followed through ``len(delta_b_sq)`` steps: the log e trajectory and the first step at which the
        observation gate is open (None if it never opens).  The sample is slot 0 of the trainer's state."""
        d = torch.as_tensor(delta_b_sq, dtype=torch.float32).flatten()
        if d.numel() == 0:
            return torch.zeros(0), None
        eps = self._vec("epsilon", epsilon, d, self.config.epsilon_max)
        inc, _ = self.expected_increment_profile(d, eps, self._vec("cos_sq_phi", cos_sq_phi, d, self.config.cos_phi_min))
        self.config.hitting_time_bound()                      # a non-positive worst-case drift is an error, as in step()
        start = self._log_e[:1].to(d.device) if self._log_e is not None and self._log_e.numel() == 1 else torch.zeros(1, device=d.device)
        traj = start + torch.cumsum(inc, 0)
        self._log_e = traj[-1:].clone()
        self.log_e_mean = float(traj[-1])
        self.iteration += d.numel()
        hits = torch.nonzero(traj >= self.threshold())
        return traj, (int(hits[0]) if hits.numel() else None)

    def aggregate_family(self, step: SyncStep, policy: str = "any") -> FamilyAggregation:
        if policy not in FAMILY_POLICIES:
            raise SyncError(f"unknown family policy {policy!r}; one of {FAMILY_POLICIES}")
        n = step.log_e.numel()
        if n == 0:
            raise SyncError("family aggregation requires at least one pair contribution")
        log_family = float(step.log_e.mean())
        confidence = 1.0 - math.exp(-log_family)
        gates = step.structure_gate
        structure = bool(gates.any()) if policy == "any" else bool(gates.all()) if policy == "all" else int(gates.sum()) * 2 > n
        observation = log_family >= self.threshold()
        label = "critical" if structure and observation else "safe" if (not structure and not observation and confidence >= 1.0 - self.config.alpha) else "abstain"
        dom = int(torch.argmax(step.log_e))
        agg = FamilyAggregation(log_family, confidence, structure, observation, label, n, dom, float(step.log_e[dom]))
        _obs.emit_tensor_op("sync_family_aggregate", [n], [1, 6])
        _obs.emit_tensor_op_meta("sync_family_aggregate", lambda: {
            "backend": "cpu", "requested_backend": "auto", "kind": "st_core_sync_family_aggregate", "policy": policy, "pair_count": n,
            "log_e_family": log_family, "confidence": confidence, "structure_gate": structure, "observation_gate": observation,
            "label": label, "dominant_pair": dom, "threshold": self.threshold(), "alpha": self.config.alpha})
        return agg

    def _emit_step(self, step: SyncStep) -> None:
        n = step.log_e.numel()
        _obs.emit_tensor_op("sync_theorem_step", [n, 3], [max(n, 1), 5])

        def build():
            def stats(t: torch.Tensor):
                t = t[torch.isfinite(t)]
                return (float(t.min()), float(t.max()), float(t.mean())) if t.numel() else (0.0, 0.0, 0.0)
            lo, hi, mean = stats(step.log_e)
            counts = torch.bincount(step.labels.to(torch.int64), minlength=3).tolist() if n else [0, 0, 0]
            cfg = self.config
            return {"backend": "cpu" if step.log_e.device.type == "cpu" else "cuda", "requested_backend": "auto", "kind": "st_core_sync_theorem_step",
                    "iteration": self.iteration, "batch": n, "alpha": cfg.alpha, "tau_b": cfg.tau_b, "epsilon_max": cfg.epsilon_max,
                    "cos_phi_min": cfg.cos_phi_min, "slew_steps": cfg.slew_steps, "threshold": cfg.threshold(),
                    "hitting_time_bound": step.hitting_time_bound, "log_e_min": lo, "log_e_max": hi, "log_e_mean": mean,
                    "structure_open": int(step.structure_gate.sum()), "observation_open": int(step.observation_gate.sum()),
                    "critical": counts[CRITICAL], "safe": counts[SAFE], "abstain": counts[ABSTAIN], "has_azuma_c": cfg.azuma_c is not None}
        _obs.emit_tensor_op_meta("sync_theorem_step", build)
