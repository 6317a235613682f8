"""BlackCat: a contextual-bandit picker of runtime knobs rewarded by step metrics.

Restated from crates/st-core/src/runtime/blackcat.rs: choice groups (knob → candidate values), one
linear bandit per candidate (ridge posterior ``A = λI + Σ x xᵀ``, ``b = Σ r x``; UCB score
``θ·x + c·sqrt(xᵀ A⁻¹ x)``, :4402-4520), ``choose(context)`` (:772) picks the best candidate of every
group and remembers the selection, ``post_step(metrics)`` (:879) turns ``StepMetrics`` into a utility
``-(λ_speed·t/scale + λ_mem·m/scale + λ_stab·retry/scale)`` (``RewardCfg`` :271-295) and credits the
pending selection once.  Invalid contexts are rejected without touching any state.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import plugin
from ..nn.trainer import StepMetrics


class BlackCatError(ValueError):
    pass


@dataclass
class RewardCfg:
    lam_speed: float = 0.5
    lam_mem: float = 0.3
    lam_stab: float = 0.2
    scale_speed: float = 10.0
    scale_mem: float = 1024.0
    scale_stab: float = 1.0

    def utility(self, m: StepMetrics) -> float:
        for v in (m.step_time_ms, m.mem_peak_mb, m.retry_rate):
            if not math.isfinite(v) or v < 0:
                raise BlackCatError("step metrics must be finite and non-negative")
        return -(self.lam_speed * m.step_time_ms / self.scale_speed + self.lam_mem * m.mem_peak_mb / self.scale_mem
                 + self.lam_stab * m.retry_rate / self.scale_stab)


class LinUcb:
    def __init__(self, dim: int, lam: float = 1.0):
        if dim <= 0 or not (lam > 0 and math.isfinite(lam)):
            raise BlackCatError("bandit needs a positive dimension and regularisation")
        self.dim = dim
        self.A = torch.eye(dim, dtype=torch.float64) * lam
        self.b = torch.zeros(dim, dtype=torch.float64)
        self.observations = 0

    def project(self, x: torch.Tensor) -> tuple:
        inv = torch.linalg.inv(self.A)
        theta = inv @ self.b
        return float(theta @ x), math.sqrt(max(float(x @ inv @ x), 0.0))

    def ucb_score(self, x: torch.Tensor, c: float) -> float:
        mean, std = self.project(x)
        return mean + c * std

    def update(self, x: torch.Tensor, reward: float) -> None:
        self.A += torch.outer(x, x)
        self.b += reward * x
        self.observations += 1


class BlackCat:
    def __init__(self, groups: dict, context_dim: int, reward: Optional[RewardCfg] = None, exploration: float = 1.0):
        if not groups or any(not v for v in groups.values()):
            raise BlackCatError("every choice group needs at least one candidate")
        if context_dim <= 0:
            raise BlackCatError("context dimension must be positive")
        self.groups = {g: [str(v) for v in vals] for g, vals in groups.items()}
        self.context_dim, self.reward, self.exploration = context_dim, reward or RewardCfg(), exploration
        self._bandits = {g: {v: LinUcb(context_dim) for v in vals} for g, vals in self.groups.items()}
        self._pending: Optional[tuple] = None
        self.selections, self.steps = 0, 0
        self.mean_utility = 0.0

    def _context(self, context) -> torch.Tensor:
        x = torch.as_tensor(context, dtype=torch.float64).reshape(-1)
        if x.numel() != self.context_dim:
            raise BlackCatError(f"context has {x.numel()} features, expected {self.context_dim}")
        if not bool(torch.isfinite(x).all()):
            raise BlackCatError("context must be finite")
        return x

    def try_choose(self, context) -> dict:
        return self.try_choose_with_hints(context, {})

    def choice_domains(self) -> dict:
        """Knob → the complete list of values the runtime may emit for it."""
        return {g: list(vals) for g, vals in self.groups.items()}

    def try_choose_with_hints(self, context, hints: dict) -> dict:
        """As ``try_choose``; a hinted value wins only among candidates whose upper confidence bounds are
        equivalent (within 1e-9), otherwise the bandit's own decision stands
        (crates/st-core/src/runtime/autopilot.rs:61-71 ``AutoMode::Hint``)."""
        x = self._context(context)          # a selection still pending is replaced: only the latest one is credited
        picks, witness = {}, {}
        for g, vals in self.groups.items():
            scores = [(self._bandits[g][v].ucb_score(x, self.exploration), -i, v) for i, v in enumerate(vals)]
            best = max(scores)
            pick = best[2]                     # ties go to the earlier candidate
            hinted = hints.get(g)
            if hinted is not None and hinted in vals:
                hs = next(sc for sc in scores if sc[2] == hinted)
                if abs(hs[0] - best[0]) <= 1e-9:
                    pick = hinted
            picks[g] = pick
            witness[g] = {"pick": pick, "score": best[0], "hinted": hinted if hinted in vals else None}
        self.selections += 1
        self._pending = (x, dict(picks))
        self._selection_id = self.selections
        self._witness = {"selection_id": self.selections, "groups": witness, "exploration": self.exploration}
        return picks

    def abandon_pending_selection(self) -> Optional[int]:
        """Drop the pending selection without crediting it; returns its id (None when nothing was pending)."""
        if self._pending is None:
            return None
        self._pending = None
        return getattr(self, "_selection_id", None)

    def last_selection_witness(self) -> Optional[dict]:
        return getattr(self, "_witness", None)

    def choose(self, context) -> dict:
        try:
            return self.try_choose(context)
        except BlackCatError as exc:
            if plugin.has_listeners("BlackCatChooseRejected"):
                plugin.publish("BlackCatChooseRejected", {"error": str(exc)})
            return {}

    def try_post_step(self, metrics: StepMetrics) -> float:
        u = self.reward.utility(metrics)
        self.steps += 1
        self.mean_utility += (u - self.mean_utility) / self.steps
        if self._pending is not None:
            x, picks = self._pending
            for g, v in picks.items():
                self._bandits[g][v].update(x, u)
            self._pending = None                # a selection is credited at most once
        return u

    def post_step(self, metrics: StepMetrics) -> float:
        try:
            return self.try_post_step(metrics)
        except BlackCatError as exc:
            if plugin.has_listeners("BlackCatRewardRejected"):
                plugin.publish("BlackCatRewardRejected", {"error": str(exc)})
            return -math.inf

    def observations(self, group: str, value: str) -> int:
        return self._bandits[group][str(value)].observations
