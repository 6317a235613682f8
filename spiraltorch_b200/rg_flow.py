"""Renormalisation-group flows on a log-scale lattice, and a channel-keyed gravity potential.

Parity: crates/st-core/src/theory/rg_flow.rs — `RgFlowLattice::{new_with_beta, from_mellin_grid, evaluate_mellin(_many),
fixed_points}` (:93-222), `RgFlowNode` / `ScaleFixedPoint` (:32-82); crates/st-core/src/theory/renormalization_flow.rs —
`ResonanceProfile` (:24-68), `RGOperator` (:70-98), `RGFlowModel::{new, from_lattice, propagate, sample_beta,
narrative_depth, gaussian_resonance, breathing_resonance}` (:124-292) with ``beta = (Delta - 4) g + c g^2 + Re
resonance(log mu) - damping g``; crates/st-core/src/theory/gravity.rs — `GravityField::potential` (:58-67).

`RGFlowModel.propagate` advances every registered operator together: the resonance drive of each operator does not
depend on the couplings, so it is evaluated for the whole lattice in one Mellin plan (a vertical line ``s = pole + i log
mu``) before the Euler recurrence runs as vector updates over the operators.
"""
from __future__ import annotations

import cmath
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from . import observability
from .mellin import MellinError, MellinEvalPlan, MellinLogGrid


class RgFlowError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass
class RgFlowNode:
    log_scale: float
    scale: float
    couplings: List[float]
    beta: List[float]

    def narrative_depth(self) -> float:
        return self.scale

    def beta_norm(self) -> float:
        return math.sqrt(sum(b * b for b in self.beta))


@dataclass
class ScaleFixedPoint:
    log_scale: float
    scale: float
    couplings: List[float]

    def narrative_depth(self) -> float:
        return self.scale


class RgFlowLattice:
    """Explicit Euler integration ``g_{k+1} = g_k + h beta(log mu_k, g_k)`` of a user beta function over a log lattice."""

    def __init__(self, log_start: float, log_step: float, nodes: List[RgFlowNode], mellin_series: Optional[torch.Tensor] = None):
        self.log_start, self.log_step, self.nodes, self._mellin = log_start, log_step, nodes, mellin_series

    @classmethod
    def new_with_beta(cls, log_start: float, log_step: float, steps: int, root_couplings: Sequence[float],
                      beta: Callable[[float, List[float]], Sequence[float]]) -> "RgFlowLattice":
        if not math.isfinite(log_start):
            raise RgFlowError("invalid_log_start", "log_start must be finite")
        if not (math.isfinite(log_step) and log_step > 0.0):
            raise RgFlowError("invalid_log_step", "log_step must be positive and finite")
        if steps == 0:
            raise RgFlowError("empty_lattice", "RG flow requires at least one lattice step")
        current = [float(c) for c in root_couplings]
        if not current:
            raise RgFlowError("empty_couplings", "at least one coupling is required")
        nodes, log_scale = [], float(log_start)
        for step in range(steps):
            b = [float(v) for v in beta(log_scale, list(current))]
            if len(b) != len(current):
                raise RgFlowError("beta_dimension", f"beta function returned {len(b)} entries, expected {len(current)}")
            nodes.append(RgFlowNode(log_scale, math.exp(log_scale), list(current), b))
            if step + 1 < steps:
                current = [c + log_step * d for c, d in zip(current, b)]
                log_scale += log_step
        return cls(float(log_start), float(log_step), nodes)

    @classmethod
    def from_mellin_grid(cls, grid: MellinLogGrid, root_couplings: Sequence[float], beta) -> "RgFlowLattice":
        lattice = cls.new_with_beta(grid.log_start, grid.log_step, len(grid), root_couplings, beta)
        lattice._mellin = grid.weighted_series()
        return lattice

    def __len__(self) -> int:
        return len(self.nodes)

    def mellin_series(self) -> Optional[torch.Tensor]:
        return self._mellin

    def evaluate_mellin_many(self, s_values) -> torch.Tensor:
        if self._mellin is None:
            raise RgFlowError("missing_mellin_series", "Mellin projection unavailable for this flow")
        return MellinEvalPlan.many(self.log_start, self.log_step, s_values).evaluate(self._mellin)

    def evaluate_mellin(self, s: complex) -> complex:
        return complex(self.evaluate_mellin_many([complex(s)])[0])

    def fixed_points(self, tolerance: float) -> List[ScaleFixedPoint]:
        points = [ScaleFixedPoint(n.log_scale, n.scale, list(n.couplings)) for n in self.nodes if n.beta_norm() <= tolerance]
        dim = len(self.nodes[0].couplings) if self.nodes else 0
        observability.emit_tensor_op("rg_flow_fixed_points", (len(self.nodes), dim), (len(points), max(dim, 1)))

        def meta():
            norms = [n.beta_norm() for n in self.nodes if math.isfinite(n.beta_norm())]
            return {"backend": "host", "kind": "rg_flow_fixed_points", "nodes": len(self.nodes), "coupling_dim": dim,
                    "fixed_points": len(points), "tolerance": tolerance if math.isfinite(tolerance) else 0.0, "log_start": self.log_start,
                    "log_step": self.log_step, "has_mellin_series": self._mellin is not None,
                    "beta_norm_min": min(norms, default=0.0), "beta_norm_mean": sum(norms) / max(len(self.nodes), 1),
                    "beta_norm_max": max(norms, default=0.0), "fixed_scale_min": min((p.scale for p in points), default=0.0),
                    "fixed_scale_max": max((p.scale for p in points), default=0.0)}
        observability.emit_tensor_op_meta("rg_flow_fixed_points", meta)
        return points


# ---- operator flows with Mellin resonances --------------------------------------------------------------------------------
class ResonanceProfile:
    """``residue * M[grid](pole + i log mu)``: a drive that breathes with the log scale."""

    def __init__(self, grid: MellinLogGrid, pole: complex, residue: complex = 1.0 + 0j):
        self.grid, self.pole, self.residue = grid, complex(pole), complex(residue)

    def evaluate(self, log_scale: float) -> complex:
        return self.grid.evaluate(complex(self.pole.real, self.pole.imag + log_scale)) * self.residue

    def evaluate_lattice(self, log_scales: Sequence[float]) -> torch.Tensor:
        imag = torch.as_tensor(log_scales, dtype=torch.float64) + self.pole.imag
        return self.grid.evaluate_vertical_line(self.pole.real, imag) * self.residue


@dataclass
class RGOperator:
    name: str
    scaling_dimension: float
    initial_coupling: float
    resonance: Optional[ResonanceProfile] = None
    nonlinear_feedback: float = 0.0

    def with_resonance(self, resonance: ResonanceProfile) -> "RGOperator":
        self.resonance = resonance
        return self

    def with_nonlinear_feedback(self, coefficient: float) -> "RGOperator":
        self.nonlinear_feedback = float(coefficient)
        return self


@dataclass
class RGFlowTrajectory:
    name: str
    values: List[float]

    def at(self, index: int) -> Optional[float]:
        return self.values[index] if 0 <= index < len(self.values) else None


class RGFlowSolution:
    def __init__(self, lattice: List[float], trajectories: List[RGFlowTrajectory], tensor: torch.Tensor):
        self.lattice, self.trajectories, self.tensor = lattice, trajectories, tensor        # tensor: [operators, depth]

    def trajectory(self, name: str) -> Optional[RGFlowTrajectory]:
        return next((t for t in self.trajectories if t.name == name), None)

    def __iter__(self):
        return iter(self.trajectories)


class RGFlowModel:
    def __init__(self, log_start: float, log_step: float, depth: int):
        if depth == 0:
            raise RgFlowError("empty_lattice", "log lattice must contain at least one point")
        if not (math.isfinite(log_step) and log_step > 0.0):
            raise RgFlowError("invalid_log_step", "log step must be finite and positive")
        self.log_step = float(log_step)
        self.lattice = [log_start + log_step * i for i in range(depth)]
        self.operators: List[RGOperator] = []
        self.damping = 0.0

    @classmethod
    def from_lattice(cls, lattice: Sequence[float]) -> "RGFlowModel":
        lattice = [float(v) for v in lattice]
        if not lattice:
            raise RgFlowError("empty_lattice", "log lattice must contain at least one point")
        model = cls.__new__(cls)
        model.log_step = lattice[1] - lattice[0] if len(lattice) > 1 else 1.0
        model.lattice, model.operators, model.damping = lattice, [], 0.0
        return model

    @classmethod
    def narrative_depth(cls, depth: int, start: float) -> "RGFlowModel":
        """A lattice whose total span is the golden-ratio conjugate, however many levels it has."""
        golden = (math.sqrt(5.0) - 1.0) / 2.0
        return cls(start, max(golden / max(depth, 1), 1e-3), depth)

    def register_operator(self, operator: RGOperator) -> None:
        self.operators.append(operator)

    def _beta_parts(self):
        ops = self.operators
        linear = torch.tensor([o.scaling_dimension - 4.0 for o in ops], dtype=torch.float64)
        if self.damping > 0.0:
            linear = linear - self.damping
        quad = torch.tensor([o.nonlinear_feedback for o in ops], dtype=torch.float64)
        drive = torch.zeros(len(ops), len(self.lattice), dtype=torch.float64)
        for i, o in enumerate(ops):
            if o.resonance is not None:
                drive[i] = o.resonance.evaluate_lattice(self.lattice).real
        return linear, quad, drive

    def propagate(self) -> RGFlowSolution:
        depth = len(self.lattice)
        if not self.operators:
            solution = RGFlowSolution(list(self.lattice), [], torch.zeros(0, depth, dtype=torch.float64))
            self._emit(solution)
            return solution
        linear, quad, drive = self._beta_parts()
        values = torch.zeros(len(self.operators), depth, dtype=torch.float64)
        g = torch.tensor([o.initial_coupling for o in self.operators], dtype=torch.float64)
        values[:, 0] = g
        for k in range(1, depth):
            g = g + self.log_step * (linear * g + quad * g * g + drive[:, k])
            values[:, k] = g
        solution = RGFlowSolution(list(self.lattice), [RGFlowTrajectory(o.name, values[i].tolist()) for i, o in enumerate(self.operators)], values)
        self._emit(solution)
        return solution

    def sample_beta(self, coupling: float, operator_index: int, log_scale: float) -> float:
        if not 0 <= operator_index < len(self.operators):
            raise RgFlowError("initial_couplings", f"initial couplings mismatch: expected {len(self.operators)}, got {operator_index}")
        o = self.operators[operator_index]
        res = o.resonance.evaluate(log_scale).real if o.resonance is not None else 0.0
        damp = -self.damping * coupling if self.damping > 0.0 else 0.0
        return (o.scaling_dimension - 4.0) * coupling + o.nonlinear_feedback * coupling * coupling + res + damp

    @staticmethod
    def gaussian_resonance(log_start: float, log_step: float, n: int, center: float, bandwidth: float, amplitude: float) -> ResonanceProfile:
        """A Gaussian bump of the abscissa around `center`, sampled on the lattice, with its pole at ``s = 2``."""
        sigma = max(bandwidth, 1e-3)
        grid = MellinLogGrid.from_function(log_start, log_step, n, lambda x: amplitude * torch.exp(-0.5 * ((x - center) / sigma) ** 2))
        return ResonanceProfile(grid, 2.0 + 0j, 1.0 + 0j)

    @staticmethod
    def breathing_resonance(grid: MellinLogGrid, pole: complex, phase: float, strength: float) -> ResonanceProfile:
        return ResonanceProfile(grid, pole, cmath.rect(strength, phase))

    def _emit(self, solution: RGFlowSolution) -> None:
        n = len(self.operators)
        observability.emit_tensor_op("rg_mellin_flow_propagate", (len(solution.lattice), max(n, 1)), (max(n, 1), max(len(solution.lattice), 1)))

        def meta():
            t = solution.tensor
            fin = torch.isfinite(t)
            return {"backend": "torch", "kind": "rg_mellin_flow_propagate", "operator_count": n, "lattice_len": len(solution.lattice),
                    "log_step": self.log_step, "damping": self.damping, "resonance_count": sum(o.resonance is not None for o in self.operators),
                    "nonlinear_count": sum(abs(o.nonlinear_feedback) > 1.2e-7 for o in self.operators),
                    "unstable_trajectory_count": int((~fin.all(1)).sum()) if n else 0,
                    "final_abs_mean": float(t[:, -1].abs().mean()) if n else 0.0, "max_abs_coupling": float(t[fin].abs().max()) if n and fin.any() else 0.0,
                    "drift_abs_mean": float((t[:, -1] - t[:, 0]).abs().mean()) if n else 0.0}
        observability.emit_tensor_op_meta("rg_mellin_flow_propagate", meta)


# ---- gravity ---------------------------------------------------------------------------------------------------------------
@dataclass
class GravityWell:
    mass: float
    speed_of_light: Optional[float] = None              # None: Newtonian; a value: the potential is damped by 1 / (1 + r / c)

    @classmethod
    def newtonian(cls, mass: float) -> "GravityWell":
        return cls(mass)

    @classmethod
    def relativistic(cls, mass: float, speed_of_light: float) -> "GravityWell":
        return cls(mass, speed_of_light)

    def factor(self, radius: float) -> float:
        return 1.0 if self.speed_of_light is None else 1.0 / (1.0 + radius / max(self.speed_of_light, 1e-6))


class GravityField:
    """``-G m / r`` per named channel (times the well's relativistic factor); 0 inside ``r <= 1e-6``."""

    def __init__(self, constant: float = 6.67430e-11, wells: Optional[Dict[str, GravityWell]] = None):
        self.constant, self.wells = float(constant), dict(wells or {})

    def add_well(self, channel: str, well: GravityWell) -> None:
        self.wells[channel] = well

    def potential(self, channel: str, radius: float) -> Optional[float]:
        well = self.wells.get(channel)
        if well is None:
            return None
        if radius <= 1e-6:
            return 0.0
        return -self.constant * well.mass / radius * well.factor(radius)

    def __call__(self, channel: str, radius: float) -> float:
        """The callable form `robotics.DesireLagrangianField` takes for its gravity term."""
        return self.potential(channel, radius) or 0.0
