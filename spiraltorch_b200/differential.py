"""Spiral differentials: homotopy flows, functor linearisation, the recursive barycenter path and the
hierarchy of levels, resonating together under one topos.

Parity: crates/st-tensor/src/pure/differential.rs:119-760 (`HomotopyDifferential`, `FunctorDifferential`,
`RecursiveDifferential`, `InfinityDifferential`, `DifferentialResonance`, `SpiralDifferential`).
All arithmetic is vectorised torch on the operands' device; the functor products go through `Tensor.matmul`
(the tcgen05 GEMM on a GPU).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .measure import ZSpaceBarycenter
from .tensor import Tensor, TensorError
from .topos import OpenCartesianTopos


def _finite(label: str, t: Tensor) -> torch.Tensor:
    raw = t.torch()
    if not bool(torch.isfinite(raw).all()):
        raise TensorError(f"non-finite value for {label}")
    return raw


def _same(a: Tensor, b: Tensor) -> None:
    if a.shape() != b.shape():
        raise TensorError(f"shape mismatch: {a.shape()} vs {b.shape()}")


def _guarded(topos: Optional[OpenCartesianTopos], label: str, raw: torch.Tensor) -> Tensor:
    if topos is None:
        return Tensor._wrap(raw)
    out = topos.saturate(raw.float())
    topos.guard_tensor(label, out)
    return Tensor._wrap(out)


class HomotopyDifferential:
    """`flow(x) = x + generator * direction` (element-wise); the commutator of two flows measures how far
    they are from commuting at the seed."""

    def __init__(self, seed: Tensor, generator: Tensor, direction: Tensor):
        _same(generator, seed)
        _same(direction, seed)
        for label, t in (("homotopy_seed", seed), ("homotopy_generator", generator), ("homotopy_direction", direction)):
            _finite(label, t)
        self.seed, self.generator, self.direction = seed, generator, direction

    def flow_from(self, state: Tensor) -> Tensor:
        _same(state, self.seed)
        return Tensor._wrap(_finite("homotopy_state", state) + self.generator.torch() * self.direction.torch())

    def flow(self) -> Tensor:
        return self.flow_from(self.seed)

    def flow_guarded(self, topos: OpenCartesianTopos) -> Tensor:
        return _guarded(topos, "homotopy_flow", self.flow().torch())

    def commutator(self, other: "HomotopyDifferential", topos: Optional[OpenCartesianTopos] = None) -> Tensor:
        _same(self.seed, other.seed)
        forward = other.flow_from(self.flow_from(self.seed)).torch()
        backward = self.flow_from(other.flow_from(self.seed)).torch()
        return _guarded(topos, "homotopy_commutator", forward - backward)

    def directional_energy(self) -> float:
        return float(((self.generator.torch().double() * self.direction.torch().double()) ** 2).sum())


class FunctorDifferential:
    """A linear functor `X -> X K`; `linearise(d) = d K` is its differential in direction `d`."""

    def __init__(self, source: Tensor, kernel: Tensor, epsilon: float):
        if not math.isfinite(epsilon):
            raise TensorError(f"non-finite value for functor_epsilon: {epsilon}")
        if epsilon <= 0:
            raise TensorError(f"learning rate must be positive, got {epsilon}")
        if source.shape()[1] != kernel.shape()[0]:
            raise TensorError(f"shape mismatch: {source.shape()} vs {kernel.shape()}")
        _finite("functor_source", source)
        _finite("functor_kernel", kernel)
        self.source, self.kernel, self.epsilon = source, kernel, float(epsilon)

    def apply(self) -> Tensor:
        return self.source.matmul(self.kernel)

    def apply_to(self, functional: Tensor) -> Tensor:
        if functional.shape()[1] != self.kernel.shape()[0]:
            raise TensorError(f"shape mismatch: {functional.shape()} vs {self.kernel.shape()}")
        return functional.matmul(self.kernel)

    def linearise(self, direction: Tensor) -> Tensor:
        _same(direction, self.source)
        return direction.matmul(self.kernel)


class RecursiveDifferential:
    """The barycenter's interpolation path as a differential: interpolations must rise within [0, 1], the
    objective must not rise along the path, and the path must end at the barycenter density."""

    def __init__(self, barycenter: ZSpaceBarycenter):
        for label in ("kl_energy", "entropy", "coupling_energy", "objective", "effective_weight"):
            v = getattr(barycenter, label)
            if not math.isfinite(v):
                raise TensorError(f"non-finite value for recursive_barycenter_{label}: {v}")
        if barycenter.kl_energy < -1e-6 or barycenter.entropy < 0 or barycenter.coupling_energy < 0:
            raise TensorError("invalid value: recursive_barycenter_energy")
        if barycenter.effective_weight <= 0:
            raise TensorError(f"degenerate barycenter: effective weight {barycenter.effective_weight}")
        if not barycenter.intermediates:
            raise TensorError("empty input: recursive_barycenter_intermediates")
        prev_a, prev_obj = -math.inf, math.inf
        for st in barycenter.intermediates:
            _same(st.density, barycenter.density)
            d = _finite("recursive_intermediate_density", st.density)
            if bool((d < 0).any()) or abs(float(d.sum()) - 1.0) > 1e-3:
                raise TensorError("invalid value: recursive_intermediate_density is not a probability tensor")
            if not 0.0 <= st.interpolation <= 1.0 or st.interpolation < prev_a:
                raise TensorError("invalid value: recursive_interpolation")
            if st.objective > prev_obj + 1e-4:
                raise TensorError("invalid value: recursive_objective_curve")
            prev_a, prev_obj = st.interpolation, st.objective
        if float((barycenter.intermediates[-1].density.torch() - barycenter.density.torch()).abs().max()) > 1e-4:
            raise TensorError("invalid value: recursive_barycenter_endpoint")
        self.barycenter = barycenter

    @classmethod
    def from_barycenter(cls, barycenter: ZSpaceBarycenter) -> "RecursiveDifferential":
        return cls(barycenter)

    def density(self) -> Tensor:
        return self.barycenter.density

    def intermediates(self) -> list:
        return self.barycenter.intermediates

    def objective_curve(self) -> list:
        return [s.objective for s in self.barycenter.intermediates]

    def kl_curve(self) -> list:
        return [s.kl_energy for s in self.barycenter.intermediates]

    def entropy_curve(self) -> list:
        return [s.entropy for s in self.barycenter.intermediates]

    def objective_curve_tensor(self) -> Tensor:
        return Tensor._wrap(torch.tensor([self.objective_curve()], dtype=torch.float32))

    def accumulate(self, hypergrad) -> None:
        hypergrad.accumulate_barycenter_path(self.barycenter.intermediates)


class InfinityDifferential:
    """A tower of same-shaped levels: `collapse` is their mean, the hierarchical energy `|c_i| * ||L_i||^2`."""

    def __init__(self, levels: Sequence[Tensor], curvatures: Sequence[float] = ()):
        if not levels:
            raise TensorError("empty input: infinity_levels")
        if curvatures and len(curvatures) != len(levels):
            raise TensorError(f"data length mismatch: expected {len(levels)}, got {len(curvatures)}")
        for lv in levels:
            _same(lv, levels[0])
            _finite("infinity_level", lv)
        if not all(math.isfinite(c) for c in curvatures):
            raise TensorError("non-finite value for infinity_curvature")
        self.levels, self.curvatures = list(levels), [float(c) for c in curvatures]

    def shape(self) -> tuple:
        return self.levels[0].shape()

    def collapse(self) -> Tensor:
        return Tensor._wrap(torch.stack([lv.torch().double() for lv in self.levels]).mean(0).float())

    def hierarchical_energy_tensor(self) -> Tensor:
        e = [float((lv.torch().double() ** 2).sum()) * abs(self.curvatures[i] if self.curvatures else 1.0)
             for i, lv in enumerate(self.levels)]
        return Tensor._wrap(torch.tensor([e], dtype=torch.float32))


@dataclass
class DifferentialResonance:
    homotopy_flow: Tensor
    functor_linearisation: Tensor
    recursive_objective: Tensor
    infinity_projection: Tensor
    infinity_energy: Tensor


class SpiralDifferential:
    """The four differentials over one shape; `resonate` evaluates them (saturated and guarded by the topos
    when there is one) and optionally feeds the barycenter path to a hypergrad tape."""

    def __init__(self, topos: Optional[OpenCartesianTopos], homotopy: HomotopyDifferential, functor: FunctorDifferential,
                 recursive: RecursiveDifferential, infinity: InfinityDifferential):
        shape = homotopy.seed.shape()
        for actual in (functor.source.shape(), recursive.density().shape(), infinity.shape(),
                       (functor.source.shape()[0], functor.kernel.shape()[1])):
            if actual != shape:
                raise TensorError(f"shape mismatch: {shape} vs {actual}")
        if topos is not None:
            for label, t in (("spiral_homotopy_seed", homotopy.seed), ("spiral_homotopy_generator", homotopy.generator),
                             ("spiral_homotopy_direction", homotopy.direction), ("spiral_functor_source", functor.source),
                             ("spiral_functor_kernel", functor.kernel), ("spiral_recursive_density", recursive.density())):
                topos.guard_tensor(label, t)
            for lv in infinity.levels:
                topos.guard_tensor("spiral_infinity_level", lv)
            if len(infinity.levels) > topos.max_volume:
                raise TensorError(f"tensor volume exceeded for spiral_infinity_energy: {len(infinity.levels)} > {topos.max_volume}")
        self.topos, self.homotopy, self.functor, self.recursive, self.infinity = topos, homotopy, functor, recursive, infinity

    def resonate(self, hypergrad=None) -> DifferentialResonance:
        t = self.topos
        out = DifferentialResonance(
            _guarded(t, "spiral_resonance_homotopy", self.homotopy.flow().torch()),
            _guarded(t, "spiral_resonance_functor", self.functor.linearise(self.homotopy.direction).torch()),
            _guarded(t, "spiral_resonance_objective", self.recursive.objective_curve_tensor().torch()),
            _guarded(t, "spiral_resonance_infinity", self.infinity.collapse().torch()),
            _guarded(t, "spiral_resonance_energy", self.infinity.hierarchical_energy_tensor().torch()))
        if hypergrad is not None:
            self.recursive.accumulate(hypergrad)
        return out
