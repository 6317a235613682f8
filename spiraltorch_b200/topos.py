"""Open-cartesian topos guards: validated envelope, probability projection, rewrite monad, biome.

Parity: crates/st-tensor/src/pure/topos.rs — `LawvereTierneyGuard::project_slice` (:2649-2790),
`ToposControlSignal::from_observation` (:2038-2100), `OpenCartesianTopos` (:3207-3522),
`RewriteMonad` (:4860-4910), `TensorBiome` (:5021-5420).

The optimizer tapes carry the plain `optim.amegagrad.Topos` parameter record (its `saturate` is
the fused porous-mix kernel on the GPU); the classes here add the validation, guarding and
aggregation API around the same six parameters and work on tensors of either device with
vectorised torch ops — no per-element host loop.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Callable, Optional

import torch

from .ops import optim as K
from .optim.amegagrad import Topos
from .tensor import Tensor, TensorError


def _raw(x) -> torch.Tensor:
    return x.torch() if isinstance(x, Tensor) else torch.as_tensor(x, dtype=torch.float32)


class LawvereTierneyGuard:
    """Projects a non-negative slice onto `{p : sum p = 1, density_min <= p_i <= density_max}` over
    its strictly positive entries (zeros stay zero)."""

    def __init__(self, density_min: float = 1e-6, density_max: float = 1e3, mass_tolerance: float = 1e-5):
        for label, v in (("density_min", density_min), ("density_max", density_max), ("mass_tolerance", mass_tolerance)):
            if not math.isfinite(v):
                raise TensorError(f"non-finite value for lawvere_tierney_{label}: {v}")
        if density_min <= 0 or density_max < density_min:
            raise TensorError("invalid value: lawvere_tierney_density_window")
        if not (1.1920929e-07 <= mass_tolerance < 1.0):
            raise TensorError("invalid value: lawvere_tierney_mass_tolerance")
        self.density_min, self.density_max, self.mass_tolerance = density_min, density_max, mass_tolerance

    def project(self, label: str, values, saturation: float) -> torch.Tensor:
        v = _raw(values).double().flatten()
        if v.numel() == 0:
            raise TensorError(f"empty input: {label}")
        if not math.isfinite(saturation):
            raise TensorError(f"non-finite value for lawvere_tierney_saturation: {saturation}")
        if saturation <= 0:
            raise TensorError(f"saturation must be positive, got {saturation}")
        hi = min(self.density_max, saturation)
        g = torch.nan_to_num(v, nan=0.0, posinf=0.0, neginf=0.0).clamp(0.0, hi)
        active = g > 0
        n = int(active.sum())
        if n == 0 or n * self.density_min > 1 + self.mass_tolerance or n * hi < 1 - self.mass_tolerance:
            raise TensorError(f"probability projection infeasible: {n} active values in "
                              f"[{self.density_min}, {hi}]")
        a = g[active]
        lo_s, hi_s = 0.0, float((hi / a).max())
        for _ in range(80):                      # bisection on the common scale; mass is monotone in it
            s = 0.5 * (lo_s + hi_s)
            if float((a * s).clamp(self.density_min, hi).sum()) < 1.0:
                lo_s = s
            else:
                hi_s = s
        a = (a * (0.5 * (lo_s + hi_s))).clamp(self.density_min, hi)
        for _ in range(4):                       # spread what the clamps left over, inside the window
            delta = 1.0 - float(a.sum())
            if abs(delta) <= 0.25 * self.mass_tolerance:
                break
            room = (hi - a) if delta > 0 else (a - self.density_min)
            tot = float(room.sum())
            if tot <= 0:
                break
            a = a + room * (min(abs(delta), tot) / tot) * (1 if delta > 0 else -1)
        if abs(float(a.sum()) - 1.0) > self.mass_tolerance:
            raise TensorError(f"probability projection infeasible: mass {float(a.sum())}")
        out = torch.zeros_like(g)
        out[active] = a
        return out.float()


@dataclass
class ToposControlSignal:
    """How close a traversal is to the envelope, folded into trainer-facing scales."""
    curvature: float
    tolerance: float
    saturation: float
    porosity: float
    max_depth: int
    max_volume: int
    observed_depth: int
    visited_volume: int
    remaining_volume: int
    depth_pressure: float
    volume_pressure: float
    closure_pressure: float
    openness: float
    guard_strength: float
    stability_hint: float
    exploration_hint: float
    step_damping: float
    learning_rate_scale: float
    temperature_scale: float
    regularization_scale: float
    sampling_focus: float

    def as_dict(self) -> dict:
        return asdict(self)


def _clamp(x, lo, hi):
    return min(max(x, lo), hi)


class OpenCartesianTopos(Topos):
    """The validated envelope: negative curvature, positive tolerance / saturation, non-zero depth
    and volume horizons, porosity in [0, 1]."""

    def __init__(self, curvature: float, tolerance: float, saturation: float, max_depth: int, max_volume: int,
                 porosity: float = 0.2, guard: Optional[LawvereTierneyGuard] = None):
        for label, v in (("topos_curvature", curvature), ("topos_tolerance", tolerance), ("topos_saturation", saturation)):
            if not math.isfinite(v):
                raise TensorError(f"non-finite value for {label}: {v}")
        if curvature >= 0:
            raise TensorError(f"curvature must be negative, got {curvature}")
        if tolerance <= 0:
            raise TensorError(f"tolerance must be positive, got {tolerance}")
        if saturation <= 0:
            raise TensorError(f"saturation must be positive, got {saturation}")
        if max_depth <= 0:
            raise TensorError("empty input: topos max depth")
        if max_volume <= 0:
            raise TensorError("empty input: topos max volume")
        super().__init__(curvature, tolerance, saturation, int(max_depth), int(max_volume), 0.2)
        self.guard = guard or LawvereTierneyGuard()
        self.porosity = self._check_porosity(porosity)

    @staticmethod
    def _check_porosity(p: float) -> float:
        if not math.isfinite(p) or not 0.0 <= p <= 1.0:
            raise TensorError(f"invalid value: topos_porosity {p}")
        return float(p)

    def with_porosity(self, porosity: float) -> "OpenCartesianTopos":
        return OpenCartesianTopos(self.curvature, self.tolerance, self.saturation, self.max_depth, self.max_volume,
                                  porosity, self.guard)

    def checkpoint(self) -> dict:
        return {"curvature": self.curvature, "tolerance": self.tolerance, "saturation": self.saturation,
                "porosity": self.porosity, "max_depth": self.max_depth, "max_volume": self.max_volume,
                "density_min": self.guard.density_min, "density_max": self.guard.density_max,
                "mass_tolerance": self.guard.mass_tolerance}

    @classmethod
    def from_checkpoint(cls, ck: dict) -> "OpenCartesianTopos":
        g = LawvereTierneyGuard(ck.get("density_min", 1e-6), ck.get("density_max", 1e3), ck.get("mass_tolerance", 1e-5))
        return cls(ck["curvature"], ck["tolerance"], ck["saturation"], ck["max_depth"], ck["max_volume"],
                   ck.get("porosity", 0.2), g)

    # -- guards ---------------------------------------------------------------------------------
    def guard_slice(self, label: str, values) -> None:
        v = _raw(values)
        if not bool(torch.isfinite(v).all()):
            bad = v[~torch.isfinite(v)].flatten()[0].item()
            raise TensorError(f"non-finite value for {label}: {bad}")

    def guard_tensor(self, label: str, tensor) -> None:
        v = _raw(tensor)
        if v.numel() > self.max_volume:
            raise TensorError(f"tensor volume exceeded for {label}: {v.numel()} > {self.max_volume}")
        self.guard_slice(label, v)

    def guard_probability_tensor(self, label: str, tensor) -> Tensor:
        """Row-major flattening of `tensor` projected onto the simplex window; returns the new tensor."""
        v = _raw(tensor)
        if v.numel() > self.max_volume:
            raise TensorError(f"tensor volume exceeded for {label}: {v.numel()} > {self.max_volume}")
        out = self.guard.project(label, v, self.saturation).reshape(v.shape).to(v.device)
        self.guard_slice(label, out)
        return Tensor._wrap(out)

    def guard_probability_slice(self, label: str, values) -> list:
        return self.guard.project(label, values, self.saturation).tolist()

    def ensure_loop_free(self, depth: int) -> None:
        if depth >= self.max_depth:
            raise TensorError(f"loop detected at depth {depth} (max {self.max_depth})")

    # -- saturation -----------------------------------------------------------------------------
    def saturate_scalar(self, value: float) -> float:
        return float(K.porous_mix(torch.tensor([value], dtype=torch.float32), self.saturation, self.porosity)[0])

    def saturate_with_slope(self, value: float) -> tuple:
        if not math.isfinite(value):
            return 0.0, 0.0
        x = torch.tensor([value], dtype=torch.float32, requires_grad=True)
        with torch.enable_grad():
            y = K.porous_mix(x, self.saturation, self.porosity)
            y.backward()
        return float(y.detach()), float(x.grad)

    # -- control signal -------------------------------------------------------------------------
    def control_signal(self, observed_depth: int = 0, visited_volume: int = 0) -> ToposControlSignal:
        dp = _clamp(observed_depth / self.max_depth, 0.0, 1.0)
        vp = _clamp(visited_volume / self.max_volume, 0.0, 1.0)
        cp = max(dp, vp)
        op = _clamp(1 - cp, 0.0, 1.0)
        gs = _clamp(_clamp(1 - self.porosity, 0.0, 1.0) * 0.7 + cp * 0.3, 0.0, 1.0)
        ex = _clamp(self.porosity * op + (1 - gs) * 0.25, 0.0, 1.0)
        sd = _clamp(cp * gs, 0.0, 1.0)
        return ToposControlSignal(
            self.curvature, self.tolerance, self.saturation, self.porosity, self.max_depth, self.max_volume,
            observed_depth, visited_volume, max(0, self.max_volume - visited_volume), dp, vp, cp, op, gs,
            stability_hint=_clamp(op * (1 - 0.4 * self.porosity), 0.0, 1.0), exploration_hint=ex, step_damping=sd,
            learning_rate_scale=_clamp(1 - 0.65 * sd + 0.25 * ex, 0.1, 1.25),
            temperature_scale=_clamp(0.75 + 0.75 * ex + 0.25 * op - 0.35 * gs, 0.5, 1.5),
            regularization_scale=_clamp(0.5 + gs + 0.5 * cp - 0.25 * ex, 0.5, 2.0),
            sampling_focus=_clamp(gs * (1 - 0.5 * ex) + 0.25 * cp, 0.0, 1.0))


class RewriteMonad:
    """Saturate-then-guard rewrites under one topos; a failed rewrite leaves its input untouched."""

    def __init__(self, topos: OpenCartesianTopos):
        self.topos = topos

    def rewrite_scalar(self, value: float) -> float:
        return self.topos.saturate_scalar(value)

    def rewrite_tensor(self, label: str, tensor) -> Tensor:
        out = self.topos.saturate(_raw(tensor).float())
        self.topos.guard_tensor(label, out)
        return Tensor._wrap(out)

    lift_tensor = rewrite_tensor

    def guard_probability_slice(self, label: str, values) -> list:
        return self.topos.guard_probability_slice(label, values)


class TensorBiome:
    """Weighted collection of same-shaped guarded tensors ("shoots") that collapses to their
    weighted mean ("canopy"), itself rewritten through the topos.  The whole biome may hold at most
    `max_volume` values."""

    def __init__(self, topos: OpenCartesianTopos):
        self._topos, self._shoots, self._weights, self._shape = topos, [], [], None

    def topos(self) -> OpenCartesianTopos:
        return self._topos

    def monad(self) -> RewriteMonad:
        return RewriteMonad(self._topos)

    def __len__(self) -> int:
        return len(self._shoots)

    def is_empty(self) -> bool:
        return not self._shoots

    def total_weight(self) -> float:
        return float(sum(self._weights))

    def weights(self) -> list:
        return list(self._weights)

    def shape(self):
        return self._shape

    def stored_volume(self) -> int:
        return len(self._shoots) * (self._shape[0] * self._shape[1] if self._shape else 0)

    def remaining_volume(self) -> int:
        return max(0, self._topos.max_volume - self.stored_volume())

    def control_signal(self) -> ToposControlSignal:
        return self._topos.control_signal(0, self.stored_volume())

    def _push(self, label: str, raw: torch.Tensor, weight: float) -> None:
        if not math.isfinite(weight) or weight <= 0:
            raise TensorError(f"weight must be positive and finite, got {weight}")
        shape = tuple(raw.shape)
        if self._shape is not None and shape != self._shape:
            raise TensorError(f"shape mismatch: {self._shape} vs {shape}")
        if (len(self._shoots) + 1) * raw.numel() > self._topos.max_volume:
            raise TensorError(f"tensor volume exceeded for tensor_biome_storage: "
                              f"{(len(self._shoots) + 1) * raw.numel()} > {self._topos.max_volume}")
        self._shoots.append(raw)
        self._weights.append(float(weight))
        self._shape = shape

    def absorb(self, label: str, tensor) -> None:
        self.absorb_weighted(label, tensor, 1.0)

    def absorb_weighted(self, label: str, tensor, weight: float) -> None:
        if not math.isfinite(weight) or weight <= 0:
            raise TensorError(f"weight must be positive and finite, got {weight}")
        self._push(label, self.monad().lift_tensor(label, tensor).torch(), weight)

    def absorb_fractal_patch(self, patch: "FractalPatch") -> None:
        """Guard the patch's depth and relation, then absorb the relation under the patch's weight."""
        self._topos.ensure_loop_free(patch.depth)
        self._topos.guard_tensor("tensor_biome_fractal_patch", patch.relation())
        self.absorb_weighted("tensor_biome_fractal_patch", patch.relation(), patch.weight)

    def absorb_with(self, label: str, build: Callable) -> None:
        self.absorb(label, build(self.monad()))

    def map_shoots(self, label: str, f: Callable) -> "TensorBiome":
        out, m = TensorBiome(self._topos), self.monad()
        for s, w in zip(self._shoots, self._weights):
            out._push(label, m.lift_tensor(label, f(m, Tensor._wrap(s))).torch(), w)
        return out

    def bind_shoots(self, label: str, f: Callable) -> None:
        """Replace every shoot by `f(monad, shoot)`, all or nothing."""
        other = self.map_shoots(label, f)
        self._shoots, self._shape = other._shoots, other._shape

    def renormalise_weights(self) -> None:
        if not self._weights:
            raise TensorError("empty input: tensor_biome_weights")
        self._weights = [float(w) for w in self.monad().guard_probability_slice("tensor_biome_weights", self._weights)]

    def clear(self) -> None:
        self._shoots, self._weights, self._shape = [], [], None

    def canopy(self) -> Tensor:
        if not self._shoots:
            raise TensorError("empty input: tensor_biome")
        tot = sum(self._weights)
        if not math.isfinite(tot) or tot <= 0:
            raise TensorError(f"weight must be positive and finite, got {tot}")
        w = torch.tensor(self._weights, dtype=torch.float32, device=self._shoots[0].device) / tot
        acc = torch.einsum("s,sij->ij", w, torch.stack(self._shoots))
        return self.monad().rewrite_tensor("tensor_biome_canopy", acc / float(w.sum()))


# ----------------------------------------------------------------------------------------------
# Fractal patches and their bounded scheduler
# ----------------------------------------------------------------------------------------------
class FractalPatch:
    """A relation tensor with a coherence / tension pair; its weight is `coherence / (1 + tension)`.

    Parity: crates/st-tensor/src/pure/fractal.rs:40-150."""

    def __init__(self, relation, coherence: float, tension: float, depth: int = 0):
        for label, v in (("coherence", coherence), ("tension", tension)):
            if not math.isfinite(v):
                raise TensorError(f"non-finite value for fractal_patch_{label}: {v}")
            if v <= 0:
                raise TensorError(f"{label} must be positive, got {v}")
        r = _raw(relation).float()
        if not bool(torch.isfinite(r).all()):
            raise TensorError("non-finite value for fractal_patch_relation")
        self._relation, self.coherence, self.tension, self.depth = r, float(coherence), float(tension), int(depth)
        self.weight = coherence / (1.0 + tension)

    def relation(self) -> Tensor:
        return Tensor._wrap(self._relation)

    def normalized_relation(self) -> Tensor:
        n = float(self._relation.double().norm())
        return Tensor._wrap(torch.zeros_like(self._relation) if n == 0.0 else (self._relation.double() / n).float())


@dataclass
class FractalSchedulerSnapshot:
    capacity: int
    queued: int
    total_weight: float
    relation_shape: Optional[tuple]
    oldest_depth: Optional[int]
    newest_depth: Optional[int]

    def is_empty(self) -> bool:
        return self.queued == 0


class UringFractalScheduler:
    """Bounded FIFO ring of same-shaped patches, safe to share between threads; a push into a full
    ring evicts the oldest patch, and a rejected push changes nothing.

    Parity: crates/st-tensor/src/pure/fractal.rs:202-400 (`push`, `pop`, `snapshot`,
    `fold_coherence`).  Folding stacks the queued relations and reduces them with one weighted
    sum on the relations' device."""

    def __init__(self, capacity: int):
        import threading
        from collections import deque
        if capacity <= 0:
            raise TensorError("empty input: fractal scheduler capacity")
        self._cap, self._q, self._lock = int(capacity), deque(), threading.Lock()

    def capacity(self) -> int:
        return self._cap

    def __len__(self) -> int:
        with self._lock:
            return len(self._q)

    def is_empty(self) -> bool:
        return len(self) == 0

    def push(self, patch: FractalPatch) -> None:
        with self._lock:
            evict = max(0, len(self._q) - (self._cap - 1))
            if len(self._q) > evict and self._q[evict]._relation.shape != patch._relation.shape:
                raise TensorError(f"shape mismatch: {tuple(self._q[evict]._relation.shape)} vs {tuple(patch._relation.shape)}")
            for _ in range(evict):
                self._q.popleft()
            self._q.append(patch)

    def pop(self) -> Optional[FractalPatch]:
        with self._lock:
            return self._q.popleft() if self._q else None

    async def push_async(self, patch: FractalPatch) -> None:
        self.push(patch)

    async def pop_async(self) -> Optional[FractalPatch]:
        return self.pop()

    def total_weight(self) -> float:
        with self._lock:
            return float(sum(p.weight for p in self._q))

    def relation_shape(self) -> Optional[tuple]:
        with self._lock:
            return tuple(self._q[0]._relation.shape) if self._q else None

    def snapshot(self) -> FractalSchedulerSnapshot:
        with self._lock:
            q = list(self._q)
        return FractalSchedulerSnapshot(self._cap, len(q), float(sum(p.weight for p in q)),
                                        tuple(q[0]._relation.shape) if q else None,
                                        q[0].depth if q else None, q[-1].depth if q else None)

    def fold_coherence(self) -> Tensor:
        """Weight-normalised sum of the unit-norm relations in the ring."""
        with self._lock:
            q = list(self._q)
        if not q:
            raise TensorError("empty input: fractal scheduler queue")
        w = torch.tensor([p.weight for p in q], dtype=torch.float64, device=q[0]._relation.device)
        stack = torch.stack([p._relation.double() for p in q])
        norms = stack.flatten(1).norm(dim=1).clamp(min=1e-300)
        unit = stack / norms.reshape(-1, *([1] * (stack.dim() - 1)))
        unit[norms <= 1e-300] = 0.0
        return Tensor._wrap(torch.tensordot(w / w.sum(), unit, dims=1).float())

    def fold_coherence_into(self, target: Tensor) -> None:
        folded = self.fold_coherence()
        if target.shape() != folded.shape():
            raise TensorError(f"shape mismatch: {target.shape()} vs {folded.shape()}")
        target.torch().copy_(folded.torch())
