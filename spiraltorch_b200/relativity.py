"""Lorentzian geometry on the Z-space manifold: metric validation, Levi-Civita connection, Riemann / Ricci / Einstein
tensors, Weyl self-dual diagnostics, the vacuum field equation, and the product geometry (spacetime x internal
Z-space) with its Kaluza-Klein style reduction into an effective metric, a gauge field and scalar moduli.

Parity: crates/st-core/src/theory/general_relativity.rs — `LorentzianMetric` (:412-505), `InternalMetric` (:509-580),
`MixedBlock` / `GaugeField` / `WarpFactor` (:585-716), `ProductMetric` (:721-857), `DimensionalReduction` (:904-966),
`ZRelativityModel::assemble` (:1077-1127), `finite_difference_metric_data` (:1517-1607), `LeviCivitaConnection`
(:1611-1648), `ConnectionDerivatives` (:1652-1710), `RiemannTensor` (:1714-1778), `RicciTensor` (:1781-1857),
`EinsteinTensor` (:1861-1891), `FieldEquation` (:1956-1992), `CurvatureDiagnostics::from_fields` (:2151-2405),
`GeneralRelativityModel::new` (:2435-2470).

Every tensor here is a float64 torch tensor with optional leading batch dimensions: the contractions are einsum calls,
so one call evaluates the curvature at a whole cloud of sample points (`curvature_at_points`), on whichever device the
metric samples live.  The reference works one point at a time with fixed 4x4x4x4 arrays.
"""
from __future__ import annotations

import cmath
import itertools
import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from . import observability

DIM = 4
BIVECTOR_BASIS = ((0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3))
_TOL = 1e-12


class MetricError(ValueError):
    """A metric (or one of its companions) failed validation; ``kind`` names the rule."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def _f64(x, shape=None) -> torch.Tensor:
    t = torch.as_tensor(x, dtype=torch.float64)
    if shape is not None and tuple(t.shape[-len(shape):]) != tuple(shape):
        raise MetricError("shape", f"expected trailing shape {tuple(shape)}, found {tuple(t.shape)}")
    return t


def _check_symmetric(m: torch.Tensor, tol: float) -> None:
    if m.shape[-1] != m.shape[-2]:
        raise MetricError("non_square", f"matrix must be square, found {m.shape[-2]}x{m.shape[-1]}")
    if bool(((m - m.transpose(-1, -2)).abs() > tol).any()):
        raise MetricError("non_symmetric", f"matrix is not symmetric within {tol}")


# ---- charts -------------------------------------------------------------------------------------------------------------
@dataclass
class CoordinatePatch:
    name: str
    coordinates: Sequence[str]

    def __post_init__(self):
        self.coordinates = tuple(str(c) for c in self.coordinates)
        if len(self.coordinates) != DIM:
            raise MetricError("shape", f"a spacetime chart has {DIM} coordinates")


@dataclass
class ZManifold:
    name: str
    patches: List[CoordinatePatch] = field(default_factory=list)

    @classmethod
    def canonical(cls) -> "ZManifold":
        return cls("Z-space", [CoordinatePatch("global", ("t", "x", "y", "z"))])

    def add_patch(self, patch: CoordinatePatch) -> None:
        self.patches.append(patch)

    def dimension(self) -> int:
        return DIM


@dataclass
class InternalPatch:
    name: str
    coordinates: Sequence[str]

    def __post_init__(self):
        self.coordinates = tuple(str(c) for c in self.coordinates)


@dataclass
class InternalSpace:
    name: str
    patches: List[InternalPatch]

    def __init__(self, name: str, patch: InternalPatch):
        self.name, self.patches = name, [patch]

    def dimension(self) -> int:
        return len(self.patches[0].coordinates)

    def add_patch(self, patch: InternalPatch) -> None:
        if len(patch.coordinates) != self.dimension():
            raise MetricError("shape", "every internal chart has the same number of coordinates")
        self.patches.append(patch)


# ---- metrics ------------------------------------------------------------------------------------------------------------
class LorentzianMetric:
    """Symmetric, non-degenerate 4x4 metric with one negative and three positive eigenvalues."""

    def __init__(self, components):
        g = _f64(components, (DIM, DIM))
        if g.dim() != 2:
            raise MetricError("shape", "a single metric is a 4x4 matrix; batches go through curvature_at_points")
        _check_symmetric(g, _TOL)
        if abs(float(torch.linalg.det(g))) == 0.0 or not bool(torch.isfinite(g).all()):
            raise MetricError("degenerate", "metric is degenerate")
        ev = torch.linalg.eigvalsh(g)
        sig = [1 if v > _TOL else (-1 if v < -_TOL else 0) for v in ev.tolist()]
        if sig.count(-1) != 1 or sig.count(1) != 3:
            raise MetricError("non_lorentzian", "metric signature is not (-,+,+,+)")
        self.components = g
        self.inverse = torch.linalg.inv(g)
        self.signature = tuple(sig)

    @classmethod
    def minkowski(cls) -> "LorentzianMetric":
        return cls(torch.diag(torch.tensor([-1.0, 1.0, 1.0, 1.0], dtype=torch.float64)))

    @classmethod
    def try_scaled(cls, components, scale: float) -> "LorentzianMetric":
        return cls(_f64(components) * float(scale))

    def scaled(self, scale: float) -> "LorentzianMetric":
        return LorentzianMetric(self.components * float(scale))

    def determinant(self) -> float:
        return float(torch.linalg.det(self.components))

    def volume_element(self) -> Optional[float]:
        det = self.determinant()
        return None if det >= 0.0 else math.sqrt(-det)


class InternalMetric:
    """Symmetric positive-definite metric on the internal directions."""

    def __init__(self, components, learnable: bool = False):
        h = _f64(components)
        if h.dim() != 2:
            raise MetricError("non_square", "internal metric is a matrix")
        _check_symmetric(h, _TOL)
        if abs(float(torch.linalg.det(h))) == 0.0:
            raise MetricError("degenerate", "internal metric is degenerate")
        if bool((torch.linalg.eigvalsh(h) <= _TOL).any()):
            raise MetricError("non_positive_definite", "internal metric is not positive definite")
        self.components, self.inverse, self.learnable = h, torch.linalg.inv(h), bool(learnable)

    def with_learnable(self, learnable: bool) -> "InternalMetric":
        return InternalMetric(self.components, learnable)

    def volume_density(self) -> float:
        return math.sqrt(float(torch.linalg.det(self.components)))

    def dimension(self) -> int:
        return self.components.shape[0]


class MixedBlock:
    """Cross terms g_{mu A} between spacetime and internal directions."""

    def __init__(self, components, base_dim: int = DIM, internal_dim: Optional[int] = None, learnable: bool = False):
        c = _f64(components)
        internal_dim = c.shape[-1] if internal_dim is None else internal_dim
        if c.dim() != 2 or tuple(c.shape) != (base_dim, internal_dim):
            raise MetricError("cross_term_shape", f"cross terms must be {base_dim}x{internal_dim}, found {tuple(c.shape)}")
        self.components, self.learnable = c, bool(learnable)

    @classmethod
    def zeros(cls, base_dim: int, internal_dim: int) -> "MixedBlock":
        return cls(torch.zeros(base_dim, internal_dim, dtype=torch.float64), base_dim, internal_dim)

    def with_learnable(self, learnable: bool) -> "MixedBlock":
        return MixedBlock(self.components, *self.components.shape, learnable=learnable)

    def component(self, mu: int, a: int) -> float:
        return float(self.components[mu, a])


class GaugeField:
    def __init__(self, components, internal_dim: int):
        c = _f64(components)
        if c.dim() != 2 or tuple(c.shape) != (DIM, internal_dim):
            raise MetricError("cross_term_shape", f"gauge field must be {DIM}x{internal_dim}, found {tuple(c.shape)}")
        self.components = c

    def internal_dimension(self) -> int:
        return self.components.shape[1]

    def component(self, mu: int, a: int) -> float:
        return float(self.components[mu, a])


@dataclass(frozen=True)
class WarpFactor:
    scale: float
    learnable: bool = False

    def __post_init__(self):
        if not self.scale > 0.0:
            raise MetricError("invalid_warp", "warp factor must be positive")

    @classmethod
    def from_multiplier(cls, scale: float) -> "WarpFactor":
        return cls(float(scale))

    @classmethod
    def from_exponent(cls, exponent: float) -> "WarpFactor":
        return cls(math.exp(2.0 * exponent))

    def with_learnable(self, learnable: bool) -> "WarpFactor":
        return WarpFactor(self.scale, bool(learnable))


@dataclass(frozen=True)
class LearnableFlags:
    warp: bool = False
    mixed: bool = False
    internal: bool = False


@dataclass(frozen=True)
class PhysicalConstants:
    gravitational_constant: float = 6.67430e-11
    speed_of_light: float = 299_792_458.0

    def einstein_prefactor(self) -> float:
        return 8.0 * math.pi * self.gravitational_constant / self.speed_of_light ** 4


class ProductMetric:
    """Block metric ``[[warp * g, mixed], [mixedᵀ, h]]`` on spacetime x internal space."""

    def __init__(self, base: LorentzianMetric, internal: InternalMetric, mixed: Optional[MixedBlock] = None,
                 warp: Optional[WarpFactor] = None):
        n = internal.dimension()
        mixed = mixed or MixedBlock.zeros(DIM, n)
        if tuple(mixed.components.shape) != (DIM, n):
            raise MetricError("cross_term_shape", f"cross terms must be {DIM}x{n}")
        scale = warp.scale if warp else 1.0
        block = torch.zeros(DIM + n, DIM + n, dtype=torch.float64)
        block[:DIM, :DIM] = scale * base.components
        block[DIM:, DIM:] = internal.components
        block[:DIM, DIM:] = mixed.components
        block[DIM:, :DIM] = mixed.components.T
        self.base, self.internal, self.mixed, self.warp, self.block = base, internal, mixed, warp, block

    def total_dimension(self) -> int:
        return DIM + self.internal.dimension()

    def internal_volume_density(self) -> float:
        return self.internal.volume_density()

    def learnable_flags(self) -> LearnableFlags:
        return LearnableFlags(bool(self.warp and self.warp.learnable), self.mixed.learnable, self.internal.learnable)

    def block_matrix(self) -> torch.Tensor:
        return self.block

    def effective_base_metric(self) -> LorentzianMetric:
        return LorentzianMetric(self.base.components * (self.warp.scale if self.warp else 1.0))

    def effective_newton_constant(self, constants: PhysicalConstants, internal_volume: float) -> float:
        if not internal_volume > 0.0:
            raise MetricError("invalid_volume", "internal volume must be positive")
        return constants.gravitational_constant / internal_volume


@dataclass
class ProductGeometry:
    spacetime: ZManifold
    internal: InternalSpace
    metric: ProductMetric

    def internal_volume_density(self) -> float:
        return self.metric.internal_volume_density()

    def total_dimension(self) -> int:
        return self.metric.total_dimension()


def _abs_summary(t: torch.Tensor) -> dict:
    fin = torch.isfinite(t)
    v = t[fin]
    n = int(v.numel())
    return {"finite": n, "non_finite": int(t.numel()) - n, "abs_mean": float(v.abs().mean()) if n else 0.0,
            "abs_max": float(v.abs().max()) if n else 0.0, "frobenius_norm": float(v.pow(2).sum().sqrt()) if n else 0.0}


@dataclass
class DimensionalReduction:
    effective_metric: LorentzianMetric
    gauge_field: GaugeField
    scalar_moduli: InternalMetric
    effective_newton_constant: float

    @classmethod
    def project(cls, geometry: ProductGeometry, constants: PhysicalConstants, internal_volume: float) -> "DimensionalReduction":
        m = geometry.metric
        out = cls(m.effective_base_metric(), GaugeField(m.mixed.components.clone(), geometry.internal.dimension()),
                  m.internal, m.effective_newton_constant(constants, internal_volume))
        total = geometry.total_dimension()
        observability.emit_tensor_op("zrelativity_dimensional_reduction", (total, total), (total, total))
        observability.emit_tensor_op_meta("zrelativity_dimensional_reduction", lambda: {
            "backend": "torch", "kind": "zrelativity_dimensional_reduction", "base_dim": DIM,
            "internal_dim": geometry.internal.dimension(), "total_dim": total, "has_warp": m.warp is not None,
            "warp_scale": m.warp.scale if m.warp else 1.0, "internal_volume": internal_volume,
            "effective_newton_constant": out.effective_newton_constant,
            **{f"block_{k}": v for k, v in _abs_summary(m.block).items()}})
        return out

    def gauge_component(self, mu: int, a: int) -> float:
        return self.gauge_field.component(mu, a)

    def modulus_component(self, a: int, b: int) -> float:
        return float(self.scalar_moduli.components[a, b])


class ExtendedStressEnergy:
    def __init__(self, components, tolerance: float = 1e-9):
        c = _f64(components)
        _check_symmetric(c, tolerance)
        self.components = c

    @classmethod
    def zeros(cls, dimension: int) -> "ExtendedStressEnergy":
        return cls(torch.zeros(dimension, dimension, dtype=torch.float64))


@dataclass
class ZRelativityFieldEquation:
    lhs: torch.Tensor
    prefactor: float

    def residual(self, stress_energy: ExtendedStressEnergy) -> torch.Tensor:
        return self.lhs - self.prefactor * stress_energy.components


# ---- curvature (batched) ------------------------------------------------------------------------------------------------
class MetricDerivatives:
    """``partials[..., rho, mu, nu] = d_rho g_{mu nu}``."""

    def __init__(self, partials):
        self.partials = _f64(partials, (DIM, DIM, DIM))

    @classmethod
    def zero(cls) -> "MetricDerivatives":
        return cls(torch.zeros(DIM, DIM, DIM, dtype=torch.float64))

    @classmethod
    def from_fn(cls, f: Callable[[int, int, int], float]) -> "MetricDerivatives":
        return cls([[[f(r, m, n) for n in range(DIM)] for m in range(DIM)] for r in range(DIM)])

    def partial(self, rho: int, mu: int, nu: int) -> float:
        return float(self.partials[rho, mu, nu])


class MetricSecondDerivatives:
    """``partials[..., lam, rho, mu, nu] = d_lam d_rho g_{mu nu}``."""

    def __init__(self, partials):
        self.partials = _f64(partials, (DIM, DIM, DIM, DIM))

    @classmethod
    def zero(cls) -> "MetricSecondDerivatives":
        return cls(torch.zeros(DIM, DIM, DIM, DIM, dtype=torch.float64))

    @classmethod
    def from_fn(cls, f: Callable[[int, int, int, int], float]) -> "MetricSecondDerivatives":
        return cls([[[[f(l, r, m, n) for n in range(DIM)] for m in range(DIM)] for r in range(DIM)] for l in range(DIM)])

    def partial(self, lam: int, rho: int, mu: int, nu: int) -> float:
        return float(self.partials[lam, rho, mu, nu])


def _stencil_offsets() -> torch.Tensor:
    """The 33 offsets of the second-order central stencil: origin, +-e_i, and (+-e_i +- e_j) for i < j."""
    offs = [(0, 0, 0, 0)]
    for i in range(DIM):
        for s in (1, -1):
            o = [0] * DIM
            o[i] = s
            offs.append(tuple(o))
    for i, j in itertools.combinations(range(DIM), 2):
        for si, sj in ((1, 1), (1, -1), (-1, 1), (-1, -1)):
            o = [0] * DIM
            o[i], o[j] = si, sj
            offs.append(tuple(o))
    return torch.tensor(offs, dtype=torch.float64)


def finite_difference_batch(metric_fn: Callable[[torch.Tensor], torch.Tensor], points, step: float):
    """Central differences of a metric field at ``points[N, 4]``.  ``metric_fn`` maps ``[M, 4]`` coordinates to
    ``[M, 4, 4]`` metrics and is called once on all ``33 N`` stencil points.  Returns ``(g, dg, ddg)`` with shapes
    ``[N,4,4]``, ``[N,4,4,4]``, ``[N,4,4,4,4]``."""
    if not step > 0.0:
        raise ValueError("finite difference step must be positive")
    pts = _f64(points)
    pts = pts.reshape(-1, DIM)
    offs = _stencil_offsets().to(pts.device)
    n = pts.shape[0]
    samples = _f64(metric_fn((pts[:, None, :] + step * offs[None, :, :]).reshape(-1, DIM))).reshape(n, offs.shape[0], DIM, DIM)
    g = samples[:, 0]
    plus = samples[:, 1:9:2]                                   # [N, 4, 4, 4]: +e_rho
    minus = samples[:, 2:9:2]
    dg = (plus - minus) / (2.0 * step)
    ddg = torch.zeros(n, DIM, DIM, DIM, DIM, dtype=torch.float64, device=pts.device)
    diag = (plus - 2.0 * g[:, None] + minus) / (step * step)
    for i in range(DIM):
        ddg[:, i, i] = diag[:, i]
    for p, (i, j) in enumerate(itertools.combinations(range(DIM), 2)):
        pp, pm, mp, mm = (samples[:, 9 + 4 * p + q] for q in range(4))
        cross = (pp - pm - mp + mm) / (4.0 * step * step)
        ddg[:, i, j] = cross
        ddg[:, j, i] = cross
    return g, dg, ddg


def finite_difference_metric_data(metric_fn: Callable[[Sequence[float]], object], point: Sequence[float], step: float):
    """Single-point form: ``metric_fn`` takes one 4-vector of coordinates and returns a 4x4 matrix."""
    def batched(coords: torch.Tensor) -> torch.Tensor:
        return torch.stack([_f64(metric_fn(c.tolist()), (DIM, DIM)) for c in coords])
    g, dg, ddg = finite_difference_batch(batched, [list(point)], step)
    return LorentzianMetric(g[0]), MetricDerivatives(dg[0]), MetricSecondDerivatives(ddg[0])


def christoffel(g_inv: torch.Tensor, dg: torch.Tensor) -> torch.Tensor:
    """``Gamma^rho_{mu nu} = 1/2 g^{rho s} (d_mu g_{nu s} + d_nu g_{mu s} - d_s g_{mu nu})``."""
    sym = dg.permute(*range(dg.dim() - 3), -3, -2, -1)          # [.., a, b, c] = d_a g_{bc}
    t = sym + sym.transpose(-3, -2) - sym.permute(*range(dg.dim() - 3), -2, -1, -3)   # [.., mu, nu, s]
    return 0.5 * torch.einsum("...rs,...mns->...rmn", g_inv, t)


def christoffel_derivatives(g_inv: torch.Tensor, dg: torch.Tensor, ddg: torch.Tensor) -> torch.Tensor:
    """``out[..., lam, rho, mu, nu] = d_lam Gamma^rho_{mu nu}`` with ``d_lam g^{rs} = -g^{ra} g^{sb} d_lam g_{ab}``."""
    nb = dg.dim() - 3
    lead = tuple(range(nb))
    first = dg + dg.transpose(-3, -2) - dg.permute(*lead, nb + 1, nb + 2, nb)            # [.., mu, nu, s]
    d_inv = -torch.einsum("...ra,...sb,...lab->...lrs", g_inv, g_inv, dg)
    second = ddg + ddg.transpose(-3, -2) - ddg.permute(*lead, nb, nb + 2, nb + 3, nb + 1)  # [.., lam, mu, nu, s]
    return 0.5 * (torch.einsum("...lrs,...mns->...lrmn", d_inv, first) + torch.einsum("...rs,...lmns->...lrmn", g_inv, second))


def riemann_from_connection(gamma: torch.Tensor, dgamma: torch.Tensor) -> torch.Tensor:
    """``R^s_{m n r} = d_n Gamma^s_{m r} - d_r Gamma^s_{m n} + Gamma^s_{l n} Gamma^l_{m r} - Gamma^s_{l r} Gamma^l_{m n}``."""
    nb = gamma.dim() - 3
    lead = tuple(range(nb))
    a = dgamma.permute(*lead, nb + 1, nb + 2, nb, nb + 3)       # [.., s, m, n, r] = d_n Gamma^s_{m r}
    quad = torch.einsum("...sln,...lmr->...smnr", gamma, gamma)
    return a - a.transpose(-1, -2) + quad - quad.transpose(-1, -2)


def ricci_from_riemann(riemann: torch.Tensor) -> torch.Tensor:
    return torch.einsum("...smsn->...mn", riemann)


class LeviCivitaConnection:
    def __init__(self, coefficients: torch.Tensor):
        self.coefficients = coefficients

    @classmethod
    def from_metric(cls, metric: LorentzianMetric, derivatives: MetricDerivatives) -> "LeviCivitaConnection":
        return cls(christoffel(metric.inverse, derivatives.partials))

    def coefficient(self, rho: int, mu: int, nu: int) -> float:
        return float(self.coefficients[rho, mu, nu])


class ConnectionDerivatives:
    def __init__(self, partials: torch.Tensor):
        self.partials = partials

    @classmethod
    def from_metric(cls, metric: LorentzianMetric, first: MetricDerivatives, second: MetricSecondDerivatives):
        return cls(christoffel_derivatives(metric.inverse, first.partials, second.partials))

    def partial(self, lam: int, rho: int, mu: int, nu: int) -> float:
        return float(self.partials[lam, rho, mu, nu])


class RiemannTensor:
    def __init__(self, components):
        self.components = _f64(components, (DIM,) * 4)

    @classmethod
    def from_connection(cls, connection: LeviCivitaConnection, derivatives: ConnectionDerivatives) -> "RiemannTensor":
        return cls(riemann_from_connection(connection.coefficients, derivatives.partials))

    def component(self, sigma: int, mu: int, nu: int, rho: int) -> float:
        return float(self.components[sigma, mu, nu, rho])

    def is_near_zero(self, tolerance: float) -> bool:
        return not bool((self.components.abs() > tolerance).any())


class RicciTensor:
    def __init__(self, components):
        self.components = _f64(components, (DIM, DIM))

    @classmethod
    def from_riemann(cls, riemann: RiemannTensor) -> "RicciTensor":
        return cls(ricci_from_riemann(riemann.components))

    def component(self, mu: int, nu: int) -> float:
        return float(self.components[mu, nu])

    def is_near_zero(self, tolerance: float) -> bool:
        return not bool((self.components.abs() > tolerance).any())

    def scalar_curvature(self, metric: LorentzianMetric) -> float:
        return float((metric.inverse * self.components).sum())

    def contracted_square(self, metric: LorentzianMetric) -> float:
        """``R_{mu nu} g^{mu a} R_{a nu}`` — the reference raises one index only (general_relativity.rs:1836-1857); for
        metrics that commute with the Ricci tensor up to sign conventions this is the mixed-tensor square."""
        return float((self.components * (metric.inverse @ self.components)).sum())


class EinsteinTensor:
    def __init__(self, components):
        self.components = _f64(components, (DIM, DIM))

    @classmethod
    def from_ricci(cls, ricci: RicciTensor, scalar_curvature: float, metric: LorentzianMetric) -> "EinsteinTensor":
        return cls(ricci.components - 0.5 * scalar_curvature * metric.components)

    def component(self, mu: int, nu: int) -> float:
        return float(self.components[mu, nu])


class EnergyMomentumTensor:
    def __init__(self, components, tolerance: float = 1e-9):
        c = _f64(components, (DIM, DIM))
        _check_symmetric(c, tolerance)
        self.components = c

    @classmethod
    def zero(cls) -> "EnergyMomentumTensor":
        return cls(torch.zeros(DIM, DIM, dtype=torch.float64))

    def component(self, mu: int, nu: int) -> float:
        return float(self.components[mu, nu])


class FieldEquation:
    """``G_{mu nu} + Lambda g_{mu nu}``; `residual` subtracts ``8 pi G / c^4 T_{mu nu}``."""

    def __init__(self, lhs: torch.Tensor):
        self.lhs = lhs

    @classmethod
    def vacuum(cls, einstein: EinsteinTensor, cosmological_constant: float, metric: LorentzianMetric) -> "FieldEquation":
        return cls(einstein.components + cosmological_constant * metric.components)

    def residual(self, energy_momentum: EnergyMomentumTensor, constants: PhysicalConstants) -> torch.Tensor:
        return self.lhs - constants.einstein_prefactor() * energy_momentum.components


def _levi_civita() -> torch.Tensor:
    eps = torch.zeros((DIM,) * 4, dtype=torch.float64)
    for perm in itertools.permutations(range(DIM)):
        inv = sum(1 for i in range(DIM) for j in range(i + 1, DIM) if perm[i] > perm[j])
        eps[perm] = -1.0 if inv % 2 else 1.0
    return eps


def _raise_all(t: torch.Tensor, g_inv: torch.Tensor) -> torch.Tensor:
    return torch.einsum("...ma,...nb,...rc,...sd,...abcd->...mnrs", g_inv, g_inv, g_inv, g_inv, t)


def solve_self_dual_eigenvalues(i: complex, j: complex) -> List[complex]:
    """Roots of ``x^3 - I x + 2 J = 0`` (the characteristic polynomial of a trace-free 3x3 matrix with invariants
    ``I = tr(Q^2)/2`` and ``J = -tr(Q^3)/6``), by the trigonometric form when everything is real and three roots exist,
    Cardano otherwise."""
    tol = 1e-12
    i, j = complex(i), complex(j)
    if abs(i.imag) <= tol and abs(j.imag) <= tol:
        p, q = -i.real, 2.0 * j.real
        disc = q * q / 4.0 + p ** 3 / 27.0
        cbrt = lambda v: math.copysign(abs(v) ** (1.0 / 3.0), v)
        if abs(disc) <= tol:
            u = cbrt(-q / 2.0)
            return [complex(2.0 * u), complex(-u), complex(-u)]
        if disc > 0.0:
            s = math.sqrt(disc)
            u = cbrt(-q / 2.0 + s)
            v = -p / (3.0 * u) if abs(u) > tol else cbrt(-q / 2.0 - s)
            re, im = -0.5 * (u + v), math.sqrt(3.0) * 0.5 * (u - v)
            return [complex(u + v), complex(re, im), complex(re, -im)]
        base = max(-p / 3.0, 0.0)
        if base <= tol:
            r = cbrt(-q / 2.0)
            return [complex(r)] * 3
        r = math.sqrt(base)
        phi = math.acos(min(max(-q / (2.0 * r ** 3), -1.0), 1.0))
        return [complex(2.0 * r * math.cos((phi + 2.0 * math.pi * k) / 3.0)) for k in range(3)]
    p3, hq = -i / 3.0, j
    sq = cmath.sqrt(hq * hq + p3 ** 3)
    cb = lambda z: 0j if z == 0 else cmath.rect(abs(z) ** (1.0 / 3.0), cmath.phase(z) / 3.0)
    u = cb(-hq + sq)
    v = cb(-hq - sq) if abs(u) <= 1e-24 else -p3 / u
    w = complex(-0.5, math.sqrt(3.0) / 2.0)
    return [u + v, w * u + w.conjugate() * v, w.conjugate() * u + w * v]


def _self_dual_projectors():
    s = 1.0 / math.sqrt(2.0)
    plus = torch.zeros(6, 3, dtype=torch.complex128)
    for col, (e, b, sign) in enumerate(((0, 5, 1), (1, 4, -1), (2, 3, 1))):     # electric row, magnetic row, orientation
        plus[e, col] = s
        plus[b, col] = sign * 1j * s
    return plus, plus.conj()


@dataclass
class CurvatureDiagnostics:
    scalar_curvature: float
    ricci_square: float = 0.0
    kretschmann: float = 0.0
    weyl_square: float = 0.0
    weyl_dual_contraction: float = 0.0
    weyl_self_dual_squared: float = 0.0
    weyl_anti_self_dual_squared: float = 0.0
    weyl_self_dual_matrix: torch.Tensor = field(default_factory=lambda: torch.zeros(3, 3, dtype=torch.complex128))
    weyl_anti_self_dual_matrix: torch.Tensor = field(default_factory=lambda: torch.zeros(3, 3, dtype=torch.complex128))
    weyl_self_dual_invariant_i: complex = 0j
    weyl_self_dual_invariant_j: complex = 0j
    weyl_self_dual_discriminant: complex = 0j
    weyl_self_dual_eigenvalues: List[complex] = field(default_factory=lambda: [0j, 0j, 0j])

    @classmethod
    def from_fields(cls, riemann: RiemannTensor, metric: LorentzianMetric, ricci: RicciTensor, scalar_curvature: float):
        if riemann.is_near_zero(_TOL) and ricci.is_near_zero(_TOL) and abs(scalar_curvature) <= _TOL:
            return cls(scalar_curvature)
        g, gi, ric = metric.components, metric.inverse, ricci.components
        lower = torch.einsum("ma,anrs->mnrs", g, riemann.components)
        return cls._from_lower(lower, weyl_lower(lower, g, ric, scalar_curvature), metric, ricci, scalar_curvature)

    @classmethod
    def _from_lower(cls, lower, weyl, metric, ricci, scalar_curvature):
        g, gi = metric.components, metric.inverse
        kretschmann = float((lower * _raise_all(lower, gi)).sum())
        weyl_up = _raise_all(weyl, gi)
        det = metric.determinant()
        eps = (metric.volume_element() or math.sqrt(abs(det))) * _levi_civita()
        eps_raised = torch.einsum("ga,db,fsgd->fsab", gi, gi, eps)     # eps_{rho sigma}^{alpha beta}
        dual = 0.5 * torch.einsum("rsab,mnab->mnrs", eps_raised, weyl)
        weyl_sq, dual_c = float((weyl * weyl_up).sum()), float((dual * weyl_up).sum())
        idx = torch.tensor(BIVECTOR_BASIS)
        biv = 0.5 * weyl[idx[:, 0], idx[:, 1]][:, idx[:, 0], idx[:, 1]].to(torch.complex128)       # 6 x 6
        plus, minus = _self_dual_projectors()
        qp = plus.conj().T @ biv @ plus
        qm = minus.conj().T @ biv @ minus
        qp, qm = 0.5 * (qp + qp.T), 0.5 * (qm + qm.T)
        q2 = qp @ qp
        inv_i = complex(0.5 * torch.trace(q2))
        inv_j = complex(-torch.trace(q2 @ qp) / 6.0)
        eig = sorted(solve_self_dual_eigenvalues(inv_i, inv_j), key=lambda z: (z.real, z.imag))
        return cls(scalar_curvature, ricci.contracted_square(metric), kretschmann, weyl_sq, dual_c, 0.5 * (weyl_sq + dual_c),
                   0.5 * (weyl_sq - dual_c), qp, qm, inv_i, inv_j, inv_i ** 3 - 27.0 * inv_j ** 2, eig)


def weyl_lower(riemann_lower: torch.Tensor, g: torch.Tensor, ricci: torch.Tensor, scalar) -> torch.Tensor:
    """``C_{mnrs} = R_{mnrs} - 1/2 (g_{mr} R_{ns} - g_{ms} R_{nr} - g_{nr} R_{ms} + g_{ns} R_{mr}) + R/6 (g_{mr} g_{ns} - g_{ms} g_{nr})``."""
    gr = torch.einsum("...mr,...ns->...mnrs", g, ricci)
    trace = gr - gr.transpose(-1, -2) - gr.transpose(-3, -4) + gr.transpose(-1, -2).transpose(-3, -4)
    gg = torch.einsum("...mr,...ns->...mnrs", g, g)
    scalar = torch.as_tensor(scalar, dtype=torch.float64)
    return riemann_lower - 0.5 * trace + (scalar / 6.0)[..., None, None, None, None] * (gg - gg.transpose(-1, -2))


@dataclass
class CurvatureField:
    """Curvature at a cloud of points (all tensors carry the leading ``N``)."""
    metric: torch.Tensor
    connection: torch.Tensor
    riemann: torch.Tensor
    ricci: torch.Tensor
    scalar: torch.Tensor
    einstein: torch.Tensor
    kretschmann: torch.Tensor
    weyl_square: torch.Tensor


def curvature_from_derivatives(g: torch.Tensor, dg: torch.Tensor, ddg: torch.Tensor) -> CurvatureField:
    gi = torch.linalg.inv(g)
    gamma = christoffel(gi, dg)
    riem = riemann_from_connection(gamma, christoffel_derivatives(gi, dg, ddg))
    ric = ricci_from_riemann(riem)
    scalar = (gi * ric).sum((-1, -2))
    lower = torch.einsum("...ma,...anrs->...mnrs", g, riem)
    weyl = weyl_lower(lower, g, ric, scalar)
    return CurvatureField(g, gamma, riem, ric, scalar, ric - 0.5 * scalar[..., None, None] * g,
                          (lower * _raise_all(lower, gi)).sum((-1, -2, -3, -4)), (weyl * _raise_all(weyl, gi)).sum((-1, -2, -3, -4)))


def curvature_at_points(metric_fn: Callable[[torch.Tensor], torch.Tensor], points, step: float = 1e-3) -> CurvatureField:
    """Connection, Riemann, Ricci, Einstein, Kretschmann and Weyl-square at every row of ``points[N, 4]`` in one pass."""
    return curvature_from_derivatives(*finite_difference_batch(metric_fn, points, step))


# ---- models -------------------------------------------------------------------------------------------------------------
SYMMETRY_DESCRIPTIONS = {"static_spherical": "Static, spherically symmetric metric ansatz",
                         "homogeneous_isotropic": "Homogeneous and isotropic cosmological ansatz"}
TOPOLOGIES = {"r4": "ℝ^4", "r3xs1": "ℝ^3 × S^1"}
BOUNDARY_KINDS = {"asymptotically_flat": "Asymptotically flat", "regularity": "Regularity condition", "periodic": "Periodic boundary"}


@dataclass(frozen=True)
class SymmetryAnsatz:
    kind: str                                    # a key of SYMMETRY_DESCRIPTIONS, or free text (a custom ansatz)

    def description(self) -> str:
        return SYMMETRY_DESCRIPTIONS.get(self.kind, self.kind)

    def seed_metric(self) -> torch.Tensor:
        if self.kind in SYMMETRY_DESCRIPTIONS:
            return torch.diag(torch.tensor([-1.0, 1.0, 1.0, 1.0], dtype=torch.float64))
        return torch.eye(DIM, dtype=torch.float64)


SymmetryAnsatz.STATIC_SPHERICAL = SymmetryAnsatz("static_spherical")
SymmetryAnsatz.HOMOGENEOUS_ISOTROPIC = SymmetryAnsatz("homogeneous_isotropic")


@dataclass(frozen=True)
class Topology:
    kind: str

    def __str__(self) -> str:
        return TOPOLOGIES.get(self.kind, self.kind)


Topology.R4 = Topology("r4")
Topology.R3XS1 = Topology("r3xs1")


@dataclass
class BoundaryCondition:
    kind: str
    location: Optional[str] = None
    notes: Optional[str] = None

    def description(self) -> str:
        return BOUNDARY_KINDS.get(self.kind, self.kind)

    def with_location(self, location: str) -> "BoundaryCondition":
        return BoundaryCondition(self.kind, location, self.notes)

    def with_notes(self, notes: str) -> "BoundaryCondition":
        return BoundaryCondition(self.kind, self.location, notes)


class GeneralRelativityModel:
    def __init__(self, manifold: ZManifold, metric: LorentzianMetric, first: MetricDerivatives, second: MetricSecondDerivatives,
                 symmetry: SymmetryAnsatz = SymmetryAnsatz.STATIC_SPHERICAL, topology: Topology = Topology.R4,
                 boundary_conditions: Sequence[BoundaryCondition] = ()):
        self.manifold, self.metric = manifold, metric
        self.connection = LeviCivitaConnection.from_metric(metric, first)
        self.riemann = RiemannTensor.from_connection(self.connection, ConnectionDerivatives.from_metric(metric, first, second))
        self.ricci = RicciTensor.from_riemann(self.riemann)
        scalar = self.ricci.scalar_curvature(metric)
        self.einstein = EinsteinTensor.from_ricci(self.ricci, scalar, metric)
        self.diagnostics = CurvatureDiagnostics.from_fields(self.riemann, metric, self.ricci, scalar)
        self.symmetry, self.topology, self.boundary_conditions = symmetry, topology, list(boundary_conditions)

    @classmethod
    def from_metric_fn(cls, metric_fn, point, step: float = 1e-3, **kw) -> "GeneralRelativityModel":
        metric, first, second = finite_difference_metric_data(metric_fn, point, step)
        return cls(ZManifold.canonical(), metric, first, second, **kw)


@dataclass
class ZRelativityTensorBundle:
    block_metric: torch.Tensor
    effective_metric: torch.Tensor
    gauge_field: torch.Tensor
    scalar_moduli: torch.Tensor
    field_equation: torch.Tensor
    warp: Optional[torch.Tensor]
    internal_volume_density: float
    field_prefactor: float


class ZRelativityModel:
    """Spacetime curvature + product geometry + reduction + the extended field-equation left-hand side
    ``[[G + Lambda g_eff, Lambda mixed], [Lambda mixedᵀ, Lambda h]]`` with prefactor ``8 pi G_eff / c^4``."""

    def __init__(self, geometry, base_model, reduction, field_equations):
        self.geometry, self.base_model, self.reduction, self.field_equations = geometry, base_model, reduction, field_equations

    @classmethod
    def assemble(cls, geometry: ProductGeometry, base_model: GeneralRelativityModel, constants: PhysicalConstants = PhysicalConstants(),
                 internal_volume: float = 1.0, cosmological_constant: float = 0.0) -> "ZRelativityModel":
        reduction = DimensionalReduction.project(geometry, constants, internal_volume)
        m = geometry.metric
        lhs = cosmological_constant * m.block.clone()
        lhs[:DIM, :DIM] = base_model.einstein.components + cosmological_constant * reduction.effective_metric.components
        prefactor = 8.0 * math.pi * reduction.effective_newton_constant / constants.speed_of_light ** 4
        model = cls(geometry, base_model, reduction, ZRelativityFieldEquation(lhs, prefactor))
        total = geometry.total_dimension()
        observability.emit_tensor_op("zrelativity_model_assemble", (total, total), (total, total))
        observability.emit_tensor_op_meta("zrelativity_model_assemble", lambda: {
            "backend": "torch", "kind": "zrelativity_model_assemble", "total_dim": total, "internal_volume": internal_volume,
            "cosmological_constant": cosmological_constant, "field_prefactor": prefactor,
            "base_scalar_curvature": base_model.diagnostics.scalar_curvature, "base_kretschmann": base_model.diagnostics.kretschmann,
            **{f"lhs_{k}": v for k, v in _abs_summary(lhs).items()}})
        return model

    def as_tensor(self) -> torch.Tensor:
        return self.geometry.metric.block.to(torch.float32)

    def to_dlpack(self):
        return torch.utils.dlpack.to_dlpack(self.as_tensor())

    def gauge_tensor(self) -> torch.Tensor:
        return self.reduction.gauge_field.components.to(torch.float32)

    def scalar_moduli_tensor(self) -> torch.Tensor:
        return self.reduction.scalar_moduli.components.to(torch.float32)

    def effective_metric_tensor(self) -> torch.Tensor:
        return self.reduction.effective_metric.components.to(torch.float32)

    def field_equation_tensor(self) -> torch.Tensor:
        return self.field_equations.lhs.to(torch.float32)

    def tensor_bundle(self) -> ZRelativityTensorBundle:
        warp = self.geometry.metric.warp
        return ZRelativityTensorBundle(self.as_tensor(), self.effective_metric_tensor(), self.gauge_tensor(), self.scalar_moduli_tensor(),
                                       self.field_equation_tensor(), torch.tensor([[warp.scale]], dtype=torch.float32) if warp else None,
                                       self.geometry.internal_volume_density(), self.field_equations.prefactor)

    def learnable_flags(self) -> LearnableFlags:
        return self.geometry.metric.learnable_flags()
