"""Closed-form stability helpers of the psi-spiral control loop: the hard / soft barrier on the effective growth rate
``mu_eff = mu0 + gamma c``, the logistic audit force and its derivatives, steady radii of the cubic normal form, the
audit / container gain balance, the Hopf normal-form coefficient and regime, the Ito mean-square bound, and Gershgorin
contraction margins.

Parity: crates/st-core/src/theory/spiral_dynamics.rs — `hard_barrier_max_c` (:54), `LogisticForce::evaluate` (:159),
`soft_barrier_*` (:174-218), `cbf_boundary_projection` / `cbf_dot_h` (:220-247), `steady_radius*` (:249-320),
`audit_container_balance` (:322), `hopf_normal_form` (:340-385), `ito_mean_square_bound` (:387),
`dimensionless_parameters` (:432), `psi_spiral_metrics` (:473), `gershgorin_contraction_bound` (:650),
`contraction_with_cubic` (:670).  Scalars in, scalars out: these run once per controller update on the host.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from . import observability

EPS = 2.220446049250313e-16


def _logistic(x: float) -> float:
    if x >= 0.0:
        return 1.0 / (1.0 + math.exp(-x))
    e = math.exp(x)
    return e / (1.0 + e)


def hard_barrier_max_c(mu0: float, gamma: float) -> Optional[float]:
    """Largest ``c`` with ``mu0 + gamma c <= 0`` (``inf`` when ``gamma`` vanishes and ``mu0 <= 0``), or ``None``."""
    if abs(gamma) < EPS:
        return math.inf if mu0 <= 0.0 else None
    bound = -mu0 / gamma
    return bound if math.isfinite(bound) and bound >= 0.0 else None


def hard_barrier_satisfied(mu0: float, gamma: float, c_max: float) -> bool:
    return c_max >= 0.0 and mu0 + gamma * c_max <= 0.0


@dataclass(frozen=True)
class LogisticForce:
    value: float = 0.0
    du: float = 0.0
    ds: float = 0.0

    @classmethod
    def evaluate(cls, u: float, s: float, c_max: float, sigma_s: float) -> "LogisticForce":
        if c_max <= 0.0:
            return cls()
        sig = _logistic(u - sigma_s * s)
        value = c_max * sig
        du = value * (1.0 - sig)
        return cls(value, du, -sigma_s * du)


def soft_barrier_ceiling(c_base: float, kappa_b: float, s: float) -> float:
    return 0.0 if c_base <= 0.0 else c_base / max(1.0 + kappa_b * s, 1e-9)


def soft_barrier_force(u: float, s: float, c_base: float, kappa_b: float, sigma_s: float) -> float:
    return soft_barrier_ceiling(c_base, kappa_b, s) * _logistic(u - sigma_s * s) if c_base > 0.0 else 0.0


def soft_barrier_mu_eff(mu0: float, gamma: float, c_base: float, kappa_b: float, s: float) -> float:
    return mu0 + gamma * soft_barrier_ceiling(c_base, kappa_b, s)


def soft_barrier_margin_satisfied(mu0: float, gamma: float, c_base: float, kappa_b: float, margin: float) -> bool:
    return margin >= 0.0 and mu0 + gamma * c_base <= -margin


def cbf_boundary_projection(kappa, alpha, beta, theta, re_z, im_z, tau, u, sigma_s, lam, s, rho) -> float:
    return kappa * (alpha * re_z - beta * im_z - theta) - tau * u + sigma_s * lam * s - sigma_s * rho * im_z


def cbf_dot_h(gamma: float, force: LogisticForce, dot_u_minus_sigma_dot_s: float) -> float:
    return -gamma * force.du * dot_u_minus_sigma_dot_s


def steady_radius_squared(mu0, eta, gamma, c1, q, nu, sigma_s, s) -> Optional[float]:
    """Non-negative root ``y = r^2`` of ``q nu y^2 + a1 y + a0 = 0`` (saturating audit ``c1 / (1 + q y)``)."""
    if not (math.isfinite(q) and math.isfinite(nu)) or q <= 0.0 or nu <= 0.0:
        return None
    a = mu0 - eta
    a2 = q * nu
    a1 = nu - q * a + q * gamma * sigma_s * s
    a0 = -a + gamma * sigma_s * s - gamma * c1
    disc = a1 * a1 - 4.0 * a2 * a0
    if disc < 0.0:
        return None
    root = (-a1 + math.sqrt(disc)) / (2.0 * a2)
    return root if math.isfinite(root) and root >= 0.0 else None


def steady_radius(mu0, eta, gamma, c1, q, nu, sigma_s, s) -> Optional[float]:
    y = steady_radius_squared(mu0, eta, gamma, c1, q, nu, sigma_s, s)
    return None if y is None else math.sqrt(y)


def steady_radius_sensitivity(mu0, eta, gamma, c1, q, nu, sigma_s, s) -> Optional[float]:
    """``d(r^2) / ds`` at the steady state."""
    y = steady_radius_squared(mu0, eta, gamma, c1, q, nu, sigma_s, s)
    if y is None:
        return None
    denom = -(gamma * c1 * q) / (1.0 + q * y) ** 2 - nu
    return None if abs(denom) < 1e-12 else gamma * sigma_s / denom


@dataclass(frozen=True)
class AuditContainerBalance:
    audit_gain: float
    container_gain: float
    difference: float


def audit_container_balance(kappa, a, tau, sigma_s, rho, lam) -> Optional[AuditContainerBalance]:
    if tau <= 0.0 or lam <= 0.0:
        return None
    audit, container = kappa * a / tau, sigma_s * rho / lam
    return AuditContainerBalance(audit, container, audit - container)


@dataclass(frozen=True)
class HopfNormalForm:
    forcing: LogisticForce
    mu_eff0: float
    center_manifold_c: float
    alpha3: float
    regime: str                          # "supercritical" (alpha3 > 0), "subcritical" (< 0), "degenerate" (0)


def hopf_normal_form(mu0, gamma, nu, omega, kappa, a, tau, theta, sigma_s, rho, lam, c_max) -> Optional[HopfNormalForm]:
    if not all(math.isfinite(v) and v > 0.0 for v in (nu, lam, tau)):
        return None
    balance = audit_container_balance(kappa, a, tau, sigma_s, rho, lam)
    force = LogisticForce.evaluate(-kappa * theta / tau, 0.0, c_max, sigma_s)
    ratio = min(max(force.du / force.value, 0.0), 1.0) if force.value > EPS else 0.0
    c_corr = ratio * (1.0 - ratio) * balance.difference if force.value > EPS else 0.0
    alpha3 = nu - gamma * c_corr
    regime = "supercritical" if alpha3 > 0.0 else ("subcritical" if alpha3 < 0.0 else "degenerate")
    return HopfNormalForm(force, mu0 + gamma * force.value, c_corr, alpha3, regime)


def ito_mean_square_bound(mu_eff: float, nu: float, noise_power: float) -> Optional[float]:
    """Stationary bound of ``E[r^2]`` for ``dr = (mu r - nu r^3) dt + noise``: the positive root of ``nu y^2 - mu y - D/2``."""
    if not (math.isfinite(nu) and nu > 0.0 and math.isfinite(noise_power) and noise_power >= 0.0 and math.isfinite(mu_eff)):
        return None
    return (mu_eff + math.sqrt(mu_eff * mu_eff + 2.0 * nu * noise_power)) / (2.0 * nu)


@dataclass(frozen=True)
class DimensionlessParameters:
    mu_bar: float
    gamma_bar: float
    omega_bar: float
    audit_cluster: float
    container_cluster: float


def dimensionless_parameters(mu0, gamma, omega, nu, kappa, a, tau, sigma_s, rho, lam) -> Optional[DimensionlessParameters]:
    if not all(math.isfinite(v) and v > 0.0 for v in (nu, tau, lam)):
        return None
    return DimensionlessParameters(mu0 / nu, gamma / nu, omega / nu, kappa * a / (tau * nu), sigma_s * rho / (lam * nu))


@dataclass(frozen=True)
class PsiSpiralMetrics:
    hopf: HopfNormalForm
    dimensionless: DimensionlessParameters
    balance: AuditContainerBalance


def psi_spiral_metrics(mu0, gamma, omega, nu, kappa, a, tau, theta, sigma_s, rho, lam, c_max) -> Optional[PsiSpiralMetrics]:
    hopf = hopf_normal_form(mu0, gamma, nu, omega, kappa, a, tau, theta, sigma_s, rho, lam, c_max)
    dims = dimensionless_parameters(mu0, gamma, omega, nu, kappa, a, tau, sigma_s, rho, lam)
    balance = audit_container_balance(kappa, a, tau, sigma_s, rho, lam)
    if hopf is None or dims is None or balance is None:
        return None
    m = PsiSpiralMetrics(hopf, dims, balance)
    observability.emit_tensor_op("psi_spiral_metrics", (1, 12), (1, 16))
    observability.emit_tensor_op_meta("psi_spiral_metrics", lambda: {
        "backend": "host", "kind": "psi_spiral_metrics", "hopf_regime": hopf.regime, "hopf_mu_eff0": hopf.mu_eff0, "hopf_alpha3": hopf.alpha3,
        "hopf_center_manifold_c": hopf.center_manifold_c, "forcing_value": hopf.forcing.value, "forcing_du": hopf.forcing.du,
        "forcing_ds": hopf.forcing.ds, "audit_gain": balance.audit_gain, "container_gain": balance.container_gain,
        "balance_difference": balance.difference, "mu_bar": dims.mu_bar, "gamma_bar": dims.gamma_bar, "omega_bar": dims.omega_bar,
        "audit_cluster": dims.audit_cluster, "container_cluster": dims.container_cluster,
        "hard_barrier_max_c": (lambda b: b if b is not None and math.isfinite(b) else 0.0)(hard_barrier_max_c(mu0, gamma)),
        "hard_barrier_satisfied": hard_barrier_satisfied(mu0, gamma, c_max), "soft_mu_eff_zero": soft_barrier_mu_eff(mu0, gamma, c_max, 0.0, 0.0),
        "noise_free_bound": ito_mean_square_bound(hopf.mu_eff0, nu, 0.0) or 0.0})
    return m


def gershgorin_contraction_bound(a, gamma, kappa, alpha, beta, sigma_s, rho, tau, lam) -> float:
    """Smallest Gershgorin margin of the linearised loop; positive means every disc lies in the contracting half-plane."""
    gk = abs(gamma - kappa * alpha)
    return min(a - 0.5 * gk, a - 0.5 * (abs(kappa * beta) + abs(sigma_s - rho)), tau - 0.5 * (gk + abs(kappa * beta) + abs(sigma_s)),
               lam - 0.5 * (abs(sigma_s - rho) + abs(sigma_s)))


def contraction_with_cubic(eps_lin: float, nu: float, radius: float) -> float:
    return eps_lin + nu * radius * radius
