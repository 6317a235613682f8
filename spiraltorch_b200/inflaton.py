"""Slow-roll inflation backgrounds on the logarithmic Z-space lattice: uniformly spaced samples of the e-folding time
tau = ln a with trapezoid (optionally Hann-tapered) weights, the weighted Z transform of a background channel at many
points at once, and the slow-roll scalar power spectrum P_zeta = H^2 / (8 pi^2 epsilon M_Pl^2) assembled from the
transformed H and epsilon channels.

Reference parity: crates/st-core/src/theory/inflaton_zspace.rs (`LogLattice` :234-330, `z_transform` :337-353,
`assemble_primordial_spectrum` :361-386, `PrimordialProjection` and its telemetry record :33-231).  The transform is
evaluated for a whole tensor of z points per Horner step (complex128), so a spectrum over thousands of modes is a
handful of tensor operations on whichever device holds the samples.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch

from . import observability as _obs

_ArrayLike = Union[torch.Tensor, Sequence[float], Sequence[complex]]


def _real(x: _ArrayLike, device=None) -> torch.Tensor:
    return torch.as_tensor(x, dtype=torch.float64, device=device)


def _cplx(x: _ArrayLike, device=None) -> torch.Tensor:
    t = torch.as_tensor(x, device=device)
    return t.to(torch.complex128)


class LogLattice:
    """Samples of one background channel at tau0 + k delta_tau with quadrature weights that sum to one."""

    def __init__(self, tau0: float, delta_tau: float, samples: _ArrayLike):
        if not (math.isfinite(delta_tau) and delta_tau > 0.0):
            raise ValueError("delta_tau must be positive")
        self.samples = _real(samples)
        n = self.samples.numel()
        if self.samples.dim() != 1 or n < 2:
            raise ValueError("at least two samples are required for a trapezoidal rule")
        self.tau0, self.delta_tau = float(tau0), float(delta_tau)
        w = torch.ones(n, dtype=torch.float64, device=self.samples.device)
        w[0] = w[-1] = 0.5
        self.weights = w / w.sum()

    from_samples = classmethod(lambda cls, tau0, delta_tau, samples: cls(tau0, delta_tau, samples))

    def apply_hann_window(self) -> "LogLattice":
        """Multiplies the weights by a Hann taper and renormalises them (a taper that removes all weight is skipped)."""
        n = self.weights.numel()
        k = torch.arange(n, dtype=torch.float64, device=self.weights.device)
        w = self.weights * 0.5 * (1.0 - torch.cos(2.0 * math.pi * k / (n - 1)))
        total = float(w.sum())
        if total > 0.0:
            self.weights = w / total
        return self

    def tau(self) -> torch.Tensor:
        return self.tau0 + self.delta_tau * torch.arange(len(self), dtype=torch.float64, device=self.samples.device)

    def __len__(self) -> int:
        return self.samples.numel()

    def is_empty(self) -> bool:
        return len(self) == 0

    def __iter__(self):
        return iter(zip(self.samples.tolist(), self.weights.tolist()))

    def z_transform(self, z: _ArrayLike) -> torch.Tensor:
        return z_transform(self.weights, self.samples, z)


def z_transform(weights: _ArrayLike, samples: _ArrayLike, z: _ArrayLike) -> torch.Tensor:
    """sum_k w_k x_k z^k by Horner's rule, for every entry of ``z`` at once (complex128, the shape of ``z``)."""
    x = _real(samples)
    w = _real(weights, x.device)
    if w.shape != x.shape or x.dim() != 1:
        raise ValueError("weights and samples must be vectors of the same length")
    zz = _cplx(z, x.device)
    coeff = (w * x).to(torch.complex128)
    acc = torch.zeros_like(zz)
    for k in range(coeff.numel() - 1, -1, -1):
        acc = acc * zz + coeff[k]
    return acc


def assemble_primordial_spectrum(z_points: _ArrayLike, h_z: _ArrayLike, epsilon_z: _ArrayLike, planck_mass: float) -> torch.Tensor:
    """Re(H)^2 / (8 pi^2 max(Re(epsilon), 1e-20) M_Pl^2) per evaluation point (float64)."""
    zp = _cplx(z_points)
    h, eps = _cplx(h_z, zp.device), _cplx(epsilon_z, zp.device)
    if h.shape != zp.shape or eps.shape != zp.shape:
        raise ValueError("H(z) / epsilon(z) channel length mismatch")
    if not planck_mass > 0.0:
        raise ValueError("Planck mass must be positive")
    return h.real ** 2 / (8.0 * math.pi ** 2 * eps.real.clamp_min(1e-20) * planck_mass ** 2)


@dataclass
class PrimordialProjection:
    """The transformed channels of one background and the spectrum assembled from them."""
    log_start: float
    log_step: float
    lattice_len: int
    s_values: torch.Tensor
    z_points: torch.Tensor
    h_z: torch.Tensor
    epsilon_z: torch.Tensor
    spectrum: torch.Tensor

    @classmethod
    def new(cls, log_start: float, log_step: float, lattice_len: int, s_values: _ArrayLike, z_points: _ArrayLike, h_z: _ArrayLike,
            epsilon_z: _ArrayLike, planck_mass: float) -> "PrimordialProjection":
        if not log_step > 0.0:
            raise ValueError("log_step must be positive")
        if not math.isfinite(log_start):
            raise ValueError("log_start must be finite")
        if lattice_len < 2:
            raise ValueError("lattice length must be at least 2")
        s, zp = _cplx(s_values), _cplx(z_points)
        h, eps = _cplx(h_z, s.device), _cplx(epsilon_z, s.device)
        if not (s.shape == zp.shape == h.shape == eps.shape):
            raise ValueError("s_values / z_points / H(z) / epsilon(z) length mismatch")
        out = cls(float(log_start), float(log_step), int(lattice_len), s, zp, h, eps, assemble_primordial_spectrum(zp, h, eps, planck_mass))
        out._emit(planck_mass)
        return out

    @classmethod
    def from_background(cls, hubble: LogLattice, epsilon: LogLattice, s_values: _ArrayLike, planck_mass: float) -> "PrimordialProjection":
        """Evaluates both channels at z = exp(s delta_tau) for every Mellin ordinate ``s`` and assembles the spectrum."""
        if len(hubble) != len(epsilon) or hubble.delta_tau != epsilon.delta_tau or hubble.tau0 != epsilon.tau0:
            raise ValueError("the H and epsilon channels must live on the same lattice")
        s = _cplx(s_values, hubble.samples.device)
        z = torch.exp(s * hubble.delta_tau)
        return cls.new(hubble.tau0, hubble.delta_tau, len(hubble), s, z, hubble.z_transform(z), epsilon.z_transform(z), planck_mass)

    def __len__(self) -> int:
        return self.s_values.numel()

    def is_empty(self) -> bool:
        return len(self) == 0

    def _emit(self, planck_mass: float) -> None:
        _obs.emit_tensor_op("inflaton_primordial_projection", [self.lattice_len, len(self)], [max(self.spectrum.numel(), 1), 3])

        def build():
            fin = lambda v: float(v) if math.isfinite(float(v)) else 0.0                 # noqa: E731
            spec = self.spectrum
            ok = torch.isfinite(spec)
            good = spec[ok]
            habs, eabs = self.h_z.abs(), self.epsilon_z.abs()
            empty = len(self) == 0
            return {"backend": "cpu" if spec.device.type == "cpu" else "cuda", "requested_backend": "auto",
                    "kind": "st_core_inflaton_primordial_projection", "log_start": fin(self.log_start), "log_step": fin(self.log_step),
                    "lattice_len": self.lattice_len, "evaluation_count": len(self), "z_point_count": self.z_points.numel(),
                    "spectrum_count": spec.numel(), "planck_mass": fin(planck_mass),
                    "h_abs_mean": 0.0 if empty else fin(habs.mean()), "h_abs_max": 0.0 if empty else fin(habs.max()),
                    "epsilon_abs_mean": 0.0 if empty else fin(eabs.mean()), "epsilon_abs_max": 0.0 if empty else fin(eabs.max()),
                    "epsilon_real_min": 0.0 if empty else fin(self.epsilon_z.real.min()),
                    "epsilon_clamp_count": int((self.epsilon_z.real < 1e-20).sum()),
                    "spectrum_min": fin(good.min()) if good.numel() else 0.0, "spectrum_max": fin(good.max()) if good.numel() else 0.0,
                    "spectrum_mean": fin(good.sum() / max(good.numel(), 1)) if spec.numel() else 0.0,
                    "spectrum_non_finite": int((~ok).sum())}
        _obs.emit_tensor_op_meta("inflaton_primordial_projection", build)
