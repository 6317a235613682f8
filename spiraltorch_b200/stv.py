"""Spino-tensor-vector kernels: the mixed tensor T = [[s0, E^T], [E, D]] with D = A + [omega]_x (A symmetric), its
determinant, the scalar invariants alpha = E^T adj(D) E / det D and beta = E^T (D D^T)^-1 E, the causal class of the
kernel vector (1, -D^-1 E), the ellipse in which the quadric E^T adj(D) E = s0 det D meets the ellipsoid
E^T (D D^T)^-1 E = 1, the smallest electric field / vorticity that makes T singular, and the projection of a Pauli
spinor's Bloch current through T onto a Z pulse.

Reference parity: crates/st-core/src/theory/stv.rs (`PauliSpinor` :60-154, `SpinoTensorVector` :157-275, `ZProjection`
:277-309, the telemetry record :335-408, `SpinoTensorKernel` :847-1230).  Every quantity is computed for a whole batch
of kernels at once: ``s0`` may carry any leading shape ``[...]`` with ``a`` ``[..., 3, 3]`` and ``e``, ``omega``
``[..., 3]``, and the invariants come back with that shape (0-dim for a single kernel), in float64 on the tensors'
device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import observability as _obs
from .zpulse import ZPulse, ZScale, ZSupport, source_label

TOLERANCE = 1e-9


class StvError(ValueError):
    pass


class NonSymmetric(StvError):
    pass


class SingularD(StvError):
    pass


class SingularDdT(StvError):
    pass


class NonPositiveGamma(StvError):
    pass


class ZeroSpinor(StvError):
    pass


class InvalidBlochVector(StvError):
    pass


def _t(x, device=None) -> torch.Tensor:
    return torch.as_tensor(x, dtype=torch.float64, device=device)


def _skew(w: torch.Tensor) -> torch.Tensor:
    z = torch.zeros_like(w[..., 0])
    return torch.stack([torch.stack([z, -w[..., 2], w[..., 1]], -1), torch.stack([w[..., 2], z, -w[..., 0]], -1),
                        torch.stack([-w[..., 1], w[..., 0], z], -1)], -2)


def _adjugate(m: torch.Tensor) -> torch.Tensor:
    """adj(M) for 3x3 matrices: its rows are the cross products of M's columns."""
    c0, c1, c2 = m[..., :, 0], m[..., :, 1], m[..., :, 2]
    return torch.stack([torch.linalg.cross(c1, c2), torch.linalg.cross(c2, c0), torch.linalg.cross(c0, c1)], -2)


def _quad(v: torch.Tensor, m: torch.Tensor, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    w = v if w is None else w
    return (v * (m @ w.unsqueeze(-1)).squeeze(-1)).sum(-1)


# ---------------------------------------------------------------------------------------------------------------
# spinors
# ---------------------------------------------------------------------------------------------------------------
class PauliSpinor:
    """A normalised two-component spinor ``[..., 2]`` (complex128)."""

    def __init__(self, components):
        c = torch.as_tensor(components).to(torch.complex128)
        if c.shape[-1] != 2:
            raise StvError("a Pauli spinor has two components")
        n2 = (c.abs() ** 2).sum(-1, keepdim=True)
        if bool((n2 <= TOLERANCE).any()):
            raise ZeroSpinor("spinor must have non-zero norm")
        self.components = c / n2.sqrt()

    @classmethod
    def from_bloch_angles(cls, theta, phi) -> "PauliSpinor":
        th = _t(theta).clamp(0.0, math.pi) * 0.5
        ph = _t(phi, th.device)
        return cls(torch.stack([torch.complex(th.cos(), torch.zeros_like(th)), torch.polar(th.sin(), ph)], -1))

    @classmethod
    def from_bloch_vector(cls, bloch) -> "PauliSpinor":
        b = _t(bloch)
        norm = b.norm(dim=-1, keepdim=True)
        if bool((~torch.isfinite(norm)).any()) or bool((norm <= TOLERANCE).any()):
            raise InvalidBlochVector(f"bloch vector must have a finite non-zero norm (norm = {float(norm.flatten()[0]):.3e})")
        b = b / norm
        return cls.from_bloch_angles(torch.acos(b[..., 2].clamp(-1.0, 1.0)), torch.atan2(b[..., 1], b[..., 0]))

    def phase_shift(self, phase) -> "PauliSpinor":
        out = object.__new__(PauliSpinor)
        out.components = self.components * torch.polar(torch.ones((), dtype=torch.float64), _t(phase)).unsqueeze(-1)
        return out

    def bloch_current(self) -> torch.Tensor:
        """(j0, jx, jy, jz) with j0 = |a|^2 + |b|^2 = 1 and the Bloch vector behind it."""
        a, b = self.components[..., 0], self.components[..., 1]
        coh = a * b.conj()
        return torch.stack([a.abs() ** 2 + b.abs() ** 2, 2.0 * coh.real, -2.0 * coh.imag, a.abs() ** 2 - b.abs() ** 2], -1)

    def bloch_vector(self) -> torch.Tensor:
        return self.bloch_current()[..., 1:]

    def bloch_angles(self) -> Tuple[torch.Tensor, torch.Tensor]:
        b = self.bloch_vector()
        return torch.acos(b[..., 2].clamp(-1.0, 1.0)), torch.atan2(b[..., 1], b[..., 0])


# ---------------------------------------------------------------------------------------------------------------
# kernels
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class MinimalVectorSolution:
    magnitude_squared: torch.Tensor        # NaN where no solution exists
    vector: torch.Tensor

    def exists(self) -> torch.Tensor:
        return torch.isfinite(self.magnitude_squared)

    def direction(self) -> torch.Tensor:
        n = self.magnitude_squared.clamp_min(0.0).sqrt().unsqueeze(-1)
        return torch.where(n > 0.0, self.vector / n.clamp_min(1e-300), torch.zeros_like(self.vector))


@dataclass
class IntersectionEllipse:
    """E(t) = R^T Gamma^-1/2 Q (a1 cos t, a2 sin t, +-sqrt(1 - a1^2 cos^2 t - a2^2 sin^2 t))."""
    rotation: torch.Tensor
    gamma_inv_sqrt: torch.Tensor
    q: torch.Tensor
    a1: torch.Tensor
    a2: torch.Tensor

    def parameters(self):
        return self.a1, self.a2

    def electric_field(self, t, branch: int = 1) -> torch.Tensor:
        """Points of the curve for parameters ``t`` (any shape, broadcast against the batch); ``branch`` is +1 or -1."""
        tt = _t(t, self.a1.device)
        z1, z2 = self.a1 * tt.cos(), self.a2 * tt.sin()
        z3 = (1.0 - z1 ** 2 - z2 ** 2).clamp_min(0.0).sqrt() * (1.0 if branch >= 0 else -1.0)
        z = torch.stack([z1, z2, z3], -1).unsqueeze(-1)
        return (self.rotation.transpose(-1, -2) @ (self.gamma_inv_sqrt @ (self.q @ z))).squeeze(-1)


class SpinoTensorKernel:
    def __init__(self, s0, a, e, omega):
        self.a = _t(a)
        dev = self.a.device
        self.s0, self.e, self.omega = _t(s0, dev), _t(e, dev), _t(omega, dev)
        if self.a.shape[-2:] != (3, 3) or self.e.shape[-1] != 3 or self.omega.shape[-1] != 3:
            raise StvError("a must be [..., 3, 3] and e, omega [..., 3]")
        dev_max = float((self.a - self.a.transpose(-1, -2)).abs().max())
        if dev_max > TOLERANCE:
            raise NonSymmetric(f"spatial tensor must be symmetric (max deviation {dev_max:.3e} exceeds tolerance {TOLERANCE:.3e})")

    # ---- the tensor itself ----
    def d(self) -> torch.Tensor:
        return self.a + _skew(self.omega)

    def dd_t(self) -> torch.Tensor:
        d = self.d()
        return d @ d.transpose(-1, -2)

    def block_tensor(self) -> torch.Tensor:
        d = self.d()
        top = torch.cat([self.s0.unsqueeze(-1), self.e.expand(*d.shape[:-2], 3)], -1).unsqueeze(-2)
        return torch.cat([top, torch.cat([self.e.expand(*d.shape[:-2], 3).unsqueeze(-1), d], -1)], -2)

    def apply_tensor(self, vector) -> torch.Tensor:
        return (self.block_tensor() @ _t(vector, self.a.device).unsqueeze(-1)).squeeze(-1)

    # ---- invariants ----
    def det_d(self) -> torch.Tensor:
        return torch.linalg.det(self.d())

    def adj_d(self) -> torch.Tensor:
        return _adjugate(self.d())

    def det_t(self) -> torch.Tensor:
        return self.s0 * self.det_d() - _quad(self.e, self.adj_d())

    def alpha(self) -> torch.Tensor:
        det = self.det_d()
        if bool((det.abs() <= TOLERANCE).any()):
            raise SingularD("matrix D is singular (determinant ~ 0)")
        return _quad(self.e, self.adj_d()) / det

    def beta(self) -> torch.Tensor:
        g = self.dd_t()
        det = torch.linalg.det(g)
        if bool((det.abs() <= TOLERANCE).any()):
            raise SingularDdT("matrix D D^T is singular (determinant ~ 0)")
        return _quad(self.e, _adjugate(g) / det[..., None, None])

    def z_scale_hint(self) -> Optional[ZScale]:
        return _z_scale_from_beta(float(self.beta()))

    def kernel_direction(self) -> torch.Tensor:
        det = self.det_d()
        if bool((det.abs() <= TOLERANCE * 1e-3).any()):
            raise SingularD("matrix D is singular (determinant ~ 0)")
        spatial = torch.linalg.solve(self.d(), self.e.expand(*det.shape, 3).unsqueeze(-1)).squeeze(-1)
        return torch.cat([torch.ones_like(spatial[..., :1]), -spatial], -1)

    def classify(self, tolerance: float = TOLERANCE):
        """``"lightlike"`` where |beta - 1| <= tolerance, ``"timelike"`` below one, ``"spacelike"`` above: a string for a
        single kernel, an int8 tensor (-1 timelike, 0 lightlike, +1 spacelike) for a batch."""
        beta = self.beta()
        code = torch.where((beta - 1.0).abs() <= tolerance, 0, torch.where(beta < 1.0, -1, 1)).to(torch.int8)
        return ("timelike", "lightlike", "spacelike")[int(code) + 1] if code.dim() == 0 else code

    def normalise_kernel(self, tolerance: float = TOLERANCE):
        """(class code as in :meth:`classify`, vector, beta): timelike kernel vectors are scaled to unit Minkowski norm,
        the others are returned as directions."""
        direction, beta = self.kernel_direction(), self.beta()
        n2 = 1.0 - beta
        timelike = (n2.abs() > tolerance) & (n2 > 0.0)
        vec = torch.where(timelike.unsqueeze(-1), direction / n2.clamp_min(1e-300).sqrt().unsqueeze(-1), direction)
        return self.classify(tolerance), vec, beta

    # ---- the singular set ----
    def intersection_curve(self, tolerance: float = TOLERANCE) -> Optional[IntersectionEllipse]:
        """The ellipse of electric fields with det T = 0 on the ellipsoid beta = 1, for a single kernel (None where the two
        surfaces do not meet)."""
        if self.s0.dim() != 0:
            raise StvError("intersection_curve takes a single kernel")
        d, g = self.d(), self.dd_t()
        if abs(float(torch.linalg.det(g))) <= TOLERANCE:
            raise SingularDdT("matrix D D^T is singular (determinant ~ 0)")
        inv = torch.linalg.inv(g)
        gvals, gvecs = torch.linalg.eigh(0.5 * (inv + inv.T))
        if bool((gvals <= tolerance).any()):
            raise NonPositiveGamma(f"intersection requires positive definite D D^T (encountered eigenvalue {float(gvals.min()):.3e})")
        gis = torch.diag(1.0 / gvals.sqrt())
        rot = gvecs.T
        adj = _adjugate(d)
        c = gis @ (rot @ (0.5 * (adj + adj.T)) @ rot.T) @ gis
        cvals, q = torch.linalg.eigh(0.5 * (c + c.T))
        c1, c2, c3 = (float(v) for v in cvals)
        if abs(c1 - c3) <= tolerance or abs(c2 - c3) <= tolerance:
            return None
        kappa = float(self.s0 * torch.linalg.det(d))
        a1, a2 = (kappa - c3) / (c1 - c3), (kappa - c3) / (c2 - c3)
        if not (math.isfinite(a1) and math.isfinite(a2)) or a1 < -tolerance or a2 < -tolerance or a1 > 1.0 + tolerance or a2 > 1.0 + tolerance:
            return None
        clamp = lambda v: min(max(v, 0.0), 1.0)                                             # noqa: E731
        return IntersectionEllipse(rot, gis, q, _t(math.sqrt(clamp(a1))), _t(math.sqrt(clamp(a2))))

    def minimal_electric_field(self) -> MinimalVectorSolution:
        """The smallest E with det T = 0 for E = 0 kernels: |E|^2 = s0 (det A + omega^T A omega) / lambda_max(adj A + omega omega^T)."""
        num = self.s0 * (torch.linalg.det(self.a) + _quad(self.omega, self.a))
        k = _adjugate(self.a) + self.omega.unsqueeze(-1) * self.omega.unsqueeze(-2)
        vals, vecs = torch.linalg.eigh(0.5 * (k + k.transpose(-1, -2)))
        lam, direction = vals[..., -1], vecs[..., :, -1]
        m2 = torch.where((num > 0.0) & (lam > TOLERANCE), num / lam.clamp_min(1e-300), torch.full_like(num, float("nan")))
        return MinimalVectorSolution(m2, direction * m2.clamp_min(0.0).nan_to_num(0.0).sqrt().unsqueeze(-1))

    def minimal_vorticity(self) -> MinimalVectorSolution:
        """The smallest omega with det T = 0: |omega|^2 = mu / lambda with mu = E^T adj(A) E - s0 det A and lambda the extreme
        eigenvalue of s0 A - E E^T on mu's side (zero vorticity where mu vanishes)."""
        mu = _quad(self.e, _adjugate(self.a)) - self.s0 * torch.linalg.det(self.a)
        k = self.s0[..., None, None] * self.a - self.e.unsqueeze(-1) * self.e.unsqueeze(-2)
        vals, vecs = torch.linalg.eigh(0.5 * (k + k.transpose(-1, -2)))
        pos = mu > 0.0
        lam = torch.where(pos, vals[..., -1], vals[..., 0])
        direction = torch.where(pos.unsqueeze(-1), vecs[..., :, -1], vecs[..., :, 0])
        ok = torch.where(pos, lam > TOLERANCE, lam < -TOLERANCE)
        m2 = torch.where(ok, mu / torch.where(lam == 0.0, torch.ones_like(lam), lam), torch.full_like(mu, float("nan")))
        m2 = torch.where(m2 > 0.0, m2, torch.full_like(mu, float("nan")))
        zero = mu.abs() <= TOLERANCE
        m2 = torch.where(zero, torch.zeros_like(mu), m2)
        return MinimalVectorSolution(m2, direction * m2.nan_to_num(0.0).clamp_min(0.0).sqrt().unsqueeze(-1))


# ---------------------------------------------------------------------------------------------------------------
# spinor x kernel -> Z pulse
# ---------------------------------------------------------------------------------------------------------------
def _z_scale_from_beta(beta: float) -> ZScale:
    return ZScale.new(math.sqrt(1.0 + beta)) if 1.0 + beta > 0.0 else ZScale.ONE


def _bloch_support(b) -> ZSupport:
    w = [min(max((float(x) + 1.0) / 2.0, 0.0), 1.0) for x in b]
    s = sum(w)
    if s > TOLERANCE:
        w = [x / s for x in w]
    return ZSupport.new(w[0], w[2], w[1])


@dataclass
class ZProjection:
    tempo: float
    band_energy: Tuple[float, float, float]
    drift: float
    z_bias: float
    support: ZSupport
    scale: Optional[ZScale]
    quality: float
    stderr: float

    def into_pulse(self, ts: int, source: str) -> ZPulse:
        return ZPulse(source=source, ts=int(ts), tempo=self.tempo, band_energy=self.band_energy,
                      density_fluctuation=ZPulse.density_fluctuation_for(self.band_energy), drift=self.drift, z_bias=self.z_bias,
                      support=self.support, scale=self.scale, quality=self.quality, stderr=self.stderr, latency_ms=0.0)


class SpinoTensorVector:
    """One spinor riding on one kernel."""

    def __init__(self, spinor: PauliSpinor, kernel: SpinoTensorKernel):
        self.spinor, self.kernel = spinor, kernel

    @classmethod
    def from_components(cls, components, kernel: SpinoTensorKernel) -> "SpinoTensorVector":
        return cls(PauliSpinor(components), kernel)

    def bloch_current(self) -> torch.Tensor:
        return self.spinor.bloch_current()

    def bloch_vector(self) -> torch.Tensor:
        return self.spinor.bloch_vector()

    def induced_vector(self) -> torch.Tensor:
        return self.kernel.apply_tensor(self.bloch_current())

    def with_phase_shift(self, phase) -> "SpinoTensorVector":
        return SpinoTensorVector(self.spinor.phase_shift(phase), self.kernel)

    def with_kernel(self, kernel: SpinoTensorKernel) -> "SpinoTensorVector":
        return SpinoTensorVector(self.spinor, kernel)

    def with_bloch_vector(self, bloch) -> "SpinoTensorVector":
        return SpinoTensorVector(PauliSpinor.from_bloch_vector(bloch), self.kernel)

    def z_projection(self) -> ZProjection:
        bloch = self.bloch_current()
        if bloch.dim() != 1:
            raise StvError("z_projection takes a single spinor and kernel")
        spatial = self.induced_vector()[1:]
        norm = float(spatial.norm())
        e = [abs(float(spatial[0])), abs(float(spatial[2])), abs(float(spatial[1]))]
        tot = sum(e)
        scale = norm if math.isfinite(norm) and norm > 0.0 else 0.0
        bands = tuple((x / tot) * scale for x in e) if tot > TOLERANCE else (0.0, 0.0, 0.0)
        beta = float(self.kernel.beta())
        quality = {"timelike": 1.0, "lightlike": 0.75, "spacelike": 0.5}[self.kernel.classify(TOLERANCE)]
        return ZProjection(norm, bands, float(bloch[3]), 1.0 - beta, _bloch_support(bloch[1:].tolist()), _z_scale_from_beta(beta), quality,
                           math.sqrt(abs(float(self.kernel.det_t()))))

    def project_to_zpulse(self, ts: int, source: str) -> ZPulse:
        pulse = self.z_projection().into_pulse(ts, source)
        k = self.kernel
        _obs.emit_tensor_op("spino_tensor_zpulse_project", [4, 3], [1, 14])

        def build():
            fin = lambda v: float(v) if math.isfinite(float(v)) else 0.0                    # noqa: E731
            try:
                alpha = float(k.alpha())
            except StvError:
                alpha = None
            beta = float(k.beta())
            return {"backend": "cpu" if k.a.device.type == "cpu" else "cuda", "requested_backend": "auto",
                    "kind": "st_core_spino_tensor_zpulse_project", "ts": pulse.ts, "source": source_label(pulse.source),
                    "causal_class": k.classify(TOLERANCE), "s0": fin(k.s0), "det_d": fin(k.det_d()), "det_t": fin(k.det_t()),
                    "has_alpha": alpha is not None, "alpha": fin(alpha or 0.0), "has_beta": True, "beta": fin(beta), "tempo": fin(pulse.tempo),
                    "band_above": fin(pulse.band_energy[0]), "band_here": fin(pulse.band_energy[1]), "band_beneath": fin(pulse.band_energy[2]),
                    "band_total": fin(pulse.total_energy()), "support": fin(pulse.support.total()),
                    "density_fluctuation": fin(pulse.density_fluctuation), "drift": fin(pulse.drift), "z_bias": fin(pulse.z_bias),
                    "quality": fin(pulse.quality), "stderr": fin(pulse.stderr), "scale_present": pulse.scale is not None,
                    "scale_physical_radius": fin(pulse.scale.physical_radius) if pulse.scale else 0.0,
                    "scale_log_radius": fin(pulse.scale.log_radius) if pulse.scale else 0.0}
        _obs.emit_tensor_op_meta("spino_tensor_zpulse_project", build)
        return pulse
