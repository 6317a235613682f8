"""Z-space field layers: topos resonator, Klein–Gordon / Hamilton–Jacobi / Schrödinger dynamic
fields, continuous wavelet features, Z-space projector and the relativity scaler.

The element-wise arithmetic restates the reference's tensor-utility shaders
(crates/st-tensor/src/wgpu_shaders/tensor_utils.wgsl: ``porous_mix`` :44-61,
``topos_resonator_forward`` :126-143, ``dynamic_klein_gordon_forward`` :173-250 — one leap-frog step
with a periodic feature Laplacian, cubic self-interaction, per-column mass² and source —,
``dynamic_hamilton_jacobi_forward`` :352-378, ``dynamic_schrodinger_forward`` :416-447) and the
layers built on them (crates/st-nn/src/layers/{topos_resonator,dynamic_field,continuous_wavelet,
zspace_projector,zrelativity}.rs).  Expressed as PyTorch tensor math on the caller's device, so the
module base class derives the backward passes; the hot kernels of this framework are not involved.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..tensor import TensorError
from .modules import Module, _mm


def porous_mix(value: torch.Tensor, saturation: float, porosity: float) -> torch.Tensor:
    """Identity inside ``[-saturation, saturation]``; outside, the magnitude is the limit softened by
    ``1 - min(porosity/4, 1) * bleed`` with ``bleed = (|v| - limit) / (|v| + limit)``."""
    if saturation <= 0:
        return torch.zeros_like(value)
    limit = abs(saturation)
    mag = value.abs()
    if porosity <= 1.1920929e-07:
        out = torch.sign(value) * limit
    else:
        bleed = ((mag - limit) / (mag + limit)).clamp(max=1.0)
        out = torch.sign(value) * limit * (1.0 - min(porosity * 0.25, 1.0) * bleed).clamp(min=0.0)
    return torch.where(mag <= limit, value, out)


def _roll(x: torch.Tensor, shift: int) -> torch.Tensor:
    return torch.roll(x, shifts=shift, dims=1)


def _laplacian(x: torch.Tensor) -> torch.Tensor:
    if x.shape[1] == 1:
        return torch.zeros_like(x)
    return _roll(x, 1) - 2.0 * x + _roll(x, -1)


class ToposResonator(Module):
    """``r_{t+1} = porous_mix(x·gate + feedback·r_t)`` iterated ``iterations`` times from ``r_0 = 0``;
    ``gate`` is a learned per-feature vector."""

    def __init__(self, name: str, features: int, *, feedback: float = 0.5, iterations: int = 3, saturation: float = 1.0,
                 porosity: float = 0.5):
        super().__init__()
        if features <= 0 or iterations <= 0:
            raise TensorError("topos resonator needs positive features and iterations")
        self.name, self.features = name, features
        self.feedback, self.iterations, self.saturation, self.porosity = feedback, iterations, saturation, porosity
        self.gate = self._register(f"{name}::gate", torch.ones(1, features))

    def _fwd(self, x, p):
        drive = x * p[f"{self.name}::gate"]
        r = torch.zeros_like(drive)
        for _ in range(self.iterations):
            r = porous_mix(drive + self.feedback * r, self.saturation, self.porosity)
        return r


class DynamicKleinGordonField(Module):
    """One leap-frog step of ``φ'' = κ·Δφ − m²φ − λφ³ + s`` over the feature axis (periodic).  Input
    columns are ``[field | momentum]``; output has the same layout."""

    def __init__(self, name: str, features: int, *, dt: float = 0.1, stiffness: float = 1.0, self_interaction: float = 0.0,
                 momentum_decay: float = 1.0):
        super().__init__()
        self.name, self.features = name, features
        self.dt, self.stiffness, self.lam, self.decay = dt, stiffness, self_interaction, momentum_decay
        self.mass2 = self._register(f"{name}::mass_squared", torch.ones(1, features))
        self.source = self._register(f"{name}::source", torch.zeros(1, features))

    def _force(self, field, p):
        return self.stiffness * _laplacian(field) - p[f"{self.name}::mass_squared"] * field - self.lam * field ** 3 \
            + p[f"{self.name}::source"]

    def _fwd(self, x, p):
        if x.shape[1] != 2 * self.features:
            raise TensorError(f"{self.name}: expected {2 * self.features} columns (field | momentum), got {x.shape[1]}")
        field, mom = x[:, : self.features], x[:, self.features:]
        half = self.decay * mom + 0.5 * self.dt * self._force(field, p)
        new_field = field + self.dt * half
        new_mom = self.decay * (half + 0.5 * self.dt * self._force(new_field, p))
        return torch.cat([new_field, new_mom], 1)


class DynamicHamiltonJacobiField(Module):
    """``S ← S − dt·(½·k·(∇S)² + V) + ν·ΔS`` with a centred periodic gradient scaled by ``grad_scale``
    and a learned per-feature potential ``V``."""

    def __init__(self, name: str, features: int, *, dt: float = 0.1, kinetic: float = 1.0, viscosity: float = 0.0,
                 grad_scale: float = 0.5):
        super().__init__()
        self.name, self.features = name, features
        self.dt, self.kinetic, self.viscosity, self.grad_scale = dt, kinetic, viscosity, grad_scale
        self.potential = self._register(f"{name}::potential", torch.zeros(1, features))

    def _fwd(self, x, p):
        grad = (_roll(x, -1) - _roll(x, 1)) * self.grad_scale if x.shape[1] > 1 else torch.zeros_like(x)
        ham = 0.5 * self.kinetic * grad * grad + p[f"{self.name}::potential"]
        return x - self.dt * ham + self.viscosity * _laplacian(x)


class DynamicSchrodingerField(Module):
    """Split-step phase rotation of a real amplitude: each feature picks up the phase ``V·dt`` and
    hops to its pair partner (columns ``2i``, ``2i+1``) with angle ``hopping·dt``; output columns are
    ``[real | imaginary]``, damped by ``exp(−½·γ·dt)``."""

    def __init__(self, name: str, features: int, *, dt: float = 0.1, hopping: float = 0.0, damping: float = 0.0):
        super().__init__()
        self.name, self.features, self.dt, self.hopping, self.damping = name, features, dt, hopping, damping
        self.potential = self._register(f"{name}::potential", torch.zeros(1, features))

    def _fwd(self, x, p):
        phase = (p[f"{self.name}::potential"] * self.dt).expand_as(x)
        damp = math.exp(-0.5 * self.damping * self.dt)
        n = self.features - self.features % 2
        if n >= 2 and self.hopping != 0.0:
            idx = torch.arange(self.features, device=x.device)
            partner = torch.where(idx < n, idx ^ 1, idx)
            has = (idx < n).to(x.dtype)
            xp, pp = x[:, partner], phase[:, partner]
            mean_phase = 0.5 * phase + 0.5 * pp
            c, s = math.cos(self.hopping * self.dt), math.sin(self.hopping * self.dt)
            re = damp * (torch.where(has > 0, torch.tensor(c, device=x.device), torch.tensor(1.0, device=x.device)) * x * torch.cos(phase)
                         - has * s * xp * torch.sin(mean_phase))
            im = damp * (-torch.where(has > 0, torch.tensor(c, device=x.device), torch.tensor(1.0, device=x.device)) * x * torch.sin(phase)
                         - has * s * xp * torch.cos(mean_phase))
        else:
            re, im = damp * x * torch.cos(phase), -damp * x * torch.sin(phase)
        return torch.cat([re, im], 1)


class ContinuousWavelet(Module):
    """Morlet wavelet features of a signal laid out along the columns: for each learned scale ``a`` the
    response ``Σ_t x_t · exp(−t²/2a²)·cos(ω0·t/a) / √a`` over the whole row (scales are positive through
    a softplus), giving ``(rows, scales)``."""

    def __init__(self, name: str, length: int, scales: int = 4, omega0: float = 5.0):
        super().__init__()
        if length <= 0 or scales <= 0:
            raise TensorError("wavelet needs a positive length and at least one scale")
        self.name, self.length, self.n_scales, self.omega0 = name, length, scales, omega0
        init = torch.log(torch.expm1(torch.linspace(1.0, max(1.0, length / 4), scales))).reshape(1, scales)
        self.raw_scales = self._register(f"{name}::scales", init)

    def _fwd(self, x, p):
        if x.shape[1] != self.length:
            raise TensorError(f"{self.name}: expected {self.length} columns, got {x.shape[1]}")
        a = torch.nn.functional.softplus(p[f"{self.name}::scales"]).reshape(-1, 1)                 # [S, 1]
        t = (torch.arange(self.length, device=x.device, dtype=x.dtype) - (self.length - 1) / 2).reshape(1, -1)
        bank = torch.exp(-0.5 * (t / a) ** 2) * torch.cos(self.omega0 * t / a) / torch.sqrt(a)       # [S, L]
        return _mm(x, bank.t().contiguous())


class ZSpaceProjector(Module):
    """Linear map followed by projection into the open Poincaré ball of curvature ``c < 0``: rows whose
    norm reaches ``1/√−c`` are pulled just inside it."""

    def __init__(self, name: str, input_dim: int, output_dim: int, curvature: float = -1.0, margin: float = 1e-3):
        super().__init__()
        if not curvature < 0:
            raise TensorError("curvature must be negative")
        self.name, self.curvature, self.margin = name, curvature, margin
        g = torch.Generator().manual_seed(17)
        self.weight = self._register(f"{name}::weight", torch.randn(input_dim, output_dim, generator=g) / math.sqrt(input_dim))
        self.bias = self._register(f"{name}::bias", torch.zeros(1, output_dim))

    def _fwd(self, x, p):
        y = _mm(x, p[f"{self.name}::weight"]) + p[f"{self.name}::bias"]
        radius = (1.0 - self.margin) / math.sqrt(-self.curvature)
        norm = y.norm(dim=1, keepdim=True).clamp(min=1e-12)
        return torch.where(norm > radius, y * (radius / norm), y)


class ZRelativity(Module):
    """Per-feature Lorentz rescaling ``y = x · √(1 − β²)`` with a learned rapidity ``β = tanh(w)``."""

    def __init__(self, name: str, features: int):
        super().__init__()
        self.name = name
        self.rapidity = self._register(f"{name}::rapidity", torch.zeros(1, features))

    def _fwd(self, x, p):
        beta = torch.tanh(p[f"{self.name}::rapidity"])
        return x * torch.sqrt((1.0 - beta * beta).clamp(min=1e-12))


class Conv1d(Module):
    """1-D convolution over rows laid out ``(batch, C·L)``; weight ``(OC, IC·k)`` and bias ``(1, OC)`` as
    in the reference's N-D convolutions (crates/st-nn/src/layers/conv.rs:330)."""

    def __init__(self, name: str, in_channels: int, out_channels: int, kernel: int, length: int, *, stride: int = 1,
                 padding: int = 0):
        super().__init__()
        self.name, self.ic, self.oc, self.k, self.length, self.stride, self.padding = \
            name, in_channels, out_channels, kernel, length, stride, padding
        g = torch.Generator().manual_seed(29)
        self.weight = self._register(f"{name}::weight", torch.randn(out_channels, in_channels * kernel, generator=g)
                                     / math.sqrt(in_channels * kernel))
        self.bias = self._register(f"{name}::bias", torch.zeros(1, out_channels))

    def output_length(self) -> int:
        return (self.length + 2 * self.padding - self.k) // self.stride + 1

    def _fwd(self, x, p):
        if x.shape[1] != self.ic * self.length:
            raise TensorError(f"{self.name}: expected {self.ic * self.length} columns, got {x.shape[1]}")
        xs = torch.nn.functional.pad(x.reshape(-1, self.ic, self.length), (self.padding, self.padding))
        cols = xs.unfold(2, self.k, self.stride)                                   # [B, IC, OL, k]
        B, _, OL, _ = cols.shape
        cols = cols.permute(0, 2, 1, 3).reshape(B * OL, self.ic * self.k)
        y = _mm(cols, p[f"{self.name}::weight"].t().contiguous()) + p[f"{self.name}::bias"]
        return y.reshape(B, OL, self.oc).permute(0, 2, 1).reshape(B, self.oc * OL)
