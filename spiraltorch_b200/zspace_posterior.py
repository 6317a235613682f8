"""Latent Z-space posterior: decoding a latent state into the five control metrics, and projecting observed metric
overrides onto it.

Decoding a state z of n values:  speed = tanh(mean|dz| + 0.25 ||z|| / n),  memory = tanh(mean z + 0.25 ||z||^2 / n),
stability = tanh(1.5 ((1 + mean|d2z|)^-1 + (1 + mean|dz|)^-1) - 1),  frac = tanh(E_alpha / ||z||^2) with the fractional
energy E_alpha = sum_k (2k / n)^(2 alpha) P_k over the one-sided, Parseval-normalised spectrum P_k,  drs = tanh((E_high -
E_low) / (E_high + E_low)) with the split at normalised frequency 0.5;  the latent gradient is the centred difference with
zero exterior boundaries scaled to max(1, ||g||_inf);  the barycentric weights are the normalised softplus of (speed,
memory, stability).  Projection blends the prior barycentre with the one recomputed after the overrides
(smoothing * prior + (1 - smoothing) * override), reports the RMS residual over the overridden base metrics and the
confidence exp(-residual), and scales that confidence by a telemetry reliability (1 + variance)^-1 x clamp(1 + 0.25
focus, 0.75, 1).  External gradients stay basis-tagged controls and never replace the latent gradient.

Reference parity: crates/st-core/src/inference/zspace_posterior.rs (formulas :30-43, spectrum and energies :212-330,
gradient / barycentre :332-403, `decode_zspace_posterior` :405-490, `project_zspace_posterior` :560-676).  Decoding is
batched: a ``[..., n]`` tensor of states is decoded with one real FFT and a few reductions on the tensor's device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from .telemetry import ZSpaceTelemetrySummary, canonical_metric_name

CONTRACT_VERSION = "spiraltorch.zspace_posterior.v2"
LATENT_GRADIENT_BASIS = "spiraltorch.zspace.latent_state.centered_difference.v1"
MAX_DIMENSION = 4096
BASE_METRICS = ("speed", "memory", "stability", "frac", "drs")
DEFAULT_FRACTIONAL_ORDER = 0.35
DEFAULT_SMOOTHING = 0.35


class ZSpacePosteriorError(ValueError):
    pass


@dataclass
class ZSpacePosteriorDecode:
    z_state: torch.Tensor
    alpha: float
    metrics: Dict[str, torch.Tensor]          # each of the state's leading shape
    gradient: torch.Tensor
    barycentric: torch.Tensor                 # [..., 3]
    energy: torch.Tensor
    spectral_energy: torch.Tensor
    parseval_relative_error: torch.Tensor
    frac_energy: torch.Tensor
    fractional_energy_ratio: torch.Tensor
    spectral_centroid: torch.Tensor
    spectral_bins: int
    gradient_basis: str = LATENT_GRADIENT_BASIS
    contract_version: str = CONTRACT_VERSION

    def metric_floats(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self.metrics.items()}


def _softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.softplus(x, threshold=20.0)


def _barycentric(speed: torch.Tensor, memory: torch.Tensor, stability: torch.Tensor) -> torch.Tensor:
    w = _softplus(torch.stack([speed, memory, stability], -1))
    total = w.sum(-1, keepdim=True)
    if not bool((torch.isfinite(total) & (total > 0.0)).all()):
        raise ZSpacePosteriorError("invalid barycentric mass")
    return w / total


def decode_zspace_posterior(z_state, alpha: float = DEFAULT_FRACTIONAL_ORDER) -> ZSpacePosteriorDecode:
    z = torch.as_tensor(z_state, dtype=torch.float64)
    n = z.shape[-1] if z.dim() else 0
    if n == 0 or n > MAX_DIMENSION:
        raise ZSpacePosteriorError(f"z_state needs 1..{MAX_DIMENSION} values per state, got {n}")
    if not bool(torch.isfinite(z).all()):
        raise ZSpacePosteriorError("z_state must be finite")
    if not (math.isfinite(alpha) and alpha >= 0.0):
        raise ZSpacePosteriorError(f"alpha must be finite and non-negative, received {alpha}")
    dz = z[..., 1:] - z[..., :-1]
    d2z = z[..., 2:] - 2.0 * z[..., 1:-1] + z[..., :-2]
    mean_velocity = dz.abs().sum(-1) / max(n - 1, 1)
    curvature = d2z.abs().sum(-1) / max(n - 2, 1)
    energy = (z * z).sum(-1)
    centre = z.mean(-1)
    spec = torch.fft.rfft(z, dim=-1)
    mult = torch.full((spec.shape[-1],), 2.0, dtype=torch.float64, device=z.device)
    mult[0] = 1.0
    if n % 2 == 0:
        mult[n // 2] = 1.0
    bins = mult * (spec.real ** 2 + spec.imag ** 2) / n
    spectral_energy = bins.sum(-1)
    safe = torch.where(energy == 0.0, torch.ones_like(energy), energy)
    parseval = torch.where(energy == 0.0, torch.zeros_like(energy), (spectral_energy - energy).abs() / safe)
    omega = 2.0 * torch.arange(spec.shape[-1], dtype=torch.float64, device=z.device) / n
    if bins.shape[-1] > 1:
        weight = torch.where(omega > 0.0, omega.clamp_min(1e-300) ** (2.0 * alpha), torch.full_like(omega, 1.0 if alpha == 0.0 else 0.0))
        frac_energy = (weight * bins).sum(-1)
        low = bins[..., omega < 0.5].sum(-1)
        high = bins[..., omega >= 0.5].sum(-1)
        tot = high + low
        drs = torch.where(tot == 0.0, torch.zeros_like(tot), torch.tanh((high - low) / torch.where(tot == 0.0, torch.ones_like(tot), tot)))
    else:
        frac_energy = torch.zeros_like(energy)
        drs = torch.zeros_like(energy)
    ratio = torch.where(energy == 0.0, torch.zeros_like(energy), frac_energy / safe)
    se_safe = torch.where(spectral_energy == 0.0, torch.ones_like(spectral_energy), spectral_energy)
    centroid = torch.where(spectral_energy == 0.0, torch.zeros_like(spectral_energy), (omega * bins).sum(-1) / se_safe)
    pad = torch.nn.functional.pad(z, (1, 1))
    grad = 0.5 * ((pad[..., 1:-1] - pad[..., :-2]) + (pad[..., 2:] - pad[..., 1:-1]))
    grad = grad / grad.abs().amax(-1, keepdim=True).clamp_min(1.0)
    speed = torch.tanh(mean_velocity + 0.25 * energy.sqrt() / n)
    memory = torch.tanh(centre + 0.25 * energy / n)
    stability = torch.tanh((1.0 / (1.0 + curvature) + 1.0 / (1.0 + mean_velocity)) * 1.5 - 1.0)
    metrics = {"speed": speed, "memory": memory, "stability": stability, "frac": torch.tanh(ratio), "drs": drs}
    return ZSpacePosteriorDecode(z, float(alpha), metrics, grad, _barycentric(speed, memory, stability), energy, spectral_energy, parseval,
                                 frac_energy, ratio, centroid, spec.shape[-1])


@dataclass
class ZSpacePosteriorControlGradient:
    basis: str
    values: List[float]
    l2: float
    linf: float
    source: str = "partial"

    @property
    def dimension(self) -> int:
        return len(self.values)


@dataclass
class ZSpacePosteriorTelemetryAdjustment:
    variance_reliability: float
    focus_reliability: float
    combined_reliability: float
    residual_before: float
    confidence_before: float


@dataclass
class ZSpacePosteriorProjection:
    smoothing: float
    metrics: Dict[str, float]
    gradient: torch.Tensor
    control_gradient: Optional[ZSpacePosteriorControlGradient]
    barycentric: List[float]
    residual: float
    residual_metric_count: int
    confidence: float
    telemetry_reliability: float
    applied: Dict[str, float]
    prior: ZSpacePosteriorDecode
    telemetry: Optional[ZSpaceTelemetrySummary]
    telemetry_adjustment: Optional[ZSpacePosteriorTelemetryAdjustment]
    gradient_basis: str = LATENT_GRADIENT_BASIS
    gradient_source: str = "latent_state"


def _numeric_leaves(value: Any, out: List[float]) -> None:
    if isinstance(value, bool):
        return
    if isinstance(value, (int, float)):
        out.append(float(value))
    elif isinstance(value, dict):
        for k in sorted(value):
            _numeric_leaves(value[k], out)
    elif isinstance(value, (list, tuple)):
        for v in value:
            _numeric_leaves(v, out)


def project_zspace_posterior(z_state, partial: Optional[Dict[str, Any]] = None, alpha: float = DEFAULT_FRACTIONAL_ORDER,
                             smoothing: float = DEFAULT_SMOOTHING, gradient_basis: Optional[str] = None,
                             telemetry: Sequence[Any] = ()) -> ZSpacePosteriorProjection:
    """``partial`` maps metric labels (aliases allowed) to scalars; a ``gradient`` entry is a vector and needs ``gradient_basis``."""
    if not (math.isfinite(smoothing) and 0.0 <= smoothing <= 1.0):
        raise ZSpacePosteriorError(f"smoothing must lie in [0, 1], received {smoothing}")
    prior = decode_zspace_posterior(z_state, alpha)
    if prior.z_state.dim() != 1:
        raise ZSpacePosteriorError("projection takes a single state")
    metrics = prior.metric_floats()
    applied: Dict[str, float] = {}
    control: Optional[ZSpacePosteriorControlGradient] = None
    sq, count = 0.0, 0
    for label, value in sorted((partial or {}).items()):
        name = canonical_metric_name(label)
        if name is None:
            raise ZSpacePosteriorError(f"unknown metric {label!r}")
        if name == "gradient":
            vals = [float(v) for v in value]
            if not vals or not all(math.isfinite(v) for v in vals):
                raise ZSpacePosteriorError("control gradient must be a non-empty finite vector")
            if not gradient_basis:
                raise ZSpacePosteriorError("a control gradient needs its basis named")
            control = ZSpacePosteriorControlGradient(gradient_basis, vals, math.sqrt(sum(v * v for v in vals)), max(abs(v) for v in vals))
            continue
        v = float(value)
        if not math.isfinite(v):
            raise ZSpacePosteriorError(f"metric {label!r} must be finite")
        if name in BASE_METRICS:
            sq += (v - metrics[name]) ** 2
            count += 1
        metrics[name] = v
        applied[name] = v
    if gradient_basis and control is None:
        raise ZSpacePosteriorError("a gradient basis was named without a gradient")
    override = _barycentric(*(torch.tensor(metrics[m], dtype=torch.float64) for m in ("speed", "memory", "stability")))
    bary = smoothing * prior.barycentric + (1.0 - smoothing) * override
    mass = float(bary.sum())
    if not (math.isfinite(mass) and mass > 0.0):
        raise ZSpacePosteriorError("invalid barycentric mass")
    bary = bary / mass
    residual = math.sqrt(sq / count) if count else 0.0
    confidence_before = math.exp(-residual)
    confidence, reliability, summary, adjustment = confidence_before, 1.0, None, None
    if telemetry:
        leaves: List[float] = []
        for payload in telemetry:
            _numeric_leaves(payload, leaves)
        summary = ZSpaceTelemetrySummary.from_values(leaves)
        r_var = 1.0 / (1.0 + max(summary.variance, 0.0))
        r_focus = min(max(1.0 + 0.25 * summary.focus, 0.75), 1.0)
        reliability = r_var * r_focus
        confidence = min(max(confidence * reliability, 0.0), confidence_before)
        adjustment = ZSpacePosteriorTelemetryAdjustment(r_var, r_focus, reliability, residual, confidence_before)
    return ZSpacePosteriorProjection(smoothing, metrics, prior.gradient, control, bary.tolist(), residual, count, confidence, reliability,
                                     applied, prior, summary, adjustment)
