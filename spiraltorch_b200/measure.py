"""Measures on probability tensors: the Z-space barycenter and the NIRT weight update.

Restated from crates/st-tensor/src/pure/measure.rs: ``z_space_barycenter`` (:365-500 — weighted
geometric mean of normalised densities at temperature ``Σw + entropy_weight``, KL energy, entropy,
optional coupling energy ``½·β·Σ_uv J_uv·symKL(p_u, p_v)``, objective ``KL + coupling − γ·H``) and
``nirt_weight_update`` (:653-735 — additive similarity step, clamp at zero, renormalise).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .tensor import Tensor, TensorError

_TINY = 1e-12


@dataclass
class BarycenterIntermediate:
    """A point on the straight path from the weighted arithmetic mean (interpolation 0) to the barycenter (1)."""
    interpolation: float
    density: Tensor
    kl_energy: float
    entropy: float
    objective: float


@dataclass
class ZSpaceBarycenter:
    objective: float
    density: Tensor
    kl_energy: float
    entropy: float
    coupling_energy: float
    effective_weight: float
    intermediates: list = field(default_factory=list)


def _normalise(t: torch.Tensor) -> torch.Tensor:
    t = t.double()
    if not bool(torch.isfinite(t).all()) or bool((t < 0).any()):
        raise TensorError("densities must be finite and non-negative")
    s = t.sum()
    if s <= 0:
        raise TensorError("density has no mass")
    return (t / s).clamp(min=_TINY)


def _kl(p: torch.Tensor, q: torch.Tensor) -> float:
    return float((p * (p / q).log()).sum())


def z_space_barycenter(weights: Sequence[float], densities: Sequence[Tensor], entropy_weight: float, beta_j: float,
                       coupling: Optional[Tensor] = None) -> ZSpaceBarycenter:
    if not densities:
        raise TensorError("z_space_barycenter: empty input")
    if len(weights) != len(densities):
        raise TensorError(f"z_space_barycenter: {len(densities)} densities but {len(weights)} weights")
    if not math.isfinite(entropy_weight) or not math.isfinite(beta_j) or beta_j < 0:
        raise TensorError("entropy_weight must be finite and beta_j finite and non-negative")
    if any((not math.isfinite(w)) or w < 0 for w in weights):
        raise TensorError("barycenter weights must be finite and non-negative")
    effective = float(sum(weights)) + entropy_weight
    if effective <= 0:
        raise TensorError(f"degenerate barycenter (effective weight {effective})")
    shape = densities[0].shape()
    dists = []
    for d in densities:
        if d.shape() != shape:
            raise TensorError(f"shape mismatch: {shape} vs {d.shape()}")
        dists.append(_normalise(d.torch().reshape(-1)))
    log_mode = sum(w * p.log() for w, p in zip(weights, dists)) / effective
    bary = torch.softmax(log_mode, 0) if isinstance(log_mode, torch.Tensor) else torch.full_like(dists[0], 1.0 / dists[0].numel())
    coupling_energy = 0.0
    if coupling is not None:
        J = coupling.torch().double()
        n = len(dists)
        if tuple(J.shape) != (n, n):
            raise TensorError(f"coupling must be {n} x {n}")
        if not bool(torch.isfinite(J).all()) or bool((J < 0).any()):
            raise TensorError("barycenter_coupling must be finite and non-negative")
        acc = 0.0
        for u in range(n):
            for v in range(n):
                if J[u, v] != 0:
                    acc += float(J[u, v]) * (_kl(dists[u], dists[v]) + _kl(dists[v], dists[u]))
        coupling_energy = 0.5 * beta_j * acc
    kl_energy = sum(w * _kl(bary, p) for w, p in zip(weights, dists))
    entropy = float(-(bary * bary.log()).sum())
    wsum = float(sum(weights))
    baseline = _normalise(sum(w * p for w, p in zip(weights, dists)) / wsum) if wsum > 0 else \
        torch.full_like(dists[0], 1.0 / dists[0].numel())          # no chart carries weight: start from the uniform density
    stages = []
    for alpha in (0.0, 0.25, 0.5, 0.75, 1.0):
        mix = _normalise((1.0 - alpha) * baseline + alpha * bary)
        kl_a = float(sum(w * _kl(mix, p) for w, p in zip(weights, dists)))
        ent_a = float(-(mix * mix.clamp(min=_TINY).log()).sum())
        stages.append(BarycenterIntermediate(alpha, Tensor._wrap(mix.float().reshape(shape)), kl_a, ent_a,
                                             kl_a + coupling_energy - entropy_weight * ent_a))
    return ZSpaceBarycenter(kl_energy + coupling_energy - entropy_weight * entropy,
                            Tensor._wrap(bary.float().reshape(shape)), float(kl_energy), entropy, coupling_energy, effective,
                            stages)


def nirt_weight_update(weights: Sequence[float], similarities: Sequence[float], coherence_rate: float, eta: float) -> list:
    """``w_i ← max(0, w_i + η·ρ·s_i)`` renormalised to sum to one; returns the new weights."""
    if not weights:
        raise TensorError("nirt_weight_update: empty weights")
    if len(weights) != len(similarities):
        raise TensorError(f"nirt_weight_update: {len(weights)} weights but {len(similarities)} similarities")
    if not (math.isfinite(eta) and eta > 0):
        raise TensorError(f"learning rate must be positive, got {eta}")
    if not (math.isfinite(coherence_rate) and 0.0 <= coherence_rate <= 1.0):
        raise TensorError("nirt_coherence_rate must lie in [0, 1]")
    out = []
    for w, s in zip(weights, similarities):
        if not math.isfinite(w) or w < 0:
            raise TensorError(f"weights must be finite and non-negative, got {w}")
        if not math.isfinite(s) or not -1.0 <= s <= 1.0:
            raise TensorError("nirt_similarity must lie in [-1, 1]")
        out.append(max(0.0, w + eta * coherence_rate * s))
    total = sum(out)
    if total <= 0:
        raise TensorError("degenerate weights after the update")
    return [v / total for v in out]
