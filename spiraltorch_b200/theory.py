"""Theory helpers used by the telemetry / language pipelines: Maxwell-coded envelopes and their
sequential Z detector, the Leech-lattice projector, and the RoPE table cache.

Parity: crates/st-core/src/theory/maxwell.rs:113-600 (`MaxwellFingerprint`, `MeaningGate`,
`expected_z_curve`, `simulate_z_curve`, `SequentialZ`, `MaxwellZProjector`, `MaxwellZPulse`),
crates/st-core/src/util/math.rs:59-175 (`LeechProjector`, `ramanujan_pi`),
crates/st-core/src/util/rope_lru.rs (`RopeLRU`).

The per-block statistics are scalar host arithmetic (one float per block arrives from a matched
filter); curves and envelope series are vectorised torch ops and the RoPE tables are produced
directly as device tensors, so a cached entry is what the rotary kernel consumes.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .nn.conv import _LEECH_PACKING_DENSITY, ramanujan_pi


class MaxwellSeriesError(ValueError):
    pass


class MaxwellExpectationError(ValueError):
    pass


# ----------------------------------------------------------------------------------------------
# Leech projector
# ----------------------------------------------------------------------------------------------
class LeechProjector:
    """`enrich(g) = weight * density(Leech) * g * sqrt(rank) * (pi / ramanujan_pi(iterations))`."""

    def __init__(self, rank: int, weight: float, ramanujan_iterations: int = 0):
        self.sqrt_rank = math.sqrt(max(int(rank), 1))
        self.weight = max(float(weight), 0.0)
        self.ramanujan_iterations = int(ramanujan_iterations)
        self.ramanujan_pi = math.pi if ramanujan_iterations == 0 else max(ramanujan_pi(ramanujan_iterations), 2.2e-16)
        self.ramanujan_ratio = math.pi / self.ramanujan_pi

    def ramanujan_delta(self) -> float:
        return abs(self.ramanujan_pi - math.pi)

    def enrich(self, geodesic: float) -> float:
        if self.weight <= 2.2e-16 or geodesic <= 2.2e-16:
            return 0.0
        return self.weight * _LEECH_PACKING_DENSITY * geodesic * self.sqrt_rank * self.ramanujan_ratio


# ----------------------------------------------------------------------------------------------
# Maxwell fingerprint, gate, expected / simulated Z curves
# ----------------------------------------------------------------------------------------------
@dataclass
class MaxwellFingerprint:
    """`lambda = gamma * alpha * |H_tis| * 10^(-S_dB/20) * G * |cos(theta)| / r`."""
    gamma: float
    modulation_depth: float
    tissue_response: float
    shielding_db: float
    transmit_gain: float
    polarization_angle: float
    distance_m: float

    def __post_init__(self):
        self.gamma, self.modulation_depth = max(self.gamma, 0.0), max(self.modulation_depth, 0.0)
        self.tissue_response, self.transmit_gain = max(self.tissue_response, 0.0), max(self.transmit_gain, 0.0)
        self.distance_m = max(self.distance_m, 2.2e-16)

    def shielding_factor(self) -> float:
        return 10.0 ** (-self.shielding_db / 20.0)

    def polarization_alignment(self) -> float:
        return abs(math.cos(self.polarization_angle))

    def lambda_(self) -> float:
        return (self.gamma * self.modulation_depth * self.tissue_response * self.shielding_factor()
                * self.transmit_gain * self.polarization_alignment() / self.distance_m)

    def expected_block_mean(self, kappa: float) -> float:
        return kappa * self.lambda_()


@dataclass
class MeaningGate:
    """`u_tot(t) = [lambda + mu * rho(t)] * c(t)` with `rho` clamped to [-1, 1]."""
    physical_gain: float
    semantic_gain: float

    def __post_init__(self):
        self.semantic_gain = max(self.semantic_gain, 0.0)

    def envelope(self, rho: float) -> float:
        return self.physical_gain + self.semantic_gain * min(max(rho, -1.0), 1.0)

    def envelope_series(self, rho_values, code_values) -> torch.Tensor:
        rho = torch.as_tensor(rho_values, dtype=torch.float64)
        code = torch.as_tensor(code_values, dtype=torch.float64).to(rho.device)
        if rho.shape != code.shape:
            raise MaxwellSeriesError(f"rho and code lengths must match (rho={rho.numel()}, code={code.numel()})")
        for name, t in (("rho", rho), ("code", code)):
            bad = (~torch.isfinite(t)).nonzero()
            if bad.numel():
                i = int(bad[0])
                raise MaxwellSeriesError(f"{name}[{i}] is not finite: {float(t.flatten()[i])}")
        return (self.physical_gain + self.semantic_gain * rho.clamp(-1.0, 1.0)) * code


def _check_curve_args(sigma: float, kappa: float, lam: float) -> float:
    if not (math.isfinite(sigma) and sigma > 0):
        raise MaxwellExpectationError(f"sigma must be finite and > 0, got {sigma}")
    if not math.isfinite(kappa):
        raise MaxwellExpectationError(f"kappa must be finite, got {kappa}")
    if not math.isfinite(lam):
        raise MaxwellExpectationError(f"lambda must be finite, got {lam}")
    mean = kappa * lam
    if not math.isfinite(mean) or not math.isfinite(mean / sigma):
        raise MaxwellExpectationError("expected z coefficient became non-finite")
    return mean


def expected_z_curve(blocks: int, sigma: float, kappa: float, lam: float) -> torch.Tensor:
    """`z_n = (kappa * lambda / sigma) * sqrt(n)` for n = 1..blocks."""
    if blocks == 0:
        return torch.zeros(0, dtype=torch.float64)
    mean = _check_curve_args(sigma, kappa, lam)
    return (mean / sigma) * torch.sqrt(torch.arange(1, blocks + 1, dtype=torch.float64))


def simulate_z_curve(blocks: int, sigma: float, kappa: float, lam: float, seed: int = 0) -> torch.Tensor:
    """Running Z statistic of `blocks` Gaussian block means drawn from a seeded generator, computed
    for all prefixes at once from cumulative sums (0 where fewer than two blocks or zero spread)."""
    if blocks == 0:
        return torch.zeros(0, dtype=torch.float64)
    mean = _check_curve_args(sigma, kappa, lam)
    g = torch.Generator().manual_seed(int(seed))
    x = mean + sigma * torch.randn(blocks, dtype=torch.float64, generator=g)
    n = torch.arange(1, blocks + 1, dtype=torch.float64)
    m = torch.cumsum(x, 0) / n
    var = (torch.cumsum(x * x, 0) - n * m * m).clamp(min=0.0) / (n - 1).clamp(min=1.0)
    se = torch.sqrt(var / n)
    z = torch.where((n >= 2) & (se > 0), m / se.clamp(min=1e-300), torch.zeros_like(m))
    return torch.nan_to_num(z, nan=0.0, posinf=0.0, neginf=0.0)


def expected_z_curve_from_fingerprint(blocks: int, sigma: float, kappa: float, fp: MaxwellFingerprint) -> torch.Tensor:
    return expected_z_curve(blocks, sigma, kappa, fp.lambda_())


def envelope_series_from_fingerprint(fp: MaxwellFingerprint, semantic_gain: float, rho_values, code_values) -> torch.Tensor:
    return MeaningGate(fp.lambda_(), semantic_gain).envelope_series(rho_values, code_values)


# ----------------------------------------------------------------------------------------------
# Sequential Z detector and its projection to a Z pulse
# ----------------------------------------------------------------------------------------------
class SequentialZ:
    """Welford running mean / variance of block means; `z = mean / stderr` once it is defined."""

    def __init__(self):
        self.count, self._mean, self._m2 = 0, 0.0, 0.0

    def __len__(self) -> int:
        return self.count

    def is_empty(self) -> bool:
        return self.count == 0

    def push(self, sample: float) -> Optional[float]:
        self.count += 1
        d = sample - self._mean
        self._mean += d / self.count
        self._m2 += d * (sample - self._mean)
        return self.z_stat()

    def extend(self, samples: Sequence[float]) -> Optional[float]:
        z = None
        for s in samples:
            z = self.push(float(s))
        return z

    def mean(self) -> float:
        return self._mean

    def variance(self) -> Optional[float]:
        return None if self.count < 2 else self._m2 / (self.count - 1.0)

    def standard_error(self) -> Optional[float]:
        v = self.variance()
        if v is None:
            return None
        se = math.sqrt(v / self.count)
        return se if math.isfinite(se) and se > 0 else None

    def z_stat(self) -> Optional[float]:
        se = self.standard_error()
        return None if se is None else self._mean / se


@dataclass
class MaxwellZPulse:
    blocks: int
    mean: float
    standard_error: float
    z_score: float
    band_energy: tuple
    z_bias: float

    def magnitude(self) -> float:
        return abs(self.z_score)

    def quality(self) -> float:
        """tanh(|z|) scaled by min(1, 1/stderr)."""
        snr = min(1.0 / self.standard_error, 1.0) if self.standard_error > 0 else 1.0
        return math.tanh(abs(self.z_score)) * snr

    def into_softlogic_feedback(self, psi_total: float, weighted_loss: float) -> dict:
        return {"psi_total": psi_total, "weighted_loss": weighted_loss, "band_energy": self.band_energy,
                "drift": self.mean, "z_signal": self.z_bias, "scale": None, "events": [], "attributions": []}


class MaxwellZProjector:
    """Turns a detector state into a pulse: `z_bias = sign(z) * leech.enrich(|z|) * bias_gain`, band
    energy `(max(mean,0), stderr, max(-mean,0))`; silent below `min_blocks` or `min_z`."""

    def __init__(self, rank: int, weight: float, bias_gain: float = 1.0, min_blocks: int = 2, min_z: float = 0.0):
        self.projector = LeechProjector(rank, weight)
        self.bias_gain, self.min_blocks, self.min_z = float(bias_gain), max(int(min_blocks), 1), max(float(min_z), 0.0)
        self._last: Optional[MaxwellZPulse] = None
        self.last_reason = "none"

    def project(self, tracker: SequentialZ) -> Optional[MaxwellZPulse]:
        if len(tracker) < self.min_blocks:
            self.last_reason = "min_blocks"
            return None
        se = tracker.standard_error()
        if se is None:
            self.last_reason = "undefined_stderr"
            return None
        mean = tracker.mean()
        z = mean / se
        if abs(z) < self.min_z:
            self.last_reason = "min_z"
            return None
        enriched = self.projector.enrich(abs(z))
        bias = math.copysign(enriched * self.bias_gain, z) if enriched > 1.2e-7 and abs(self.bias_gain) > 1.2e-7 else 0.0
        self._last = MaxwellZPulse(len(tracker), mean, se, z, (max(mean, 0.0), max(se, 0.0), max(-mean, 0.0)), bias)
        self.last_reason = "emitted"
        return self._last

    def last_pulse(self) -> Optional[MaxwellZPulse]:
        return self._last


# ----------------------------------------------------------------------------------------------
# RoPE table cache
# ----------------------------------------------------------------------------------------------
class RopeLRU:
    """Least-recently-used cache of `(cos, sin)` tables `cos[t] = cos(t * theta mod 2pi)`.

    Keys are `(theta, length, dtype, device)`, with `theta` matched to 1e-9.  A hit returns the very
    same tensors (no re-allocation), already on the requested device."""

    def __init__(self, capacity: int):
        self.capacity = max(int(capacity), 1)
        self._entries: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.hits = self.misses = 0

    @staticmethod
    def _key(theta: float, t: int, dtype, device) -> tuple:
        return (round(float(theta) / 1e-9), int(t), str(dtype), str(torch.device(device)))

    def get(self, theta: float, t: int, dtype=torch.float32, device="cpu") -> tuple:
        k = self._key(theta, t, dtype, device)
        if k in self._entries:
            self._entries.move_to_end(k)
            self.hits += 1
            return self._entries[k]
        self.misses += 1
        phase = torch.remainder(torch.arange(t, dtype=torch.float64, device=device) * float(theta), 2 * math.pi)
        entry = (torch.cos(phase).to(dtype), torch.sin(phase).to(dtype))
        self._entries[k] = entry
        if len(self._entries) > self.capacity:
            self._entries.popitem(last=False)
        return entry

    def __len__(self) -> int:
        return len(self._entries)
