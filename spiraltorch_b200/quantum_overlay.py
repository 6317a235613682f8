"""Quantum overlay of the QR studio: Maxwell Z pulses become a resonance (a spectrum with shell weights and a coupling
hint), the resonance is spread over a register of qubits on a hyperbolic chart with a Leech-lattice packing term, and a
measurement of that register gives the active qubits, policy logits and the packing pressure a policy head consumes.

Reference parity: crates/st-qr-studio/src/quantum_overlay.rs (`QuantumOverlayConfig` :8-60, `ZResonance` :69-124,
`ZOverlayCircuit` :127-199, `normalize_shells` :201-225, `QuantumMeasurement` :228-250).  The register weights are
computed as one tensor expression, and :meth:`ZOverlayCircuit.synthesize_batch` builds the registers of many
resonances at once (one row each).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Sequence

import torch

from .theory import MaxwellZPulse


class QuantumOverlayConfig:
    def __init__(self, curvature: float = -1.0, qubits: int = 24):
        self.curvature = float(curvature) if math.isfinite(curvature) else -1.0
        self.qubits = max(int(qubits), 1)
        self.packing_bias = 0.35
        self.leech_shells = 24

    def with_packing_bias(self, packing_bias: float) -> "QuantumOverlayConfig":
        if math.isfinite(packing_bias):
            self.packing_bias = min(max(float(packing_bias), 0.0), 1.0)
        return self

    def with_leech_shells(self, shells: int) -> "QuantumOverlayConfig":
        self.leech_shells = max(int(shells), 1)
        return self


@dataclass
class ZResonance:
    spectrum: List[float] = field(default_factory=list)
    eta_hint: float = 0.0
    shell_weights: List[float] = field(default_factory=list)

    @classmethod
    def from_pulses(cls, pulses: Sequence[MaxwellZPulse]) -> "ZResonance":
        """Spectrum = the pulses' means, shell weight = a pulse's total band energy, hint = mean |z_bias| capped at 2."""
        if not pulses:
            return cls.from_spectrum([], 0.0)
        return cls([float(p.mean) for p in pulses], min(sum(abs(float(p.z_bias)) for p in pulses) / len(pulses), 2.0),
                   [max(float(sum(p.band_energy)), 0.0) for p in pulses])

    @classmethod
    def from_spectrum(cls, spectrum: Sequence[float], eta_hint: float) -> "ZResonance":
        spec = [float(v) for v in spectrum]
        return cls(spec, max(float(eta_hint), 0.0), [abs(v) * (i + 1.0) for i, v in enumerate(spec)])


def normalize_shells(resonance: ZResonance, shells: int) -> torch.Tensor:
    """Shell weights cycled up to ``shells`` entries and scaled to unit L1 norm; 1 / (k + 1) when the resonance has none."""
    shells = max(shells, 1)
    base = resonance.shell_weights
    if not base:
        return 1.0 / torch.arange(1, shells + 1, dtype=torch.float64)
    w = torch.tensor(base, dtype=torch.float64)
    if w.numel() < shells:
        extra = torch.tensor([abs(base[i % len(base)]) for i in range(shells - w.numel())], dtype=torch.float64)
        w = torch.cat([w, extra])
    norm = float(w.abs().sum())
    return torch.ones(shells, dtype=torch.float64) if norm <= 0.0 else w / norm


@dataclass
class QuantumMeasurement:
    active_qubits: List[int]
    eta_bar: float
    policy_logits: List[float]
    packing_pressure: float


class ZOverlayCircuit:
    def __init__(self, config: QuantumOverlayConfig, weights: torch.Tensor, eta_bar: float, packing_pressure: float):
        self.config, self.weights, self.eta_bar, self.packing_pressure = config, weights, eta_bar, packing_pressure

    @staticmethod
    def _register(config: QuantumOverlayConfig, shell_per_qubit: torch.Tensor) -> torch.Tensor:
        """weights[..., q] = tanh(|shell_q| |kappa|) (1 - b) + |sin(2 pi q / L) b| b, shell_q being the shell qubit q sits on."""
        q = torch.arange(config.qubits, dtype=torch.float64)
        hyper = torch.tanh(shell_per_qubit.abs() * max(abs(config.curvature), 1e-6))
        packing = (torch.sin(q / config.leech_shells * 2.0 * math.pi) * config.packing_bias).abs()
        return hyper * (1.0 - config.packing_bias) + packing * config.packing_bias

    @staticmethod
    def _shell_per_qubit(config: QuantumOverlayConfig, shells: torch.Tensor) -> torch.Tensor:
        return shells[torch.arange(config.qubits) % shells.numel()]

    @classmethod
    def synthesize(cls, config: QuantumOverlayConfig, resonance: ZResonance) -> "ZOverlayCircuit":
        shells = normalize_shells(resonance, config.leech_shells)
        pressure = float(shells.sum() / max(shells.numel(), 1))
        return cls(config, cls._register(config, cls._shell_per_qubit(config, shells)), abs(math.tanh(resonance.eta_hint + pressure)), pressure)

    from_config = synthesize

    @classmethod
    def synthesize_batch(cls, config: QuantumOverlayConfig, resonances: Sequence[ZResonance]) -> torch.Tensor:
        """Register weights of many resonances, one row each ([len(resonances), qubits])."""
        if not resonances:
            return torch.zeros(0, config.qubits, dtype=torch.float64)
        per_qubit = torch.stack([cls._shell_per_qubit(config, normalize_shells(r, config.leech_shells)) for r in resonances])
        return cls._register(config, per_qubit)

    def measure(self, threshold: float) -> QuantumMeasurement:
        """Qubits in decreasing weight; those at or above the threshold are active (the strongest one always is)."""
        thr = threshold if math.isfinite(threshold) else 0.0
        order = torch.argsort(self.weights, descending=True, stable=True)
        sorted_w = self.weights[order]
        active = [int(i) for i, w in zip(order.tolist(), sorted_w.tolist()) if w >= thr]
        if not active and order.numel():
            active = [int(order[0])]
        return QuantumMeasurement(active, float(self.eta_bar), [float(w) for w in sorted_w.tolist()], float(self.packing_pressure))
