"""Latency advisor and the Z-tiger gain tracker.

Parity: crates/julia-ffi-poc/src/lib.rs:6-66 (`rust_latency_score`, `ZTigerOptim`).  The reference
keeps these as the pure mirror of functions it can also evaluate through an embedded Julia
runtime; no Julia runtime exists in this build, so `latency_score(..., engine="julia")` raises.
"""
from __future__ import annotations

import math
from collections import deque
from typing import Sequence


def latency_score(tile: int, slack: int, engine: str = "native") -> float:
    """sqrt(tile) + slack / 2 — cheap ranking of (tile size, slack width) pairs."""
    if engine != "native":
        raise RuntimeError(f"latency advisor engine {engine!r} is not available; use 'native'")
    if tile < 0 or slack < 0:
        raise ValueError("tile and slack must be non-negative")
    return math.sqrt(float(tile)) + float(slack) / 2.0


class ZTigerOptim:
    """Gain in [1, 2) from a 32-step moving average of phase-weighted resonance magnitudes."""

    def __init__(self, curvature: float = -1.0):
        self._curvature = curvature if math.isfinite(curvature) and curvature < 0 else -1.0
        self._gain, self._history = 1.0, deque(maxlen=32)

    def curvature(self) -> float:
        return self._curvature

    def gain(self) -> float:
        return self._gain

    def update(self, lora_pid: float, resonance: Sequence[float]) -> float:
        n = len(resonance)
        mean = sum(abs(v) * (i + 1) / n for i, v in enumerate(resonance)) / n if n else 0.0
        self._history.append(mean)
        smooth = sum(self._history) / len(self._history)
        boost = max(abs(math.tanh(self._curvature)), 1e-3)
        self._gain = abs(math.tanh(smooth * boost / max(lora_pid, 1e-6))) + 1.0
        return self._gain


# ----------------------------------------------------------------------------------------------
# Temporal-spectral fusion of a lane window
# (crates/st-core/src/backend/temporal_fusion.rs:19-260, unison_heuristics.rs:207-215)
# ----------------------------------------------------------------------------------------------
from dataclasses import dataclass

import torch

MAX_HARMONICS = 8


@dataclass(frozen=True)
class LaneWindow:
    """Candidate lane counts `lower, lower+stride, ..., upper` around `target`."""
    target: int
    lower: int
    upper: int
    min_lane: int = 1
    max_lane: int = 1024
    slack: int = 0
    stride: int = 1

    def lanes(self) -> list:
        if self.upper <= self.lower:
            return [self.lower]
        return list(range(self.lower, self.upper + 1, max(self.stride, 1)))


@dataclass
class TemporalSpectralFusion:
    """Occupancy series over a lane window, the magnitudes of its first harmonics, and their outer
    product (`fusion[h, t] = spectral[h] * temporal[t]`).

    `temporal[t] = log1p(k / lane_t) + 0.5 log1p(rows / lanes) + 0.25 log1p(cols / lanes)`; the
    spectrum is the zero-padded power-of-two FFT's first half, `dominant_frequency` its arg-max bin
    over the FFT length, `tempo_hint` the dominant magnitude's share of the half-spectrum's sum."""
    temporal: torch.Tensor
    spectral: torch.Tensor
    fusion: torch.Tensor
    dominant_frequency: float
    tempo_hint: float
    spectral_energy: float

    @classmethod
    def analyse(cls, window: LaneWindow, rows: int, cols: int, k: int, lanes: int) -> "TemporalSpectralFusion":
        lane = torch.tensor(window.lanes(), dtype=torch.float32).clamp(min=1.0)
        lf = float(max(lanes, 1))
        temporal = torch.log1p(max(k, 1) / lane) + 0.5 * math.log1p(max(rows, 1) / lf) + 0.25 * math.log1p(max(cols, 1) / lf)
        n = max(1 << max(temporal.numel() - 1, 0).bit_length(), 2)
        mag = torch.nan_to_num(torch.fft.fft(temporal, n=n).abs()[: n // 2], nan=0.0, posinf=0.0, neginf=0.0)
        energy = max(float(mag.sum()), 1.1920929e-07)
        dom = int(mag.argmax())
        spectral = mag[: min(MAX_HARMONICS, mag.numel())].clone()
        return cls(temporal, spectral, spectral[:, None] * temporal[None, :], dom / n,
                   min(max(float(mag[dom]) / energy, 0.0), 1.0), energy)
