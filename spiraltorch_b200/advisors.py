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
