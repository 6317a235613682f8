"""Turns training telemetry into short narrative text and an audio-like wave.

Restated from crates/st-text/src/lib.rs:37-200 (``TextResonator``: describe a resonance / chrono
summary in words — energy level, drift direction, stability — and synthesise a wave whose amplitude
follows the energy and whose frequency follows the drift).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from .telemetry import ChronoSummary, ChronoTimeline


@dataclass
class ResonanceNarrative:
    summary: str
    highlights: list


@dataclass
class WaveSynthesis:
    samples: list
    sample_rate: int
    base_frequency: float


class TextResonator:
    def __init__(self, curvature: float = -1.0, temperature: float = 0.5):
        if not curvature < 0 or not temperature > 0:
            raise ValueError("curvature must be negative and temperature positive")
        self.curvature, self.temperature = curvature, temperature

    def describe_summary(self, s: ChronoSummary) -> ResonanceNarrative:
        level = "quiet" if s.mean_energy < 0.1 else "steady" if s.mean_energy < 1.0 else "energetic"
        drift = "flat" if abs(s.mean_drift) < 1e-3 else "rising" if s.mean_drift > 0 else "falling"
        stable = s.drift_std <= max(1e-3, 0.5 * s.mean_abs_drift + 1e-3) and s.energy_std <= 0.25 * max(s.mean_energy, 1e-6)
        hl = [f"{s.frames} frames over {s.duration:.2f}s", f"energy {s.min_energy:.3f}–{s.max_energy:.3f}",
              f"mean decay {s.mean_decay:+.3f}/s"]
        if not stable:
            hl.append("unstable: drift or energy varies strongly inside the window")
        text = (f"The run is {level}: mean energy {s.mean_energy:.3f} with curvature {drift} "
                f"({s.mean_drift:+.4f}/s); it looks {'stable' if stable else 'unsettled'}.")
        return ResonanceNarrative(text, hl)

    def describe_timeline(self, timeline: ChronoTimeline, window: int = 32) -> Optional[ResonanceNarrative]:
        s = timeline.summarise(window)
        return None if s is None else self.describe_summary(s)

    def synthesize_wave(self, timeline: ChronoTimeline, sample_rate: int = 8000, seconds_per_frame: float = 0.05,
                        base_frequency: float = 220.0) -> WaveSynthesis:
        samples, phase = [], 0.0
        per = max(1, int(sample_rate * seconds_per_frame))
        for f in timeline.frames():
            amp = math.tanh(f.total_energy * self.temperature)
            freq = base_frequency * 2.0 ** max(-2.0, min(2.0, f.curvature_drift * math.sqrt(-self.curvature)))
            for _ in range(per):
                phase += 2 * math.pi * freq / sample_rate
                samples.append(amp * math.sin(phase))
        return WaveSynthesis(samples, sample_rate, base_frequency)
