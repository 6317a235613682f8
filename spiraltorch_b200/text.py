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

    def describe_resonance(self, resonance) -> ResonanceNarrative:
        """Narrative of a differential resonance (its five channels' squared norms): which band dominates, its share,
        the total energy and the observed curvature -sqrt(homotopy energy).  crates/st-text/src/lib.rs:115-120, 656-760."""
        return resonance_narrative(resonance)

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

    def describe_frame(self, frame) -> ResonanceNarrative:
        return _frame_narrative(frame)

    def describe_atlas(self, atlas, chrono_summary=None, maintainer_status: Optional[str] = None) -> ResonanceNarrative:
        return _atlas_narrative(atlas, chrono_summary, maintainer_status)

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


# ---- frame / atlas narratives, realtime narrator, token semantics ------------------------------------------------
_BAND_LABELS = ("Above band accelerating curvature", "Here band weaving functor linearisation",
                "Beneath band anchoring recursive objective", "∞ projection tightening geodesics", "∞ hierarchy storing latent energy")
_EPS32 = 1.1920929e-07


def _sq_norm(t) -> float:
    data = t.torch() if hasattr(t, "torch") else t
    import torch
    return float((torch.as_tensor(data, dtype=torch.float32) ** 2).sum())


def resonance_narrative(resonance) -> ResonanceNarrative:
    """``resonance`` has the channels homotopy_flow, functor_linearisation, recursive_objective, infinity_projection,
    infinity_energy (tensors or anything array-like)."""
    e = [_sq_norm(getattr(resonance, n)) for n in ("homotopy_flow", "functor_linearisation", "recursive_objective", "infinity_projection",
                                                    "infinity_energy")]
    e = [v if math.isfinite(v) and v > 0.0 else 0.0 for v in e]
    total = sum(e)
    if total <= _EPS32:
        return ResonanceNarrative("Resonance geometry is quiescent; no meaningful curvature pulses detected.", ["all bands below activation threshold"])
    curvature = -math.sqrt(e[0]) if e[0] > 0.0 else -1.0
    lead = max(range(5), key=lambda i: (e[i], -i))                      # the first of equal bands leads
    pct = [v / total for v in e]
    summary = (f"{_BAND_LABELS[lead]} commanding {min(max(pct[lead], 0.0), 1.0) * 100.0:.1f}% of the field while total energy sits at "
               f"{total:.3f} with curvature {curvature:+.3f}.")
    highlights = [f"Above {pct[0] * 100:.1f}%", f"Here {pct[1] * 100:.1f}%", f"Beneath {pct[2] * 100:.1f}%", f"∞ proj {pct[3] * 100:.1f}%",
                  f"∞ tower {pct[4] * 100:.1f}%", f"curvature {curvature:+.3f}"]
    entropy = -sum(p * math.log(p) for p in pct if p > 0.0)
    if entropy > 0.0:
        highlights.append(f"band entropy {entropy:.2f}")
    ordered = sorted(pct, reverse=True)
    if ordered[0] - ordered[1] > 0.0:
        highlights.append(f"dominant contrast {(ordered[0] - ordered[1]) * 100:.1f}%")
    mean = sum(pct) / 5.0
    spread = math.sqrt(sum((p - mean) ** 2 for p in pct) / 5.0)
    if spread > 0.0:
        highlights.append(f"band spread σ {spread * 100:.1f}%")
    if entropy > 0.0:
        highlights.append(f"band evenness {entropy / math.log(5.0) * 100:.1f}%")
    active = sum(1 for p in pct if p > 0.05)
    if active:
        highlights.append(f"active bands {active}")
    return ResonanceNarrative(summary, highlights)


def describe_resonance(resonance) -> str:
    return TextResonator(-1.0, 0.6).describe_resonance(resonance).summary


def _frame_narrative(frame) -> ResonanceNarrative:
    """One temporal frame in words (crates/st-text/src/lib.rs:122-146)."""
    if frame.total_energy <= 1.1920929e-07:
        summary = (f"At t={frame.timestamp:.3f} the resonance settled; curvature drift {frame.curvature_drift:+.3f} "
                   "with negligible energy.")
    else:
        summary = (f"At t={frame.timestamp:.3f} the resonance carried {frame.total_energy:.3f} energy with curvature "
                   f"drift {frame.curvature_drift:+.3f}.")
    hl = [f"homotopy {frame.homotopy_ratio() * 100:.1f}%", f"functor {frame.functor_ratio() * 100:.1f}%",
          f"recursive {frame.recursive_ratio() * 100:.1f}%", f"projection {frame.projection_ratio() * 100:.1f}%",
          f"infinity {frame.infinity_ratio() * 100:.1f}%", f"energy decay {frame.energy_decay:+.3f}"]
    return ResonanceNarrative(summary, hl)


def _atlas_narrative(atlas, chrono_summary=None, maintainer_status: Optional[str] = None) -> ResonanceNarrative:
    """An atlas snapshot in words: span / energy / drift when a chrono summary is known, then loop support, collapse
    total, Z bias, every metric, the notes and the script hint as highlights (crates/st-text/src/lib.rs:475-537)."""
    if chrono_summary is not None:
        summary = (f"Atlas at t={atlas.timestamp:.3f} spans {chrono_summary.duration:.3f}s with energy "
                   f"{chrono_summary.mean_energy:.3f} and drift {chrono_summary.mean_drift:+.3f}.")
    else:
        summary = f"Atlas snapshot at t={atlas.timestamp:.3f}."
    if maintainer_status:
        summary += f" Maintainer {maintainer_status}."
    hl = []
    if atlas.loop_support > 0.0:
        hl.append(f"loop support {atlas.loop_support:.3f}")
    if atlas.collapse_total is not None:
        hl.append(f"collapse total {atlas.collapse_total:.3f}")
    if atlas.z_signal is not None:
        hl.append(f"z bias {atlas.z_signal:+.3f}")
    hl += [f"{name} {value:.3f}" for name, value in atlas.metrics.items()]
    hl += list(atlas.notes)
    if atlas.script_hint:
        hl.append(f"script {atlas.script_hint}")
    return ResonanceNarrative(summary, hl)


class RealtimeNarrator:
    """Timeline → audio samples at a fixed rate (crates/st-text/src/lib.rs:595-627)."""

    def __init__(self, curvature: float = -1.0, temperature: float = 0.6, sample_rate: int = 8000):
        self.inner, self.sample_rate = TextResonator(curvature, temperature), max(1, sample_rate)

    @classmethod
    def from_resonator(cls, resonator: TextResonator, sample_rate: int) -> "RealtimeNarrator":
        n = cls.__new__(cls)
        n.inner, n.sample_rate = resonator, max(1, sample_rate)
        return n

    def narrate_timeline(self, timeline: ChronoTimeline) -> list:
        return self.inner.synthesize_wave(timeline, self.sample_rate).samples


def describe_frame(frame) -> str:
    return TextResonator(-1.0, 0.6).describe_frame(frame).summary


def describe_timeline(timeline: ChronoTimeline) -> Optional[str]:
    n = TextResonator(-1.0, 0.6).describe_timeline(timeline)
    return None if n is None else n.summary


def describe_atlas(atlas) -> str:
    return TextResonator(-1.0, 0.6).describe_atlas(atlas).summary


def token_scale_stack(embeddings, scales, threshold: float, metric: str = "euclidean"):
    """Scale stack of a token sequence: tokens are samples along the sequence, the embedding dimension is the
    semantic feature axis (crates/st-text/src/semantics.rs:16-31).  Returns the same :class:`ScaleStack` the
    fractal module builds for vector-valued fields, so persistence, boundary dimension and coherence breaks apply."""
    import torch
    from .frac import ScaleStack
    e = embeddings.torch() if hasattr(embeddings, "torch") else torch.as_tensor(embeddings, dtype=torch.float32)
    if e.dim() != 2:
        raise ValueError(f"token_scale_stack needs a [tokens, dims] matrix, got shape {tuple(e.shape)}")
    if metric not in ("euclidean", "cosine"):
        raise ValueError(f"unknown semantic metric '{metric}'")
    return ScaleStack.from_semantic_field(e, list(scales), float(threshold), 1, metric)


def token_coherence_levels(embeddings, scales, threshold: float, metric: str = "euclidean", levels=(0.25, 0.5, 0.75)):
    """Per level, the smallest scale whose gate fraction reaches it, else ``None``
    (crates/st-text/src/semantics.rs:34-43)."""
    return token_scale_stack(embeddings, scales, threshold, metric).coherence_profile(list(levels))
