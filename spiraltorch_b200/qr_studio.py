"""The studio driven by the Maxwell-desire bridge: every pulse captured on a channel becomes a frame that carries the
bridge's concept window and narrative hint (or the meta-narrative layer's released beat), a causal annotation (the
previous event of the same channel and of every shared concept token are its parents), an overlay of glyphs stitched
from narrative, temporal and sheaf tags, and a Z-space signature.  Frames go to sinks; a Z-space sink keeps one
log-lattice of pulse magnitudes per channel and projects it through the Mellin transform.

Parity: crates/st-qr-studio/src/lib.rs — `StudioConceptHint` / `ConceptWindow` (:133-186), `StudioFrame` /
`MetaNarrative` (:331-367), `SemanticTagger::from_bridge` (:412-430), `OverlayComposer::compose` (:433-458),
`StudioSink` and the outlet (:461-475, :760-828), `ZSpaceSink` (:553-756), `QuantumRealityStudio::ingest` (:911-980),
`infer_concept_window` (:1005), `stitch_narrative_tags` (:1017); crates/st-qr-studio/src/meta.rs — the studio's own
causal annotation engine (:9-70, :167-256) and running sheaf per channel (:72-165).  The capture primitives
(`SignalCaptureConfig`, `PulseSnapshot`, `RecordedPulse`, `OverlayFrame`) are the ones in `logic.py`.
"""
from __future__ import annotations

import json
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Deque, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .language import ConceptHint, MaxwellDesireBridge, NarrativeHint, NarrativeSummary
from .logic import OverlayFrame, OverlayGlyph, PulseSnapshot, RecordedPulse, SignalCaptureConfig, SignalCaptureSession, StudioError
from .mellin import MellinLogGrid
from .meta_narrative import MetaNarrativeLayer, ResolvedNarrative, ZSpace
from .theory import MaxwellZPulse

EPS = 1.1920929e-07


def snapshot_of(pulse: MaxwellZPulse) -> PulseSnapshot:
    return PulseSnapshot(pulse.blocks, pulse.mean, pulse.standard_error, pulse.z_score, tuple(pulse.band_energy), pulse.z_bias)


def pulse_of(snapshot: PulseSnapshot) -> MaxwellZPulse:
    return MaxwellZPulse(snapshot.blocks, snapshot.mean, snapshot.standard_error, snapshot.z_score, tuple(snapshot.band_energy), snapshot.z_bias)


def weighted_window(hint: ConceptHint) -> List[Tuple[int, float]]:
    """``(token, weight)`` pairs with a positive weight, from either form of a concept hint."""
    pairs = list(enumerate(hint.distribution)) if hint.distribution is not None else list(hint.window)
    return [(int(t), float(w)) for t, w in pairs if w > EPS]


@dataclass
class ConceptWindow:
    channel: str
    timestamp: float
    weights: List[Tuple[int, float]]
    magnitude: float

    @classmethod
    def from_hint(cls, record: RecordedPulse, hint: ConceptHint) -> Optional["ConceptWindow"]:
        weights = sorted(weighted_window(hint), key=lambda w: w[0])
        return cls(record.channel, record.timestamp, weights, record.pulse.magnitude()) if weights else None


@dataclass
class TemporalCausalAnnotation:
    event_id: int
    ordinal: int
    timestamp: float
    channel: str
    magnitude: float
    depth: int
    parents: List[int]
    parent_channels: List[str]

    def is_root(self) -> bool:
        return not self.parents


class StudioTemporalEngine:
    """Append-only causal record of the captured pulses."""

    def __init__(self):
        self.events: List[TemporalCausalAnnotation] = []
        self._by_channel: Dict[str, int] = {}
        self._by_token: Dict[int, int] = {}

    def observe(self, record: RecordedPulse, concept: Optional[ConceptWindow]) -> TemporalCausalAnnotation:
        tokens = [t for t, _ in concept.weights] if concept else []
        parents = sorted({p for p in [self._by_channel.get(record.channel)] + [self._by_token.get(t) for t in tokens] if p is not None})
        depth = (max(self.events[p].depth for p in parents) + 1) if parents else 0
        eid = len(self.events)
        names = [self.events[p].channel if self.events[p].channel != record.channel else f"{record.channel}#{p}" for p in parents]
        ann = TemporalCausalAnnotation(eid, eid, float(record.timestamp), record.channel, record.pulse.magnitude(), depth, parents, names)
        self.events.append(ann)
        self._by_channel[record.channel] = eid
        for t in tokens:
            self._by_token[t] = eid
        return ann

    def snapshot(self) -> List[TemporalCausalAnnotation]:
        return list(self.events)

    @staticmethod
    def temporal_tags(a: TemporalCausalAnnotation) -> List[str]:
        return [f"ordinal:{a.ordinal}", f"time:{a.timestamp:.3f}", f"magnitude:{a.magnitude:.3f}", f"depth:{a.depth}"] + \
               [f"after:{c}" for c in a.parent_channels]


class _SheafSection:
    def __init__(self):
        self.total_weight, self.tokens, self.signature = 0.0, {}, []

    def integrate(self, record: RecordedPulse, concept: Optional[ConceptWindow], depth: int) -> None:
        p = record.pulse
        sig = [p.z_score, float(p.band_energy[0]), float(p.band_energy[1]), float(p.band_energy[2]), float(p.z_bias), p.mean]
        if not self.signature:
            self.signature = sig
        else:
            f = 1.0 / (self.total_weight + 1.0)
            self.signature = [d * (1.0 - f) + s * f for d, s in zip(self.signature, sig)]
        gain = 1.0 + depth
        if concept is not None:
            gain *= max(concept.magnitude, 1e-3)
            for token, weight in concept.weights:
                self.tokens[token] = self.tokens.get(token, 0.0) + weight * gain
        self.total_weight += gain

    def semantic_tags(self, annotation: TemporalCausalAnnotation) -> List[str]:
        tags = []
        if self.signature:
            tags.append(f"sheaf|curvature:{self.signature[0]:+.3f}")
            for name, v in zip(("above", "here", "beneath"), self.signature[1:4]):
                tags.append(f"sheaf|{name}:{v:.3f}")
        total = max(self.total_weight, 1e-6)
        for token, weight in sorted(self.tokens.items(), key=lambda kv: -kv[1])[:3]:
            tags.append(f"sheaf|token#{token}:{min(max(weight / total, 0.0), 1.0):.2f}")
        tags.append(f"sheaf|depth:{annotation.depth}")
        return tags


class StudioToposBridge:
    """A running mean of the pulse signature and accumulated concept-token weights per channel."""

    def __init__(self):
        self.sections: Dict[str, _SheafSection] = {}

    def update(self, record: RecordedPulse, concept: Optional[ConceptWindow], annotation: TemporalCausalAnnotation) -> List[str]:
        sec = self.sections.setdefault(record.channel, _SheafSection())
        sec.integrate(record, concept, annotation.depth)
        return sec.semantic_tags(annotation)

    def meaning_sheaf(self, channel: str) -> Optional[ZSpace]:
        sec = self.sections.get(channel)
        return None if sec is None else ZSpace(list(sec.signature))


@dataclass
class MetaNarrative:
    event_id: str
    channel: str
    tags: List[str]
    intensity: float
    z_space: ZSpace

    @classmethod
    def from_resolved(cls, r: ResolvedNarrative) -> "MetaNarrative":
        return cls(r.event_id, r.channel, list(r.tags), r.intensity, ZSpace(list(r.z_space.signature)))

    def signature(self) -> List[float]:
        return self.z_space.signature


@dataclass
class StudioFrame:
    record: RecordedPulse
    concept: Optional[ConceptHint]
    narrative: Optional[NarrativeHint]
    narrative_summary: Optional[NarrativeSummary]
    causal: TemporalCausalAnnotation
    overlay: OverlayFrame
    z_space: ZSpace
    meta: Optional[MetaNarrative] = None


class SemanticTagger:
    def __init__(self, fallback_tags: Dict[str, List[str]]):
        self.fallback_tags = fallback_tags

    @classmethod
    def from_bridge(cls, bridge: MaxwellDesireBridge) -> "SemanticTagger":
        return cls({c: list(bridge.narrative_tags(c)) for c in bridge.channel_names() if bridge.narrative_tags(c) is not None})

    def fallback_for(self, channel: str) -> Optional[List[str]]:
        return self.fallback_tags.get(channel)


def compose_overlay(record: RecordedPulse, narrative: Optional[NarrativeHint], fallback: Optional[Sequence[str]]) -> OverlayFrame:
    """The first glyph: the narrative's dominant tag, else the channel's first fallback tag, else the channel name; its
    intensity is the narrative's quantum emphasis when it has one, else ``max(narrative intensity, |z|)``, else ``|z|``."""
    glyph = (narrative.dominant_tag() if narrative is not None else None) or (fallback[0] if fallback else None) or record.channel
    if narrative is None:
        intensity = record.pulse.magnitude()
    else:
        emph = narrative.quantum_emphasis()
        intensity = emph if emph > EPS else max(narrative.intensity, record.pulse.magnitude())
    return OverlayFrame.from_pairs(record.channel, record.timestamp, [(glyph, intensity)])


class StudioSink:
    name = "sink"

    def send(self, frame: StudioFrame) -> None:
        raise NotImplementedError

    def flush(self) -> None:
        return None


@dataclass
class ZSpaceProjection:
    channel: str
    lattice_len: int
    evaluations: List[Tuple[complex, complex, complex]]       # (s, z = e^{s h}, value)

    def signature_components(self) -> List[float]:
        out = []
        for s, z, v in self.evaluations:
            out += [s.real, s.imag, z.real, z.imag, v.real, v.imag]
        return out

    def to_zspace(self) -> ZSpace:
        return ZSpace(self.signature_components())


class ZSpaceSink(StudioSink):
    """Appends each frame's pulse magnitude (real) and Z bias (imaginary) to its channel's log lattice and, once the lattice
    has two samples, records the Mellin transform of the lattice at the configured points."""

    def __init__(self, name: str, log_start: float, log_step: float, s_values: Sequence[complex]):
        self.name, self.log_start, self.log_step = name, float(log_start), float(log_step)
        self.s_values = [complex(s) for s in s_values]
        self.samples: Dict[str, List[complex]] = {}
        self.projections: List[ZSpaceProjection] = []

    @classmethod
    def vertical_line(cls, name: str, log_start: float, log_step: float, sigma: float, tau_samples: Sequence[float]) -> "ZSpaceSink":
        return cls(name, log_start, log_step, [complex(sigma, t) for t in tau_samples])

    def send(self, frame: StudioFrame) -> None:
        series = self.samples.setdefault(frame.record.channel, [])
        series.append(complex(frame.record.pulse.magnitude(), frame.record.pulse.z_bias))
        if len(series) < 2 or not self.s_values:
            return
        grid = MellinLogGrid(self.log_start, self.log_step, torch.tensor(series, dtype=torch.complex128))
        plan = grid.plan_many(self.s_values)
        values = grid.evaluate_plan(plan)
        self.projections.append(ZSpaceProjection(frame.record.channel, len(series),
                                                 [(s, complex(z), complex(v)) for s, z, v in zip(self.s_values, plan.z_points, values)]))

    def take_projections(self) -> List[ZSpaceProjection]:
        out, self.projections = self.projections, []
        return out

    def take_logic_signatures(self) -> List[Tuple[str, ZSpace]]:
        return [(p.channel, p.to_zspace()) for p in self.take_projections()]


class QuantumRealityStudio:
    def __init__(self, config: SignalCaptureConfig, bridge: MaxwellDesireBridge):
        self.capture = SignalCaptureSession(config)
        self.tagger = SemanticTagger.from_bridge(bridge)
        self.sinks: List[StudioSink] = []
        self.frames: Deque[StudioFrame] = deque(maxlen=config.history_limit)
        self.meta_layer: Optional[MetaNarrativeLayer] = None
        self.temporal, self.topos = StudioTemporalEngine(), StudioToposBridge()

    def with_sink(self, sink: StudioSink) -> "QuantumRealityStudio":
        self.sinks.append(sink)
        return self

    register_sink = with_sink

    def with_meta_layer(self, layer: MetaNarrativeLayer) -> "QuantumRealityStudio":
        self.meta_layer = layer
        return self

    def set_meta_layer(self, layer: MetaNarrativeLayer) -> None:
        self.meta_layer = layer

    def clear_meta_layer(self) -> None:
        self.meta_layer = None

    def sink_count(self) -> int:
        return len(self.sinks)

    def _each_sink(self, call) -> None:
        failures = []
        for sink in self.sinks:
            try:
                call(sink)
            except Exception as exc:                                   # noqa: BLE001 - every sink gets the frame; failures are reported together
                failures.append(f"sink `{getattr(sink, 'name', type(sink).__name__)}` failed: {exc}")
        if len(failures) == 1:
            raise StudioError(failures[0])
        if failures:
            raise StudioError("multiple sinks failed: " + "; ".join(failures))

    def flush_sinks(self) -> None:
        self._each_sink(lambda s: s.flush())

    def record_pulse(self, channel: str, pulse: MaxwellZPulse, timestamp: Optional[float] = None) -> RecordedPulse:
        return self.capture.ingest(channel, snapshot_of(pulse), timestamp)

    def stitch_narrative_tags(self, overlay: OverlayFrame, tags: Iterable[str]) -> OverlayFrame:
        base = max(overlay.glyphs[0].intensity if overlay.glyphs else 1.0, 1e-6)
        overlay.extend_tags(tags, base)
        return overlay

    def ingest(self, bridge: MaxwellDesireBridge, channel: str, pulse: MaxwellZPulse, timestamp: Optional[float] = None) -> StudioFrame:
        meta = self.meta_layer.next_with_pulse(channel, pulse) if self.meta_layer is not None else None
        emission = bridge.emit(channel, pulse)
        concept, narrative = emission if emission is not None else (None, None)
        z_space, meta_details = ZSpace.from_pulse(pulse), None
        if meta is not None:
            meta_details = MetaNarrative.from_resolved(meta)
            z_space = meta_details.z_space
            narrative = NarrativeHint(meta_details.channel, meta_details.tags, meta_details.intensity)
        record = self.record_pulse(channel, pulse, timestamp)
        window = ConceptWindow.from_hint(record, concept) if concept is not None else None
        annotation = self.temporal.observe(record, window)
        fallback = self.tagger.fallback_for(channel)
        overlay = compose_overlay(record, narrative, fallback)
        if narrative is not None:
            overlay = self.stitch_narrative_tags(overlay, narrative.tags)
        elif fallback:
            overlay = self.stitch_narrative_tags(overlay, fallback)
        overlay = self.stitch_narrative_tags(overlay, StudioTemporalEngine.temporal_tags(annotation))
        overlay = self.stitch_narrative_tags(overlay, self.topos.update(record, window, annotation))
        frame = StudioFrame(record, concept, narrative, narrative.summary() if narrative is not None else None, annotation, overlay, z_space, meta_details)
        self._each_sink(lambda s: s.send(frame))
        self.frames.append(frame)
        return frame

    def records(self) -> List[RecordedPulse]:
        return self.capture.records()

    def causal_snapshot(self) -> List[TemporalCausalAnnotation]:
        return self.temporal.snapshot()

    def meaning_sheaf(self, channel: str) -> Optional[ZSpace]:
        return self.topos.meaning_sheaf(channel)

    def emit_concept_window(self, frame: StudioFrame) -> Optional[ConceptWindow]:
        return ConceptWindow.from_hint(frame.record, frame.concept) if frame.concept is not None else None

    def infer_concept_window(self, bridge: MaxwellDesireBridge, record: RecordedPulse) -> Optional[ConceptWindow]:
        hint = bridge.hint_for(record.channel, pulse_of(record.pulse))
        return None if hint is None else ConceptWindow.from_hint(record, hint)

    # ---- storyboard --------------------------------------------------------------------------------------------------------
    def export_storyboard(self) -> dict:
        frames = []
        for ordinal, f in enumerate(self.frames):
            frames.append({
                "ordinal": ordinal, "channel": f.record.channel, "timestamp": f.record.timestamp, "z_score": f.record.pulse.z_score,
                "band_energy": list(f.record.pulse.band_energy), "z_bias": f.record.pulse.z_bias,
                "glyphs": [asdict(g) for g in f.overlay.glyphs],
                "narrative": None if f.narrative_summary is None else {"dominant_tag": f.narrative_summary.dominant_tag,
                                                                      "tags": list(f.narrative_summary.tags), "intensity": f.narrative_summary.intensity},
                "concept": None if f.concept is None else weighted_window(f.concept),
                "causal": {"depth": f.causal.depth, "parents": list(f.causal.parents), "parent_channels": list(f.causal.parent_channels)},
                "meta": None if f.meta is None else {"event_id": f.meta.event_id, "tags": list(f.meta.tags), "intensity": f.meta.intensity},
                "z_space": list(f.z_space.signature)})
        return {"frames": frames, "channels": sorted({fr["channel"] for fr in frames})}

    def export_storyboard_grouped(self) -> dict:
        grouped: Dict[str, list] = {}
        for fr in self.export_storyboard()["frames"]:
            grouped.setdefault(fr["channel"], []).append(fr)
        return {"channels": grouped}

    def export_storyboard_ndjson(self) -> str:
        return "\n".join(json.dumps(fr, sort_keys=True) for fr in self.export_storyboard()["frames"])
