"""Bridge-driven studio: frames, causal annotations, overlay stitching, meta layer, sinks and Z-space projections."""
import json

import pytest

from spiraltorch_b200.language import MaxwellDesireBridge
from spiraltorch_b200.logic import SignalCaptureConfig, StudioError
from spiraltorch_b200.mellin import MellinLogGrid
from spiraltorch_b200.meta_narrative import MeaningSection, MeaningSheaf, MetaNarrativeLayer, NarrativeBeat
from spiraltorch_b200.qr_studio import (ConceptWindow, QuantumRealityStudio, SemanticTagger, StudioSink, StudioTemporalEngine, ZSpaceSink,
                                        compose_overlay, snapshot_of)
from spiraltorch_b200.theory import MaxwellZPulse
import torch


def pulse(z, bias=0.18):
    return MaxwellZPulse(16, 0.12, 0.05, z, (0.4, 0.3, 0.2), bias)


def bridge():
    b = MaxwellDesireBridge()
    b.register_channel("alpha", [(3, 0.7), (5, 0.3)], tags=["glimmer", "tide"], gain=1.0)
    b.register_channel("beta", [(5, 1.0)], tags=["ember"])
    b.register_channel("mute", [(9, 1.0)])
    return b


def test_frames_carry_concept_narrative_causality_and_overlay():
    b = bridge()
    studio = QuantumRealityStudio(SignalCaptureConfig(100.0, history_limit=3), b)
    assert SemanticTagger.from_bridge(b).fallback_for("alpha") == ["glimmer", "tide"]
    f0 = studio.ingest(b, "alpha", pulse(2.0), timestamp=1.0)
    assert f0.causal.is_root() and f0.causal.depth == 0 and f0.narrative.dominant_tag() in ("glimmer", "tide")
    win = studio.emit_concept_window(f0)
    assert [t for t, _ in win.weights] == [3, 5] and win.magnitude == 2.0 and win.weights[0][1] == pytest.approx((0.7 + 1e-4) * 2.0)
    glyphs = [g.glyph for g in f0.overlay.glyphs]
    assert glyphs[0] == f0.narrative.dominant_tag() and {"glimmer", "tide", "ordinal:0", "time:1.000", "magnitude:2.000", "depth:0"} <= set(glyphs)
    assert "sheaf|curvature:+2.000" in glyphs and "sheaf|above:0.400" in glyphs and "sheaf|depth:0" in glyphs and any(g.startswith("sheaf|token#3:") for g in glyphs)
    assert f0.overlay.glyphs[0].intensity == pytest.approx(f0.narrative.quantum_emphasis()) and f0.z_space.signature[3] == 2.0
    f1 = studio.ingest(b, "beta", pulse(-1.0), timestamp=2.0)        # shares token 5 with the alpha event
    assert f1.causal.parents == [0] and f1.causal.parent_channels == ["alpha"] and f1.causal.depth == 1 and "after:alpha" in [g.glyph for g in f1.overlay.glyphs]
    f2 = studio.ingest(b, "alpha", pulse(0.5), timestamp=3.0)
    assert f2.causal.parents == [0, 1] and f2.causal.parent_channels == ["alpha#0", "beta"] and f2.causal.depth == 2
    f3 = studio.ingest(b, "mute", pulse(1.5), timestamp=4.0)         # a channel without tags: the channel name is the glyph
    assert f3.narrative is None and f3.overlay.glyphs[0].glyph == "mute" and f3.overlay.glyphs[0].intensity == 1.5 and f3.narrative_summary is None
    assert len(studio.frames) == 3 and len(studio.records()) == 3 and len(studio.causal_snapshot()) == 4
    sheaf = studio.meaning_sheaf("alpha")
    assert sheaf.signature[0] == pytest.approx(2.0 * (2 / 3) + 0.5 / 3)      # the first event left a weight of (1 + depth 0) * |z| = 2
    assert studio.meaning_sheaf("nope") is None
    assert studio.infer_concept_window(b, f0.record).weights == win.weights
    with pytest.raises(StudioError):
        QuantumRealityStudio(SignalCaptureConfig(100.0, channels=["alpha"]), b).ingest(b, "beta", pulse(1.0))
    board = studio.export_storyboard()
    assert board["channels"] == ["alpha", "beta", "mute"] and board["frames"][0]["causal"]["parents"] == [0] and board["frames"][0]["ordinal"] == 0
    assert list(studio.export_storyboard_grouped()["channels"]) == ["beta", "alpha", "mute"]
    lines = studio.export_storyboard_ndjson().splitlines()
    assert len(lines) == 3 and json.loads(lines[2])["channel"] == "mute"


def test_overlay_composition_rules():
    b = bridge()
    studio = QuantumRealityStudio(SignalCaptureConfig(10.0), b)
    rec = studio.record_pulse("alpha", pulse(3.0), 0.0)
    assert compose_overlay(rec, None, ["fallback", "x"]).glyphs[0].glyph == "fallback" and compose_overlay(rec, None, None).glyphs[0].glyph == "alpha"
    from spiraltorch_b200.language import NarrativeHint
    quiet = NarrativeHint("alpha", ["soft"], 0.5).with_quantum_state(0.0, 0.0, 1.0, 0.0)
    assert compose_overlay(rec, quiet, None).glyphs[0].intensity == 3.0      # no emphasis: max(narrative intensity, |z|)
    loud = NarrativeHint("alpha", ["loud"], 0.5).with_quantum_state(4.0, 0.0, 0.5, 0.5)
    assert compose_overlay(rec, loud, None).glyphs[0].intensity == pytest.approx(1.0)
    eng = StudioTemporalEngine()
    a = eng.observe(rec, ConceptWindow("alpha", 0.0, [(1, 0.5)], 3.0))
    assert StudioTemporalEngine.temporal_tags(a) == ["ordinal:0", "time:0.000", "magnitude:3.000", "depth:0"]


def test_meta_layer_overrides_the_narrative():
    b = bridge()
    layer = MetaNarrativeLayer()
    layer.engine_mut().insert_event("open", NarrativeBeat("alpha", "root", ["prologue"]).with_intensity_scale(2.0))
    layer.bridge_mut().attach("open", MeaningSheaf().with_section(MeaningSection.for_open("root", ["lumen"], 0.5)))
    studio = QuantumRealityStudio(SignalCaptureConfig(10.0), b).with_meta_layer(layer)
    f = studio.ingest(b, "alpha", pulse(1.5), 0.0)
    assert f.meta.event_id == "open" and f.meta.tags == ["lumen", "prologue"] and f.meta.intensity == pytest.approx(3.0 * 1.5)
    assert f.narrative.tags == ["lumen", "prologue"] and f.narrative.intensity == pytest.approx(4.5) and f.z_space.signature == f.meta.signature()
    assert f.overlay.glyphs[0].intensity == pytest.approx(4.5)
    g = studio.ingest(b, "alpha", pulse(1.5), 1.0)                   # the beat is spent: back to the bridge's narrative
    assert g.meta is None and set(g.narrative.tags) == {"glimmer", "tide"}
    studio.clear_meta_layer()
    assert studio.meta_layer is None


def test_sinks_and_zspace_projection():
    b = bridge()
    seen = []

    class Collect(StudioSink):
        name = "collect"

        def send(self, frame):
            seen.append(frame.record.channel)

    class Broken(StudioSink):
        name = "broken"

        def send(self, frame):
            raise IOError("pipe closed")
    zs = ZSpaceSink.vertical_line("zspace", -1.0, 0.5, 1.2, [-0.5, 0.0, 0.5])
    studio = QuantumRealityStudio(SignalCaptureConfig(10.0), b).with_sink(Collect()).with_sink(zs)
    assert studio.sink_count() == 2
    studio.ingest(b, "alpha", pulse(2.0, 0.1), 0.0)
    assert zs.take_projections() == []                               # one sample is not a lattice yet
    studio.ingest(b, "alpha", pulse(-1.0, -0.2), 1.0)
    studio.ingest(b, "beta", pulse(0.5), 2.0)
    studio.ingest(b, "alpha", pulse(3.0, 0.3), 3.0)
    projs = zs.take_projections()
    assert [(p.channel, p.lattice_len) for p in projs] == [("alpha", 2), ("alpha", 3)] and zs.take_projections() == []
    grid = MellinLogGrid(-1.0, 0.5, torch.tensor([2.0 + 0.1j, 1.0 - 0.2j, 3.0 + 0.3j], dtype=torch.complex128))
    s, z, v = projs[1].evaluations[1]
    assert s == 1.2 + 0j and z == pytest.approx(complex(torch.exp(torch.tensor(0.6)))) and v == pytest.approx(grid.evaluate(1.2 + 0j))
    assert len(projs[1].signature_components()) == 18 and projs[1].to_zspace().signature[0] == 1.2
    assert seen == ["alpha", "alpha", "beta", "alpha"]
    studio.flush_sinks()
    studio.register_sink(Broken())
    with pytest.raises(StudioError) as e:
        studio.ingest(b, "beta", pulse(0.5), 4.0)
    assert "sink `broken` failed: pipe closed" in str(e.value) and seen[-1] == "beta"          # the healthy sinks still got the frame
    studio.register_sink(Broken())
    with pytest.raises(StudioError) as e:
        studio.ingest(b, "beta", pulse(0.5), 5.0)
    assert str(e.value).startswith("multiple sinks failed")
