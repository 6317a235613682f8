"""Text side of the telemetry: narratives for frames, timelines and atlas snapshots, the realtime narrator, and the
token scale stack (behaviour of crates/st-text/src/lib.rs and semantics.rs)."""
import pytest
import torch

from spiraltorch_b200 import text
from spiraltorch_b200.telemetry import AtlasFrame, ChronoFrame, ChronoTimeline


def _frame(step, t, energy, drift=0.0, **parts):
    return ChronoFrame(step=step, timestamp=t, dt=0.1, total_energy=energy, curvature_drift=drift, **parts)


def test_frame_narrative_reports_energy_shares():
    f = _frame(0, 1.25, 2.0, -0.2, homotopy_energy=1.0, functor_energy=0.5)
    n = text.TextResonator().describe_frame(f)
    assert "t=1.250" in n.summary and "2.000 energy" in n.summary and "-0.200" in n.summary
    assert n.highlights[0] == "homotopy 50.0%" and n.highlights[1] == "functor 25.0%"
    quiet = text.describe_frame(_frame(1, 2.0, 0.0))
    assert "settled" in quiet and "negligible" in quiet


def test_atlas_narrative_lists_metrics_notes_and_hint():
    a = AtlasFrame(timestamp=2.0, loop_support=0.4, collapse_total=1.5, z_signal=-0.25, script_hint="tile 128")
    a.push_metric("psi.total", 0.75)
    a.notes.append("maintainer clamp engaged")
    n = text.TextResonator().describe_atlas(a, maintainer_status="clamp")
    assert n.summary == "Atlas snapshot at t=2.000. Maintainer clamp."
    assert n.highlights == ["loop support 0.400", "collapse total 1.500", "z bias -0.250", "psi.total 0.750",
                            "maintainer clamp engaged", "script tile 128"]
    assert text.describe_atlas(AtlasFrame(timestamp=0.5)) == "Atlas snapshot at t=0.500."


def test_realtime_narrator_emits_samples_per_frame():
    tl = ChronoTimeline(capacity=8)
    for i in range(4):
        tl.record(0.1, {"total_energy": 1.0 + i, "observed_curvature": -1.0 + 0.05 * i})
    narrator = text.RealtimeNarrator(sample_rate=1000)
    samples = narrator.narrate_timeline(tl)
    assert len(samples) == 4 * 50 and max(abs(s) for s in samples) <= 1.0
    assert text.describe_timeline(tl) is not None
    assert text.describe_timeline(ChronoTimeline(capacity=4)) is None


def test_token_scale_stack_flags_semantic_boundary():
    e = torch.tensor([[0.0, 0.0], [0.0, 0.0], [1.0, 1.0], [1.0, 1.0]])
    stack = text.token_scale_stack(e, [1.0, 2.0], 0.25)
    assert stack.mode.startswith("semantic")
    assert stack.samples[0][1] == pytest.approx(0.5)        # tokens 1 and 2 see the jump at radius 1
    assert stack.samples[1][1] == pytest.approx(1.0)
    levels = text.token_coherence_levels(e, [1.0, 2.0, 3.0], 0.25, levels=[0.25, 0.5, 0.75])
    assert levels == [1.0, 1.0, 2.0]
    with pytest.raises(ValueError):
        text.token_scale_stack(e, [1.0], 0.25, metric="manhattan")
    with pytest.raises(ValueError):
        text.token_scale_stack(e[0], [1.0], 0.25)
