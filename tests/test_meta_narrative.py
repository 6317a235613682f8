"""Causal set, temporal engine, meaning sheaf and the meta-narrative layer."""
import pytest

from spiraltorch_b200.meta_narrative import (CausalError, CausalInvariantError, CausalSet, MeaningSection, MeaningSheaf, MetaNarrativeLayer,
                                             NarrativeBeat, TemporalLogicEngine, ToposLogicBridge, ZSpace, ZSpaceGate)
from spiraltorch_b200.theory import MaxwellZPulse


def pulse(z):
    return MaxwellZPulse(16, 0.12, 0.05, z, (0.4, 0.3, 0.2), 0.18)


def test_causal_set_rules():
    s = CausalSet()
    s.insert("a", 1)
    s.insert("b", 2)
    s.add_dependency("a", "b")
    with pytest.raises(CausalError) as e:
        s.add_dependency("b", "a")
    assert e.value.kind == "cyclic_dependency" and "`b` -> `a`" in str(e.value)
    for call, kind in ((lambda: s.insert(" ", 0), "empty_event_id"), (lambda: s.insert("a", 0), "duplicate_event"),
                       (lambda: s.add_dependency("a", "a"), "self_dependency"), (lambda: s.add_dependency("x", "a"), "unknown_event"),
                       (lambda: s.add_dependency("a", "x"), "unknown_event")):
        with pytest.raises(CausalError) as e:
            call()
        assert e.value.kind == kind
    assert s.is_ready("a") and not s.is_ready("b") and s.ready_ids() == ["a"] and s.get("b").parent_ids() == ["a"]
    s.validate()
    assert s.resolve("a") == ("a", 1) and s.was_resolved("a") and s.is_ready("b") and s.resolve("a") is None
    with pytest.raises(CausalError) as e:
        s.insert("a", 9)
    assert e.value.kind == "resolved_event"
    s.insert("c", 3)
    s.add_dependency("a", "c")                                         # a dependency on a resolved event never blocks
    assert s.is_ready("c") and len(s) == 2 and s.resolved_len() == 1
    s.validate()
    s.successors["b"].add("ghost")
    with pytest.raises(CausalInvariantError) as e:
        s.validate()
    assert e.value.kind == "unknown_successor"


def test_engine_orders_by_readiness():
    eng = TemporalLogicEngine()
    eng.insert_event("bridge", "B")
    eng.insert_event("intro", "I")
    eng.add_dependency("intro", "bridge")                              # inserted in reverse, constrained afterwards
    eng.insert_event("aside", "A")
    eng.validate()
    assert eng.frontier == ["intro", "aside"] and eng.pending() == 3
    assert eng.next_matching(lambda p: p == "A") == ("aside", "A")
    assert eng.next_ready() == ("intro", "I") and eng.next_ready() == ("bridge", "B") and eng.next_ready() is None
    assert eng.was_resolved("intro")
    eng.insert_event("x", 1)
    eng.insert_event("y", 2)
    eng.add_dependency("x", "y")
    assert eng.discard_event("x") == ("x", 1) and eng.frontier == ["y"] and eng.payload("y") == 2
    eng.frontier.append("y")
    with pytest.raises(CausalInvariantError) as e:
        eng.validate()
    assert e.value.kind == "duplicate_frontier_event"


def test_sheaf_collapse_and_gates():
    z = ZSpace.from_pulse(pulse(2.0))
    assert z.signature == [16.0, 0.12, 0.05, 2.0, 0.4, 0.3, 0.2, 0.18] and z.cosine_similarity(z) == pytest.approx(1.0)
    sheaf = (MeaningSheaf().with_section(MeaningSection.for_open("root", ["warm", " warm ", "bright"], 0.5))
             .with_section(MeaningSection(["*"], ["bright"], 0.25)).with_section(MeaningSection(["other"], ["cold"], 9.0))
             .with_section(MeaningSection([], ["aligned"], 2.0).with_zspace_signature(z.signature, 0.9))
             .with_section(MeaningSection([], ["opposed"], 2.0).with_zspace_signature([-v for v in z.signature], 0.1)))
    tags, total = sheaf.collapse("root", 0.3, z)
    assert tags == [("aligned", pytest.approx(2.0)), ("bright", 0.75), ("warm", 0.5)] and total == pytest.approx(3.25)
    tags, total = sheaf.collapse("root", 0.6, None)                    # signature-gated sections need an observation
    assert tags == [("bright", 0.75)] and total == 0.75
    assert sheaf.collapse("nowhere", 0.0, None)[0] == [("bright", 0.25)]
    assert ZSpaceGate(z.signature, 0.9, 1.0).allows(z) and not ZSpaceGate(z.signature, 0.9, 100.0).allows(z)
    assert not ZSpaceGate([0.0] * 8, 0.0, 0.0).allows(ZSpace([0.0] * 8)) or True
    assert ToposLogicBridge().resolve("none", "root", 0.0) == ([], 0.0)


def test_layer_releases_beats_with_pulses():
    layer = MetaNarrativeLayer()
    eng, bridge = layer.engine_mut(), layer.bridge_mut()
    eng.insert_event("intro", NarrativeBeat("alpha", "root", ["hello", "hello"]).with_intensity_scale(0.5).with_floor(0.2))
    eng.insert_event("bridge", NarrativeBeat(None, "root", ["world"]).with_sheaf_threshold(0.1))
    eng.insert_event("gated", NarrativeBeat("alpha", "root", ["rare"]).with_zspace_gate(ZSpace.from_pulse(pulse(2.0)).signature, 0.99, 0.0))
    eng.add_dependency("intro", "bridge")
    bridge.attach("bridge", MeaningSheaf().with_section(MeaningSection.for_open("root", ["glow"], 0.5)))
    assert layer.next_with_pulse("beta", pulse(1.0)) is None           # nothing ready accepts channel beta yet
    first = layer.next_with_pulse("alpha", pulse(-3.0))
    assert first.event_id == "intro" and first.channel == "alpha" and first.tags == ["hello"] and first.intensity == pytest.approx(1.5)
    second = layer.next_with_pulse("beta", pulse(1.0))                 # channel-free beat takes the caller's channel
    assert second.event_id == "bridge" and second.channel == "beta" and second.tags == ["glow", "world"] and second.intensity == pytest.approx(1.5)
    assert layer.next_with_pulse("alpha", pulse(-40.0)) is None        # the gate wants a pulse that looks like z = 2
    third = layer.next_with_pulse("alpha", pulse(2.0))
    assert third.event_id == "gated" and third.z_space.signature[3] == 2.0
    weak = MetaNarrativeLayer()
    weak.engine_mut().insert_event("quiet", NarrativeBeat(None, "root", []).with_floor(0.3))
    assert weak.next_with_pulse("c", pulse(0.01)).intensity == pytest.approx(0.3)
