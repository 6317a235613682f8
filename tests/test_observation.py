"""Observation accounting: orbit counts against brute force, the bridge against the values of the unit tests of
crates/st-core/src/theory/observation.rs."""
import itertools

import pytest
import torch

from spiraltorch_b200 import observability as obs
from spiraltorch_b200 import observation as O
from spiraltorch_b200.hub import SoftlogicZFeedback
from spiraltorch_b200.macro_model import MacroTemplateBank, MinimalCardConfig, PhasePair
from spiraltorch_b200.microlocal import InterfaceSignature, InterfaceZFused, InterfaceZLift, InterfaceZPulse, InterfaceZReport
from spiraltorch_b200.theory import LeechProjector
from spiraltorch_b200.zpulse import ZScale


def _brute(symmetry, c, b):
    seen = set()
    for tup in itertools.product(range(c), repeat=b):
        if symmetry == "trivial":
            images = [tup]
        elif symmetry == "symmetric":
            images = [tuple(sorted(tup))]
        else:
            images = [tup[i:] + tup[:i] for i in range(b)]
            if symmetry == "dihedral":
                images += [t[::-1] for t in images]
        seen.add(min(images))
    return len(seen)


@pytest.mark.parametrize("symmetry", O.SLOT_SYMMETRIES)
@pytest.mark.parametrize("c,b", [(1, 1), (2, 3), (3, 4), (4, 2), (2, 6), (3, 5), (0, 3)])
def test_orbit_counts_match_enumeration(symmetry, c, b):
    assert O.slot_orbits(symmetry, c, b) == _brute(symmetry, c, b)


def test_coalgebra_unfolds_and_assesses():
    co = O.ObservationalCoalgebra(O.ObservabilityConfig(2, 2, "symmetric"))
    # s0 = 2; s1 = 2 * C(3, 2) = 6; s2 = 2 * C(7, 2) = 42
    assert co.unfold(2) == [2, 6, 42] and co.unique_signatures(1) == 6
    a = co.assess([1, 3, 42, 5])
    assert a.expected[:3] == [2, 6, 42] and a.efficiency[:3] == [0.5, 0.5, 1.0] and a.saturated_depths() == [2]
    assert O.slot_orbits("trivial", 10, 60) == (1 << 128) - 1                     # saturates
    cfg = O.ObservabilityConfig(5, 2).with_color_action(O.ColorAction(5, "cyclic"))
    assert cfg.effective_roots() == 1 and not cfg.color_action.singleton_observable()
    assert O.ColorAction(5).observable_classes() == 5 and O.ColorAction(5).singleton_observable()
    with pytest.raises(ValueError):
        O.ObservabilityConfig(1, 2, "octahedral")


def _report(active: bool) -> InterfaceZReport:
    one = lambda v: torch.full((1,), v)                                            # noqa: E731
    sig = InterfaceSignature(one(1.0 if active else 0.0), one(0.5), one(1.0), one(0.25), None, None, 1.0, 1, 1.0)
    pulse = InterfaceZPulse(support=1.0, interface_cells=1.0, band_energy=(0.2, 0.6, 0.2), scale=ZScale.ONE, drift=0.1, z_bias=0.05,
                            quality_hint=0.8) if active else InterfaceZPulse()
    fused = InterfaceZFused(None, pulse.z_bias, pulse.support, [("microlocal", 1.0)], [])
    return InterfaceZReport(["macro"], [sig], InterfaceZLift([1.0], LeechProjector(1, 0.0)), [pulse], [0.9], pulse, fused, SoftlogicZFeedback(), 1.0)


def test_bridge_links_microlocal_and_macro_feedback():
    bank = MacroTemplateBank().with_card("macro", MinimalCardConfig(PhasePair("A", "B"), 1.0, 1.0))
    bridge = O.ObservationBridge.with_templates(O.ObservabilityConfig(1, 3, "symmetric"), bank)
    seen = []
    handle = obs.add_observer(seen.append) if hasattr(obs, "add_observer") else None
    try:
        snap = bridge.ingest(_report(True))
    finally:
        if handle is not None and hasattr(obs, "remove_observer"):
            obs.remove_observer(handle)
    assert snap.depth_counts == [1, 1, 1, 1, 1] and snap.counts.total_gauges == 1 and snap.counts.active_pulses == 1
    assert len(snap.assessment.expected) >= 5 and snap.microlocal_feedback is not None and list(snap.drives) == ["macro"]
    assert snap.has_interface() and snap.counts.coverage() == 1.0 and snap.counts.pulse_activation_rate() == 1.0
    g = snap.gauges[0]
    assert g.matched_template and g.is_active() and g.pulse_support == 1.0 and g.quality == 0.9
    p = snap.pulses
    assert (p.total, p.active, p.inactive) == (1, 1, 0) and p.mean_support == 1.0 and p.max_support == 1.0
    assert abs(p.mean_z_bias - 0.05) < 1e-7 and p.activation_rate() == 1.0
    if seen:
        meta = [e for e in seen if e.get("kind") == "tensor_op_meta" and e.get("op") == "observation_bridge_ingest"]
        assert meta and meta[0]["meta"]["matched_macro_drives"] == 1 and meta[0]["meta"]["has_microlocal_feedback"]


def test_bridge_handles_empty_reports():
    snap = O.ObservationBridge(O.ObservabilityConfig(1, 2, "symmetric")).ingest(_report(False))
    assert snap.depth_counts == [0, 0, 0, 0, 0] and snap.counts.total_gauges == 1 and snap.counts.active_gauges == 0
    assert snap.microlocal_feedback is None and not snap.drives and not snap.has_interface()
    assert snap.counts.inactive_gauges() == 1 and snap.counts.pulse_activation_rate() == 0.0 and snap.pulses.inactive == 1
