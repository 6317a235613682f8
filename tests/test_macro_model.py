"""Macro-scale interface templates: goldens of crates/st-core/src/theory/macro.rs (its unit tests' values)."""
import math

import pytest
import torch

from spiraltorch_b200 import macro_model as M
from spiraltorch_b200.microlocal import (InterfaceGauge, InterfaceSignature, InterfaceZConductor, InterfaceZLift, InterfaceZPulse,
                                          MicrolocalGaugeBank)
from spiraltorch_b200.theory import LeechProjector


def _sig(shape, r, perim, mean, signed=None, orientation=None):
    t = lambda v: torch.tensor(v, dtype=torch.float32).reshape(shape)      # noqa: E731
    return InterfaceSignature(t(r), torch.zeros(shape), t(perim), t(mean), t(signed) if signed is not None else None,
                              orientation, 1.0, 1, 1.0)


def _minimal(sigma=0.2, **kw):
    return M.MacroModelTemplate.from_card(M.MinimalCardConfig(M.PhasePair("A", "B"), sigma, 1.0, **kw))


def test_dimensionless_groups_match_the_reference_values():
    g = M.DimensionlessGroups.from_scales(M.PhysicalScales(0.072, 0.01, 0.02, 1.0e-3, 100.0, 9.81, 1.0e-6, 1.0e-9, 1.0e-19, 1.0e-7, 0.5))
    assert abs(g.capillary - 2.7777778e-4) < 1e-10
    assert abs(g.bond - 1.3625) < 1e-4
    assert abs(g.cahn - 1.0e-4) < 1e-10
    assert abs(g.peclet - 2.0e5) < 1e-2
    assert abs(g.bending_length - 1.1785113e-9) < 1e-15
    assert abs(g.line_tension_length - 1.3888889e-6) < 1e-12
    assert g.mobility_ratio == 0.5 and g.sharp_interface_ok()
    assert M.DimensionlessGroups.from_scales(M.PhysicalScales(0.1)).capillary is None


def test_cards_build_the_expected_templates():
    t = _minimal(0.1, volume=1.0)
    assert len(t.functional.surface_terms) == 1 and not t.functional.bending_terms
    assert len(t.functional.constraints.volumes) == 1 and t.kinetics.flow == "non_conserved" and t.numerics.algorithm == "mbo"
    assert len(t.numerics.steps) == 3
    mem = M.MacroModelTemplate.from_card(M.MembraneCardConfig(M.PhasePair("A", "C"), 0.2, 0.05, 0.5, spontaneous_curvature=0.1, pressure_jump=0.02))
    assert mem.numerics.algorithm == "level_set" and mem.functional.bending_terms[0].spontaneous_curvature == 0.1
    assert abs(mem.nondimensional.bending_length - math.sqrt(0.05 / 0.2)) < 1e-12
    assert mem.kinetics.forcing_from_pulse(None) == pytest.approx(0.02)
    pat = M.MacroModelTemplate.from_card(M.PatternCardConfig("oil", 0.1, M.Kernel("gaussian", 0.3, 2.0), 1.0))
    assert pat.functional.surface_terms[0].pair == M.PhasePair("oil_in", "out") and pat.kinetics.forcing_from_pulse(None) == pytest.approx(0.3)
    assert not pat.analysis.constraint_handling
    con = M.MacroModelTemplate.from_card(M.ContactCardConfig(M.PhasePair("L", "G"), 0.07, 1.0, 2.0, 1.0, "S", line_tension=1e-3))
    assert con.functional.line_tensions[0].triple == M.PhaseTriple("L", "G", "S") and con.nondimensional.line_tension_length == pytest.approx(1e-3 / 0.07)
    pulse = InterfaceZPulse(z_bias=1.5)
    assert con.kinetics.forcing_from_pulse(pulse) == pytest.approx(-2.0 * 0.5) and con.kinetics.forcing_from_pulse(None) == 0.0
    ani = M.MacroModelTemplate.from_card(M.AnisotropicCardConfig(M.PhasePair("A", "B"), 0.1, M.Anisotropy.custom("facets"), 1.0, bending_regularisation=0.01))
    assert ani.analysis.regularity and len(ani.functional.bending_terms) == 1


def test_kinetics_velocity():
    c = M.CurvatureContributions(0.5, 0.6, 0.1, 0.2)
    assert M.MacroKinetics.non_conserved(2.0).evaluate_velocity(c) == pytest.approx(1.4)
    assert M.MacroKinetics.surface_diffusion(2.0).evaluate_velocity(c) == pytest.approx(-0.2)
    assert M.MacroKinetics.surface_diffusion(2.0).evaluate_velocity(M.CurvatureContributions(0.5)) == pytest.approx(-1.0)


def test_bank_registers_and_couples_in_order():
    bank = M.MacroTemplateBank()
    assert bank.register("minimal", _minimal(0.1)) and not bank.register("minimal", _minimal(0.1))
    bank.with_card("membrane", M.MembraneCardConfig(M.PhasePair("A", "C"), 0.2, 0.05, 0.5))
    assert len(bank) == 2 and bank.get("membrane") is not None
    lift = InterfaceZLift([1.0], LeechProjector(24, 0.15))
    assert bank.couple("minimal", lift).template.kinetics.flow == "non_conserved" and bank.couple("nope", lift) is None
    assert list(bank.couple_all(lift)) == ["minimal", "membrane"]


def test_bridge_turns_a_signature_into_a_drive():
    scales = M.PhysicalScales(0.1, reference_length=1.0, velocity_scale=0.5, viscosity=0.2, interface_thickness=0.2, density_difference=1.0, gravity=9.81)
    bridge = _minimal(0.1, physical_scales=scales).couple_with(InterfaceZLift([1.0], LeechProjector(24, 0.1)))
    drive = bridge.ingest_signature(_sig((1, 1, 1), [1.0], [0.1], [0.5], [0.55]))
    assert drive.velocity > 0.0 and abs(drive.contributions.mean_curvature - 0.5) < 1e-6 and drive.pulse.support > 0.0
    assert not drive.sharp_interface_ok()
    fb = drive.microlocal_feedback()
    assert fb.bias_gain > 0.0 and fb.smoothing >= 0.2 and fb.tempo_hint > 0.0 and fb.threshold_scale < 1.0


def test_perimeter_weighting_and_fourier_anisotropy():
    bridge = _minimal(0.2).couple_with(InterfaceZLift([1.0], LeechProjector(24, 0.2)))
    d = bridge.ingest_signature(_sig((1, 2), [1.0, 0.0], [1.0, 0.0], [2.0, 20.0], [2.0, 20.0]))
    assert abs(d.contributions.mean_curvature - 2.0) < 1e-6 and abs(d.contributions.anisotropic_curvature - 2.0) < 1e-6 and abs(d.velocity - 2.0) < 1e-6
    fn = M.MacroInterfacialFunctional.minimal(M.PhasePair("A", "B"), 0.3)
    fn.surface_terms[0].anisotropy = M.Anisotropy.fourier([(4, 0.5)])
    t = M.MacroModelTemplate(fn, M.MacroKinetics.non_conserved(1.0), M.DimensionlessGroups(), M.AnalysisChecklist.minimal_surface(), M.NumericalRecipe.mbo(False))
    bridge = M.MacroZBridge(t, InterfaceZLift([1.0, 0.0], LeechProjector(24, 0.5)))
    orient = torch.tensor([0.0, 1.0]).reshape(2, 1, 1)
    d = bridge.ingest_signature(_sig((1, 1), [1.0], [1.0], [2.0], [2.0], orient))
    assert abs(d.contributions.anisotropic_curvature - 3.0) < 1e-6 and abs(d.velocity - 3.0) < 1e-6


@pytest.mark.parametrize("bands,tight", [((2.0, 0.0, 0.0), True), ((0.5, 0.5, 0.5), False)])
def test_density_fluctuation_tightens_or_relaxes_the_controls(bands, tight):
    bridge = _minimal(0.2).couple_with(InterfaceZLift([1.0], LeechProjector(24, 0.0)))
    c = M.CurvatureContributions(1.0)
    v = bridge.template.kinetics.evaluate_velocity(c)
    pulse = InterfaceZPulse(support=1.0, interface_cells=8.0, band_energy=bands, drift=0.1, quality_hint=0.7, standard_error=0.05)
    fb = bridge.derive_feedback(c, v, pulse)
    if tight:
        assert pulse.density_fluctuation() > 0.45
        assert fb.threshold_scale < 1.0 and fb.smoothing >= 0.55 and fb.bias_gain < 1.0 and fb.tempo_hint >= v
    else:
        assert pulse.density_fluctuation() < 0.25
        assert fb.threshold_scale > 1.0 and fb.smoothing < 0.3 and fb.bias_gain > 1.0 and fb.tempo_hint < v


def test_drive_matched_feeds_back_into_the_conductor():
    gauges = MicrolocalGaugeBank().with_registered("minimal", InterfaceGauge(1.0, 1.0))
    conductor = InterfaceZConductor(gauges, InterfaceZLift([1.0], LeechProjector(24, 0.25)))
    report = conductor.step(torch.tensor([[0.0, 0.0], [0.0, 1.0]]))
    assert report.gauge_id(0) == "minimal"
    bank = M.MacroTemplateBank().with_card("minimal", M.MinimalCardConfig(M.PhasePair("A", "B"), 0.1, 1.0))
    drives = bank.drive_matched(report)
    assert list(drives) == ["minimal"]
    fb0 = drives["minimal"].microlocal_feedback()
    assert fb0.threshold_scale is not None or fb0.bias_gain is not None
    before = (conductor.gauge_thresholds(), conductor.bias_gain())
    conductor.apply_feedback(bank.feedback_from_report(report))
    after = (conductor.gauge_thresholds(), conductor.bias_gain())
    assert before != after
