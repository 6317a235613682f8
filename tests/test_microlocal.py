"""Microlocal interface gauges, the Z lift, pulse algebra, quality policies and the interface conductor."""
import itertools
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.microlocal import (BandPolicy, BudgetPolicy, CompositePolicy, DefaultZSourcePolicy, FixedPolicy, InterfaceGauge,
                                         InterfaceZConductor, InterfaceZLift, InterfaceZPulse, MicrolocalFeedback, MicrolocalGaugeBank,
                                         ZSourcePolicy, unit_sphere_area)
from spiraltorch_b200.theory import LeechProjector
from spiraltorch_b200.zpulse import ZScale

MASK = torch.tensor([[0.0, 0.0, 0.0], [0.0, 1.0, 1.0], [0.0, 1.0, 1.0]])
LABEL = torch.where(MASK > 0.5, 1.0, -1.0)


def naive(mask, label, threshold):
    """Cell-by-cell restatement of the stencil."""
    shape, dim = mask.shape, mask.dim()
    var, r, lap_t, grad = torch.zeros(shape), torch.zeros(shape), torch.zeros(shape), torch.zeros((dim,) + tuple(shape))
    for idx in itertools.product(*[range(n) for n in shape]):
        c, lap, iface = float(mask[idx]), 0.0, False
        for ax in range(dim):
            f = b = None
            if idx[ax] + 1 < shape[ax]:
                f = float(mask[idx[:ax] + (idx[ax] + 1,) + idx[ax + 1:]]) - c
                grad[(ax,) + idx] += f
                var[idx] = max(float(var[idx]), abs(f))
                iface |= abs(f) >= threshold
            if idx[ax] > 0:
                b = c - float(mask[idx[:ax] + (idx[ax] - 1,) + idx[ax + 1:]])
                grad[(ax,) + idx] -= b
                var[idx] = max(float(var[idx]), abs(b))
                iface |= abs(b) >= threshold
            if f is not None and b is not None:
                lap += f - b
        r[idx], lap_t[idx] = float(iface), lap
    norm = grad.pow(2).sum(0).sqrt()
    orient = torch.where(norm > 0, grad / norm.clamp(min=1e-6), grad)
    return var, r, lap_t, orient


def test_gauge_matches_the_cell_loop_in_2d_and_3d():
    g = torch.Generator().manual_seed(3)
    for shape in ((5, 7), (3, 4, 5), (6,)):
        mask = torch.rand(shape, generator=g)
        label = torch.where(mask > 0.5, 1.0, -1.0)
        sig = InterfaceGauge(1.0, 2.0).with_threshold(0.3).analyze_with_label(mask, label)
        var, r, lap, orient = naive(mask, label, 0.3)
        kappa = unit_sphere_area(len(shape))
        assert torch.allclose(sig.raw_density, var) and torch.equal(sig.r_machine, r) and torch.allclose(sig.perimeter_density, r * kappa)
        assert torch.allclose(sig.mean_curvature, (lap.abs() * 0.25).clamp(max=kappa), atol=1e-6)
        assert torch.allclose(sig.signed_mean_curvature, lap * torch.sign(label), atol=1e-6) and torch.allclose(sig.orientation, orient, atol=1e-6)
        assert sig.radius == 2 and sig.physical_radius == 2.0
    assert unit_sphere_area(2) == pytest.approx(2 * math.pi) and unit_sphere_area(3) == pytest.approx(4 * math.pi) and unit_sphere_area(0) == 0.0


def test_boundary_detection_and_normals():
    sig = InterfaceGauge(1.0, 1.0).analyze(MASK)
    assert sig.has_interface() and sig.kappa_d == pytest.approx(2 * math.pi) and sig.orientation is None and sig.signed_mean_curvature is None
    assert float(sig.perimeter_density[1, 1]) == pytest.approx(sig.kappa_d) and float(sig.perimeter_density[0, 0]) == 0.0
    assert not InterfaceGauge(1.0, 1.0).analyze(torch.zeros(3, 3)).has_interface()
    sig = InterfaceGauge(1.0, 1.0).analyze_with_label(MASK, LABEL)
    ny, nx = float(sig.orientation[0, 1, 1]), float(sig.orientation[1, 1, 1])
    assert abs(ny) > 0.5 and abs(nx) == pytest.approx(abs(ny)) and nx < 0
    wide = InterfaceGauge(1.0, 2.0).analyze_with_label(MASK, LABEL)
    assert torch.allclose(wide.orientation, sig.orientation) and wide.radius == 2
    sigs = InterfaceGauge(1.0, 1.0).analyze_multiradius(MASK, LABEL, [1.0, 1.5, 3.0])
    assert [s.radius for s in sigs] == [1, 2, 3] and sigs[1].physical_radius == 1.5 and all(s.orientation is not None for s in sigs)
    with pytest.raises(ValueError):
        InterfaceGauge(1.0, 1.0).analyze_with_label(MASK, torch.zeros(2, 2))
    bank = MicrolocalGaugeBank().with_registered("fine", InterfaceGauge(1.0, 1.0)).with_registered("coarse", InterfaceGauge(1.0, 2.5))
    assert not bank.register("fine", InterfaceGauge(1.0, 9.0)) and bank.ids() == ["fine", "coarse"] and len(bank) == 2
    assert set(bank.analyze_all(MASK)) == {"fine", "coarse"} and bank.remove("fine") is not None and bank.get("fine") is None


def test_lift_and_pulse_algebra():
    lift = InterfaceZLift([1.0, 0.0], LeechProjector(24, 0.5))
    pulse = lift.project(InterfaceGauge(1.0, 1.0).analyze_with_label(MASK, LABEL))
    above, here, beneath = pulse.band_energy
    assert above > beneath and here > 0 and pulse.z_bias > 0 and pulse.scale == ZScale.ONE and pulse.interface_cells == pulse.support
    fb = pulse.into_softlogic_feedback()
    assert fb.band_energy == pulse.band_energy and fb.z_signal == pulse.z_bias and fb.scale == pulse.scale
    plain = lift.project(InterfaceGauge(1.0, 1.0).analyze(MASK))
    assert plain.band_energy[0] == plain.band_energy[2] == 0.0 and plain.band_energy[1] > 0 and plain.z_bias == 0.0
    a = InterfaceZPulse(support=2.0, interface_cells=2.0, band_energy=(0.2, 0.4, 0.1), scale=ZScale.new(1.0), drift=0.1, z_bias=0.5)
    b = InterfaceZPulse(support=6.0, interface_cells=5.0, band_energy=(0.1, 0.2, 0.3), scale=ZScale.new(3.0), drift=-0.1, z_bias=-0.1)
    agg = InterfaceZPulse.aggregate([a, b])
    assert agg.support == 8.0 and agg.interface_cells == 7.0 and agg.band_energy == pytest.approx((0.3, 0.6, 0.4))
    assert agg.drift == pytest.approx((0.1 * 2 - 0.1 * 6) / 8) and agg.z_bias == pytest.approx((0.5 * 2 - 0.1 * 6) / 8) and agg.scale.physical_radius == pytest.approx(2.5)
    assert InterfaceZPulse.aggregate([]).is_empty() and InterfaceZPulse.aggregate([]).scale == ZScale.ONE
    mid = InterfaceZPulse.lerp(a, b, 0.25)
    assert mid.support == 3.0 and mid.z_bias == pytest.approx(0.35) and mid.scale.physical_radius == pytest.approx(1.5)
    half = a.scaled(0.5)
    assert half.support == 1.0 and half.band_energy == pytest.approx((0.1, 0.2, 0.05)) and half.z_bias == 0.25 and a.scaled(-1).support == 0.0
    with pytest.raises(ValueError):
        InterfaceZLift([], LeechProjector(24, 0.5))


def test_policies():
    p = InterfaceZPulse(support=0.6, band_energy=(0.5, 0.4, 0.3), z_bias=0.4)
    assert DefaultZSourcePolicy().quality(p) == pytest.approx(0.5) and DefaultZSourcePolicy().quality(InterfaceZPulse()) == 0.0
    assert FixedPolicy(1.7).quality(p) == 1.0
    comp = CompositePolicy(DefaultZSourcePolicy()).with_source("Maxwell", FixedPolicy(0.9))
    assert comp.quality(p) == pytest.approx(0.5) and comp.quality(InterfaceZPulse(source="maxwell", support=1.0)) == 0.9
    lop = InterfaceZPulse(support=1.0, band_energy=(0.9, 0.05, 0.05))
    band = BandPolicy([0.2, 0.5, 0.2])
    assert band.project_quality(lop) == pytest.approx((0.05 / 0.5) * (0.05 / 0.2)) and band.project_quality(InterfaceZPulse(band_energy=(0.25, 0.5, 0.25))) == 1.0
    assert BandPolicy([0.2, 0.5, 0.2], hysteresis=0.5).project_quality(lop) == 1.0
    pc = BandPolicy.positive_curvature(1.0)
    assert pc.min_quality[0] == pytest.approx(0.2 + 0.15 * math.tanh(1.0)) and pc.min_quality[1] == pytest.approx(0.5 + 0.25 * math.tanh(1.0))
    budget = BudgetPolicy(0.1)
    assert budget.apply(p) == pytest.approx(0.25) and p.z_bias == pytest.approx(0.1) and p.band_energy == pytest.approx((0.125, 0.4, 0.075))
    assert p.support == pytest.approx(0.15) and budget.apply(p) == 1.0
    fbk = MicrolocalFeedback().with_threshold_scale(0.5).with_bias_gain(2.0).merge(MicrolocalFeedback().with_threshold_scale(0.5).with_smoothing(1.5))
    assert fbk.threshold_scale == 0.25 and fbk.bias_gain == 2.0 and fbk.smoothing == 1.0 and fbk.tempo_hint is None
    assert MicrolocalFeedback().with_bias_gain(-1.0).bias_gain is None


def test_conductor_fuses_gauges_with_smoothing_budget_and_feedback():
    big = torch.zeros(4, 4)
    big[1:, 1:] = 1.0
    flipped = big.clone()
    flipped[1, 2] = flipped[2, 2] = 0.0
    label = torch.where(big > 0.5, 1.0, -1.0)
    lift = InterfaceZLift([1.0, 0.0], LeechProjector(24, 0.5)).with_bias_gain(0.5)
    cond = InterfaceZConductor([InterfaceGauge(1.0, 1.0), InterfaceGauge(1.0, 2.5)], lift).with_smoothing(0.5)
    events = []
    with st.observability.observe(events.append):
        first = cond.step(big, label)
    assert first.has_interface() and first.fused_pulse.z_bias > 0 and len(first.qualities) == len(first.pulses) == len(first.signatures) == 2
    assert first.budget_scale == 1.0 and first.gauge_ids == [None, None] and "smoothing.applied" not in first.fused_z.events
    assert any(e["kind"] == "tensor_op_meta" and e["op"] == "microlocal_conductor_step" and e["meta"]["gauges"] == 2 for e in events)
    second = cond.step(flipped, -label)
    raw = InterfaceZPulse.aggregate(second.pulses)
    assert "smoothing.applied" in second.fused_z.events and second.feedback.has_event("smoothing.applied")
    a, h, b = second.fused_pulse.band_energy
    assert second.fused_z.pulse.band_energy == second.fused_pulse.band_energy and second.feedback.band_energy == second.fused_pulse.band_energy
    assert (second.fused_z.pulse.support.leading, second.fused_z.pulse.support.central, second.fused_z.pulse.support.trailing) == pytest.approx((a, h, b))
    assert second.fused_pulse.z_bias == pytest.approx(0.5 * (first.fused_pulse.z_bias + InterfaceZPulse.aggregate(
        [p.scaled(q) for p, q in zip(second.pulses, second.qualities)]).z_bias))
    assert second.feedback.attributions and second.feedback.attributions[0][0] == "microlocal"
    assert cond.last_fused_pulse().z_bias == second.fused_pulse.z_bias and raw.support > 0

    class Half(ZSourcePolicy):
        def quality(self, pulse):
            return 0.5
    solo = InterfaceZConductor([InterfaceGauge(1.0, 1.0)], InterfaceZLift([1.0], LeechProjector(24, 0.5))).with_policy(Half())
    rep = solo.step(big, label)
    assert rep.qualities == [0.5] and rep.fused_pulse.support == pytest.approx(rep.pulses[0].support * 0.5)
    assert rep.fused_pulse.z_bias == pytest.approx(rep.pulses[0].z_bias * 0.5) and rep.fused_z.pulse.quality == 0.5
    clamp = InterfaceZConductor([InterfaceGauge(1.0, 1.0)], InterfaceZLift([1.0], LeechProjector(24, 0.5), bias_gain=1000.0)).with_budget_policy(BudgetPolicy(0.02))
    rep = clamp.step(big, label, tempo_hint=3.0, stderr_hint=0.1)
    assert rep.budget_scale < 1.0 and abs(rep.fused_pulse.z_bias) <= 0.02 + 1e-9 and rep.fused_z.pulse.tempo == 3.0 and rep.fused_z.pulse.stderr == 0.1
    bank = MicrolocalGaugeBank().with_registered("fine", InterfaceGauge(1.0, 1.0))
    named = InterfaceZConductor.from_bank(bank, lift).reinforce_positive_curvature(2.0)
    named.apply_feedback(MicrolocalFeedback().with_threshold_scale(0.5).with_bias_gain(2.0).with_smoothing(0.3).with_tempo_hint(4.0).with_stderr_hint(0.2))
    assert named.gauge_thresholds() == [0.125] and named.bias_gain() == 2.0 and named.smoothing == 0.3 and named.band_policy is not None
    rep = named.step(big, label)
    assert rep.gauge_id(0) == "fine" and rep.signature_for("fine") is rep.signatures[0] and rep.signature_for("nope") is None
    assert rep.fused_z.pulse.tempo == 4.0 and rep.fused_z.pulse.stderr == 0.2 and rep.lift.bias_gain() == 2.0
    with pytest.raises(ValueError):
        InterfaceZConductor([], lift)
