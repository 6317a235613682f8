"""Elliptic warp: Lie frames, telemetry of one orientation, the batched differentiable feature map, accumulation, and the
warped microlocal lift."""
import math

import pytest
import torch

from spiraltorch_b200.elliptic import (EllipticAccumulator, EllipticTelemetry, EllipticWarp, FEATURES, LieFrame, homology_index)
from spiraltorch_b200.microlocal import InterfaceGauge, InterfaceZConductor, InterfaceZLift, MicrolocalFeedback
from spiraltorch_b200.theory import LeechProjector


def test_lie_frame_algebra():
    f = LieFrame.from_axis_angle([0, 0, 2.0], math.pi / 2)
    assert f.apply([1, 0, 0]) == pytest.approx([0, 1, 0], abs=1e-12) and f.apply_inverse([0, 1, 0]) == pytest.approx([1, 0, 0], abs=1e-12)
    assert f.log() == pytest.approx([0, 0, math.pi / 2]) and LieFrame.exp(f.log()).quaternion == pytest.approx(f.quaternion)
    g = LieFrame.from_axis_angle([1, 0, 0], 0.3)
    fg = f.compose(g)
    assert fg.apply([0.2, -0.4, 0.9]) == pytest.approx(f.apply(g.apply([0.2, -0.4, 0.9])))
    assert fg.relative_to(f).quaternion == pytest.approx(g.quaternion) and f.compose(f.inverse()).quaternion == pytest.approx([1, 0, 0, 0])
    assert LieFrame.from_matrix(fg.rotation_matrix()).quaternion == pytest.approx(fg.quaternion)
    for axis, ang in (([1, 0, 0], 3.0), ([0, 1, 0], 3.0), ([0, 0, 1], 3.0)):       # the three non-trace branches of the matrix route
        h = LieFrame.from_axis_angle(axis, ang)
        assert LieFrame.from_matrix(h.rotation_matrix()).quaternion == pytest.approx(h.quaternion, abs=1e-9)
    assert LieFrame([0, 0, 0, 0]).quaternion == [1, 0, 0, 0] and LieFrame([-1, 0, 0, 0]).quaternion == [1, 0, 0, 0]
    assert LieFrame.from_axis_angle([0, 0, 0], 1.0).quaternion == [1, 0, 0, 0] and LieFrame.exp([0, 0, 0]).log() == [0, 0, 0]
    assert f.transport([1, 0, 0], g) == pytest.approx(g.apply_inverse(f.apply([1, 0, 0])))


def test_telemetry_of_one_orientation():
    warp = EllipticWarp(2.0).with_sheet_count(4).with_spin_harmonics(2)
    assert warp.max_geodesic() == pytest.approx(2 * math.pi) and warp.map_orientation([]) is None and warp.map_orientation([0, 0, 0]) is None
    t = warp.map_orientation([1.0, 1.0, 0.0])                              # on the equator, azimuth 45 degrees
    assert t.geodesic_radius == pytest.approx(math.pi) and t.normalized_radius == pytest.approx(0.5) and t.normal_bias == pytest.approx(0.0, abs=1e-12)
    assert t.spin_alignment == pytest.approx(math.sin(0.25 * 2)) and t.sheet_position == pytest.approx(0.625) and t.sheet_index == 2
    assert t.topological_sector == (2 << 1) and t.homology_index == homology_index(2, 4, t.spin_alignment, 0.5)
    assert t.rotor_field == pytest.approx([-math.sqrt(0.5) * math.pi / 2, math.sqrt(0.5) * math.pi / 2, 0.0])
    assert t.lie_frame.apply([0, 0, 1]) == pytest.approx([math.sqrt(0.5), math.sqrt(0.5), 0.0], abs=1e-9)      # the frame carries the pole onto the direction
    assert t.lie_log == pytest.approx(t.rotor_field) and t.noise_density == pytest.approx(0.0, abs=1e-6)
    assert t.curvature_tensor[0][1] == pytest.approx(0.25) and t.resonance_heat == pytest.approx(0.5 * abs(t.spin_alignment), rel=1e-5)
    assert t.event_tags() == ["elliptic.sheet:02", "elliptic.sector:04", "elliptic.radius:0.5000", f"elliptic.spin:{t.spin_alignment:.3f}",
                              f"elliptic.heat:{t.resonance_heat:.3f}"]
    pole = warp.map_orientation([0, 0, 3.0])
    assert pole.geodesic_radius == 0.0 and pole.rotor_field == [0.0, 0.0, 0.0] and pole.noise_density == 1.0
    south = warp.map_orientation([0.0, -1e-3, -1.0])
    assert south.topological_sector & 1 == 1 and south.normalized_radius > 0.99
    assert set(t.as_dict()) >= {"quaternion", "rotation", "lie_log", "rotor_transport", "curvature_tensor", "homology_index"}
    warp.configure(sheet_count=1)
    assert warp.map_orientation([1.0, 1.0, 0.0]).sheet_position == 0.0 and warp.sheet_count() == 1 and warp.spin_harmonics() == 2


def test_batched_features_match_and_differentiate():
    warp = EllipticWarp(1.5).with_sheet_count(3).with_spin_harmonics(2)
    g = torch.Generator().manual_seed(1)
    o = torch.randn(64, 3, generator=g, dtype=torch.float64)
    feats = warp.features(o)
    assert feats.shape == (64, 9) and len(FEATURES) == 9
    for i in (0, 7, 33):
        t = warp.map_orientation(o[i].tolist())
        want = [t.geodesic_radius, t.normalized_radius, t.spin_alignment, t.sheet_position, t.normal_bias, t.resonance_heat] + t.rotor_field
        assert feats[i].tolist() == pytest.approx(want, abs=1e-9)
    tel, diff = warp.map_orientation_differential(o[5].tolist())
    assert diff.features == pytest.approx(feats[5].tolist()) and len(diff.jacobian) == 9 and len(diff.jacobian[0]) == 3
    eps = 1e-6
    for j in range(3):
        d = torch.zeros(3, dtype=torch.float64)
        d[j] = eps
        fd = (warp.features((o[5] + d)[None])[0] - warp.features((o[5] - d)[None])[0]) / (2 * eps)
        assert [row[j] for row in diff.jacobian] == pytest.approx(fd.tolist(), abs=1e-5)
    # scale invariance: the features see the direction only, so the Jacobian annihilates the radial direction
    radial = torch.tensor(diff.jacobian, dtype=torch.float64) @ o[5]
    assert radial.abs().max() < 1e-9
    loss = warp.features(o.clone().requires_grad_(True)).sum()
    assert loss.requires_grad


def test_lerp_and_accumulator():
    warp = EllipticWarp(1.0).with_sheet_count(4)
    a, b = warp.map_orientation([1, 0, 0.5]), warp.map_orientation([-0.2, 1, -0.5])
    m = a.lerp(b, 0.25)
    assert m.normalized_radius == pytest.approx(0.75 * a.normalized_radius + 0.25 * b.normalized_radius) and m.topological_sector == a.topological_sector
    assert a.lerp(b, 0.75).homology_index == b.homology_index and abs(sum(q * q for q in m.lie_frame.quaternion) - 1) < 1e-12
    assert a.lerp(b, 7.0).geodesic_radius == pytest.approx(b.geodesic_radius)
    acc = EllipticAccumulator()
    acc.accumulate(a, 1.0)
    acc.accumulate(b, 3.0)
    acc.accumulate(b, float("nan"))
    out = acc.finish()
    assert out.normal_bias == pytest.approx((a.normal_bias + 3 * b.normal_bias) / 4) and out.topological_sector == b.topological_sector
    assert out.sheet_count == 4 and 0 <= out.sheet_index < 4 and EllipticAccumulator().finish() is None


def test_warped_lift_and_conductor_feedback():
    mask = torch.zeros(4, 4)
    mask[1:, 1:] = 1.0
    label = torch.where(mask > 0.5, 1.0, -1.0)
    sig = InterfaceGauge(1.0, 1.0).analyze_with_label(mask, label)
    flat = InterfaceZLift([1.0, 0.0], LeechProjector(24, 0.5)).project(sig)
    warped = InterfaceZLift([1.0, 0.0], LeechProjector(24, 0.5)).with_elliptic_warp(EllipticWarp(2.0)).project(sig)
    assert flat.elliptic is None and warped.elliptic is not None and warped.band_energy[1] == flat.band_energy[1]
    a, h, b = warped.band_energy
    assert a > 0 and b > 0 and a + b == pytest.approx(h)                       # the warp splits the whole "here" energy between the outer bands
    assert warped.into_softlogic_feedback().elliptic["sheet_count"] == 2 and flat.into_softlogic_feedback().elliptic is None
    cond = InterfaceZConductor([InterfaceGauge(1.0, 1.0), InterfaceGauge(1.0, 2.0)], InterfaceZLift([1.0], LeechProjector(24, 0.5)))
    cond = cond.reinforce_positive_curvature(2.0).with_smoothing(0.5)
    assert cond.lift().elliptic_warp().curvature_radius() == 2.0 and cond.band_policy is not None
    first = cond.step(mask, label)
    assert first.fused_pulse.elliptic is not None and any(e.startswith("elliptic.sheet:") for e in first.fused_z.events)
    assert first.feedback.elliptic is not None and first.feedback.has_event(first.fused_pulse.elliptic.event_tags()[0])
    second = cond.step(mask.T.contiguous(), label.T.contiguous())
    assert second.fused_pulse.elliptic is not None and "smoothing.applied" in second.fused_z.events
    cond.apply_feedback(MicrolocalFeedback().with_elliptic_sheet_count(6).with_elliptic_spin_harmonics(3))
    w = cond.lift().elliptic_warp()
    assert (w.curvature_radius(), w.sheet_count(), w.spin_harmonics()) == (2.0, 6, 3)
    cond.apply_feedback(MicrolocalFeedback().with_elliptic_radius(5.0))
    w = cond.lift().elliptic_warp()
    assert (w.curvature_radius(), w.sheet_count(), w.spin_harmonics()) == (5.0, 6, 3)
    merged = MicrolocalFeedback().with_elliptic_radius(1.0).merge(MicrolocalFeedback().with_elliptic_sheet_count(3).with_elliptic_radius(-1.0))
    assert merged.elliptic_radius == 1.0 and merged.elliptic_sheet_count == 3
