"""Telemetry hub (blackboard slots, atlas merge / route / observers, psi subscriptions, loopback buffer), chrono
harmonics / loop signal / time warps, the timeline maintainer, and the desire-psi bridge."""
import math

import pytest

import spiraltorch_b200 as st
from spiraltorch_b200 import hub, telemetry as T
from spiraltorch_b200.psi import PsiComponent, PsiEvent, PsiReading
from spiraltorch_b200.zpulse import ZScale


@pytest.fixture(autouse=True)
def clean_hub():
    hub.reset()
    yield
    hub.reset()


def frame(step, drift, energy, decay=-0.01):
    return T.ChronoFrame(step, step * 0.1 + 0.1, 0.1, -1.0 + drift, energy, 0.4 * energy, 0.2 * energy, 0.2 * energy, 0.1 * energy,
                         0.1 * energy, drift, decay)


def wave(n=16, period=8, amp=0.2):
    return [frame(k, amp * math.sin(2 * math.pi * k / period), 1.0 + abs(math.cos(2 * math.pi * k / period))) for k in range(n)]


def test_harmonics_find_the_drift_tone_and_build_a_script():
    frames = wave()
    h = T.ChronoHarmonics.from_frames(frames, 8)
    assert h.frames == 16 and h.duration == pytest.approx(1.6) and h.sample_rate == pytest.approx(10.0) and h.nyquist == pytest.approx(5.0)
    assert len(h.drift_power) == 8 and h.dominant_drift.frequency == pytest.approx(10.0 * 2 / 16)        # period 8 of 16 samples: bin 2
    assert h.dominant_drift.magnitude == pytest.approx(0.1, rel=1e-6)                                   # amp / 2
    assert h.dominant_energy.frequency == pytest.approx(10.0 * 4 / 16)                                  # |cos| doubles the tone
    assert T.ChronoHarmonics.from_frames(frames[:1], 8) is None and T.ChronoHarmonics.from_frames(frames, 0) is None
    tl = T.ChronoTimeline(64)
    for k in range(16):
        tl.record(0.1, {"observed_curvature": -1 + 0.2 * math.sin(2 * math.pi * k / 8), "total_energy": 1.0 + 0.1 * k})
    sig = tl.loop_signal(16, 8)
    assert sig.summary.frames == 16 and sig.harmonics is not None
    fields = [h.field for h in sig.spiralk_hints]
    assert fields[:3] == ["radix", "segments", "tile_cols"] and "kl" in fields and "wg" in fields
    assert "soft (radix" in sig.spiralk_script.replace("soft(", "soft (")
    assert tl.loop_signal(1, 8).harmonics is None and T.ChronoTimeline().loop_signal(4, 4) is None


def test_time_warps():
    tl = T.ChronoTimeline(16)
    for k in range(4):
        tl.record(0.5, {"observed_curvature": -1.0, "total_energy": 2.0 - 0.1 * k})
    decay = tl.latest().energy_decay
    tl.dilate(2.0)
    assert [f.timestamp for f in tl.frames()] == pytest.approx([1.0, 2.0, 3.0, 4.0]) and tl.latest().dt == pytest.approx(1.0)
    assert tl.latest().energy_decay == pytest.approx(decay / 2.0)
    tl.shift(10.0)
    assert tl.latest().timestamp == pytest.approx(14.0) and next(tl.frames()).dt == pytest.approx(1.0)
    tl.align_to_progress(0.25, 8.0)                                       # the recorded span becomes [0, 2]
    assert tl.latest().timestamp == pytest.approx(2.0) and next(tl.frames()).timestamp == pytest.approx(0.5)
    nxt = tl.record(0.5, {"observed_curvature": -1.0, "total_energy": 1.0})
    assert nxt.timestamp == pytest.approx(2.5)
    for bad, kind in ((lambda: tl.dilate(0.0), "invalid_scale"), (lambda: tl.shift(float("nan")), "non_finite"),
                      (lambda: T.ChronoTimeline().dilate(2.0), "empty"), (lambda: T.TemporalWarp.fit_span(0, 0, 0, 1), "degenerate")):
        with pytest.raises(T.TemporalWarpError) as e:
            bad()
        assert e.value.kind == kind
    assert T.TemporalWarp(2.0, 1.0, 3.0).apply(5.0) == pytest.approx(3.0 + 4.0 + 1.0)


def test_maintainer_statuses():
    m = T.Maintainer()
    assert m.assess([]).status == "dormant"
    calm = [frame(k, 0.01, 1.0, 0.0) for k in range(12)]
    rep = m.assess(calm)
    assert rep.status == "stable" and rep.suggested_max_scale is None and "within expected range" in rep.diagnostic
    assert m.assess([frame(k, 0.0, 1e-5, 0.0) for k in range(4)]).status == "dormant"
    jitter = [frame(k, 0.8 if k % 2 else -0.8, 1.0, 0.0) for k in range(12)]
    rep = m.assess(jitter)
    assert rep.status == "clamp" and rep.suggested_max_scale == 3.0 and rep.suggested_pressure == pytest.approx(min(0.12 * (1 + 0.8 / 0.35), 1.0))
    assert "curvature jitter 0.800" in rep.diagnostic
    growth = [frame(k, 0.0, 1.0, -0.2) for k in range(12)]
    rep = m.assess(growth)
    assert rep.status == "rewrite" and rep.should_rewrite() and rep.suggested_pressure == pytest.approx(0.12 * (1 + 0.2 / 0.05))
    cfg = T.MaintainerConfig(jitter_threshold=-1, clamp_min=5.0, clamp_max=1.0, window=0).sanitise()
    assert cfg.jitter_threshold == 0.35 and (cfg.clamp_min, cfg.clamp_max) == (1.0, 5.0) and cfg.window == 1


def test_atlas_merge_route_and_observers():
    seen = []
    sub = hub.register_atlas_frame_observer(lambda f: seen.append(f.timestamp))
    assert hub.atlas_observer_count() == 1 and hub.get_atlas_frame() is None
    frag = T.AtlasFragment(timestamp=1.0, loop_support=0.5, z_signal=0.2)
    frag.push_metric("loop.energy", 2.0)
    frag.push_metric("bad", float("nan"))
    frag.push_note("  hello ")
    hub.merge_atlas_fragment(frag)
    hub.merge_atlas_fragment(T.AtlasFragment())                            # empty: ignored
    f2 = T.AtlasFragment(timestamp=0.5, loop_support=0.25, collapse_total=3.0)
    f2.push_metric("loop.energy", 4.0)
    f2.push_note("hello")
    hub.merge_atlas_fragment(f2)
    a = hub.get_atlas_frame()
    assert a.timestamp == 1.0 and a.loop_support == 0.75 and a.collapse_total == 3.0 and a.z_signal == 0.2
    assert a.metrics == {"loop.energy": 4.0} and a.notes == ["hello"] and seen == [1.0, 1.0]
    assert len(hub.get_atlas_route()) == 2 and len(hub.get_atlas_route(1)) == 1 and len(hub.get_atlas_route(0)) == 0
    for k in range(40):
        hub.set_atlas_frame(T.AtlasFrame(float(k + 2)))
    assert len(hub.get_atlas_route()) == hub.ATLAS_ROUTE_CAPACITY and hub.get_atlas_route().latest().timestamp == 41.0
    assert not hub.get_atlas_route_summary().is_empty()
    sub.close()
    hub.set_atlas_frame(T.AtlasFrame(99.0))
    assert hub.atlas_observer_count() == 0 and seen[-1] == 41.0
    hub.clear_atlas()
    assert hub.get_atlas_frame() is None and len(hub.get_atlas_route()) == 0
    # a fragment without any timestamp still founds a frame (at the smallest positive time) once it carries content
    only = T.AtlasFragment()
    only.push_metric("x", 1.0)
    hub.merge_atlas_fragment(only)
    assert 0 < hub.get_atlas_frame().timestamp < 1e-6


def test_softlogic_realgrad_maintainer_feed_the_atlas():
    fb = hub.SoftlogicZFeedback(psi_total=1.5, weighted_loss=0.7, band_energy=(0.2, 0.5, 0.3), drift=0.1, z_signal=-0.4,
                                scale=ZScale.new(2.0), events=["flip-held"], elliptic={"curvature_radius": 1.2, "sheet_index": 3})
    fb.set_attributions([("Maxwell", 0.6), ("lidar", -1.0)])
    assert fb.attributions == [("maxwell", 0.6), ("other.lidar", 0.0)] and fb.has_event("flip-held")
    hub.set_softlogic_z(fb)
    a = hub.get_atlas_frame()
    assert a.z_signal == -0.4 and a.metric_value("softlogic.band.total") == pytest.approx(1.0)
    assert a.metric_value("softlogic.attribution.maxwell") == 0.6 and a.metric_value("softlogic.elliptic.sheet_index") == 3.0
    assert "softlogic.event:flip-held" in a.notes and any(n.startswith("softlogic.scale.radius:2.000@0.693") for n in a.notes)
    assert hub.get_softlogic_z() is fb and hub.clear_softlogic_z() and not hub.clear_softlogic_z()
    hub.set_last_realgrad(hub.RealGradPulse(iterations=7, gradient_norm=2.0, converged=True, transparency={"gain": 0.3}))
    a = hub.get_atlas_frame()
    assert a.timestamp == 7.0 and a.metric_value("realgrad.converged") == 1.0 and a.metric_value("realgrad.transparency.gain") == 0.3
    assert hub.get_last_realgrad().gradient_summary() == {"norm": 2.0, "sparsity": 1.0}
    rep = T.Maintainer().assess([frame(k, 0.0, 1.0, -0.2) for k in range(12)])
    hub.set_maintainer_report(rep)
    a = hub.get_atlas_frame()
    assert a.maintainer_status == "rewrite" and a.suggested_pressure == rep.suggested_pressure and a.metric_value("maintainer.should_rewrite") == 1.0
    assert a.script_hint == rep.spiralk_script.strip() and hub.get_maintainer_report() is rep


def test_psi_slots_and_subscriptions():
    sub = hub.subscribe_psi_metrics()
    assert sub.snapshot().reading is None and hub.psi_subscriber_count() == 1
    reading = PsiReading(1.25, {PsiComponent.LOSS: 1.0, PsiComponent.GRAD_NORM: 0.5}, 4)
    hub.set_last_psi(reading)
    ev = PsiEvent(PsiComponent.LOSS, 1.0, 0.8, True, 4)
    hub.set_last_psi_events([ev])
    hub.set_last_psi_spiral({"regime": "supercritical"})
    hub.set_last_psi_spiral_tuning({"gain": 1.1})
    snap = sub.snapshot()
    assert snap.reading is reading and snap.events == [ev] and snap.spiral == {"regime": "supercritical"} and snap.tuning == {"gain": 1.1}
    late = hub.subscribe_psi_metrics()
    assert late.snapshot().reading is reading                                # a new subscriber starts from the current state
    a = hub.get_atlas_frame()
    assert a.metric_value("psi.total") == 1.25 and a.metric_value("psi.loss") == 1.0 and a.timestamp == 4.0 and str(ev) in a.notes
    hub.clear_last_psi()
    hub.clear_last_psi_events()
    hub.clear_last_psi_spiral()
    hub.clear_last_psi_spiral_tuning()
    assert sub.snapshot() == hub.PsiMetricsFrame() and hub.get_last_psi() is None and hub.get_last_psi_events() == []
    sub.close()
    late.close()
    assert hub.psi_subscriber_count() == 0
    assert hub.PsiMetricsSubscription.detached(hub.PsiMetricsFrame(reading)).snapshot().reading is reading


def test_loopback_dashboard_config_region_collapse():
    tl = T.ChronoTimeline(32)
    for k in range(8):
        tl.record(0.1, {"observed_curvature": -1 + 0.1 * k, "total_energy": 1.0})
    sig = tl.loop_signal(8, 4)
    hub.set_chrono_loop(sig)
    assert hub.get_chrono_loop() is sig
    for k in range(70):
        hub.push_loopback_envelope(hub.LoopbackEnvelope(sig, source=f"node-{k}", support=0.5, z_signal=0.1 if k % 2 else float("nan")))
    assert len(hub.peek_loopback_envelopes(100)) == hub.LOOPBACK_CAPACITY and hub.peek_loopback_envelopes(1)[0].source == "node-6"
    drained = hub.drain_loopback_envelopes(10)
    assert [e.source for e in drained][:2] == ["node-6", "node-7"] and len(hub.peek_loopback_envelopes(100)) == 54
    assert drained[0].z_signal is None and drained[1].z_signal == 0.1 and drained[0].timestamp == sig.summary.latest_timestamp
    a = hub.get_atlas_frame()
    assert a.loop_support == pytest.approx(35.0) and a.metric_value("loop.frames") == 8.0 and a.chrono_summary == sig.summary
    assert "source:node-69" in a.notes and a.metric_value("z.bias") == 0.1
    for k in range(70):
        hub.push_dashboard_frame(T.DashboardFrame(float(k), [T.DashboardMetric("m", float(k))], []))
    snap = hub.snapshot_dashboard_frames(3)
    assert [f.timestamp for f in snap] == [69.0, 68.0, 67.0] and hub.latest_dashboard_frame().timestamp == 69.0
    assert hub.snapshot_dashboard_frames(0) == [] and len(hub.snapshot_dashboard_frames(1000)) == hub.DASHBOARD_CAPACITY
    hub.record_config_events([hub.ConfigDiffEvent("site", "trainer.lr", 0.1, 0.2)])
    assert hub.get_config_events()[0].path == "trainer.lr"
    events = []
    with st.observability.observe(events.append):
        hub.set_region_loss_report(hub.AttributionReport(2, 2, [1.0, -2.0, float("nan"), 0.5], algorithm="grad_cam"))
        hub.set_region_loss_trend_report(hub.AttributionReport(1, 1, [0.1]))
    meta = [e["meta"] for e in events if e["kind"] == "tensor_op_meta"]
    assert meta[0]["finite_values"] == 3 and meta[0]["negative_values"] == 1 and meta[0]["max_abs_value"] == 2.0 and meta[0]["algorithm"] == "grad_cam"
    assert hub.get_region_loss_report().rows == 2 and hub.get_region_loss_trend_report().values == [0.1]
    assert hub.get_region_loss_volatility_report() is None and hub.clear_region_loss_report() and hub.get_region_loss_report() is None
    hub.set_collapse_pulse(hub.CollapsePulse(12, 2.5, {"kind": "collapse", "grad_scale": 0.5}, sig))
    a = hub.get_atlas_frame()
    assert a.collapse_total == 2.5 and "collapse.command:collapse" in a.notes and a.metric_value("collapse.command.grad_scale") == 0.5
    assert hub.get_collapse_pulse().step == 12


def test_desire_psi_bridge_pairs_steps_with_hub_state():
    from tests.test_desire_pipeline import LOGITS, _automation
    from spiraltorch_b200.desire_pipeline import DesirePipeline, DesirePsiBridge, DesireTelemetryBundle
    bridge = DesirePsiBridge()
    bundle = DesireTelemetryBundle().with_psi_bridge(bridge)
    pipe = DesirePipeline.builder(_automation()).with_telemetry_bundle(bundle).build()
    assert pipe.sink_count() == 1 and bridge.is_empty() and bridge.drain_summary() is None
    pipe.step_at(LOGITS, 0, [0.7, 0.3], 0.0, 100.0)                       # nothing in the hub yet
    hub.set_last_psi(PsiReading(2.0, {PsiComponent.LOSS: 1.5}, 3))
    hub.set_last_psi_events([PsiEvent(PsiComponent.LOSS, 1.5, 1.0, True, 3)])
    hub.set_softlogic_z(hub.SoftlogicZFeedback(z_signal=0.4))
    for i in range(1, 5):
        pipe.step_at(LOGITS, i, [0.7, 0.3], float(i), 100.0 + i)
    assert len(bridge) == 5
    last = hub.get_last_desire_step()
    assert last.psi_total == 2.0 and last.z_feedback.z_signal == 0.4 and last.phase == "integration" and last.timestamp == 104.0
    a = hub.get_atlas_frame()
    assert a.metric_value("desire.psi.total") == 2.0 and a.metric_value("desire.z_feedback.z_signal") == 0.4 and "desire.phase:integration" in a.notes
    s = bridge.drain_summary()
    assert s.steps == 5 and s.psi_samples == 4 and s.mean_psi_total == 2.0 and s.component_means == {PsiComponent.LOSS: 1.5}
    assert s.threshold_crossings == {PsiComponent.LOSS: (4, 0)} and s.mean_z_signal == pytest.approx(0.4) and s.last_timestamp == 104.0
    assert s.triggers == 1 and s.mean_entropy > 0 and bridge.is_empty()
