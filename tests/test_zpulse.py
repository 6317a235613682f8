"""Z pulses, the conductor's fusion / hysteresis / latency alignment, emitters, and scale persistence of a pulse train."""
import math

import pytest

import spiraltorch_b200 as st
from spiraltorch_b200.zpulse import (DesireEmitter, LatencyAlignerCfg, ZAdaptiveGainCfg, ZConductor, ZConductorCfg, ZFrequencyConfig,
                                     ZPulse, ZRegistry, ZScale, ZSupport, derive_quality, shift_timestamp, zpulse_coherence_levels,
                                     zpulse_scale_stack)


def pulse(source, ts, drift, quality, **kw):
    support = ZSupport(abs(drift), 0.0, abs(drift))
    bands = (support.leading, 0.0, support.trailing)
    return ZPulse(source=source, ts=ts, tempo=abs(drift), band_energy=bands, density_fluctuation=ZPulse.density_fluctuation_for(bands),
                  drift=drift, z_bias=drift, support=support, quality=quality, **kw)


def test_scale_and_support_helpers():
    s = ZScale.new(2.0)
    assert s.log_radius == pytest.approx(math.log(2.0)) and ZScale.new(0.0) is None and ZScale.new(float("nan")) is None
    assert ZScale.from_log(0.0) == ZScale.ONE and ZScale.from_log(float("inf")) is None
    mid = ZScale.lerp(ZScale.new(1.0), ZScale.new(3.0), 0.5)
    assert mid.physical_radius == pytest.approx(2.0) and mid.log_radius == pytest.approx(0.5 * math.log(3.0))
    avg = ZScale.weighted_average([(ZScale.new(1.0), 1.0), (ZScale.new(3.0), 3.0), (ZScale.new(9.0), -1.0)])
    assert avg.physical_radius == pytest.approx(2.5)
    assert ZScale.weighted_average([]) is None
    sup = ZSupport.new(-1.0, 0.5, float("nan"))
    assert (sup.leading, sup.central, sup.trailing) == (0.0, 0.5, 0.0) and sup.total() == 0.5 and not sup.is_empty()
    assert ZSupport().is_empty() and ZSupport.from_band_energy((1, 2, 3)).max_component() == 3
    assert ZPulse.density_fluctuation_for((0.4, 0.4, 0.4)) < 1e-12
    assert ZPulse.density_fluctuation_for((1.0, 0.0, 0.0)) == pytest.approx(math.sqrt(2.0 / 9.0), rel=1e-5)
    assert ZPulse.density_fluctuation_for((float("nan"), -1.0, 0.0)) == 0.0
    p = pulse("Maxwell", 0, 0.5, 1.0)
    assert p.source == "maxwell" and p.total_energy() == 1.0 and p.normalised_drift() == 0.0 and ZPulse(source="lidar").source == "other.lidar"
    assert shift_timestamp(10, -12.4, 1) == 0 and shift_timestamp(10, 2.5, 1) == 13 and shift_timestamp(10, 8.0, 4) == 12


def test_quality_is_derived_when_missing():
    p = pulse("microlocal", 0, 0.5, 0.0)
    q = derive_quality(p)
    want = (0.4 * math.tanh(1.0 / (1e-6 + 1.0)) + 0.3 * 0.5 + 0.3 * (0.5 / 1.5)) * (1.0 - 0.2 * p.density_fluctuation)
    assert q == pytest.approx(want)
    c = ZConductor()
    c.ingest(p)
    assert c.pending[0].quality == pytest.approx(q) and p.quality == 0.0           # the caller's pulse is not touched
    c.ingest(pulse("microlocal", 0, 0.5, 7.0))
    assert c.pending[1].quality == 1.0


def test_conductor_fuses_by_support_and_reports():
    events = []
    with st.observability.observe(events.append):
        c = ZConductor(ZConductorCfg(alpha_fast=1.0, alpha_slow=1.0))
        c.set_frequency_config(ZFrequencyConfig.new(0.25, 0.1))
        c.set_adaptive_gain_config(ZAdaptiveGainCfg.new(0.2, 1.4, 0.75))
        c.ingest(pulse("microlocal", 10, 0.4, 1.0))
        c.ingest(pulse("maxwell", 10, 0.8, 0.9))
        fused = c.step(10)
    # z = (0.4 * 0.8 + 0.8 * 1.6) / 2.4 = 0.6667, limited to one slew step from 0
    assert fused.support == pytest.approx(2.4) and fused.z == pytest.approx(0.35)
    assert fused.quality == pytest.approx((1.0 * 0.8 + 0.9 * 1.6) / 2.4) and fused.attributions[0][0] == "maxwell"
    meta = [e["meta"] for e in events if e["kind"] == "tensor_op_meta" and e["op"] == "zpulse_conductor_step"][0]
    assert meta["pending_before"] == 2 and meta["ready_count"] == 2 and meta["retained_count"] == 0 and meta["top_source"] == "maxwell"
    assert meta["source_microlocal_support"] == pytest.approx(0.8) and meta["frequency_configured"] and meta["latency_source_count"] > 0
    # a pulse stamped in the future waits
    c.ingest(pulse("microlocal", 50, 0.4, 1.0))
    assert c.step(11).support == 0.0 and len(c.pending) == 1
    assert c.step(50).support == pytest.approx(0.8)


def test_sign_flip_hysteresis_slew_and_budget():
    c = ZConductor(ZConductorCfg(flip_hold=2, alpha_fast=1.0, alpha_slow=1.0, slew_max=10.0, z_budget=0.9, latency=None))
    c.set_latency_aligner(None)
    seen = []
    for ts, sign in enumerate([1.0, 1.0, -1.0, -1.0, -1.0, -1.0]):
        c.ingest(pulse("microlocal", ts, sign, 1.0))
        seen.append(c.step(ts))
    assert seen[0].z == 0.9                                            # budget clamp
    assert "flip-held" in seen[2].events and seen[2].z == 0.9          # the opposite sign is held back ...
    assert "flip-held" in seen[3].events and seen[3].z == 0.9
    assert "sign-flip" in seen[4].events and seen[4].z == -0.9         # ... and goes through after flip_hold steps
    assert seen[5].events == [] and seen[5].z == -0.9
    d = ZConductor(ZConductorCfg(alpha_fast=0.5, slew_max=0.1))
    d.ingest(pulse("microlocal", 0, 1.0, 1.0))
    assert d.step(0).z == pytest.approx(0.1)                           # slew limit
    # robust_delta: a tiny opposite value still flips to at least that magnitude
    e = ZConductor(ZConductorCfg(flip_hold=1, alpha_fast=1.0, alpha_slow=1.0, slew_max=10.0, robust_delta=0.25))
    for ts, z in enumerate([0.5, -0.01, -0.01]):
        e.ingest(pulse("microlocal", ts, z, 1.0))
        out = e.step(ts)
    assert "sign-flip" in out.events and out.z == pytest.approx(-0.25)


def test_density_event_and_empty_pulses():
    c = ZConductor()
    lop = ZPulse(source="graph", ts=0, band_energy=(1.0, 0.0, 0.0), density_fluctuation=0.47, support=ZSupport(1.0, 0.0, 0.0), z_bias=0.2, quality=1.0)
    c.ingest(lop)
    c.ingest(ZPulse(source="maxwell", ts=0, quality=1.0))              # empty: ignored by the fusion
    fused = c.step(0)
    assert any(e.startswith("density.fluctuation:0.470") for e in fused.events) and len(fused.attributions) == 1
    assert fused.drift == pytest.approx(1.0)


def test_latency_aligner_tracks_seeds_holds_and_refuses():
    c = ZConductor()
    c.set_latency_aligner(LatencyAlignerCfg.from_steps(16, 0.4, 0.1, 1).with_hop(1))
    for lag in range(5, 15):
        anchor = lag * 10
        drift = math.sin(lag * 0.3)
        c.ingest(pulse("microlocal", anchor, drift, 1.0))
        c.ingest(pulse("maxwell", anchor + lag, drift, 1.0))
        c.step(anchor)
    assert abs(c.latency_for("maxwell") - 10.0) <= 10.0
    # an explicit latency hint seeds the estimate
    c = ZConductor()
    c.set_latency_aligner(LatencyAlignerCfg.from_steps(48, 0.2, 0.2, 4).with_window(192).with_hop(1))
    c.ingest(pulse("microlocal", 0, 0.4, 1.0))
    c.ingest(pulse("graph", 0, 0.5, 1.0, latency_ms=12.5))
    fused = c.step(0)
    assert c.latency_for("graph") == pytest.approx(12.5) and any(e.startswith("latency.seeded:graph:12.50") for e in fused.events)
    assert "latency.held:graph" in fused.events
    # hold_steps spaces the adjustments
    c = ZConductor()
    c.set_latency_aligner(LatencyAlignerCfg(window=256, hop=1, max_lag_steps=64, alpha=0.3, coherence_min=0.2, hold_steps=3))
    last = None
    for step in range(60):
        c.ingest(pulse("microlocal", step, 1.0, 1.0))
        c.ingest(pulse("maxwell", step + 8, 1.0, 1.0))
        if any(e.startswith("latency.adjusted") for e in c.step(step).events):
            assert last is None or step - last >= 3
            last = step
    assert last is not None
    # a coherence bar above 1 can never be met: only low-coherence notes, no adjustment
    c = ZConductor()
    c.set_latency_aligner(LatencyAlignerCfg(coherence_min=2.0))
    low = adj = False
    for ts in range(10):
        c.ingest(pulse("microlocal", ts, math.sin(ts * 0.3), 1.0))
        c.ingest(pulse("maxwell", ts + 12, math.cos(ts * 0.4), 1.0))
        ev = c.step(ts).events
        low |= any(e.startswith("latency.low_coherence") for e in ev)
        adj |= any(e.startswith("latency.adjusted") for e in ev)
    assert low and not adj
    # timestamps that run backwards are reported and ignored by the aligner
    c = ZConductor()
    c.ingest(pulse("graph", 10, 0.1, 1.0))
    c.ingest(pulse("graph", 5, 0.1, 1.0))
    assert "latency.invalid_ts:graph" in c.step(10).events
    c.set_latency_aligner(None)
    assert c.latency is None and c.latency_for("graph") is None


def test_registry_and_desire_emitter():
    em = DesireEmitter()
    reg = ZRegistry()
    reg.register(em)
    p = ZPulse(source="microlocal", support=ZSupport(0.4, 0.4, 0.4), band_energy=(0.4, 0.4, 0.4), drift=0.1)
    em.enqueue(p)
    got = reg.gather(42)
    assert len(got) == 1 and got[0].source == "desire" and p.source == "microlocal"
    em.extend([ZPulse(source="maxwell", support=ZSupport(0.4, 0.4, 0.4), band_energy=(0.4, 0.4, 0.4))] * 2)
    assert [g.source for g in reg.gather(43)] == ["desire", "desire"] and reg.gather(44) == []

    class Hinted(DesireEmitter):
        def quality_hint(self):
            return 0.7
    h = Hinted()
    h.enqueue(p)
    reg2 = ZRegistry()
    reg2.register(h)
    c = ZConductor()
    fused = c.step_from_registry(reg2, 0)
    assert fused.quality == pytest.approx(0.7) and fused.attributions == [("desire", pytest.approx(1.2))]


def test_scale_persistence_of_a_pulse_train():
    calm = [pulse("microlocal", t, 0.1, 1.0) for t in range(8)]
    jump = calm[:4] + [pulse("maxwell", t, 2.0, 1.0) for t in range(4, 8)]
    flat = zpulse_scale_stack(calm, [1.0, 2.0, 4.0], 0.5)
    assert [g for _, g in flat.samples] == [0.0, 0.0, 0.0]
    stack = zpulse_scale_stack(jump, [1.0, 2.0, 4.0], 0.5)
    gates = [g for _, g in stack.samples]
    assert gates[0] == pytest.approx(2 / 8) and gates == sorted(gates) and gates[-1] == 1.0
    levels = zpulse_coherence_levels(jump, [1.0, 2.0, 4.0], 0.5, "euclidean", [0.2, 0.9, 1.5])
    assert levels[0] == 1.0 and levels[1] == 4.0 and levels[2] is None
    with pytest.raises(ValueError):
        zpulse_scale_stack(jump, [], 0.5)
