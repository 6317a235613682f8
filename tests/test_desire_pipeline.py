"""Desire automation, logbook and pipeline (reference behaviour: crates/st-nn/src/language/automation.rs,
logbook.rs, pipeline.rs and their tests)."""
import queue

import pytest
import torch

from spiraltorch_b200 import plugin
from spiraltorch_b200.desire_pipeline import (DesireAutomation, DesireLogbook, DesireLogReplay, DesirePipeline,
                                              DesireTrainerBridge, DesireTriggerBuffer, SelfRewriteCfg)
from spiraltorch_b200.language import DesireLagrangian, DesireWeights, TemperatureController, constant, warmup


def _automation(cfg=None, V=6, C=2):
    g = torch.Generator().manual_seed(0)
    lag = DesireLagrangian(torch.randn(V, V, generator=g) * 0.1, torch.randn(V, V, generator=g) * 0.1,
                           torch.tensor([0.0, 0.9, 0.0, 0.8, 0.0, 0.0]), torch.rand(V, C, generator=g),
                           TemperatureController(1.0, 1.2, 0.05, 0.3, 2.0))
    lag.with_schedules(alpha=warmup(0.0, 0.4, 3), beta=constant(0.1), gamma=warmup(0.0, 0.3, 3), lam=constant(0.5))
    lag.with_horizons(2, 4)
    return DesireAutomation(lag, cfg or SelfRewriteCfg(score_thresh=0.0, min_samples=2, cooldown_sec=10.0))


LOGITS = [0.2, 1.5, -0.3, 1.2, 0.0, 0.4]


def test_phases_vector_and_trigger_rule():
    auto = _automation()
    phases, triggers = [], []
    for i in range(8):
        step = auto.step(LOGITS, i % 6, [0.7, 0.3], now=float(i))
        phases.append(step.solution.phase)
        triggers.append(step.trigger is not None)
    assert phases[:2] == ["observation", "observation"] and phases[2:] == ["integration"] * 6
    # integration starts once the observation horizon (2 steps) has passed; two samples are needed, so the first
    # trigger fires at step 3; the cool-down (10 s of the injected clock) suppresses the rest
    assert triggers == [False, False, False, True, False, False, False, False]
    assert auto.trigger_count == 1 and auto.penalty_samples() == 4          # cleared at the trigger, four since
    v = torch.tensor(auto.desire_vector())
    # observation steps mix the (normalised) avoidance heat in; a bias without mass only decays the vector
    assert bool((v >= 0).all()) and float(v.sum()) <= 1.0 + 1e-5 and set(torch.nonzero(v).flatten().tolist()) <= {1, 3}
    late = auto.step(LOGITS, 0, [0.7, 0.3], now=100.0)
    assert late.trigger is not None and late.trigger.samples == 5 and late.trigger.mean_penalty > 0
    assert set(late.trigger.report.tokens) <= {1, 3}                         # only repressed tokens heat up


def test_threshold_blocks_triggers():
    auto = _automation(SelfRewriteCfg(score_thresh=10.0, min_samples=1, cooldown_sec=0.0))
    assert all(auto.step(LOGITS, 0, [0.5, 0.5], now=float(i)).trigger is None for i in range(8))


def test_logbook_round_trip_and_replay(tmp_path):
    auto = _automation()
    path = tmp_path / "desire.jsonl"
    book = DesireLogbook(path, flush_every=2)
    bridge, buf, chan = DesireTrainerBridge(), DesireTriggerBuffer(), queue.Queue()
    pipe = (DesirePipeline.builder(auto).with_logbook(book).with_trainer_bridge(bridge).with_trigger_buffer(buf)
            .with_channel(chan).with_telemetry().build())
    assert pipe.sink_count() == 5
    seen = []
    sid = plugin.subscribe("DesireStep", seen.append)
    try:
        for i in range(7):
            pipe.step_at(LOGITS, i % 6, [0.6, 0.4], now=float(i), timestamp=1000.0 + i)
    finally:
        plugin.unsubscribe("DesireStep", sid)
    pipe.flush()
    assert book.ordinal() == 7 and len(seen) == 7 and len(buf) == 1 and chan.qsize() == 8
    summary = bridge.drain_summary()
    assert summary.total == 7 and summary.observation == 2 and summary.integration == 5 and summary.triggers == 1
    assert bridge.is_empty() and bridge.drain_summary() is None
    records = list(DesireLogReplay.open(path))
    assert [r.ordinal for r in records] == list(range(7)) and records[0].timestamp_ms == 1_000_000
    assert records[3].step.trigger is not None and isinstance(records[5].step.solution.weights, DesireWeights)
    # replay feeds the sinks again without running the automation
    other = DesireTrainerBridge()
    fresh = DesirePipeline(_automation())
    fresh.attach_trainer_bridge(other)
    assert fresh.replay(DesireLogReplay(path)) == 7 and len(other) == 7
    book.close()
    again = DesireLogbook(path)
    assert again.ordinal() == 7                                       # ordinals continue across re-opens
    again.close()
    with pytest.raises(FileNotFoundError):
        DesireLogReplay(tmp_path / "absent.jsonl")


def test_trainer_bridge_checkpoint():
    auto = _automation()
    bridge = DesireTrainerBridge()
    pipe = DesirePipeline.builder(auto).with_trainer_bridge(bridge).build()
    for i in range(6):
        pipe.step_at(LOGITS, 0, [0.5, 0.5], now=float(i), timestamp=float(i))
    doc = bridge.checkpoint()
    restored = DesireTrainerBridge()
    restored.restore_checkpoint(doc)
    a, b = bridge.drain_summary(), restored.drain_summary()
    assert a == b and a.total == 6


def test_roundtable_bridge_projection_summary_checkpoint_and_cooperation():
    import copy
    import math
    from spiraltorch_b200.desire_pipeline import DesireRoundtableBridge, DesireRoundtableSummary, DesireTelemetryBundle
    imp = DesireRoundtableBridge.project(DesireWeights(alpha=0.6, beta=0.1, gamma=0.3, lam=0.5), 0.6, 0.4, 7.0)
    assert imp.multipliers == pytest.approx((1 + 0.6 * (0.6 - 1 / 3), 1 + 0.6 * (0.3 - 1 / 3), 1 + 0.6 * (0.1 - 1 / 3)))
    assert imp.drift == pytest.approx(math.tanh(0.5) * 0.4) and imp.timestamp == 7.0
    flat = DesireRoundtableBridge.project(DesireWeights(alpha=-1.0, beta=0.0, gamma=0.0, lam=-50.0), 1.0, 1.0, 0.0)
    assert flat.multipliers == pytest.approx((2 / 3, 2 / 3, 2 / 3)) and flat.drift == pytest.approx(-1.0)

    rt, tr = DesireRoundtableBridge(blend=0.5, drift_gain=0.3), DesireTrainerBridge()
    assert rt.propose() == (0.0, 1.0)
    bundle = DesireTelemetryBundle().with_trainer_bridge(tr).with_roundtable_bridge(rt)
    pipe = DesirePipeline.builder(_automation()).with_telemetry_bundle(bundle).build()
    assert pipe.sink_count() == 2
    for i in range(5):
        pipe.step_at(LOGITS, 0, [0.5, 0.5], now=float(i), timestamp=10.0 + i)
    assert len(rt) == 5 and len(tr) == 5 and rt.impulse().timestamp == 14.0
    drift, weight = rt.propose()
    assert -1.0 <= drift <= 1.0 and 0.05 <= weight <= 2.0
    doc = copy.deepcopy(rt.checkpoint())
    assert doc["pending_summary"]["steps"] == 5 and doc["latest"]["timestamp"] == 14.0
    events = rt.drain()
    want = DesireRoundtableSummary.from_events(events)
    assert want.steps == 5 and want.last_timestamp == 14.0 and want.mean_above == pytest.approx(sum(e.multipliers[0] for e in events) / 5)
    other = DesireRoundtableBridge()
    other.restore_checkpoint(doc)
    assert other.blend() == 0.5 and other.drift_gain() == 0.3 and len(other) == 5
    got = other.drain_summary()
    assert (got.steps, got.triggers) == (want.steps, want.triggers)
    assert got.mean_entropy == pytest.approx(want.mean_entropy) and got.mean_drift == pytest.approx(want.mean_drift)
    assert other.drain_summary() is None and rt.drain_summary() is None
    before = other.checkpoint()
    for bad in ({**doc, "blend": float("nan")}, {**doc, "latest": {"multipliers": [1.0, 9.0, 1.0], "drift": 0.0, "timestamp": 1.0}},
                {**doc, "pending_summary": {**doc["pending_summary"], "triggers": 99}}):
        with pytest.raises(ValueError):
            other.restore_checkpoint(bad)
    assert other.checkpoint() == before                                   # a rejected document changes nothing
    b0, g0 = other.blend(), other.drift_gain()
    other.observe(-0.2, -0.6)
    assert other.blend() > b0 and other.drift_gain() > g0
    other.observe(2.0, 2.0)
    assert other.blend() < 0.5 + 0.1 and 0.1 <= other.drift_gain() <= 1.2
    other.set_blend(float("nan"))
    assert math.isfinite(other.blend())
