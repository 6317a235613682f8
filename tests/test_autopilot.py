"""Autopilot on the BlackCat bandit: context schema, suggest / report protocol, bounded profile window with
type-7 quantiles, persistence, hint mode and the trainer coupling (reference behaviour:
crates/st-core/src/runtime/autopilot.rs:297-800 and its tests :1430-2086)."""
import json

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200 import plugin
from spiraltorch_b200.device_caps import DeviceCaps
from spiraltorch_b200.nn.trainer import StepMetrics
from spiraltorch_b200.runtime.autopilot import (AutoConfig, AutoMode, Autopilot, AutopilotError, KnobSpec,
                                                PROFILE_WINDOW, neumaier_mean, quantile_type7)
from spiraltorch_b200.runtime.blackcat import BlackCat

CAPS = DeviceCaps(backend="cuda", subgroup=True, lane_width=32, max_workgroup=1024)


def _pilot(tmp_path, mode=AutoMode.AUTO, knobs=(), groups=None, feat_dim=8, extras=()):
    rt = BlackCat(groups or {"tile": ["64", "128"], "stages": ["3", "4"]}, feat_dim)
    return Autopilot(CAPS, AutoConfig(mode, knobs, feat_dim, extras), rt, profile_dir=tmp_path)


def test_quantile_and_mean_estimators():
    assert quantile_type7([], 0.5) == 0.0
    assert quantile_type7([4.0, 1.0, 3.0, 2.0], 0.5) == 2.5
    assert abs(quantile_type7([float(i) for i in range(1, 101)], 0.95) - 95.05) < 1e-9
    assert abs(neumaier_mean([1e16, 1.0, -1e16]) - 1.0 / 3.0) < 1e-12


def test_context_schema(tmp_path):
    ap = _pilot(tmp_path, feat_dim=10, extras=("loss", "curvature"))
    ctx = ap.try_build_context(32, 4, 2, 0.5, [("curvature", -1.0), ("loss", 2.0)])
    assert ctx == [1.0, 32.0, 4.0, 2.0, 32 / 1024, 1024 / 4096, 0.5, 1.0, 2.0, -1.0]
    assert ap.context_features()[-2:] == ["loss", "curvature"]
    for bad, kind in (((0, 1, 1, 0.0, [("loss", 1.0), ("curvature", 0.0)]), "NonPositiveWorkload"),
                      ((1, 1, 1, -1.0, [("loss", 1.0), ("curvature", 0.0)]), "InvalidValue"),
                      ((1, 1, 1, 0.0, [("loss", 1.0)]), "MissingFeature"),
                      ((1, 1, 1, 0.0, [("loss", 1.0), ("curvature", 0.0), ("x", 1.0)]), "UnexpectedFeature"),
                      ((1, 1, 1, 0.0, [("loss", 1.0), ("loss", 2.0), ("curvature", 0.0)]), "DuplicateFeature")):
        with pytest.raises(AutopilotError) as e:
            ap.try_build_context(*bad)
        assert e.value.kind == kind
    assert ap.build_context(0, 1, 1, 0.0, []) == []
    short = _pilot(tmp_path, feat_dim=3)
    assert short.try_build_context(8, 2, 5, 0.0) == [1.0, 8.0, 2.0]
    with pytest.raises(AutopilotError):
        _pilot(tmp_path, feat_dim=9)                      # nine features need one named extra


def test_suggest_report_protocol_and_profile(tmp_path):
    ap = _pilot(tmp_path)
    ctx = ap.build_context(16, 2, 3, 0.1)
    with pytest.raises(AutopilotError) as e:
        ap.try_report(StepMetrics(1.0, 1.0, 0.0))
    assert e.value.kind == "MissingSuggestion"
    picks = ap.try_suggest(ctx)
    assert set(picks) == {"tile", "stages"}
    with pytest.raises(AutopilotError) as e:
        ap.try_suggest(ctx)
    assert e.value.kind == "PendingSuggestion"
    with pytest.raises(AutopilotError):
        ap.try_report(StepMetrics(float("nan"), 1.0, 0.0))
    rep = ap.try_report(StepMetrics(12.0, 100.0, 0.25))
    assert rep.sample_count == 1 and rep.profile.step_ms_p50 == 12.0 and rep.profile.chosen == picks
    assert rep.reward < 0
    # abandoning a suggestion credits nothing
    ap.try_suggest(ctx)
    before = ap.runtime.steps
    assert ap.abandon_suggestion() is not None and ap.abandon_suggestion() is None
    assert ap.runtime.steps == before and not ap.suggestion_ready
    # the window is bounded
    for i in range(PROFILE_WINDOW + 4):
        ap.try_suggest(ctx)
        ap.try_report(StepMetrics(float(i), float(i), 0.0))
    assert ap.profile_sample_count() == PROFILE_WINDOW
    doc = json.loads(ap.profile_path().read_text())
    assert doc["sample_capacity"] == PROFILE_WINDOW and len(doc["samples"]["step_ms"]) == PROFILE_WINDOW
    assert doc["estimators"]["step_ms_p50"] == "exact_hyndman_fan_type_7"


def test_profile_is_reloaded_and_corrupt_profiles_are_replaced(tmp_path):
    ap = _pilot(tmp_path)
    ctx = ap.build_context(4, 1, 1, 0.0)
    for v in (5.0, 7.0, 9.0):
        ap.try_suggest(ctx)
        ap.try_report(StepMetrics(v, 10 * v, 0.0))
    again = _pilot(tmp_path)
    assert again.profile_sample_count() == 3 and again.profile.step_ms_p50 == 7.0
    again.profile_path().write_text("{ not json")
    fresh = _pilot(tmp_path)
    assert fresh.profile_sample_count() == 0 and fresh.profile.chosen == {}


def test_hint_mode_prefers_persisted_choice_among_equivalent_arms(tmp_path):
    ap = _pilot(tmp_path, mode=AutoMode.HINT)
    ap.profile.chosen = {"tile": "128", "stages": "4"}
    picks = ap.try_suggest(ap.build_context(4, 1, 1, 0.0))     # untrained bandit: every arm is equivalent
    assert picks == {"tile": "128", "stages": "4"}
    ap.abandon_suggestion()
    auto = _pilot(tmp_path, mode=AutoMode.AUTO)
    auto.profile.chosen = {"tile": "128", "stages": "4"}
    assert auto.try_suggest(auto.build_context(4, 1, 1, 0.0)) == {"tile": "64", "stages": "3"}   # hints ignored


def test_knob_contract_and_off_mode(tmp_path):
    with pytest.raises(AutopilotError):
        _pilot(tmp_path, knobs=[KnobSpec("tile", ["64"])])            # BlackCat could emit "128"
    with pytest.raises(AutopilotError) as e:
        ap = _pilot(tmp_path, knobs=[KnobSpec("tile", ["64", "128"])])
        ap.try_suggest(ap.build_context(1, 1, 1, 0.0))                # "stages" is not declared
    assert e.value.kind == "UndeclaredKnob"
    ap = _pilot(tmp_path, knobs=[KnobSpec("tile", ["64", "128"]), KnobSpec("stages", ["3", "4"]),
                                 KnobSpec("ring", ["2", "3"], default_idx=1)])
    assert ap.try_suggest(ap.build_context(1, 1, 1, 0.0))["ring"] == "3"     # default of a knob BlackCat does not own
    off = _pilot(tmp_path, mode=AutoMode.OFF)
    assert off.try_suggest([1.0] * 8) == {} and off.try_report(StepMetrics(1.0, 1.0, 0.0)) is None


def test_trainer_coupling_publishes_events(tmp_path):
    ap = _pilot(tmp_path)
    seen, applied = [], []
    sid = plugin.subscribe("AutopilotReport", lambda ev: seen.append(ev))
    try:
        model = st.nn.Sequential()
        model.add(st.nn.Linear(4, 3, name="fc"))
        x, y = st.Tensor(torch.randn(6, 4)), st.Tensor(torch.randn(6, 3))
        trainer = st.SpiralSession("cpu", seed=1).trainer()
        trainer.enable_autopilot(ap, apply_picks=applied.append)
        trainer.train_epoch(model, st.nn.MeanSquaredError(), [(x, y), (x, y)])
    finally:
        plugin.unsubscribe("AutopilotReport", sid)
    assert len(applied) == 2 and set(applied[0]) == {"tile", "stages"}
    assert ap.profile_sample_count() == 2 and ap.runtime.steps == 2
    assert len(seen) == 2
