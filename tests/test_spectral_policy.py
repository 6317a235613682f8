"""Coherence-driven learning-rate policy and its ModuleTrainer wiring (behaviour of crates/st-nn/src/trainer.rs
`SpectralLearningRatePolicy`, `CoherenceSignal`, `enable_spectral_learning_rate`, `push_coherence_diagnostics`)."""
import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import zspace_coherence as zc
from spiraltorch_b200.inference import BandEnergy
from spiraltorch_b200.nn import coherence as C
from spiraltorch_b200.nn.amp import CoherenceSignal, CurvatureDecision, CurvatureScheduler, SpectralLearningRatePolicy


def _signal(weights, energy_ratio, z_bias, dominant=0):
    dist = zc.summarize_distribution(weights)
    ctl = zc.derive_control(dist, energy_ratio, sum(weights) / len(weights))
    cls = zc.classify(energy_ratio, zc.is_swap_invariant(weights))
    return CoherenceSignal(dominant, sum(1 for w in weights if w > 0), z_bias, ctl, cls)


def _flat_policy():
    return (SpectralLearningRatePolicy().with_smoothing(1.0).with_event_smoothing(1.0).with_sheet_gain(0.0).with_spin_gain(0.0)
            .with_phase_gain(0.0).with_stuck_phase_gain(0.0).with_energy_gain(0.0))


def test_control_is_dimension_invariant_at_distribution_extremes():
    for concentrated in (False, True):
        out = []
        for n in (4, 64):
            w = [1.0 / n] * n
            if concentrated:
                w = [1.0] + [0.0] * (n - 1)
            out.append(_flat_policy().observe_signal(_signal(w, 0.8, 0.0), 0.0, BandEnergy(1.0, 1.0, 1.0)))
        a, b = out
        assert a.metrics["raw_mean_coherence"] == pytest.approx(0.25) and b.metrics["raw_mean_coherence"] == pytest.approx(1 / 64)
        for k in ("spectral_radius", "spectral_entropy", "spectral_pressure"):
            assert a.metrics[k] == pytest.approx(b.metrics[k], abs=1e-6)
        assert a.lr_scale == pytest.approx(b.lr_scale, abs=1e-6) and a.band_scale == pytest.approx(b.band_scale, abs=1e-6)
        assert a.metrics["control_kind"] == zc.CONTROL_KIND and a.metrics["distribution_channels"] == 4


def test_labels_move_learning_rate_and_bands():
    w = [0.7, 0.1, 0.1, 0.1]
    cascade = SpectralLearningRatePolicy().with_smoothing(1.0).observe_signal(_signal(w, 0.9, 0.0), -1.0, BandEnergy(1, 1, 1))
    drift = SpectralLearningRatePolicy().with_smoothing(1.0).observe_signal(_signal(w, 0.4, 0.0), -1.0, BandEnergy(1, 1, 1))
    assert cascade.metrics["label"] == "cascade_imbalance" and drift.metrics["label"] == "diffuse_drift"
    assert cascade.band_scale[1] > cascade.band_scale[0]                # cascade damps the side bands, lifts Here
    assert drift.band_scale[0] > drift.band_scale[1]                    # dominant channel 0 -> phase gain on Above
    assert 1 / 1.4 <= cascade.lr_multiplier <= 1.4 and 1 / 1.4 <= drift.lr_multiplier <= 1.4
    up = SpectralLearningRatePolicy().with_smoothing(1.0).observe_signal(_signal(w, 0.4, 1.0, dominant=3), -1.0, BandEnergy(1, 1, 1))
    down = SpectralLearningRatePolicy().with_smoothing(1.0).observe_signal(_signal(w, 0.4, -1.0, dominant=3), -1.0, BandEnergy(1, 1, 1))
    assert up.band_scale[0] > down.band_scale[0] and up.band_scale[2] < down.band_scale[2]      # spin tilts above / beneath
    p = SpectralLearningRatePolicy()
    assert p.observe_signal(None, -1.0, BandEnergy(1, 1, 1)) is None
    p.observe_signal(_signal(w, 0.4, 0.0, dominant=0), -1.0, BandEnergy(1, 1, 1))
    assert p.dominant_turnover == 0.0
    p.observe_signal(_signal(w, 0.4, 0.0, dominant=2), -1.0, BandEnergy(1, 1, 1))
    assert p.dominant_turnover == pytest.approx(0.15) and p.last_coherence_label() == "diffuse_drift"


def test_state_round_trip_bounds_and_env():
    p = SpectralLearningRatePolicy().with_lr_bounds(2.0, 3.0).with_band_bounds(1.5, 2.5)
    s = p.state()
    assert s["lr_state"] == 2.0 and s["applied_lr_scale"] == 2.0 and s["band_state"] == [1.5] * 3 and s["local_lr_state"] == [1.5] * 3
    assert SpectralLearningRatePolicy.from_state(s).state() == s
    for patch in ({"max_lr_step": 0.5}, {"local_lr_state": [9.0, 1.5, 1.5]}, {"lr_state": float("nan")}):
        with pytest.raises(ValueError):
            SpectralLearningRatePolicy.from_state({**s, **patch})
    q = SpectralLearningRatePolicy().with_smoothing(-1.0).with_lr_bounds(3.0, 2.0).with_max_lr_step(0.2)
    assert q.smoothing == 0.2 and (q.min_lr_scale, q.max_lr_scale) == (0.1, 6.0) and q.max_lr_step == 1.0
    q.apply_env_overrides({"SPIRAL_SPECTRAL_POLICY_SMOOTHING": "0.5", "SPIRAL_SPECTRAL_POLICY_LR_MIN": "0.5",
                           "SPIRAL_SPECTRAL_POLICY_LR_MAX": "2.0", "SPIRAL_SPECTRAL_POLICY_PHASE_GAIN": "oops"})
    assert q.smoothing == 0.5 and (q.min_lr_scale, q.max_lr_scale) == (0.5, 2.0) and q.phase_gain == 0.25


def test_curvature_decision_is_a_record_readable_by_key():
    d = CurvatureScheduler(-1.0, -2.0, -0.5, 0.5).observe_pressure(1.5)
    assert isinstance(d, CurvatureDecision) and d["changed"] == d.changed and d.as_dict()["curvature"] == d.curvature


def _data():
    torch.manual_seed(0)
    x = torch.randn(8, 16)
    return [(st.Tensor._wrap(x), st.Tensor._wrap(x @ torch.randn(16, 4) * 0.1))]


def test_trainer_consumes_pushed_diagnostics_and_trace_bridge():
    model = st.nn.Sequential()
    model.add(st.nn.Linear("l", 16, 4))
    trainer = st.nn.ModuleTrainer(fallback_learning_rate=1e-2)
    trainer.enable_spectral_learning_rate(SpectralLearningRatePolicy().with_smoothing(1.0))
    sched = trainer.roundtable(8, 4, st.nn.RoundtableConfig(top_k=8, mid_k=8, bottom_k=8))
    try:
        trainer.train_epoch(model, st.nn.MeanSquaredError(), _data(), sched)
        assert trainer.last_spectral_metrics is None and trainer.fallback_learning_rate == 1e-2     # nothing pending yet
        seq = C.ZSpaceCoherenceSequencer(64, 4, -1.0, st.topos.OpenCartesianTopos(-1.0, 1e-5, 10.0, 256, 8192))
        x = st.Tensor._wrap(torch.linspace(0.01, 0.5, 64).reshape(1, 64))
        assert trainer.push_coherence_diagnostics(seq.diagnostics(x))
        trainer.train_epoch(model, st.nn.MeanSquaredError(), _data(), sched)
        m = trainer.last_spectral_metrics
        assert m is not None and m["distribution_channels"] == 8 and m["label"] in zc.LABELS
        lr_after_push = trainer.fallback_learning_rate
        assert lr_after_push != 1e-2 and trainer.pending_coherence is None
        # a sequencer whose trace recorder publishes on the bus feeds the trainer without an explicit push
        seq.install_trace_recorder(C.ZSpaceTraceConfig(publish_plugin_events=True))
        seq.forward(x)
        assert trainer._bridge_latest is not None
        trainer.last_spectral_metrics = None
        trainer.train_epoch(model, st.nn.MeanSquaredError(), _data(), sched)
        assert trainer.last_spectral_metrics is not None and trainer._bridge_latest is None
        # records that do not re-derive are ignored
        st.plugin.publish("ZSpaceTrace", {"record": {"kind": "Aggregated", "payload": {"diagnostics": {"entropy": 0.1}}}})
        assert trainer._bridge_latest is None
    finally:
        trainer.disable_zspace_trace_coherence_bridge()
        trainer.disable_spectral_learning_rate()
    assert trainer.spectral_policy is None
