"""ψ meter (reference behaviour: crates/st-core/src/telemetry/psi.rs:500-690 and its tests)."""
import pytest
import torch

import spiraltorch as st
from spiraltorch_b200 import plugin
from spiraltorch_b200.psi import (PsiAutomationHint, PsiComponent, PsiConfig, PsiInput, PsiMeter, PsiSpiralTuning)


def test_component_tokens():
    assert PsiComponent.parse_list("loss, grad|attention;band curv") == (
        PsiComponent.LOSS | PsiComponent.GRAD_NORM | PsiComponent.ATTN_ENTROPY | PsiComponent.BAND_ENERGY
        | PsiComponent.POSITIVE_CURVATURE)
    with pytest.raises(ValueError):
        PsiComponent.from_token("nope")
    assert PsiComponent.defaults() & PsiComponent.ACT_DRIFT and not PsiComponent.defaults() & PsiComponent.BAND_ENERGY


def test_defaults_filled_in_and_ema():
    m = PsiMeter(PsiConfig(enabled=True))
    cfg = m.config()
    assert cfg.ema_alpha == 0.2 and cfg.sample_rate == 1 and cfg.weights[PsiComponent.POSITIVE_CURVATURE] == 0.25
    r1, _ = m.update(PsiInput(loss=2.0, grad_l2=1.0))
    assert abs(r1.breakdown[PsiComponent.LOSS] - 2.0) < 1e-9            # the first sample seeds the EMA
    assert abs(r1.total - (1.0 * 2.0 + 0.3 * 1.0)) < 1e-9
    r2, _ = m.update(PsiInput(loss=1.0, grad_l2=1.0))
    assert abs(r2.breakdown[PsiComponent.LOSS] - (0.2 * 1.0 + 0.8 * 2.0)) < 1e-9 and r2.step == 2


def test_threshold_events_and_sampling():
    cfg = PsiConfig(True, PsiComponent.LOSS, {PsiComponent.LOSS: 1.0}, 0.5, 2, {PsiComponent.LOSS: 1.5})
    m = PsiMeter(cfg)
    r, ev = m.update(PsiInput(loss=1.0))               # step 1 is not sampled
    assert r.total == 0.0 and not ev and not r.breakdown
    r, ev = m.update(PsiInput(loss=1.0))               # step 2: EMA = 1.0
    assert not ev
    m.update(PsiInput(loss=9.0))
    r, ev = m.update(PsiInput(loss=9.0))               # step 4: EMA = 5.0 crosses upwards
    assert len(ev) == 1 and ev[0].up and str(ev[0]).startswith("psi.threshold:LOSS:up:5.000:1.500@4")
    m.update(PsiInput(loss=0.0))
    r, ev = m.update(PsiInput(loss=0.0))               # 2.5, still above
    assert not ev
    m.update(PsiInput(loss=0.0))
    r, ev = m.update(PsiInput(loss=0.0))               # 1.25 crosses downwards
    assert len(ev) == 1 and not ev[0].up


def test_automated_config_and_tuning():
    cfg = PsiConfig.automated(PsiAutomationHint(above=8, here=8, beneath=16, band_focus=6.0, drift_weight=0.05))
    assert cfg.enabled and cfg.ema_alpha == 0.22 and cfg.sample_rate == 1
    assert cfg.weights[PsiComponent.ACT_DRIFT] == 0.1 and abs(cfg.weights[PsiComponent.BAND_ENERGY] - 6.0 / 32) < 1e-9
    assert cfg.weights[PsiComponent.POSITIVE_CURVATURE] == 0.5
    cfg.apply_spiral_tuning(PsiSpiralTuning(PsiComponent.ATTN_ENTROPY, {PsiComponent.LOSS: 20.0},
                                            {PsiComponent.LOSS: 0.5}, 0.4))
    assert cfg.components & PsiComponent.ATTN_ENTROPY and cfg.weights[PsiComponent.LOSS] == 10.0
    assert cfg.thresholds[PsiComponent.LOSS] == 0.5 and cfg.sample_rate == 2


def test_checkpoint_round_trip():
    m = PsiMeter(PsiConfig(True, PsiComponent.LOSS | PsiComponent.GRAD_NORM, {PsiComponent.LOSS: 1.0}, 0.3, 1,
                           {PsiComponent.LOSS: 2.0}))
    for v in (3.0, 1.0, 4.0):
        m.update(PsiInput(loss=v, grad_l2=v / 2))
    doc = m.checkpoint()
    again = PsiMeter.from_checkpoint(doc)
    a, _ = m.update(PsiInput(loss=1.5, grad_l2=0.1))
    b, _ = again.update(PsiInput(loss=1.5, grad_l2=0.1))
    assert a.total == b.total and a.step == b.step == 4 and a.breakdown == b.breakdown
    with pytest.raises(ValueError):
        PsiMeter.from_checkpoint({"kind": "other"})


def test_trainer_feeds_the_meter():
    seen = []
    sid = plugin.subscribe("PsiReading", seen.append)
    try:
        model = st.nn.Sequential()
        model.add(st.nn.Linear(4, 2, name="fc"))
        tr = st.SpiralSession("cpu", seed=0).trainer()
        tr.enable_psi(PsiMeter(PsiConfig(enabled=True)))
        x, y = st.Tensor(torch.randn(5, 4)), st.Tensor(torch.randn(5, 2))
        tr.train_epoch(model, st.nn.MeanSquaredError(), [(x, y), (x, y), (x, y)])
    finally:
        plugin.unsubscribe("PsiReading", sid)
    assert len(seen) == 3 and tr.last_psi.step == 3 and tr.last_psi.total > 0
    assert seen[0]["breakdown"]["grad_norm"] > 0
