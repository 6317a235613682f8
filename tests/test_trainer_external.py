"""External trainer state checkpoint (reference behaviour: crates/st-core/src/runtime/trainer_external.rs)."""
import json

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200.desire_pipeline import DesirePipeline, DesireTrainerBridge
from spiraltorch_b200.psi import PsiConfig, PsiMeter
from spiraltorch_b200.runtime.trainer_external import (TrainerExternalCheckpointComponents,
                                                       TrainerExternalCheckpointError,
                                                       TrainerExternalStateCheckpoint)
from tests.test_desire_pipeline import LOGITS, _automation


def _trainer_with_state():
    tr = st.SpiralSession("cpu", seed=0).trainer()
    tr.enable_psi(PsiMeter(PsiConfig(enabled=True)))
    bridge = DesireTrainerBridge()
    tr.attach_desire_bridge(bridge)
    pipe = DesirePipeline.builder(_automation()).with_trainer_bridge(bridge).build()
    for i in range(5):
        pipe.step_at(LOGITS, 0, [0.5, 0.5], now=float(i), timestamp=100.0 + i)
    model = st.nn.Sequential()
    model.add(st.nn.Linear(3, 2, name="fc"))
    x, y = st.Tensor(torch.randn(4, 3)), st.Tensor(torch.randn(4, 2))
    tr.train_epoch(model, st.nn.MeanSquaredError(), [(x, y), (x, y)])
    return tr, bridge


def test_capture_validate_round_trip_and_restore():
    tr, bridge = _trainer_with_state()
    ckpt = tr.external_state_checkpoint()
    v = ckpt.validate()
    assert v.required_components == ["psi_meter", "desire_trainer"] and v.captured_components == ["desire_trainer", "psi_meter"]
    assert v.payload_complete and v.deterministic_resume_ready and not v.unresolved_components
    doc = json.loads(json.dumps(ckpt.to_json()))
    again = TrainerExternalStateCheckpoint.from_json(doc)
    assert again.to_json() == ckpt.to_json()
    fresh = st.SpiralSession("cpu", seed=0).trainer()
    fresh.enable_psi(PsiMeter(PsiConfig(enabled=True)))
    fresh_bridge = DesireTrainerBridge()
    fresh.attach_desire_bridge(fresh_bridge)
    fresh.restore_external_state(again)
    assert fresh.psi_meter.step == tr.psi_meter.step == 2 and fresh.psi_meter.ema == tr.psi_meter.ema
    assert len(fresh_bridge) == len(bridge) == 5


def test_unresolved_and_invalid_documents():
    ckpt = TrainerExternalCheckpointComponents().require("psi_meter", "accumulator_synchronizer") \
        .with_psi_meter(PsiMeter(PsiConfig(enabled=True)).checkpoint()).build()
    v = ckpt.validate()
    assert v.unresolved_components == ["accumulator_synchronizer"] and not v.payload_complete and not v.deterministic_resume_ready
    doc = ckpt.to_json()
    for mutate, kind, fld in (
            (lambda d: d.__setitem__("kind", "other"), "InvalidMetadata", "kind"),
            (lambda d: d.__setitem__("extra", 1), "InvalidState", "extra"),
            (lambda d: d.__setitem__("required_components", ["psi_meter", "psi_meter"]), "InvalidState", "required_components"),
            (lambda d: d.__setitem__("unresolved_components", []), "InvalidState", "required_components"),
            (lambda d: d["psi_meter"].__setitem__("ema_alpha", 1.5), "InvalidState", "psi_meter.ema_alpha")):
        bad = json.loads(json.dumps(doc))
        mutate(bad)
        with pytest.raises(TrainerExternalCheckpointError) as e:
            TrainerExternalStateCheckpoint.from_json(bad)
        assert (e.value.kind, e.value.field) == (kind, fld)


def test_desire_queue_rules():
    tr, _ = _trainer_with_state()
    doc = tr.external_state_checkpoint().to_json()
    events = doc["desire_trainer"]
    trig = next(e for e in events if e["trigger"] is not None)["trigger"]
    for mutate, fld in ((lambda: events[0].__setitem__("temperature", 0.0), "desire_trainer.events[0].temperature"),
                        (lambda: events[1].__setitem__("entropy", -1.0), "desire_trainer.events[1].entropy"),
                        (lambda: events[2]["weights"].__setitem__("lam", float("nan")), "desire_trainer.events[2].weights.lam"),
                        (lambda: trig.__setitem__("samples", 0), None),
                        (lambda: trig["report"].__setitem__("tokens", [1, 1]) or trig["report"].__setitem__("scores", [0.1, 0.2]), None)):
        saved = json.dumps(doc)
        mutate()
        with pytest.raises(TrainerExternalCheckpointError) as e:
            TrainerExternalStateCheckpoint.from_json(json.loads(json.dumps(doc)))
        if fld:
            assert e.value.field == fld
        doc = json.loads(saved)
        events = doc["desire_trainer"]
        trig = next(e for e in events if e["trigger"] is not None)["trigger"]
