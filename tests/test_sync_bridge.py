"""Sync-theorem trainer: gate arithmetic, labels, the trajectory form and family aggregation
(crates/st-core/src/theory/sync_bridge.rs)."""
import math

import pytest
import torch

from spiraltorch_b200 import sync_bridge as B


def test_config_validation_and_bounds():
    cfg = B.SyncConfig(0.05, 0.2, 0.05, 0.8)
    assert cfg.threshold() == pytest.approx(math.log(20.0))
    assert cfg.hitting_time_bound() == pytest.approx(math.log(20.0) / (2 * 0.2 * 0.8 - 0.05))
    assert cfg.hitting_time_tail(1.0) is None and cfg.with_azuma_c(0.5).hitting_time_tail(2.0) == pytest.approx(math.exp(-2.0))
    assert cfg.hitting_time_tail(-1.0) == 1.0
    for bad in [(1.0, 0.2, 0.0, 0.5), (0.1, 0.0, 0.0, 0.5), (0.1, 0.2, -1.0, 0.5), (0.1, 0.2, 0.0, 0.0), (0.1, 0.2, 0.0, 1.5)]:
        with pytest.raises(B.SyncError):
            B.SyncConfig(*bad)
    with pytest.raises(B.SyncError):
        B.SyncConfig(0.05, 0.1, 0.5, 0.5).hitting_time_bound()
    with pytest.raises(B.SyncError):
        cfg.with_azuma_c(0.0)


def test_steps_accumulate_and_label():
    tr = B.SyncTheoremTrainer(B.SyncConfig(0.05, 0.2, 0.05, 0.8, slew_steps=1))
    d = torch.tensor([0.5, 0.1, 2.5])
    s1 = tr.step(d)
    assert torch.allclose(s1.increment, 2 * 0.8 * d - 0.05) and torch.allclose(s1.effective_delta_b_sq, 0.8 * d)
    assert not bool(s1.structure_gate.any())                                # the slew lag holds the structure gate shut
    assert s1.observation_gate.tolist() == [False, False, True]             # 3.95 >= ln 20
    assert s1.label_names() == ["abstain", "abstain", "abstain"]
    s2 = tr.step(d, epsilon=[0.0, 0.5, 0.0], cos_sq_phi=[1.0, 1.0, 1.0])
    assert torch.allclose(s2.log_e, s1.log_e + torch.tensor([1.0, -0.3, 5.0]))
    assert s2.structure_gate.tolist() == [True, False, True] and s2.label_names() == ["abstain", "abstain", "critical"]
    assert torch.allclose(s2.confidence, 1.0 - torch.exp(-s2.log_e)) and tr.iteration == 2
    # both gates shut: the confidence 1 - exp(-log e) stays below 1 - alpha exactly while log e is below ln(1 / alpha),
    # so the sample abstains
    tr2 = B.SyncTheoremTrainer(B.SyncConfig(0.6, 5.0, 0.0, 1.0))
    tr2.set_log_e([0.45])
    s = tr2.step([0.01])
    assert s.label_names() == ["abstain"] and float(s.log_e[0]) == pytest.approx(0.47) and float(s.log_e[0]) < tr2.threshold()
    with pytest.raises(B.SyncError):
        tr.step(d, epsilon=[0.0, 0.0])
    empty = tr.step([])
    assert empty.log_e.numel() == 0 and empty.hitting_time_bound > 0.0


def test_run_matches_repeated_steps():
    cfg = B.SyncConfig(0.05, 0.2, 0.05, 0.8)
    d = torch.tensor([0.3, 0.4, 0.9, 1.4, 0.2, 2.0])
    eps = torch.tensor([0.05, 0.0, 0.1, 0.05, 0.3, 0.0])
    traj, hit = B.SyncTheoremTrainer(cfg).run(d, eps)
    tr = B.SyncTheoremTrainer(cfg)
    ref, first = [], None
    for i in range(d.numel()):
        s = tr.step(d[i:i + 1], eps[i:i + 1])
        ref.append(float(s.log_e[0]))
        if first is None and bool(s.observation_gate[0]):
            first = i
    assert torch.allclose(traj, torch.tensor(ref), atol=1e-6) and hit == first and hit is not None
    assert B.SyncTheoremTrainer(cfg).run([0.01, 0.01])[1] is None
    assert hit <= math.ceil(cfg.hitting_time_bound() * 4)


def test_family_aggregation_policies():
    tr = B.SyncTheoremTrainer(B.SyncConfig(0.05, 0.2, 0.05, 0.8))
    step = tr.step(torch.tensor([3.0, 0.1, 2.5]), cos_sq_phi=[1.0, 1.0, 1.0])
    any_, all_, maj = (tr.aggregate_family(step, p) for p in B.FAMILY_POLICIES)
    assert any_.structure_gate and not all_.structure_gate and maj.structure_gate
    assert any_.log_e_family == pytest.approx(float(step.log_e.mean())) and any_.pair_count == 3
    assert any_.dominant_pair == 0 and any_.dominant_log_e == pytest.approx(5.95)
    assert any_.observation_gate and any_.label == "critical" and all_.label == "abstain"
    with pytest.raises(B.SyncError):
        tr.aggregate_family(tr.step([]), "any")
    with pytest.raises(B.SyncError):
        tr.aggregate_family(step, "plurality")
