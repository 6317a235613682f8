"""Study drivers of the HF bridge (bindings/st-py/spiraltorch/hf_optimizer_study.py, hf_peft.py, hf_optimizer_control.py):
plans, the chained event log, resume / quarantine, the summary, LoRA injection and the loss-feedback gate."""
import json
import math

import pytest
import torch

from spiraltorch_b200 import hf_study as H


def fake_runner(calls, fail=()):
    def run(config, out_dir):
        calls.append((config["arm"], config["seed"]))
        if (config["arm"], config["seed"]) in fail:
            raise RuntimeError("boom")
        (out_dir / "artifact.bin").write_bytes(b"x")
        offset = {"observe": 0.0, "raw_unguarded": -0.1, "raw_loss_guard": -0.2}[config["arm"]]
        return {"eval_loss_before": 3.0, "eval_loss_after": 2.0 + offset + 0.01 * config["seed"], "steps_per_second": 10.0}
    return run


def test_plan_identity_and_persistence(tmp_path):
    plan = H.build_study_plan(tmp_path / "s", seeds=[2, 0, 2], base_config={"steps": 5})
    assert [r["label"] for r in plan["runs"]][:4] == ["seed-0000-observe", "seed-0000-raw_unguarded", "seed-0000-raw_loss_guard", "seed-0002-observe"]
    assert plan["study_id"] == H.build_study_plan(tmp_path / "elsewhere", seeds=[0, 2], base_config={"steps": 5})["study_id"]   # content, not place
    assert plan["study_id"] != H.build_study_plan(tmp_path / "s", seeds=[0, 2], base_config={"steps": 6})["study_id"]
    assert len({r["run_id"] for r in plan["runs"]}) == 6
    with pytest.raises(H.StudyError):
        H.build_study_plan(tmp_path / "s", base_config={"seed": 1})
    with pytest.raises(H.StudyError):
        H.build_study_plan(tmp_path / "s", arms=["a", "a"])
    with pytest.raises(H.StudyError):
        H.build_study_plan(tmp_path / "s", arm_configs={"other": {}})
    path = H.persist_plan(plan)
    assert H.persist_plan(plan) == path                                            # same study: accepted
    with pytest.raises(H.StudyError, match="different study"):
        H.persist_plan(H.build_study_plan(tmp_path / "s", seeds=[0, 2], base_config={"steps": 6}))


def test_event_log_chain_detects_edits(tmp_path):
    log = H.EventLog(tmp_path / "e.jsonl", "sid")
    first = log.append("study_started", runs=2)
    second = log.append("run_started", run_label="a")
    assert first["previous_event_id"] is None and second["previous_event_id"] == first["event_id"] and second["sequence"] == 1
    with pytest.raises(H.StudyError, match="reserved"):
        log.append("x", sequence=9)
    assert len(H.EventLog(tmp_path / "e.jsonl", "sid").events) == 2
    with pytest.raises(H.StudyError, match="another study"):
        H.EventLog(tmp_path / "e.jsonl", "other")
    lines = (tmp_path / "e.jsonl").read_text().splitlines()
    (tmp_path / "e.jsonl").write_text(lines[0].replace('"runs": 2', '"runs": 3') + "\n" + lines[1] + "\n")
    with pytest.raises(H.StudyError, match="chain broken"):
        H.EventLog(tmp_path / "e.jsonl", "sid")
    (tmp_path / "e.jsonl").write_text(lines[1] + "\n")                              # first event dropped
    with pytest.raises(H.StudyError, match="chain broken"):
        H.EventLog(tmp_path / "e.jsonl", "sid")


def test_run_study_resumes_quarantines_and_summarises(tmp_path):
    plan = H.build_study_plan(tmp_path / "s", seeds=[0, 1])
    calls = []
    partial = H.run_study(plan, fake_runner(calls), max_runs=2)
    assert len(calls) == 2 and len(partial["pending_runs"]) == 4
    # second pass: one run fails, the rest complete; completed runs are not executed again
    summary = H.run_study(plan, fake_runner(calls, fail={("raw_unguarded", 1)}))
    assert len(calls) == 6 and summary["pending_runs"] == ["seed-0001-raw_unguarded"] == summary["failed_runs"]
    assert (tmp_path / "s" / "quarantine").is_dir() and not (tmp_path / "s" / "runs" / "seed-0001-raw_unguarded").exists()
    # third pass: the failed run is retried and the study completes
    summary = H.run_study(plan, fake_runner(calls))
    assert len(calls) == 7 and summary["pending_runs"] == [] and summary["failed_runs"] == []
    arms = summary["arms"]
    assert arms["observe"]["eval_loss_after"]["mean"] == pytest.approx(2.005) and arms["observe"]["wins_vs_reference"] is None
    assert arms["raw_loss_guard"]["paired_delta_vs_reference"]["mean"] == pytest.approx(-0.2) and arms["raw_loss_guard"]["wins_vs_reference"] == 2
    assert arms["raw_unguarded"]["improvement"]["mean"] == pytest.approx(1.095)
    assert arms["observe"]["eval_loss_after"]["std"] == pytest.approx(0.01 / math.sqrt(2))
    kinds = [e["event_type"] for e in H.EventLog(tmp_path / "s" / H.EVENTS_FILENAME, plan["study_id"]).events]
    assert kinds[0] == "study_started" and kinds[-1] == "study_completed" and kinds.count("run_completed") == 6 and kinds.count("run_failed") == 1
    # a run card edited after the fact is not trusted: the run is moved aside and executed again
    card_path = tmp_path / "s" / "runs" / "seed-0000-observe" / "run-card.json"
    card = json.loads(card_path.read_text())
    card["eval_loss_after"] = 0.1
    card_path.write_text(json.dumps(card))
    H.run_study(plan, fake_runner(calls))
    assert calls[-1] == ("observe", 0) and len(calls) == 8
    assert json.loads(card_path.read_text())["eval_loss_after"] == pytest.approx(2.0)


def test_study_lock_is_exclusive_and_reclaims_dead_owners(tmp_path):
    with H.study_lock(tmp_path, "sid"):
        with pytest.raises(H.StudyError, match="being driven"):
            with H.study_lock(tmp_path, "sid"):
                pass
    assert not (tmp_path / H.LOCK_FILENAME).exists()
    (tmp_path / H.LOCK_FILENAME).write_text(json.dumps({"pid": 2 ** 22 + 12345, "study_id": "sid"}))    # no such process
    with H.study_lock(tmp_path, "sid"):
        assert json.loads((tmp_path / H.LOCK_FILENAME).read_text())["pid"] != 2 ** 22 + 12345


def test_inject_lora_freezes_the_base_and_starts_as_identity():
    torch.manual_seed(0)
    model = H.ByteCausalLM(d_model=32, n_layer=1, n_head=2, max_len=16)
    ids = torch.randint(0, 256, (2, 16))
    ref = model(ids)
    wrapped = H.inject_lora(model, ["attn.qkv", "mlp.out"], rank=2, alpha=4.0)
    assert wrapped == ["blocks.0.attn.qkv", "blocks.0.mlp.out"]
    assert torch.allclose(model(ids), ref, atol=1e-6)                                # B = 0: the wrapped model is the base model
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all(n.endswith(("lora_a", "lora_b")) for n in trainable)
    layer = model.blocks[0].attn.qkv
    with torch.no_grad():
        layer.lora_b.normal_()
    x = torch.randn(3, 32)
    dense = x @ (layer.base.weight.t() + layer.merged_delta()) + layer.base.bias
    assert torch.allclose(layer(x), dense, atol=1e-5)
    assert set(H.lora_state(model)) == {f"blocks.0.{m}.lora_{s}" for m in ("attn.qkv", "mlp.out") for s in "ab"}
    with pytest.raises(H.StudyError):
        H.inject_lora(H.ByteCausalLM(d_model=32, n_layer=1, n_head=2), ["nothing"], rank=2)


def test_loss_feedback_gate_attenuates_halts_and_recovers():
    g = H.LossFeedbackGate(warmup_observations=1, guard=True)
    for loss in (2.0, 1.9, 1.8, 1.7):
        g.observe(loss)
    assert g.value() == 1.0 and not g.halted                                         # improving: the gate stays open
    values = [g.observe(loss) for loss in (2.6, 3.4, 4.4)]
    assert values[0] < 1.0 and g.halted and g.value() == 0.0 and g.halts == 1         # regressions in a row beyond the halt threshold
    unguarded = H.LossFeedbackGate(warmup_observations=1)
    for loss in (2.0, 1.9, 1.8, 1.7, 2.6, 3.4, 4.4):
        unguarded.observe(loss)
    assert 0.0 < unguarded.value() < 1.0 and not unguarded.halted                    # same losses, no guard: attenuated, never closed
    for loss in (3.0, 2.2, 1.8, 1.5, 1.3):
        g.observe(loss)
    assert not g.halted and g.value() > 0.0                                          # improvements in a row reopen it
    assert H.LossFeedbackGate(guard=True).observe(float("nan")) == 0.0
    assert H.gate_for_arm("observe").applied is False and H.gate_for_arm("raw_loss_guard").guard and H.gate_for_arm("adamw") is None


def test_lora_finetune_run_learns_and_the_observe_arm_never_touches_the_rate(tmp_path):
    cfg = {"steps": 30, "pretrain_steps": 20, "batch_size": 8, "seq_len": 32, "model": {"d_model": 32, "n_layer": 1, "n_head": 2}, "lr": 1e-2}
    out = H.lora_finetune_run({**cfg, "arm": "observe", "seed": 0}, tmp_path / "a")
    assert out["eval_loss_after"] < out["eval_loss_before"] and out["skipped_steps"] == 0 and out["steps_per_second"] > 0
    assert (tmp_path / "a" / "adapter.pt").exists()
    trace = [json.loads(line) for line in (tmp_path / "a" / "trainer-trace.jsonl").read_text().splitlines()]
    assert len(trace) == 30 and all(r["applied"] == 1.0 for r in trace)
    again = H.lora_finetune_run({**cfg, "arm": "observe", "seed": 0}, tmp_path / "b")
    assert again["eval_loss_after"] == pytest.approx(out["eval_loss_after"], rel=1e-5)            # a run is a function of its config
    # an over-eager guard (every rise of the loss counts) skips steps; the unguarded arm with the same gate does not
    fb = {"regression_threshold": 0.0, "halt_threshold": 0.0, "halt_regression_streak": 1, "warmup_observations": 1, "relative_delta_ema_alpha": 1.0}
    guarded = H.lora_finetune_run({**cfg, "arm": "raw_loss_guard", "seed": 0, "feedback": fb}, tmp_path / "c")
    raw = H.lora_finetune_run({**cfg, "arm": "raw_unguarded", "seed": 0, "feedback": fb}, tmp_path / "d")
    assert guarded["gate_halts"] >= 1 and guarded["skipped_steps"] >= 1 and raw["skipped_steps"] == 0


def test_cli_plans_and_runs_a_small_study(tmp_path, capsys):
    assert H.main([str(tmp_path / "s"), "--seeds", "0", "--arms", "observe", "raw_loss_guard", "--plan-only"]) == 0
    assert json.loads(capsys.readouterr().out)["runs"] == ["seed-0000-observe", "seed-0000-raw_loss_guard"]
    # the same directory with other settings is another study: refused, not overwritten
    with pytest.raises(H.StudyError, match="different study"):
        H.main([str(tmp_path / "s"), "--seeds", "0", "--arms", "observe", "raw_loss_guard", "--steps", "4"])
    assert H.main([str(tmp_path / "t"), "--seeds", "0", "--arms", "observe", "raw_loss_guard", "--steps", "4", "--pretrain-steps", "0"]) == 0
    summary = json.loads(capsys.readouterr().out)
    assert summary["pending_runs"] == [] and summary["arms"]["raw_loss_guard"]["eval_loss_after"]["n"] == 1
    assert (tmp_path / "t" / "runs" / "seed-0000-observe" / "adapter.pt").exists()
