"""Command-line entry points (CPU)."""
import json

from spiraltorch_b200 import cli


def test_model_zoo_listing_and_dry_run(capsys, tmp_path):
    assert cli.main(["model-zoo", "--list"]) == 0
    out = capsys.readouterr().out
    assert "gpt-1.3b" in out and "conv-classifier" in out and "mlp_regression" in out
    assert cli.main(["model-zoo", "gpt-1.3b", "--gpus", "8", "--dry-run"]) == 0
    cmd = capsys.readouterr().out
    assert "torch.distributed.run" in cmd and "--nproc-per-node=8" in cmd and "bench.py" in cmd and "127.0.0.1" in cmd
    assert cli.main(["model-zoo", "char-lm", "--gpus", "1", "--dry-run"]) == 0
    assert "dp_models.py --model charlm" in capsys.readouterr().out
    assert cli.main(["model-zoo", "nope"]) == 2
    run_dir = tmp_path / "mlp"
    assert cli.main(["model-zoo", "mlp_regression", "--run-dir", str(run_dir)]) == 0
    assert json.loads((run_dir / "run.json").read_text())["schema"] == "st.modelzoo.run.v1"
    keys = set(json.loads((run_dir / "weights.json").read_text())["parameters"]) if "parameters" in \
        json.loads((run_dir / "weights.json").read_text()) else set()
    assert not keys or {"fc1::weight", "head::bias"} <= keys


def test_train_export_plugin_preflight(capsys, tmp_path):
    state = tmp_path / "hpo.json"
    assert cli.main(["train", "--trials", "3", "--steps", "40", "--param", "lr=float:1e-3:1e-1", "--state", str(state)]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(lines) == 4 and "best_trial" in lines[-1] and lines[-1]["final_loss"] == min(l["final_loss"] for l in lines[:3])
    # resuming a finished search runs no new trial
    assert cli.main(["train", "--trials", "3", "--state", str(state)]) == 0
    assert len(capsys.readouterr().out.strip().splitlines()) == 1

    run_dir = tmp_path / "mlp"
    cli.main(["model-zoo", "mlp_regression", "--run-dir", str(run_dir)])
    capsys.readouterr()
    assert cli.main(["export", str(run_dir / "weights.json"), str(tmp_path / "w.bin")]) == 0
    assert "4 tensors" in capsys.readouterr().out and (tmp_path / "w.bin").stat().st_size > 0
    assert cli.main(["export", str(tmp_path / "w.bin"), str(tmp_path / "back.json")]) == 0

    ev = tmp_path / "events.jsonl"
    assert cli.main(["plugin", "--out", str(ev), "--steps", "8", "--events", "EpochEnd,TrainerStep"]) == 0
    kinds = {json.loads(l)["type"] for l in ev.read_text().splitlines()}
    assert kinds == {"EpochEnd", "TrainerStep"}
    capsys.readouterr()
    assert cli.main(["runtime-preflight", "--backend", "cpu"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert "build" in rep and "device" in rep and "native" in rep


def test_z_volume_and_xai_tools(capsys, tmp_path):
    out = tmp_path / "vol.ppm"
    assert cli.main(["z-volume", "--out", str(out), "--size", "16", "--depth", "4", "--backend", "cpu"]) == 0
    info = json.loads(capsys.readouterr().out)
    data = out.read_bytes()
    assert data.startswith(b"P6 16 16 255\n") and len(data) == len(b"P6 16 16 255\n") + 16 * 16 * 3 and info["mean"] > 0
    cam = tmp_path / "cam.ppm"
    assert cli.main(["xai", "--out", str(cam), "--size", "16", "--classes", "4", "--backend", "cpu"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["cam_shape"] == [8, 8] and cam.read_bytes().startswith(b"P6 16 16 255\n")


def test_capability_matrix():
    from benchmarks import capability_matrix as cm
    assert cm.parse_backend("B200") == "cuda" and cm.parse_backend(" CPU ") == "cpu"
    import pytest
    with pytest.raises(ValueError):
        cm.parse_backend("wgpu")
    row = cm.capability_by_name("tensor ops")
    assert row.entry("cuda").state == cm.READY and "tcgen05" in row.entry("cuda").note
    s = cm.summarize_backend("cuda")
    assert s["tracked"] == s["ready"] + s["planned"] + s["stub"] and 0 < s["readiness_ratio"] <= 1
    assert any(r.capability == "Sparse tensor ops" for r in cm.pending_capabilities_for_backend("cuda"))
    assert cm.capabilities_with_note_containing("NVLink")[0].capability == "Distributed collectives"
    md = cm.render_markdown()
    assert md.splitlines()[0].startswith("| Capability | cpu | cuda |") and len(md.splitlines()) == len(cm.MATRIX) + 2
    assert cm.matrix_summary()["capabilities"] == len(cm.MATRIX)


def test_zoo_recipes_learn_and_write_run_dirs(tmp_path):
    import json
    from spiraltorch_b200.models import recipes, zoo
    for name in recipes.RECIPES:
        out = recipes.run(name, tmp_path / name, epochs=4, quiet=True)
        assert out["final_loss"] < out["initial_loss"], name
        run = json.loads((tmp_path / name / "run.json").read_text())
        assert run["schema"] == "st.modelzoo.run.v1" and run["arch"] == name
        assert len(zoo.read_metrics(tmp_path / name)) == 4
        assert (tmp_path / name / "weights.json").exists() and (tmp_path / name / "summary.json").exists()
    from spiraltorch_b200 import cli
    assert cli.main(["model-zoo", "lstm_probe", "--run-dir", str(tmp_path / "cli_run")]) == 0
    import pytest
    with pytest.raises(KeyError):
        recipes.run("nope")
    cmp = zoo.compare_runs([tmp_path / "lstm_probe", tmp_path / "zspace_mixer_regression"])
    assert {r["rank"] for r in cmp["runs"]} == {1, 2} and cmp["runs"][0]["epochs"] == 4
    assert cmp["best_run"] in (str(tmp_path / "lstm_probe"), str(tmp_path / "zspace_mixer_regression"))
    assert cli.main(["compare-runs", str(tmp_path / "lstm_probe"), str(tmp_path / "cli_run")]) == 0
    bundle = recipes.zrba_telemetry(tmp_path / "zrba")
    assert 0.0 <= bundle["metrics"]["picp"] <= 1.0 and bundle["covariance"]["min_eigenvalue"] > 0
    assert json.loads((tmp_path / "zrba" / "zrba_telemetry.json").read_text())["gate"]["mean"] == bundle["gate"]["mean"]
