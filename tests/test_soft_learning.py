"""Learned rank-k ranker and the A/B log (crates/st-core/src/heur/soft_learning.rs, ability/ablog.rs)."""
import json
import math

import pytest

from spiraltorch_b200 import soft_learning as L
from spiraltorch_b200.unison import RankChoice


def _choice(**kw):
    from types import SimpleNamespace
    base = dict(use_2ce=False, wg=256, kl=8, ch=0, mk=1, mkd=2, tile=1024, ctile=512)
    base.update(kw)
    return SimpleNamespace(**base)


def test_features_and_bonus():
    ctx = L.SoftContext(1024, 65536, 128, "cuda", True)
    f = dict(ctx.features(_choice(use_2ce=True)))
    assert f["rows_ln"] == pytest.approx(math.log1p(1024)) and f["wg_ratio"] == 0.5 and f["kl_ratio"] == 0.25 and f["two_stage"] == 1.0
    assert f["backend_cuda"] == 1.0 and "backend_cpu" not in f and f["tile_ratio"] == 0.25 and f["mkd_kind"] == pytest.approx(0.4)
    learner = L.SoftRuleLearner({"two_stage": 2.0, "wg_ratio": -1.0}, bias=0.1, temperature=2.0)
    assert learner.learned_bonus(ctx, _choice(use_2ce=True)) == pytest.approx(math.tanh((0.1 + 2.0 - 0.5) / 2.0))
    with pytest.raises(ValueError):
        L.SoftContext(1, 1, 1, "tpu").features(_choice())
    plain = dict(ctx.features(RankChoice(True, 128, 16, 2048, 256)))          # the narrower choice record of the rank planner
    assert plain["mk_kind"] == 0.0 and plain["ch_norm"] == 0.0 and plain["kl_ratio"] == 0.5


def test_rank_respects_beam_and_non_finite_scores():
    ctx = L.SoftContext(64, 4096, 8)
    learner = L.SoftRuleLearner({"two_stage": 3.0}, beam=2)
    cands = [("a", _choice(), 0.5), ("b", _choice(use_2ce=True), 0.0), ("c", _choice(), float("nan"))]
    best, scores = learner.rank(ctx, cands)
    assert best == 1 and scores[2] == -math.inf and scores[1] == pytest.approx(math.tanh(3.0))
    assert L.SoftRuleLearner().rank(ctx, []) == (0, [])


def test_store_loading_and_validation(tmp_path, monkeypatch):
    p = tmp_path / "ranker.json"
    p.write_text(json.dumps({"weights": {"k_ln": 0.5}, "bias": -0.2, "temperature": 0.5, "beam": 3}))
    learner = L.SoftRuleLearner.try_load_from(p)
    assert learner.weights == {"k_ln": 0.5} and learner.beam == 3 and learner.temperature == 0.5
    assert L.SoftRuleLearner.try_load_from(tmp_path / "missing.json") is None
    monkeypatch.setenv(L.SOFT_RANKER_PATH_ENV, str(p))
    assert L.SoftRuleLearner.try_load().bias == -0.2
    for bad in ({"other": 1}, {"weights": {"": 1.0}}, {"weights": {"x": float("inf")}}, {"weights": {}, "temperature": 0.0},
                {"weights": {}, "beam": 0}, [1, 2]):
        p.write_text(json.dumps(bad).replace("Infinity", "1e999"))
        with pytest.raises(L.SoftRankerStoreError):
            L.SoftRuleLearner.try_load_from(p)
    assert L.SoftRuleLearner.maybe_load() is None                     # a broken store is reported and ignored


def test_ablog_appends_json_lines(tmp_path, monkeypatch):
    monkeypatch.setenv("SPIRAL_ABLOG_PATH", str(tmp_path / "logs" / "ab.jsonl"))
    L.record(L.ABEntry(128, 4096, 16, "cuda", "A", 1, 2, 1024, 512, 0.25, True))
    L.record(L.ABEntry(128, 4096, 16, "cuda", "B", 1, 2, 1024, 512, 0.31, False, ts_ms=7))
    rows = [json.loads(line) for line in (tmp_path / "logs" / "ab.jsonl").read_text().splitlines()]
    assert [r["variant"] for r in rows] == ["A", "B"] and rows[0]["ts_ms"] > 0 and rows[1]["ts_ms"] == 7 and rows[1]["ok"] is False
    assert L.wilson_lower(8, 10, 1.96) == pytest.approx(0.49, abs=0.01)
