"""Three-voice rank chooser: fallback from the device record, SpiralK environment program, key/value record and the
generated table; refinement, scoring and selection (structure of crates/st-core/src/backend/unison_heuristics.rs)."""
import pytest
import torch

from spiraltorch_b200 import kv, unison
from spiraltorch_b200.device_caps import DeviceCaps
from spiraltorch_b200.logic import Choice
from spiraltorch_b200.ops import rank


@pytest.fixture(autouse=True)
def _clean_env(monkeypatch):
    for k in ("SPIRAL_HEUR_K", "SPIRAL_HEUR_KV_URL", "SPIRAL_HEUR_KV_KEY"):
        monkeypatch.delenv(k, raising=False)


def test_fallback_refine_and_score():
    caps = DeviceCaps.cuda()
    base = unison.fallback(64, 4096, 48, caps, "midk")
    assert base.wg == caps.recommended_workgroup(64) and base.kl == 16 and base.tile == caps.recommended_tiles(4096)[0] and not base.use_2ce
    assert unison.fallback(64, 65536, 8, caps).use_2ce                                   # column-heavy rows split
    bottom = unison.fallback(64, 4096, 8, caps, "bottomk")
    assert 128 <= bottom.ctile <= bottom.tile // 2
    wild = unison.RankChoice(True, 1000, 12, 5000, 0)
    r = unison.refine(wild, base, caps, 4096)
    assert r.wg % 32 == 0 and r.wg <= 1024 and r.kl in (8, 16) and r.tile == 4096 and r.ctile == base.ctile and r.use_2ce
    assert unison.refine(unison.RankChoice(False, 0, 0, 0, 0), base, caps, 4096) == base                 # zero fields inherit
    assert unison.closeness(256, 256) == 1.0 and unison.closeness(128, 256) == 0.5 and unison.closeness(0, 256) == 0.0
    s_base = unison.score(base, base, caps, 64, 4096, 48, "midk")
    assert s_base > unison.score(r, base, caps, 64, 4096, 48, "midk")                     # the wrong strategy loses 0.35
    with pytest.raises(ValueError):
        unison.choose_unified_rank(4, 8, 9, caps)
    with pytest.raises(ValueError):
        unison.choose_unified_rank(4, 8, 2, caps, "sideways")


def test_voices_compete_and_the_best_score_wins(monkeypatch):
    caps = DeviceCaps.cuda()
    rep = unison.choose_unified_rank(512, 8192, 8, caps, table=[])
    assert rep.source == "fallback" and rep.choice == rep.baseline and set(rep.scores) == {"fallback"}
    # a tuned entry that measured the two-stage path 40 % faster than the direct kernel outranks the shape heuristics
    b = rep.baseline
    table = [{"kind": "topk", "rows": 512, "cols": 8192, "k": 8, "use_2ce": True, "wg": b.wg, "kl": b.kl, "tile": 512, "ctile": 0, "ms": 0.06, "direct_ms": 0.1},
             {"kind": "bottomk", "rows": 512, "cols": 8192, "k": 8, "use_2ce": False, "wg": 64, "kl": 8, "tile": 256, "ctile": 128}]
    rep2 = unison.choose_unified_rank(512, 8192, 8, caps, table=table)
    assert rep2.source == "generated" and rep2.choice.use_2ce and rep2.choice.tile == 512 and rep2.scores["fallback"] == rep.scores["fallback"]
    slower = [dict(table[0], ms=0.12)]                                                     # a measurement that lost stays unused
    assert unison.choose_unified_rank(512, 8192, 8, caps, table=slower).source == "fallback"
    far = unison.choose_unified_rank(4, 64, 2, caps, table=table)
    assert "generated" not in far.scores                                                 # more than three octaves away
    # the environment program: a hard assignment that contradicts the expected strategy is heard but loses
    monkeypatch.setenv("SPIRAL_HEUR_K", "u2: 1; wg: 512;")
    rep3 = unison.choose_unified_rank(512, 8192, 8, caps, table=[])
    assert "kdsl_env" in rep3.scores and rep3.source == "fallback"
    monkeypatch.setenv("SPIRAL_HEUR_K", "wg: 1024;")
    rep4 = unison.choose_unified_rank(512, 8192, 8, caps, table=[])
    wg_trade = 0.2 * (caps.occupancy_score(1024) - caps.occupancy_score(b.wg)) - 0.2      # fuller block, but far from the baseline
    assert rep4.scores["kdsl_env"] == pytest.approx(rep4.scores["fallback"] + wg_trade) and rep4.source == "fallback"
    monkeypatch.setenv("SPIRAL_HEUR_K", "this is not a program {{{")
    assert unison.choose_unified_rank(512, 8192, 8, caps, table=[]).source == "fallback"


def test_kv_voice_reads_a_shared_choice(monkeypatch):
    caps = DeviceCaps.cuda()
    with kv.MiniRespServer() as srv:
        monkeypatch.setenv("SPIRAL_HEUR_KV_URL", srv.url)
        assert "kdsl_kv" not in unison.choose_unified_rank(512, 8192, 8, caps, table=[]).scores      # nothing stored yet
        with kv.connect(srv.url) as c:
            c.set_choice(unison.kv_key(512, 8192, 8, "topk"), Choice(use_2ce=False, wg=1024, kl=8, tile_cols=8192))
        rep = unison.choose_unified_rank(500, 8000, 7, caps, table=[])                                 # same power-of-two bucket
        assert "kdsl_kv" in rep.scores and rep.scores["kdsl_kv"] < rep.scores["fallback"] and rep.source == "fallback"
    monkeypatch.setenv("SPIRAL_HEUR_KV_URL", "redis://127.0.0.1:1/0")                                  # a store that is down is ignored
    assert unison.choose_unified_rank(512, 8192, 8, caps, table=[]).source == "fallback"
    assert unison.load_table(unison.TABLE_PATH.parent / "absent.json") == []


def test_rank_select_accepts_a_choice_on_cpu():
    x = torch.randn(4, 64)
    v, i = rank.rank_select(x, 3, "topk", choice=unison.RankChoice(True, 64, 8, 16, 16))
    assert torch.equal(v, torch.topk(x, 3).values)


@pytest.mark.gpu
def test_two_stage_by_choice_matches_direct_selection():
    torch.manual_seed(0)
    x = torch.randn(64, 4096, device="cuda")
    x[:, 100] = x[:, 7]                                                                  # a tie: the lower column must win
    for kind in ("topk", "bottomk"):
        dv, di = rank.rank_select(x, 16, kind, choice=unison.RankChoice(False, 256, 16, 4096, 256))      # one full-width sort
        ref_v, ref_i = rank.rank_select_reference(x, 16, rank.MODES[kind])
        assert torch.equal(dv, ref_v) and torch.equal(di, ref_i)
        tv, ti = rank.rank_select(x, 16, kind)                                               # the tuned default
        assert torch.equal(tv, ref_v) and torch.equal(ti, ref_i)
        before = rank.launch_count
        cv, ci = rank.rank_select(x, 16, kind, choice=unison.RankChoice(True, 256, 16, 512, 256))
        assert rank.launch_count - before == 2                                           # per-chunk pass + merge pass
        assert torch.equal(dv, cv) and torch.equal(di, ci)
