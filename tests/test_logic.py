"""Host-side logic utilities: contextual observation, temporal dynamics, zeta events, KV store,
problem profiles, capture studio."""
import json
import math

import pytest
import torch

from spiraltorch_b200 import logic as L


def test_contextual_observation_is_swap_invariant():
    arr = L.Arrangement.from_line(["A", "A", "B", "A", "B", "B"])
    assert arr.boundary_edges() == 3
    assert arr.population() == (3, 3)
    assert arr.cluster_counts() == (2, 2)
    assert L.ContextObserver.is_swap_invariant(arr)
    sig = L.ContextObserver.signature(arr)
    assert sig.boundary_edges == 3 and sig.absolute_population_imbalance == 0
    assert sig.meaning_weight() == pytest.approx(3.0)
    pure = L.Arrangement.from_line(["A"] * 4)
    assert pure.is_pure() and L.ContextObserver.observe(pure) is None
    assert L.lift_to_label(pure) is None
    assert L.lift_to_label(L.Arrangement.from_line(["A", "B", "B"])) == "b"
    basis = L.MeaningBasis(L.Arrangement.from_line(["A", "B"] * 8))
    assert basis.dominant_frequency()[0] == 8            # alternation = Nyquist bin


def test_temporal_interpolation_and_integration():
    a = L.TemporalVolumeState.zeros(2, 3, 3, channels=1)
    b = L.TemporalVolumeState.zeros(2, 3, 3, channels=2)
    b.voxels += 4.0
    b.harmonics += 2.0
    b.resonance_decay += 1.0
    frames = L.interpolate_temporal_sequence(a, b, L.TemporalPropagationConfig(steps=3))
    assert len(frames) == 5
    assert torch.allclose(frames[2].voxels, torch.full((2, 3, 3), 2.0))
    assert frames[1].harmonics.shape[-1] == 2
    cfg = L.TemporalPropagationConfig(steps=2, delta_time=1.0, harmonic_blend=0.5, decay_gain=1.0)
    L.integrate_volume(a, b, cfg)
    # per sub-step decay = 0.5: 0 -> 2 -> 3
    assert torch.allclose(a.voxels, torch.full((2, 3, 3), 3.0))
    assert torch.allclose(a.harmonics, torch.full((2, 3, 3, 2), 1.5))
    with pytest.raises(ValueError):
        L.integrate_volume(a, b, L.TemporalPropagationConfig(delta_time=0.0))
    with pytest.raises(ValueError):
        L.integrate_volume(a, L.TemporalVolumeState.zeros(1, 3, 3))


def test_zeta_feedback_flushes_jsonl(tmp_path):
    path = tmp_path / "zeta.jsonl"
    z = L.ZetaFeedback("run-1", str(path), ["phase_deviation"])
    z.emit_phase_deviation(0.25)
    z.emit_collapse_resonance("spiral")
    z.emit_kernel_cache_hits(7)
    z.flush()
    rows = [json.loads(l) for l in path.read_text().splitlines()]
    assert [r["metric"] for r in rows] == ["phase_deviation", "collapse_resonance", "kernel_cache_hits"]
    assert rows[0]["value"] == 0.25 and rows[1]["pattern"] == "spiral" and rows[2]["run"] == "run-1"
    assert z.events == []


def test_memory_kv_semantics():
    now = [0.0]
    kv = L.MemoryKv(clock=lambda: now[0])
    assert kv.get("a") is None and kv.ttl("a") == -2
    kv.set("a", "1")
    assert kv.ttl("a") == -1 and kv.exists("a")
    assert not kv.set_nx("a", "2") and kv.get("a") == "1"
    kv.set_ex("t", "x", 5)
    assert kv.ttl("t") == 5
    now[0] = 5.0
    assert kv.get("t") is None and kv.set_nx("t", "y")
    assert kv.getset("a", "3") == "1" and kv.delete("a") == 1 and kv.delete("a") == 0
    assert kv.incr_by("n", 2) == 2 and kv.incr_by("n", 3) == 5
    kv.rpush("l", 1, 2, 3)
    kv.lpush("l", 0)
    assert kv.lrange("l", 0, -1) == [0, 1, 2, 3] and kv.lrange("l", -2, -1) == [2, 3]
    kv.ltrim("l", 0, 1)
    assert kv.lrange("l", 0, -1) == [0, 1]
    assert kv.hset("h", "f", 1) and not kv.hset("h", "f", 2)
    assert kv.hget("h", "f") == 2 and kv.hgetall("h") == {"f": 2} and kv.hdel("h", "f") == 1
    with pytest.raises(L.KvError):
        kv.hset("l", "x", 1)
    assert kv.set_json("j", {"k": [1, 2]}) and kv.get_json("j") == {"k": [1, 2]}
    assert not kv.set_json("j", 1, nx=True)
    assert kv.get_or_set_json("j2", lambda: {"d": 1}) == {"d": 1}
    assert kv.get_or_set_json("j2", lambda: {"d": 2}) == {"d": 1}
    c = L.Choice(use_2ce=True, wg=128, tile_cols=512)
    kv.set_choice("c", c)
    assert kv.get_choice("c") == c
    for i in range(5):
        kv.push_choice("hist", L.Choice(wg=i), keep=3)
    assert [x.wg for x in kv.lrange_choice("hist", 0, -1)] == [4, 3, 2]
    assert kv.pipeline(lambda s: (s.incr_by("n", 1), s.get("n"))) == (6, 6)
    assert L.connect("memory://t") is L.connect("memory://t")
    with pytest.raises(L.KvError):
        L.connect("redis://127.0.0.1/")


def test_problem_profile_and_wilson():
    assert L.wilson_lower_bound(0, 0) == 0.0
    lb = L.wilson_lower_bound(90, 100)
    assert 0.82 < lb < 0.9
    p = L.ProblemProfile(4096, 4096, 4096 * 8, subgroup=True)
    assert p.density_class() == "ultra_sparse" and p.aspect_class() == "square" and p.jacobi_hint() == 0
    assert p.lane_hint() == 256 and p.tile_hint() == 4096
    assert 0.15 <= p.fractional_alpha() <= 0.95
    wide = L.ProblemProfile(128, 65536, 128 * 65536 // 2, subgroup=False)
    assert wide.aspect_class() == "wide" and wide.density_class() == "dense" and wide.tile_hint() == 8192
    m = torch.zeros(6, 6)
    for i in range(6):
        m[i, i] = 1.0
        if i + 1 < 6:
            m[i, i + 1] = 2.0
    prof = L.ProblemProfile.from_sparse(m)
    assert prof.nnz == 11 and prof.diag_ratio == 1.0 and prof.bandwidth_peak == 2 and prof.max_row_nnz == 2
    learner = L.SoftRuleLearner(threshold=0.5)
    for _ in range(20):
        acc = learner.on_conversation(["wg=256"], [["wg=128"], ["wg=256"]], won=True)
    assert acc == ["wg=256"] and learner.stats["wg=128"] == [0, 20]


def test_capture_studio_storyboard():
    t = torch.arange(256, dtype=torch.float32)
    pulse = L.PulseSnapshot.from_samples(1.0 + 0.1 * torch.sin(0.05 * t))
    assert pulse.blocks == 16 and pulse.mean == pytest.approx(1.0, abs=0.05) and pulse.magnitude() > 3
    assert sum(pulse.band_energy) == pytest.approx(1.0) and pulse.band_energy[0] > 0.9
    studio = L.QuantumRealityStudio(L.SignalCaptureConfig(48.0, ["alpha", "beta"], history_limit=2),
                                    {"alpha": ["calm"]})
    seen = []
    studio.register_sink(lambda rec, frame: seen.append((rec.channel, frame.glyphs[0].glyph)))
    f0 = studio.ingest("alpha", pulse, timestamp=1.0)
    assert f0.glyphs[0].glyph == "calm" and f0.glyphs[0].intensity == pytest.approx(pulse.magnitude())
    f1 = studio.ingest("beta", pulse, narrative={"storm": 0.9, "rain": 0.2}, timestamp=2.0)
    assert f1.glyphs[0].glyph == "storm" and f1.glyphs[0].intensity == pytest.approx(0.9)
    studio.stitch_narrative_tags(f1, ["storm", "wind"])
    assert [g.glyph for g in f1.glyphs] == ["storm", "wind"]
    studio.ingest("beta", pulse, timestamp=3.0)
    with pytest.raises(L.StudioError):
        studio.ingest("gamma", pulse)
    board = studio.export_storyboard()
    assert len(board["frames"]) == 2 and board["channels"] == ["beta"]     # history limit 2
    assert seen[0] == ("alpha", "calm") and len(seen) == 3
    assert len(studio.export_storyboard_ndjson().splitlines()) == 2
    assert set(studio.export_storyboard_grouped()["channels"]) == {"beta"}
