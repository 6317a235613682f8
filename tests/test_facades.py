"""Host-side subsystems: telemetry hub, hyper-parameter search, soft logic / phase sync / refract
lowering, compression, recommenders, RL agents, robotics runtime, safety policy, metric registry."""
import math

import pytest
import torch

from spiraltorch_b200 import compress, hpo, metrics, plugin, rec, rl, robotics, safety, softlogic, telemetry
from spiraltorch_b200.nn.trainer import StepMetrics


# ---- telemetry -----------------------------------------------------------------------------------
def test_monitoring_hub_drift_and_regression_alerts():
    prom = telemetry.PrometheusExporter()
    seen = []
    hub = telemetry.MonitoringHub(drift_threshold=3.0, drift_warmup=8, perf_warmup=8)
    hub.with_exporter(prom).with_exporter(telemetry.CallbackExporter(lambda n, v, l: seen.append(n)))
    g = torch.Generator().manual_seed(0)
    for i in range(40):
        x = 1.0 + 0.01 * float(torch.randn((), generator=g))
        alerts = hub.observe(StepMetrics(10.0, 100.0, 0.0, {"grad_norm": x, "step_loss": 1.0}), reward=1.0)
        assert not alerts, (i, alerts)
    # the feature jumps far outside its frozen baseline; the loss regresses three steps in a row
    kinds = []
    for i in range(40):
        for a in hub.observe(StepMetrics(10.0, 100.0, 0.0, {"grad_norm": 5.0, "step_loss": 3.0}), reward=1.0):
            kinds.append((a.kind, a.severity))
    assert ("feature_drift", "warning") in kinds and ("performance_regression", "critical") in kinds
    assert hub.latest_alerts() and hub.last_observation() is not None
    text = prom.render()
    assert "# TYPE spiraltorch_runtime_step_time_ms gauge" in text
    assert "spiraltorch_extra_grad_norm 5.0" in text and "spiraltorch_performance_step_loss 3.0" in text
    assert "runtime_reward" in seen


def test_monitoring_alerts_reach_plugin_bus_and_prometheus_file(tmp_path):
    got = []
    sid = plugin.subscribe("Telemetry", got.append)
    hub = telemetry.MonitoringHub(2.0, 4, 4)
    for v in [1.0, 1.01, 0.99, 1.0] + [9.0] * 40:
        hub.observe(StepMetrics(extra={"f": v}))
    plugin.unsubscribe("Telemetry", sid)
    assert any(e.get("alert") == "feature_drift" for e in got)
    ex = telemetry.PrometheusExporter("st")
    ex.record_gauge("x", 1.5, [("rank", "0")])
    ex.write(tmp_path / "metrics.prom")
    assert 'st_x{rank="0"} 1.5' in (tmp_path / "metrics.prom").read_text()


def test_chrono_timeline_and_step_timer():
    tl = telemetry.ChronoTimeline(4)
    for i in range(6):
        f = tl.record(0.5, {"observed_curvature": -1.0 - 0.1 * i, "total_energy": 10.0 - i, "homotopy_energy": 2.0})
    assert len(tl) == 4 and tl.latest().step == 5
    assert abs(f.curvature_drift + 0.2) < 1e-6 and abs(f.energy_decay - 2.0) < 1e-6
    assert abs(f.homotopy_ratio() - 2.0 / 5.0) < 1e-6
    s = tl.summarise(3)
    assert s.frames == 3 and s.min_energy == 5.0 and s.max_energy == 7.0 and abs(s.mean_drift + 0.2) < 1e-6
    assert tl.rewind_steps(2) == 2 and tl.latest().step == 3
    with telemetry.StepTimer("cpu") as t:
        torch.randn(64, 64) @ torch.randn(64, 64)
    m = t.metrics(step_loss=0.5)
    assert m.step_time_ms > 0 and m.extra == {"step_loss": 0.5}


# ---- hpo -------------------------------------------------------------------------------------------
def _space():
    return hpo.SearchSpace([hpo.ParamSpec.Float("lr", 1e-4, 1e-1), hpo.ParamSpec.Int("layers", 1, 6),
                            hpo.ParamSpec.Categorical("act", ["relu", "gelu"])])


@pytest.mark.parametrize("make", [lambda: hpo.RandomStrategy(7), lambda: hpo.BayesianStrategy(7, 0.2),
                                  lambda: hpo.PopulationStrategy(7, 4, 2, 0.5)])
def test_search_loop_is_deterministic_and_resumable(make):
    def run(loop, n):
        out = []
        for _ in range(n):
            t = loop.suggest()
            loop.space().validate_suggestion(t.suggestion)
            loop.observe(t.id, (t.suggestion["lr"] - 0.01) ** 2 + 0.01 * t.suggestion["layers"])
            out.append(t.suggestion)
        return out

    a = run(hpo.SearchLoop(_space(), make()), 12)
    loop = hpo.SearchLoop(_space(), make())
    first = run(loop, 5)
    resumed = hpo.SearchLoop.from_state(_space(), loop.checkpoint())
    assert first + run(resumed, 7) == a
    best = resumed.best_trial()
    assert best is not None and best.metric == min(t.metric for t in resumed.completed())
    assert resumed.summary().completed == 12 and resumed.summary().has_best()


def test_search_space_validation_and_scheduler():
    with pytest.raises(hpo.SearchError):
        hpo.SearchSpace([]).validate()
    with pytest.raises(hpo.SearchError):
        hpo.SearchSpace([hpo.ParamSpec.Float("a", 1.0, 0.0)]).validate()
    with pytest.raises(hpo.SearchError):
        hpo.SearchSpace([hpo.ParamSpec.Int("a", 0, 1), hpo.ParamSpec.Int("a", 0, 1)]).validate()
    loop = hpo.SearchLoop(_space(), hpo.RandomStrategy(1), hpo.Objective("maximize"), hpo.ResourceConfig(max_concurrent=2))
    t0, t1 = loop.suggest(), loop.suggest()
    with pytest.raises(hpo.SearchError):
        loop.suggest()
    loop.observe(t0.id, 1.0)
    loop.observe(t1.id, 3.0)
    assert loop.best_trial().id == t1.id
    with pytest.raises(hpo.SearchError):
        loop.observe(t1.id, 0.0)
    now = [0.0]
    sch = hpo.ResourceScheduler(hpo.ResourceConfig(4, min_interval_ms=100), clock=lambda: now[0])
    assert sch.try_reserve() and not sch.try_reserve()
    now[0] = 0.2
    assert sch.try_reserve()


# ---- softlogic / sync / refract -----------------------------------------------------------------
def test_softmodes_and_beam():
    rules = [softlogic.SoftRule("a", 1.0, 2.0), softlogic.SoftRule("b", 3.0, -1.0)]
    assert softlogic.apply_softmode(rules, "sum") == -1.0
    assert abs(softlogic.apply_softmode(rules, "normalize") - (0.25 * 2 - 0.75)) < 1e-6
    sm = torch.softmax(torch.tensor([2.0, -1.0]), 0)
    assert abs(softlogic.apply_softmode(rules, "softmax") - float(sm[0] + 3 * sm[1])) < 1e-6
    p = 1 - (1 - 1 / (1 + math.exp(-2.0))) * (1 - 1 / (1 + math.exp(1.0)))
    assert abs(softlogic.apply_softmode(rules, "prob") - math.log(p / (1 - p))) < 1e-5
    assert softlogic.apply_softmode([], "sum") == 0.0
    pick = softlogic.beam_select(0, lambda c: [1, 2] if c == 0 else [], lambda c: float("nan") if c == 1 else 0.5, 2, 2)
    assert pick == 2
    expand = lambda c: [c * 2, c * 2 + 1] if c < 16 else []  # noqa: E731
    # a narrow beam drops the branch that leads to 21 (1 -> 2 -> 5 -> 10 -> 21); a wide one keeps it
    assert softlogic.beam_select(1, expand, lambda c: -abs(c - 21), 3, 6) == 26
    assert softlogic.beam_select(1, expand, lambda c: -abs(c - 21), 8, 6) == 21


def test_phase_sync_merge_rules():
    ps = softlogic.PhaseSync(0.05)
    sync = softlogic.SyncBlock("s", ["a:b"], 0.1)
    C = softlogic.PhaseCandidate
    # inside the tolerance window beats a higher-trust candidate outside it
    sel = ps.merge(sync, [C("far", 0.5, 1.0, 1.0), C("near", 0.05, 0.2, 0.0)])
    assert sel.graph_id == "near" and sel.pairs == ["a:b"]
    # equal scores: higher trust, then smaller delta, then resonance
    sel = ps.merge(sync, [C("x", 0.02, 0.5, 0.0), C("y", 0.02, 0.5, 0.3)])
    assert sel.graph_id == "y"
    assert abs(sel.score - (0.6 * 0.5 + 0.3 * 0.8 + 0.1 * math.tanh(0.3))) < 1e-6
    assert ps.merge(sync, []) is None
    with pytest.raises(ValueError, match="duplicated"):
        ps.merge(sync, [C("x", 0.0, 0.1, 0.0), C("x", 0.0, 0.1, 0.0)])
    with pytest.raises(ValueError, match="at least one pair"):
        ps.merge(softlogic.SyncBlock("s", []), [])
    with pytest.raises(ValueError):
        softlogic.PhaseSync.try_new(-1.0)


def test_refract_lowering_commits_or_rolls_back():
    calls = []

    class B(softlogic.KdslBackend):
        def __init__(self, fail=False):
            self.fail = fail

        def begin_refract(self, block): calls.append("begin")
        def set_precision(self, p): calls.append(("precision", p))
        def tune_op(self, op, flags):
            if self.fail:
                raise RuntimeError("no such op")
            calls.append(("tune", op, tuple(flags)))
        def commit_refract(self, block): calls.append("commit")
        def rollback_refract(self, block): calls.append("rollback")

    blk = softlogic.RefractBlock("main", ("graph", "gpt"), precision="bf16", backend="cuda",
                                 policies=[softlogic.RefractOpPolicy("matmul", ["tile256"])])
    softlogic.lower_refract(blk, B())
    assert calls == ["begin", ("precision", "bf16"), ("tune", "matmul", ("tile256",)), "commit"]
    calls.clear()
    with pytest.raises(RuntimeError, match="refract block 'main' failed"):
        softlogic.lower_refract(blk, B(fail=True))
    assert calls[-1] == "rollback" and "commit" not in calls
    with pytest.raises(ValueError):
        softlogic.validate_refract_block(softlogic.RefractBlock("bad name", ("graph", "g")))
    with pytest.raises(ValueError):
        softlogic.validate_refract_block(softlogic.RefractBlock("b", ("graph", "g"), precision="fp64"))
    got = []
    sid = plugin.subscribe("Telemetry", got.append)
    payload = softlogic.emit_feedback(softlogic.FeedbackBlock("fb", "out.json", ["loss", "absent"]), {"loss": 0.5})
    plugin.unsubscribe("Telemetry", sid)
    assert payload["metrics"] == {"loss": 0.5} and payload["missing"] == ["absent"] and got


# ---- compression -----------------------------------------------------------------------------------
def test_qat_observer_and_structured_pruning():
    obs = compress.QatObserver(compress.QatConfig(bit_width=4), "symmetric")
    obs.observe(torch.tensor([1.0, 2.0, 3.0]))
    obs.observe(torch.tensor([-4.0, 5.0]))
    w = torch.tensor([0.5, -0.5, 1.5, -1.5, 9.0])
    rep = obs.quantize(w)
    assert rep.bit_width == 4 and rep.scale > 0 and rep.zero_point == 0.0 and rep.observed_steps == 2
    levels = torch.unique(torch.round((w - rep.min_value) / rep.scale))
    assert len(levels) <= 16 and w.max() <= rep.max_value + 1e-6
    asym = compress.QatObserver(leveling="asymmetric")
    asym.observe(torch.tensor([0.0, 4.0]))
    r2 = asym.quantize(torch.tensor([1.0, 2.0]))
    assert r2.min_value < 0 < r2.max_value and r2.quant_error < 1e-3

    w = torch.arange(1, 65, dtype=torch.float32)
    rep = compress.StructuredPruner().apply(w, compress.StructuredPruningConfig(block_size=8, target_sparsity=0.5))
    assert rep.pruned_blocks == 4 and rep.kept_blocks == 4 and rep.achieved_sparsity == 0.5
    assert torch.all(w[:32] == 0) and torch.all(w[32:] > 0)
    assert abs(rep.l2_error - math.sqrt(sum(i * i for i in range(1, 33)))) < 1e-2
    tiny = torch.tensor([1e-6] * 4 + [1.0] * 4)
    rep = compress.StructuredPruner().apply(tiny, compress.StructuredPruningConfig(4, 0.0, 1e-4))
    assert rep.pruned_blocks == 1 and torch.all(tiny[:4] == 0)
    with pytest.raises(compress.OptimisationError):
        compress.StructuredPruner().apply(w, compress.StructuredPruningConfig(0, 0.5))
    full = compress.compress(torch.randn(256), qat=compress.QatObserver(), pruning=compress.StructuredPruningConfig(32, 0.25))
    assert full.original_params == 256 and full.remaining_params <= 192 and full.quantization and full.pruning


# ---- recommenders ----------------------------------------------------------------------------------
def test_spiral_recommender_learns_and_ranks():
    R = rec.RatingTriple
    ratings = [R(0, 0, 5.0), R(0, 1, 1.0), R(1, 0, 4.0), R(1, 2, 2.0), R(2, 1, 5.0), R(2, 2, 4.0)]
    m = rec.SpiralRecommender(3, 3, 4, 0.05, 0.01)
    assert abs(m.predict(0, 0) - sum(math.sin(f) * 0.05 * math.cos(f) * 0.05 for f in range(1, 5))) < 1e-6
    first = m.train_epoch(ratings)
    for _ in range(300):
        last = m.train_epoch(ratings)
    assert last.rmse < 0.5 * first.rmse and last.samples == 6
    top = m.recommend_top_k(0, 2, exclude=[1])
    assert [r.item for r in top][0] == 0 and all(r.item != 1 for r in top)
    with pytest.raises(rec.SpiralRecError):
        m.train_epoch([R(9, 0, 1.0)])
    with pytest.raises(rec.SpiralRecError):
        m.train_epoch([])
    nb = rec.NeighborhoodModel.fit(3, 3, ratings + [R(0, 0, 3.0)], 0.1)
    assert abs(float(nb.matrix[0, 0]) - 4.0) < 1e-6
    assert len(nb.recommend(0, 2)) == 2
    kg = rec.KnowledgeGraphRecommender(2, 4, 0.5)
    kg.add_edge("user_item", 0, 0)
    kg.add_edge("item_item", 0, 1)
    kg.add_edge("item_item", 1, 2)
    out = kg.recommend(0, 3, hops=2)
    assert [r.item for r in out] == [1, 2] and out[0].score > out[1].score and kg.item_degree(1) == 2


# ---- rl ----------------------------------------------------------------------------------------------
def test_dqn_ppo_sac_and_policy_gradient():
    dqn = rl.DqnAgent(4, 2, 0.9, 0.5)
    dqn.set_epsilon(0.0)
    for _ in range(50):
        dqn.update_batch([0, 1, 2], [1, 1, 1], [0.0, 0.0, 1.0], [1, 2, 3], [False, False, True])
    assert dqn.greedy_action(0) == 1 and abs(dqn.q_values(2)[1] - 1.0) < 1e-3 and abs(dqn.q_values(1)[1] - 0.9) < 1e-2
    assert dqn.select_action(0) == 1
    dqn.configure_epsilon_schedule(rl.EpsilonGreedySchedule(1.0, 0.0, 10))
    tr = dqn.select_action_trace(0)
    assert tr.epsilon == 1.0 and dqn.epsilon < 1.0 and dqn.schedule_step() == 1
    with pytest.raises(rl.SpiralRlError):
        rl.DqnAgent(4, 2, 1.5, 0.1)
    with pytest.raises(rl.SpiralRlError):
        dqn.update_batch([0], [0, 1], [0.0], [1])

    ppo = rl.PpoAgent(3, 2, 0.1, 0.2)
    s = [1.0, 0.5, -0.5]
    lp = ppo.log_prob(s, 1)
    ppo.update(s, 1, 2.0, lp)
    assert ppo.log_prob(s, 1) > lp and ppo.value(s) > 0

    sac = rl.SacAgent(3, 4, 0.5)
    acts = {sac.sample_action(s) for _ in range(50)}
    assert acts <= {0, 1, 2, 3} and len(acts) > 1
    sac.jitter(0.1)
    assert float(sac.policy_weights.abs().max()) <= 1.0

    pg = rl.SpiralPolicyGradient(2, 2, 0.5, 0.9)
    assert abs(float(pg.weights[0, 0]) - math.cos(1.0) * 0.01) < 1e-7
    for _ in range(60):
        for s_, a_, r_ in [([1.0, 0.0], 0, 1.0), ([1.0, 0.0], 1, -1.0), ([0.0, 1.0], 1, 1.0), ([0.0, 1.0], 0, -1.0)]:
            pg.record_transition(s_, a_, r_)
        rep = pg.finish_episode()
    assert rep.steps == 4 and pg.select_action([1.0, 0.0]) == 0 and pg.select_action([0.0, 1.0]) == 1
    with pytest.raises(rl.SpiralRlError):
        pg.finish_episode()
    pg.enable_hypergrad(-1.0, 0.05)
    pg.attach_hyper_surprise(0.01)
    pg.record_transition([1.0, 0.0], 0, 1.0)
    pg.record_transition([1.0, 0.0], 1, -3.0)
    rep = pg.finish_episode()
    assert rep.hypergrad_applied and rep.hyper_surprise["scale"] < 1.0 and pg.telemetry().hypergrad


# ---- robotics ------------------------------------------------------------------------------------------
def test_robotics_runtime_step_and_safety():
    now = [0.0]
    hub = robotics.SensorFusionHub(clock=lambda: now[0])
    hub.register_channel("imu", 3)
    hub.register_channel("lidar", 1, smoothing=0.5, optional=True, max_staleness=0.5)
    hub.calibrate("imu", bias=[0.1, 0.1, 0.1], scale=2.0)
    frame = hub.fuse({"imu": [0.2, 0.4, 0.3], "lidar": [1.0]})
    assert all(abs(a - b) < 1e-6 for a, b in zip(frame.coordinates["imu"], [0.2, 0.6, 0.4]))
    now[0] = 1.0
    frame = hub.fuse({"imu": [0.2, 0.4, 0.3], "lidar": [0.0]})
    assert 0.0 < frame.coordinates["lidar"][0] < 1.0 and frame.health["lidar"].stale
    with pytest.raises(robotics.RoboticsError):
        hub.fuse({"lidar": [0.0]})
    with pytest.raises(robotics.RoboticsError):
        hub.register_channel("imu", 3)
    assert abs(robotics.ZSpaceGeometry.non_euclidean(-1.0).metric_norm([3.0, 4.0]) - 5.0 / (1 + 25 / 6)) < 1e-6
    assert abs(robotics.ZSpaceGeometry.general_relativity([[2.0, 0.0], [0.0, 2.0]], 0.5).metric_norm([3.0, 4.0])
               - math.sqrt(50.0) * 0.5) < 1e-5

    hub2 = robotics.SensorFusionHub()
    hub2.register_channel("arm", 2)
    rt = robotics.RoboticsRuntime(hub2, robotics.DesireLagrangianField({"arm": robotics.Desire(1.0, 0.1, 2.0)}),
                                  robotics.PsiTelemetry(window=4, failure_energy=5.0, norm_limit=10.0))
    rt.attach_policy_gradient(robotics.PolicyGradientController(0.05, 0.5))
    plug = robotics.DriftSafetyPlugin("drift", hazard_cut=0.8)
    rt.attach_safety_plugin(plug)
    rt.enable_recording(2)
    ok = rt.step({"arm": [1.0, 0.0]})
    assert not ok.halted and ok.energy.total == 0.0 and ok.commands["learning_rate"] == 0.05
    hot = rt.step({"arm": [3.0, 0.0]})
    assert abs(hot.energy.total - 3.8) < 1e-5 and hot.commands["learning_rate"] < 0.05
    assert hot.halted and hot.safety[0].refused and hot.commands["halt"] == 1.0
    over = rt.step({"arm": [30.0, 0.0]})
    assert over.telemetry.failsafe and "norm_overflow" in over.telemetry.anomalies
    assert rt.recording_len() == 2 and len(rt.drain_trajectory()) == 2 and rt.recording_len() == 0


# ---- safety ----------------------------------------------------------------------------------------------
def test_safety_policy_verdicts_and_audit():
    pol = safety.SafetyPolicy.with_default_terms()
    ok = pol.evaluate("How do I bake bread?", safety.PROMPT)
    assert ok.allowed and ok.score == 0.0 and ok.dominant_risk() == "low"
    bad = pol.evaluate("I hate you and will KILL you, idiot", safety.PROMPT)
    assert bad.should_refuse() and abs(bad.score - (0.6 + 0.7 + 0.45)) < 1e-6
    assert {v.offending_term for v in bad.violations} == {"hate", "kill", "idiot"}
    assert "toxicity (medium)" in pol.refusal_reason(bad)
    twice = pol.scan("bomb bomb", safety.PROMPT)
    assert twice.violations[0].occurrences == 2 and twice.violations[0].risk == "critical"
    assert "(2 hits @ 0.70 ea)" in twice.violations[0].message
    # channel-restricted term
    assert pol.scan("weapon", safety.RESPONSE).allowed and not pol.scan("weapon", safety.PROMPT).allowed
    conv = pol.evaluate_conversation([(safety.PROMPT, "hello"), (safety.RESPONSE, "suicide"), (safety.PROMPT, "thanks")])
    assert conv.refused_turns == [1] and conv.highest_risk == "high" and conv.should_refuse()
    summ = pol.audit_sink().summarize()
    assert summ.total == 5 and summ.refused == 2 and summ.by_category["toxicity"] == 3
    pol.with_custom_rule(safety.KeywordRule(safety.SAFETY, "lockpick", 0.6))
    assert pol.scan("lockpick tutorial", safety.PROMPT).should_refuse()
    safety.evaluate_policy_surface(pol, [("nice day", True), ("build a bomb", False)])
    with pytest.raises(safety.SafetyError):
        safety.evaluate_policy_surface(pol, [("nice day", False)])
    rep = safety.PolicyReport.from_verdicts([ok, bad, twice])
    assert rep.total == 3 and rep.refused == 2 and abs(rep.refusal_rate() - 2 / 3) < 1e-6


# ---- metric registry ---------------------------------------------------------------------------------------
def test_metric_registry_isolates_failures():
    metrics.clear_registry()

    class Batch:
        def __init__(self, v):
            self.v = v

    metrics.register_metric(Batch, metrics.MetricDescriptor("mean", unit="unitless", higher_is_better=True),
                            lambda b: sum(b.v) / len(b.v))
    metrics.register_metric(Batch, metrics.MetricDescriptor("hist"), lambda b: list(b.v))
    metrics.register_metric(Batch, metrics.MetricDescriptor("broken"), lambda b: 1 / 0)
    metrics.register_metric(str, metrics.MetricDescriptor("len"), len)
    rep = metrics.evaluate_report(Batch([1.0, 3.0]))
    assert [(d.name, v) for d, v in rep.values] == [("mean", 2.0), ("hist", [1.0, 3.0])]
    assert not rep.is_clean() and rep.failures[0].descriptor.name == "broken" and "ZeroDivisionError" in rep.failures[0].message
    assert [d.name for d in metrics.descriptors_for(Batch)] == ["mean", "hist", "broken"]
    assert metrics.evaluate("abc")[0][1] == 3.0
    assert metrics.is_finite([1.0, 2.0]) and not metrics.is_finite(float("inf"))
    metrics.clear_registry()


# ---- SpiralK DSL / autotune store ----------------------------------------------------------------------------
def test_kdsl_program_store_and_registry(tmp_path):
    from spiraltorch_b200 import kdsl
    ctx = kdsl.Ctx(r=1024, c=65536, k=512, sg=True, sgc=32, kc=4, tile_cols=1024, radix=4, segments=2)
    out = kdsl.Program.parse("wg: 256; radix: log2(k);").evaluate(ctx)
    assert out.hard == {"wg": 256, "radix": 9}
    assert kdsl.Program.parse("radix: clamp(16, 2, 8);").evaluate(ctx).hard["radix"] == 8
    prog = kdsl.Program.parse("""
        let total = 0;
        for i in 0..4 { set total = total + i; }
        radix: total;
        # reference heuristics file shape
        mk:   sel(sg && (k<=128), 2, sel(k<=2048, 1, 0));
        tile: sel(log2(c)>15.0, 2048, sel(log2(c)>13.0, 1024, 256));
        ctile: sel(tile>=1024, tile/2, tile);
        if c > 100000 { wg: 512; } else { wg: 128; }
        soft(mk,   2, 0.25, sg && (k<=128));
        soft(mk,   1, 0.20, (k>128)&&(k<=2048));
        soft(tile, 2048, 0.20, log2(c)>15.0);
    """)
    out = prog.evaluate(ctx)
    assert out.hard == {"radix": 6, "mk": 1, "tile": 2048, "ctile": 1024, "wg": 128}
    assert [(s.field, s.value, s.weight) for s in out.soft] == [("mk", 1.0, 0.2), ("tile", 2048.0, 0.2)]
    for bad in ("wg 256;", "bogus: 1;", "wg: foo;", "wg: 1/0;", "while true { }", "wg: (1;"):
        with pytest.raises(kdsl.KdslError):
            kdsl.Program.parse(bad).evaluate(ctx)

    assert kdsl.wilson_lower_bound(0, 0) == 0.0
    assert abs(kdsl.wilson_lower_bound(90, 100) - 0.8256) < 1e-3
    assert kdsl.should_rewrite(kdsl.WilsonMetrics(10.0, 8.0, 95, 100), 0.1, 0.8)
    assert not kdsl.should_rewrite(kdsl.WilsonMetrics(10.0, 9.9, 95, 100), 0.1, 0.8)
    assert not kdsl.should_rewrite(kdsl.WilsonMetrics(10.0, 8.0, 3, 5), 0.1, 0.8)

    store = tmp_path / "sub" / "kernels.json"
    assert kdsl.record_best(store, "gemm", {"m": 4096, "n": 4096, "k": 1024}, 0.30, {"bn": 256, "stages": 4})
    assert not kdsl.record_best(store, "gemm", {"m": 4096, "n": 4096, "k": 1024}, 0.35, {"bn": 128, "stages": 6})
    assert kdsl.record_best(store, "gemm", {"m": 4096, "n": 4096, "k": 1024}, 0.25, {"bn": 128, "stages": 6})
    kdsl.record_best(store, "gemm", {"m": 128, "n": 128, "k": 64}, 0.01, {"bn": 128, "stages": 6})
    best = kdsl.lookup_best(store, "gemm", {"m": 4000, "n": 4096, "k": 1024})
    assert best["params"] == {"bn": 128, "stages": 6} and best["score"] == 0.25
    sim = kdsl.lookup_similar(store, "gemm", {"m": 100, "n": 128, "k": 64}, 2)
    assert sim[0][0]["context"]["m"] == 128 and sim[0][1] < sim[1][1]
    assert kdsl.lookup_best(store, "conv", {}) is None
    for i in range(40):
        kdsl.record_best(store, "many", {"i": i}, 1.0, {})
    assert len(kdsl.load_store(store)["many"]["entries"]) == kdsl.BUCKET_HISTORY_LIMIT

    key = kdsl.AutotuneKey(kdsl.DeviceProfile("NVIDIA B200", 0x100, 32, 227, "12.9"), kdsl.KernelProfile(7, "gemm:bf16:nt"))
    assert key.encode() == "NVIDIA-B200|0100|32|227|12.9|0000000000000007|gemm:bf16:nt"
    reg = kdsl.AutotuneRegistry.with_capacity(3)
    for tf in (900.0, 1500.0, 1200.0, 1100.0):
        reg.record(key, kdsl.TelemetrySample(tf, 5000.0, 0.1, {"bn": int(tf)}, regress=tf < 1000))
    log = reg.log(key)
    assert len(log) == 3 and log.best_by_tflops().tflops == 1500.0 and log.best_tile() == {"bn": 1500}
    assert log.summary()["samples"] == 3 and log.regression_rate() == 0.0
    assert kdsl.DeviceProfile.current().encode()


# ---- measures, engine hooks, operator registry, backend policy, blackcat ---------------------------------------
def test_measures_engine_and_blackcat():
    import spiraltorch_b200 as st
    from spiraltorch_b200 import engine, measure
    from spiraltorch_b200.runtime import blackcat

    d = [st.Tensor(1, 3, [0.98, 0.01, 0.01]), st.Tensor(1, 3, [0.1, 0.2, 0.7])]
    uni = measure.z_space_barycenter([0.0, 0.0], d, 0.5, 0.0)
    assert uni.density.tolist()[0] == pytest.approx([1 / 3] * 3, abs=1e-6) and uni.kl_energy == 0.0 and uni.objective < 0
    one = measure.z_space_barycenter([1.0], [st.Tensor(1, 2, [0.9, 0.1])], -0.999, 0.0)
    assert one.density.tolist()[0][0] > 0.999 and abs(sum(one.density.tolist()[0]) - 1) < 1e-6
    mix = measure.z_space_barycenter([1.0, 1.0], d, 0.0, 1.0, st.Tensor(2, 2, [0, 1, 1, 0]))
    geo = torch.tensor([[0.98 * 0.1, 0.01 * 0.2, 0.01 * 0.7]]).sqrt()
    assert torch.allclose(mix.density.torch(), geo / geo.sum(), atol=1e-6) and mix.coupling_energy > 0
    with pytest.raises(st.TensorError):
        measure.z_space_barycenter([1.0], d, 0.0, 0.0)
    with pytest.raises(st.TensorError):
        measure.z_space_barycenter([0.0, 0.0], d, 0.0, 0.0)
    w = measure.nirt_weight_update([0.5, 0.5], [1.0, -1.0], 0.5, 0.2)
    assert w == pytest.approx([0.6, 0.4]) and abs(sum(w) - 1) < 1e-9
    assert measure.nirt_weight_update([0.1, 0.9], [-1.0, 0.0], 1.0, 1.0) == pytest.approx([0.0, 1.0])
    with pytest.raises(st.TensorError):
        measure.nirt_weight_update([0.5, 0.5], [2.0, 0.0], 0.5, 0.1)

    g = torch.tensor([1.0, -2.0, 3.0])
    assert engine.call_onebit_allreduce(g, 4) is False and g.tolist() == [1.0, -2.0, 3.0]
    engine.register_onebit_allreduce(lambda grad, world: grad.copy_(torch.sign(grad) * grad.abs().mean()))
    assert engine.call_onebit_allreduce(g, 4) and g.tolist() == [2.0, -2.0, 2.0]
    engine.register_onebit_allreduce(None)
    p = torch.arange(10.0)
    assert engine.call_zero_partition(p, 1, 4) is p
    engine.register_zero_partition(engine.default_zero_partition)
    assert [engine.call_zero_partition(p, r, 4).tolist() for r in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7, 8], [9]]
    engine.register_zero_partition(None)

    reg = engine.OperatorRegistry()
    reg.register(engine.OperatorSpec("axpy", 2, lambda x, y: x.scale(2.0).add(y),
                                     lambda x, y, go: [go.scale(2.0), go], "2x + y"))
    out = reg.call("axpy", st.Tensor(1, 2, [1, 2]), st.Tensor(1, 2, [10, 20]))
    assert out.tolist() == [[12.0, 24.0]] and reg.names() == ["axpy"]
    gx, gy = reg.call_backward("axpy", [st.Tensor(1, 2, [1, 2]), st.Tensor(1, 2, [10, 20])], st.Tensor(1, 2, [1, 1]))
    assert gx.tolist() == [[2.0, 2.0]] and gy.tolist() == [[1.0, 1.0]]
    with pytest.raises(st.TensorError):
        reg.call("axpy", st.Tensor(1, 1, [1]))
    with pytest.raises(st.TensorError):
        reg.register(engine.OperatorSpec("axpy", 1, lambda x: x))
    assert reg.unregister("axpy") and not reg.unregister("axpy")

    assert engine.backend_for("matmul") == "auto"
    with engine.push_backend_policy(engine.BackendPolicy(matmul="cpu", attention="cuda")):
        assert engine.backend_for("matmul") == "cpu"
        with engine.push_backend_policy(engine.BackendPolicy(matmul="cuda")):
            assert engine.backend_for("matmul") == "cuda" and engine.backend_for("attention") == "cuda"
        assert engine.backend_for("matmul") == "cpu"
    assert engine.backend_for("matmul") == "auto"
    with pytest.raises(st.TensorError):
        engine.push_backend_policy(engine.BackendPolicy(matmul="wgpu"))

    # the bandit learns that "big" tiles are faster in context A and "small" in context B
    cat = blackcat.BlackCat({"tile": ["small", "big"]}, context_dim=2, exploration=0.5)
    ctx_a, ctx_b = [1.0, 0.0], [0.0, 1.0]
    for i in range(60):
        ctx = ctx_a if i % 2 == 0 else ctx_b
        pick = cat.choose(ctx)["tile"]
        fast = (pick == "big") == (ctx is ctx_a)
        cat.post_step(StepMetrics(step_time_ms=5.0 if fast else 20.0, mem_peak_mb=100.0))
    assert cat.choose(ctx_a)["tile"] == "big" and cat.choose(ctx_b)["tile"] == "small"
    assert cat.observations("tile", "big") + cat.observations("tile", "small") == 60
    u = cat.post_step(StepMetrics(step_time_ms=10.0, mem_peak_mb=1024.0, retry_rate=0.0))
    assert u == pytest.approx(-(0.5 + 0.3))
    n = cat.observations("tile", "small") + cat.observations("tile", "big")
    cat.post_step(StepMetrics(step_time_ms=10.0))                      # no pending selection: nothing credited
    assert cat.observations("tile", "small") + cat.observations("tile", "big") == n
    assert cat.choose([1.0]) == {} and cat.post_step(StepMetrics(step_time_ms=float("nan"))) == -math.inf


def test_language_control_and_text_resonator():
    from spiraltorch_b200 import language, text, telemetry
    assert language.entropy([0.5, 0.5]) == pytest.approx(math.log(2))
    with pytest.raises(Exception):
        language.entropy([0.5, 0.2])
    tc = language.TemperatureController(1.0, target_entropy=1.0, eta=0.5, min=0.1, max=2.0)
    assert tc.update([1.0, 0.0, 0.0]) == pytest.approx(1.5)             # too peaked -> warmer
    for _ in range(10):
        tc.update([1.0, 0.0, 0.0])
    assert tc.value() == 2.0
    assert tc.update([0.25] * 4) < 2.0                                   # too flat -> cooler
    with pytest.raises(Exception):
        language.TemperatureController(5.0, 1.0, 0.1, 0.1, 2.0)

    V, C = 6, 2
    g = torch.Generator().manual_seed(0)
    syn, par = torch.randn(V, V, generator=g) * 0.1, torch.randn(V, V, generator=g) * 0.1
    syn[0, 3] = 3.0                                                        # token 3 follows token 0
    rep = torch.zeros(V)
    rep[1] = 5.0                                                           # token 1 is repressed
    sem = torch.zeros(V, C)
    sem[4, 1] = 2.0
    lag = language.DesireLagrangian(syn, par, rep, sem, language.TemperatureController(1.0, 1.2, 0.05, 0.2, 3.0))
    logits = torch.tensor([0.0, 2.0, 0.0, 0.0, 0.0, 0.0])
    base = lag.step(logits, 0, [1.0, 0.0], language.DesireWeights())
    assert base.phase == language.OBSERVATION and max(range(V), key=lambda i: base.probabilities[i]) == 1
    sol = lag.step(logits, 0, [0.0, 1.0], language.DesireWeights(alpha=1.0, gamma=1.0, lam=1.0))
    p = dict(zip(sol.indices, sol.probabilities))
    assert sol.phase == language.INTEGRATION and p[3] > p[1] and p[4] > p[2] and abs(sum(sol.probabilities) - 1) < 1e-5
    lag2 = language.DesireLagrangian(syn, par, rep, sem, language.TemperatureController(1.0, 1.2, 0.05, 0.2, 3.0), top_k=3)
    lag2.with_schedules(alpha=language.warmup(0.0, 1.0, 4)).with_horizons(2, None)
    phases = [lag2.step_with_scheduler(logits, 0, [1.0, 0.0]).phase for _ in range(4)]
    assert phases[:2] == [language.OBSERVATION] * 2 and phases[3] == language.INJECTION
    assert len(lag2.step_with_scheduler(logits, 0, [1.0, 0.0]).indices) == 3
    with pytest.raises(Exception):
        lag.step(logits[:3], 0, [1.0, 0.0], language.DesireWeights())

    tl = telemetry.ChronoTimeline(16)
    for i in range(8):
        tl.record(0.1, {"observed_curvature": -1.0 + 0.01 * i, "total_energy": 2.0})
    tr = text.TextResonator()
    nar = tr.describe_timeline(tl)
    assert "energetic" in nar.summary and "rising" in nar.summary and "stable" in nar.summary
    wave = tr.synthesize_wave(tl, sample_rate=1000, seconds_per_frame=0.01)
    assert len(wave.samples) == 80 and max(abs(s) for s in wave.samples) <= 1.0
    assert tr.describe_timeline(telemetry.ChronoTimeline()) is None


def test_scale_stack_and_fractal_field():
    import math
    from spiraltorch_b200 import frac
    field = torch.zeros(16, 16)
    field[:, 8:] = 1.0                                   # one straight interface
    stack = frac.ScaleStack.from_scalar_field(field, [1.0, 2.0, 3.0], 0.5)
    gates = [g for _, g in stack.samples]
    assert gates == pytest.approx([2 / 16, 4 / 16, 6 / 16])
    bins = stack.persistence_measure()
    assert len(bins) == 3 and bins[0][:2] == (0.0, 1.0)
    assert stack.interface_density() == pytest.approx(2 / 16)
    dim = stack.estimate_boundary_dimension(2.0, 3)
    assert dim == pytest.approx(1.0, abs=0.05)           # a line in the plane
    assert stack.coherence_break_scale(0.2) == 2.0 and stack.coherence_break_scale(0.9) is None
    with pytest.raises(ValueError):
        frac.ScaleStack.from_scalar_field(field, [2.0, 1.0], 0.5)
    sem = torch.zeros(8, 8, 3)
    sem[:, :4, 0] = 1.0
    sem[:, 4:, 1] = 1.0
    s2 = frac.ScaleStack.from_semantic_field(sem, [1.0], 0.5, feature_axis=2, metric="cosine")
    assert s2.samples[0][1] == pytest.approx(2 / 8)
    gen = frac.FractalFieldGenerator(3, 2.0, 0.5, 16)
    fld = gen.branching_field(-2.0, 0.25, 12)
    assert fld.shape == (12,) and fld.real.abs().max() > 0 and fld.imag.abs().max() > 0
    # one octave at x = 0: c = 1 escapes after 3 iterations (0 -> 1 -> 2 -> 5)
    one = frac.FractalFieldGenerator(1, 2.0, 0.5, 8).branching_field(0.0, 1.0, 1)
    assert one[0].real == pytest.approx(3 / 8) and abs(one[0].imag) < 1e-6
    with pytest.raises(ValueError):
        frac.FractalFieldGenerator(0, 2.0, 0.5, 4)
    x = torch.randn(3, 4, 32)
    y = frac.fracdiff_gl_nd(x, 0.6, axis=2)
    assert torch.allclose(y[1, 2], frac.fracdiff_gl(x[1, 2], 0.6), atol=1e-5)
    g = torch.randn(32)
    xv = torch.randn(32)
    assert torch.dot(frac.fracdiff_gl(xv, 0.6), g) == pytest.approx(float(torch.dot(xv, frac.fracdiff_gl_vjp(g, 0.6))), rel=1e-4)
    assert len(frac.gl_coeffs_adaptive(0.5, 1e-3, 4096)) < 200


def test_video_pipeline_digests():
    from spiraltorch_b200 import vision
    frames = [(0.0, torch.zeros(4, 6)), (0.5, torch.ones(4, 6)), (1.0, torch.ones(4, 6)), (1.5, torch.ones(4, 6) * 3)]
    pipe = vision.VideoPipeline(frames, vision.VideoPipelineConfig(temporal_alpha=0.5, resonance_decay=0.5, digest_window=2))
    outs = list(pipe)
    assert [o["frame_index"] for o in outs] == [0, 1, 2, 3]
    assert outs[0]["motion_embedding"].abs().sum() == 0
    assert torch.allclose(outs[1]["motion_embedding"], torch.ones(4, 6))
    assert torch.allclose(outs[1]["volume"][0], torch.full((4, 6), 0.5))       # lerp(0, 1, 0.5)
    assert torch.allclose(outs[2]["volume"][1], torch.full((4, 6), 0.25))      # motion 1 then 0
    d = outs[3]["temporal_digest"]
    assert d["frames"] == 4 and d["duration"] == pytest.approx(1.5)
    assert d["peak_motion_energy"] == pytest.approx(2.0) and d["peak_motion_timestamp"] == 1.5
    assert d["quiescence_ratio"] == pytest.approx(0.5)                         # frames 0 and 2 are still
    assert outs[3]["window_digest"]["frames"] == 2
    assert len(outs[3]["z_dynamics"]["per_depth_energy"]) == 2 and len(pipe.atlas_timeline()) == 4
    assert outs[3]["atlas_frame"]["metrics"]["z.weight_entropy"] > 0
    assert pipe.next_frame() is None


def test_atlas_route_summary():
    from spiraltorch_b200 import telemetry as T
    assert T.metric_root_token("  .loop.frames ") == "loop" and T.infer_district("canvas_energy") == "Surface"
    assert T.infer_district("z.motion") == "Substrate" and T.infer_district("foo") == "Unknown"
    route = T.AtlasRoute()
    route.push_bounded(T.AtlasFrame(0.0))                       # dropped: no positive timestamp
    for i in range(1, 6):
        f = T.AtlasFrame(float(i), loop_support=0.1 * i, collapse_total=1.0 / i, z_signal=0.2 * i)
        f.push_metric("trainer.loss", 2.0 - 0.3 * i)
        f.push_metric("z.energy", 1.0)
        f.push_metric("custom", float(i), district="Surface")
        f.notes.append(f"n{i}")
        f.concepts.append(("spiral", "qualia"))
        route.push_bounded(f, capacity=4)
    assert len(route) == 4 and route.latest().timestamp == 5.0
    s = route.summary()
    assert s.frames == 4 and s.loop_min == pytest.approx(0.2) and s.loop_max == pytest.approx(0.5)
    assert s.collapse_trend == pytest.approx(1 / 5 - 1 / 2) and s.z_signal_trend == pytest.approx(0.6)
    assert set(s.districts) == {"Concourse", "Substrate", "Surface"}
    beacons = s.beacons()
    assert [b["metric"] for b in beacons] == ["custom", "trainer.loss"]        # z.energy did not move
    assert beacons[1]["trend"] == "falling" and "is easing" in beacons[1]["narrative"]
    assert s.beacon_for("z.energy") is None and s.latest_note() == "n5"
    assert s.concept_heatmap()["total_mentions"] == 4
    flux = s.flux()
    assert flux["coverage"] == 4 and flux["note_density"] == 1.0 and flux["loop_range"] == pytest.approx(0.3)
    import json
    json.dumps(s.to_json())
    assert T.AtlasRoute().summary().flux() is None


def test_tracking_connectors(tmp_path):
    import json
    from spiraltorch_b200 import hpo, tracking as TK
    assert TK.crc32c(b"123456789") == 0xE3069283                     # CRC-32C check value
    tb = TK.TensorBoardTracker(str(tmp_path / "tb"))
    jl = TK.JsonlTracker(str(tmp_path / "log" / "trials.jsonl"))

    class Boom(hpo.ExperimentTracker):
        def on_observe(self, trial):
            raise RuntimeError("tracker down")

    class FakeMlflow:
        def __init__(self):
            self.calls = []

        def set_experiment(self, name):
            self.calls.append(("exp", name))

        def start_run(self, run_name=None, nested=False):
            import contextlib
            self.calls.append(("run", run_name, nested))
            return contextlib.nullcontext()

        def log_params(self, p):
            self.calls.append(("params", dict(p)))

        def log_metric(self, k, v, step=None):
            self.calls.append(("metric", k, v, step))

    fake = FakeMlflow()
    ml = TK.MLflowTracker("exp1", client=fake)
    comp = TK.CompositeTracker([tb, jl, Boom(), ml, TK.ConsoleTracker()])
    space = hpo.SearchSpace([hpo.ParamSpec.Float("lr", 1e-4, 1e-1)])
    loop = hpo.SearchLoop(space, hpo.RandomStrategy(3), trackers=[comp])
    for i in range(3):
        t = loop.suggest()
        loop.observe(t.id, 1.0 / (i + 1))
    loop.checkpoint()
    comp.log_scalar("train/loss", 0.5, 7)
    events = TK.read_scalar_events(tb.path)
    assert [e["tag"] for e in events] == ["hpo/metric"] * 3 + ["train/loss"]
    assert events[1]["value"] == pytest.approx(0.5) and events[3]["step"] == 7
    rows = [json.loads(l) for l in open(jl.path)]
    assert [r["event"] for r in rows] == ["trial_start", "trial_end"] * 3 + ["checkpoint", "scalar"]
    assert ("exp", "exp1") in fake.calls and sum(1 for c in fake.calls if c[0] == "run") == 3
    assert ("metric", "train/loss", 0.5, 7) in fake.calls
    assert not TK.MLflowTracker().enabled or True                     # inert without the package, never raises
    built = TK.build_trackers(["console", f"jsonl:{tmp_path / 'b.jsonl'}", f"tensorboard:{tmp_path / 'tb2'}"])
    assert len(built.trackers) == 3
    with pytest.raises(ValueError):
        TK.build_trackers(["carrier-pigeon"])
    # a corrupted byte is detected
    blob = bytearray(open(tb.path, "rb").read())
    blob[-6] ^= 0xFF
    open(tb.path, "wb").write(bytes(blob))
    with pytest.raises(ValueError):
        TK.read_scalar_events(tb.path)


def test_api_llm_runtime(tmp_path):
    from spiraltorch_b200 import api_llm as L
    chat = {"model": "m", "choices": [{"message": {"content": "hello spiral world"}, "finish_reason": "stop",
                                       "logprobs": {"content": [{"logprob": -0.1, "top_logprobs": [{"logprob": -0.1}, {"logprob": -3.0}]}]}}],
            "usage": {"prompt_tokens": 10, "completion_tokens": 30}}
    assert L.text_from_response(chat) == "hello spiral world"
    assert L.usage_from_response(chat) == {"prompt_tokens": 10.0, "completion_tokens": 30.0, "total_tokens": 40.0}
    assert L.top_probability_from_response(chat) == pytest.approx(math.exp(-0.1))
    anthropic = {"content": [{"type": "text", "text": "abc"}, {"type": "text", "text": "def"}], "stop_reason": "max_tokens",
                 "usage": {"input_tokens": 5, "output_tokens": 2}}
    assert L.text_from_response(anthropic) == "abcdef" and L.finish_reason_from_response(anthropic) == "max_tokens"
    responses = {"output": [{"content": [{"text": "xy"}]}], "status": "completed"}
    assert L.text_from_response(responses) == "xy"

    class Obj:
        output_text = "from attr"
        usage = None
    assert L.text_from_response(Obj()) == "from attr"
    part = L.partial_from_response(chat, prompt="p" * 40, provider="x", latency_ms=500.0)
    m = part.metrics
    assert m["speed"] == pytest.approx(math.tanh(60.0 / 64.0)) and m["memory"] == pytest.approx(math.tanh(40 / 2048))
    assert m["stability"] == pytest.approx(0.65 * 0.95 + 0.35 * math.exp(-0.1)) and m["drs"] == pytest.approx(math.tanh(0.5))
    assert len(m["gradient"]) == 4 and part.telemetry["api_llm.finish_reason_stop"] == 1.0
    assert L.partial_from_response(anthropic).metrics["stability"] == pytest.approx(0.65 * 0.45 + 0.35 * 0.65)
    now = [0.0]

    def clock():
        now[0] += 0.25
        return now[0]
    rt = L.ApiLLMZSpaceRuntime(lambda prompt, **kw: {"choices": [{"text": prompt.upper(), "finish_reason": "stop"}]},
                               provider="local", model="echo", trace_path=str(tmp_path / "t.jsonl"), clock=clock)
    summary = rt.run_suite(["alpha beta", "gamma"])
    assert summary["events"] == 2 and summary["finish_reasons"] == {"stop": 2} and summary["mean_latency_ms"] == pytest.approx(250.0)
    assert rt.traces[0].text == "ALPHA BETA" and set(rt.fused) == set(L.METRIC_KEYS)
    events = L.load_trace_events(str(tmp_path / "t.jsonl"))
    assert len(events) == 2 and events[1]["model"] == "echo"
    cmp_ = L.compare_trace_runs(events[:1], events[1:])
    assert set(cmp_["delta"]) >= {"mean_speed", "mean_latency_ms"}
    with pytest.raises(ValueError):
        L.metric_gradient_projection({}, 0)


def test_latency_advisor_and_ztiger_gain():
    """Parity: crates/julia-ffi-poc/src/lib.rs."""
    import math
    from spiraltorch_b200.advisors import ZTigerOptim, latency_score
    assert latency_score(16, 6) == 7.0
    with pytest.raises(RuntimeError):
        latency_score(16, 6, engine="julia")
    z = ZTigerOptim(0.5)
    assert z.curvature() == -1.0 and z.gain() == 1.0
    g = z.update(0.5, [1.0, -2.0])
    mean = (1.0 * 0.5 + 2.0 * 1.0) / 2
    assert abs(g - (math.tanh(mean * math.tanh(1.0) / 0.5) + 1.0)) < 1e-12
    for _ in range(40):
        z.update(0.5, [])
    assert z.gain() == 1.0                                    # the 32-step window has forgotten the burst


def test_device_caps_heuristics():
    """Parity: crates/st-core/src/backend/device_caps.rs unit tests."""
    from spiraltorch_b200.device_caps import DeviceCaps, DeviceCapsError, parse_backend
    c = DeviceCaps.b200()
    assert (c.lane_width, c.max_workgroup, c.sm_count, c.shared_mem_per_workgroup) == (32, 1024, 148, 227 * 1024)
    assert c.align_workgroup(33) == 64 and c.align_workgroup(5000) == 1024 and c.align_workgroup(1) == 32
    assert c.occupancy_score(0) == 0.0 and c.occupancy_score(1024) > c.occupancy_score(64)
    assert c.recommended_workgroup() == 256 and c.recommended_workgroup(40) == 64
    assert c.preferred_tile(100_000) == 2048 and c.preferred_tile(100, hint=100) == 128
    t, ct = c.recommended_tiles(50304)
    assert t == 928 and ct == 512                       # 227 KB / (8 B x 32 lanes) = 908 -> 928 after warp alignment
    assert c.with_shared_mem(None).recommended_tiles(50304) == (16384, 512)
    small = c.with_shared_mem(16 * 1024).recommended_tiles(50304)
    assert small[0] == 128 and small[1] <= small[0]
    assert c.prefers_two_stage(50304, 8) and c.prefers_two_stage(1024, 256) and not c.prefers_two_stage(1024, 8)
    assert not c.prefers_two_stage(1024, 256, rows=64) and c.prefers_two_stage(1024, 256, rows=1024)
    assert not DeviceCaps.cpu().prefers_two_stage(50304, 8, rows=100)
    assert c.persistent_grid(10_000) == 148 and c.persistent_grid(10) == 10 and c.persistent_grid(10_000, 2) == 296
    assert DeviceCaps.default_lane_quota(64) == 32 and DeviceCaps.default_lane_quota(4) == 8
    assert parse_backend("B200") == "cuda" and parse_backend("webgpu") == "wgpu"
    assert DeviceCaps.for_backend("cpu").backend == "cpu"
    with pytest.raises(DeviceCapsError, match="not part of this build"):
        DeviceCaps.for_backend("hip")
    with pytest.raises(DeviceCapsError, match="unknown"):
        parse_backend("tpu")
    with pytest.raises(DeviceCapsError):
        DeviceCaps("cuda", True, 32, 16).validate()
    assert DeviceCaps.probe().backend in ("cpu", "cuda")


def test_collapse_drive_transitions_and_cooldown():
    """Parity: crates/st-core/src/engine/collapse_drive.rs `transitions_and_cooldown` and trend tests."""
    from spiraltorch_b200.engine import CollapseConfig, CollapseDrive
    d = CollapseDrive(CollapseConfig(enabled=True, hi=2.0, lo=0.5, warmup_steps=0, cooldown_steps=2))
    assert d.update(0.6, 1).kind == "none"
    cmd = d.update(2.2, 2)
    assert cmd.kind == "collapse" and cmd.grad_scale == 0.2 and cmd.max_norm == 1.0 and cmd.lr_decay == 0.1
    assert [d.update(1.8, s).kind for s in (3, 4, 5)] == ["none"] * 3 and d.state == "stable"
    cmd = d.update(0.3, 6)
    assert cmd.kind == "bloom" and cmd.lr_mul == 1.2 and d.diagnostics()["state_scalar"] == 3.0
    assert not CollapseDrive().enabled() and CollapseDrive().update(100.0, 1000).kind == "none"
    w = CollapseDrive(CollapseConfig(enabled=True, warmup_steps=5))
    assert w.update(100.0, 1).kind == "none" and w.state == "warmup"
    # a rising trend collapses before psi reaches `hi`
    t = CollapseDrive(CollapseConfig(enabled=True, hi=10.0, lo=-10.0, warmup_steps=0, cooldown_steps=0,
                                     trend_alpha=1.0, collapse_trend_threshold=0.5))
    assert t.update(1.0, 1).kind == "none"
    cmd = t.update(1.7, 2)
    assert cmd.kind == "collapse" and cmd.due_to_trend and not cmd.due_to_deviation
    auto = CollapseConfig.automated(24, band_focus=0.5, drift_weight=0.1)
    assert auto.enabled and 1.8 <= auto.hi <= 4.5 and 0.2 <= auto.lo <= 0.6 and auto.warmup_steps == 48 and auto.cooldown_steps == 3


def test_dashboard_ring_summary():
    """Parity: crates/st-core/src/telemetry/dashboard.rs tests."""
    from spiraltorch_b200.telemetry import (DashboardBuilder, DashboardEvent, DashboardFrame, DashboardMetric, DashboardRing)
    ring = DashboardRing(3)
    assert ring.summarize() is None
    for i in range(5):
        f = DashboardFrame(float(i))
        f.push_metric(DashboardMetric("loss", 10.0 - i).with_unit("nats").with_trend(-1))
        if i % 2 == 0:
            f.push_metric(DashboardMetric("lr", 0.1))
            f.push_event(DashboardEvent("tick", "warning"))
        ring.push(f)
    assert len(ring) == 3 and ring.latest().timestamp == 4.0
    s = ring.summarize()
    loss = next(m for m in s.metrics if m.name == "loss")
    assert (s.frame_count, s.span_seconds) == (3, 2.0) and s.events == {"warning": 2}
    assert (loss.mean, loss.min, loss.max, loss.latest, loss.samples) == (7.0, 6.0, 8.0, 6.0, 3)
    assert s.top_metric().name == "loss" and ring.summarize(1).frame_count == 1 and not s.is_empty()
    with pytest.raises(ValueError):
        DashboardEvent("x", "fatal")
    b = DashboardBuilder()
    b.record_metric(DashboardMetric("a", 1.0))
    b.record_event("hello")
    fr = b.finish_with_latency()
    assert [m.name for m in fr.metrics] == ["a", "frame_latency_ms"] and fr.events[0].severity == "info"


def test_temporal_spectral_fusion_of_a_lane_window():
    """Parity: crates/st-core/src/backend/temporal_fusion.rs tests."""
    import math
    from spiraltorch_b200.advisors import LaneWindow, TemporalSpectralFusion
    w = LaneWindow(target=64, lower=32, upper=128, stride=32)
    assert w.lanes() == [32, 64, 96, 128] and LaneWindow(8, 8, 8).lanes() == [8]
    f = TemporalSpectralFusion.analyse(w, rows=1024, cols=4096, k=64, lanes=32)
    base = 0.5 * math.log1p(32) + 0.25 * math.log1p(128)
    assert abs(float(f.temporal[0]) - (math.log1p(2.0) + base)) < 1e-5 and f.temporal.numel() == 4
    assert f.spectral.numel() == 2 and f.fusion.shape == (2, 4)
    assert abs(float(f.spectral[0]) - float(f.temporal.sum())) < 1e-4          # bin 0 is the plain sum
    assert torch.allclose(f.fusion[1], f.spectral[1] * f.temporal)
    assert f.dominant_frequency == 0.0 and 0.5 < f.tempo_hint <= 1.0 and f.spectral_energy > 0
    big = TemporalSpectralFusion.analyse(LaneWindow(64, 1, 64), 8, 8, 4, 32)
    assert big.temporal.numel() == 64 and big.spectral.numel() == 8


def test_zspace_partial_fusion():
    """Parity: crates/st-core/src/telemetry/zspace_fusion.rs (`fuse_zspace_partials`, `canonical_metric_name`)."""
    import math
    from spiraltorch_b200.telemetry import (ZSpaceFusionError, ZSpaceTelemetrySummary, canonical_metric_name,
                                            fuse_zspace_partials)
    assert canonical_metric_name("Velocity") == "speed" and canonical_metric_name("drift") == "drs"
    assert canonical_metric_name("canvas_energy") == "canvas_energy" and canonical_metric_name("spin_alignment") == "elliptic_alignment"
    assert canonical_metric_name("bogus") is None
    parts = [{"metrics": {"speed": 1.0, "mem": 4.0}, "weight": 1.0, "gradient": [1.0, 0.0]},
             None,
             {"metrics": {"velocity": 3.0, "bogus": 9.0}, "weight": 3.0, "origin": "b", "gradient": [0.0, 2.0]},
             {"metrics": {"speed": 100.0}, "weight": 0.0}]
    f = fuse_zspace_partials(parts)
    assert f["metrics"] == {"memory": 4.0, "speed": 2.5} and f["gradient"] == [0.25, 1.5]
    assert (f["active_count"], f["suppressed_count"], f["null_count"]) == (2, 1, 1)
    assert fuse_zspace_partials(parts, strategy="max")["metrics"]["speed"] == 3.0
    assert fuse_zspace_partials(parts, strategy="last")["metrics"]["speed"] == 3.0
    assert fuse_zspace_partials(parts, strategy="sum")["metrics"]["speed"] == 10.0
    assert fuse_zspace_partials(parts, strategy="median")["metrics"]["speed"] == 3.0
    assert fuse_zspace_partials(parts, weights=[1.0, 1.0, 1.0, 1.0], strategy="median")["metrics"]["speed"] == 3.0
    ragged = [{"metrics": {}, "gradient": [1.0]}, {"metrics": {}, "gradient": [1.0, 1.0]}]
    with pytest.raises(ZSpaceFusionError, match="differ"):
        fuse_zspace_partials(ragged)
    assert fuse_zspace_partials(ragged, gradient_alignment="pad_zero")["gradient"] == [1.0, 0.5]
    proj = fuse_zspace_partials([{"metrics": {"speed": 0.9, "stability": 0.2}}], metric_gradient_dimension=8)
    assert len(proj["gradient"]) == 8 and proj["sources"][0]["gradient_replaced_by_metric_projection"]
    with pytest.raises(ZSpaceFusionError):
        fuse_zspace_partials(parts, weights=[1.0])
    with pytest.raises(ZSpaceFusionError):
        fuse_zspace_partials(parts, strategy="mode")
    s = ZSpaceTelemetrySummary.from_values([3.0, -4.0])
    assert (s.l1, s.l2, s.linf, s.amplitude) == (7.0, 5.0, 4.0, 7.0) and abs(s.focus - math.tanh(1.5 * s.balance)) < 1e-12
    assert ZSpaceTelemetrySummary.from_values([]).count == 0


def test_prometheus_exporter_serves_metrics_over_http():
    import json
    import urllib.request
    from pathlib import Path
    from spiraltorch_b200.telemetry import PrometheusExporter
    exp = PrometheusExporter()
    exp.record_gauge("step_time_ms", 12.5, labels=(("rank", "0"),))
    server = exp.serve(port=0)
    try:
        port = server.server_address[1]
        body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert '# TYPE spiraltorch_step_time_ms gauge' in body and 'spiraltorch_step_time_ms{rank="0"} 12.5' in body
        with pytest.raises(Exception):
            urllib.request.urlopen(f"http://127.0.0.1:{port}/nope", timeout=5)
    finally:
        server.shutdown()
    root = Path(__file__).resolve().parent.parent / "deploy" / "observability"
    dash = json.loads((root / "grafana.json").read_text())
    assert len(dash["panels"]) == 4 and "9464" in (root / "prometheus.yml").read_text()
