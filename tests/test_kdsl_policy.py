"""Learning layers of the self-rewrite engine (crates/st-kdsl/src/self_mod.rs): update rules and their use by the engine."""
import math

import pytest

from spiraltorch_b200 import kdsl_policy as P
from spiraltorch_b200.kdsl_rewrite import SelfRewriteEngine


def test_bandit_scores_and_decay():
    b = P.HintBandit()
    assert b.score("new") == pytest.approx(0.55) and b.multiplier("new") == pytest.approx(1.0 + 0.55 / 0.65)
    b.observe_success("a", 0.4)
    assert b.arms["a"].mean_gain == pytest.approx(0.4) and b.score("a") == pytest.approx(0.4 + 0.55 * 1.25)   # below min_pulls
    b.observe_success("a", 0.2)
    assert b.arms["a"].mean_gain == pytest.approx(0.4 * 0.65 + 0.2 * 0.35)
    expected = b.arms["a"].mean_gain + 0.55 * math.sqrt(math.log1p(2) / 2)
    assert b.score("a") == pytest.approx(expected)
    b.observe_failure("a")
    assert b.arms["a"].failures == 1 and b.arms["a"].mean_gain == pytest.approx((0.4 * 0.65 + 0.2 * 0.35) / 2)
    assert b.score("a") < expected
    before = b.arms["a"].mean_gain
    b.decay()
    assert b.arms["a"].mean_gain == pytest.approx(before * 0.97) and b.snapshots()[0]["key"] == "a"
    b.observe_success("x", float("nan"))
    assert "x" not in b.arms
    assert 0.3 <= P.HintBandit(temperature=0.1).multiplier("zz") <= 4.0


def test_chain_policy_is_a_td_update_over_truncated_chains():
    m = P.ChainPolicyModel(horizon=2)
    assert m.score(["a"]) == pytest.approx(0.35) and m.score([]) == 0.0
    m.observe(["b"], 1.0, True)
    m.observe(["a", "b"], 0.5, True)                       # target = 0.5 + 0.55 * V(b) = 1.05
    assert m.values["a -> b"].value == pytest.approx(1.05)
    m.observe(["z", "a", "b"], 0.0, False)                 # truncated to the last two; blends towards 0 + 0.55 * 1.0
    assert m.values["a -> b"].value == pytest.approx(1.05 * 0.65 + 0.55 * 0.35) and "z -> a -> b" not in m.values
    v = m.values["a -> b"]
    assert m.score(["a", "b"]) == pytest.approx(v.value + 0.35 / math.sqrt(2) - 0.175)     # failed last: half the bonus off
    assert m.multiplier(["a", "b"]) == pytest.approx(1.0 + m.score(["a", "b"]) * 0.3)
    m.decay()
    assert m.values["b"].value == pytest.approx(0.96)
    assert P.chain_signature([]) == "<empty>"


def test_chain_feedback_score():
    f = P.ChainFeedback()
    f.reward(0.4, True, 0.5)
    f.reward(-1.0, False, 0.5)                             # negative rewards count as zero
    assert f.uses == 2 and f.successes == 1 and f.ema_reward == pytest.approx(0.2) and f.total_reward == pytest.approx(0.4)
    assert f.score() == pytest.approx(0.2 * 0.6 + 0.4 * 0.2 + 0.5 * 0.2) and P.ChainFeedback().score() == 0.0


def test_transition_graph_boosts_and_prunes():
    g = P.HintTransitionGraph(fanout=2)
    g.observe(None, "a", 0.2, 1.0, 1.0)
    assert g.boost(None, "a") == pytest.approx(0.5 * (1.0 + 0.2 * 0.35)) and g.boost("a", "b") == 0.0
    g.observe("a", "b", 0.4, 0.5, 0.0)
    s1 = (0.4 + 0.05) * 1.25
    g.observe("a", "b", 0.1, 0.0, 0.0)
    e = g.edges["a"][0]
    assert e.strength == pytest.approx(s1 * 0.88 + 0.15) and e.total_gain == pytest.approx(0.4 * 0.88 + 0.1) and e.hits == 2
    g.observe("a", "c", 0.0, 0.0, 0.0)
    g.observe("a", "d", 5.0, 1.0, 1.0)                     # strongest; the fan-out of 2 drops the weakest ("c")
    assert [x.to for x in g.edges["a"]] == ["d", "b"] and g.edges["a"][0].strength == 3.5
    g.penalize_target("d")
    assert g.edges["a"][0].strength == pytest.approx(1.75) or g.edges["a"][1].strength == pytest.approx(1.75)
    assert all(s["from"] != P.ROOT for s in g.snapshots())
    for _ in range(200):
        g.decay()
    assert not g.edges


def test_saga_prefers_longer_matching_prefixes():
    s = P.HintSagaTracker(depth=2)
    s.observe([], "x", 0.3, 1.0, 1.0)
    base = s.boost([], "x")
    assert base == pytest.approx(min((0.33 * 1.8) * (1.0 + 0.3 * 0.3), 4.0))
    s.observe(["a", "b"], "y", 0.3, 1.0, 1.0)
    assert set(s.sequences) == {(), ("b",), ("a", "b")}
    short, long_ = s.boost(["q", "b"], "y"), s.boost(["a", "b"], "y")
    assert long_ > short > 0.0 and s.boost(["a", "b"], "nope") == 0.0
    s.set_depth(0)
    assert not s.sequences and s.boost(["a"], "y") == 0.0


def test_relation_graph_and_diversity_governor():
    r = P.HintRelationGraph(max_neighbors=1)
    r.observe_chain(["a", "b", "c"], 0.5)
    r.observe_edge("a", "b", 1.0)
    r.observe_edge("a", "z", 0.0)                          # weaker than a -> b, dropped by the neighbour cap
    assert [e.to for e in r.adjacency["a"]] == ["b"] and r.adjacency["a"][0].strength == pytest.approx(1.5)
    assert r.snapshots()[0]["mean_reward"] == pytest.approx(0.75)
    d = P.DiversityGovernor(window=2, threshold=0.1, cooldown=2)
    d.record_success(0.01, fresh=False)
    assert d.debt == 1 and d.should_force_fresh()
    d.record_success(0.5, fresh=True)                      # a good fresh generation pays the debt and starts the cooldown
    assert d.debt == 0 and d.cooldown_left == 2 and not d.should_force_fresh()
    d.record_failure()
    assert d.debt == 0                                     # failures during the cooldown do not add debt
    d.advance_cycle(); d.advance_cycle()
    d.record_failure()
    assert d.debt == 1 and d.should_force_fresh() and d.snapshot()["mean_gain"] == pytest.approx(0.0)


def test_quality_model_learns_a_separable_rule():
    q = P.HintQualityModel(lr=0.5)
    for _ in range(300):
        q.observe(1.0, 0.8, 1.0, 0.9, 0, True)
        q.observe(0.0, 0.0, 0.0, 0.1, 20, False)
    assert q.predict(q.features(1.0, 0.8, 1.0, 0.9, 0)) > 0.8 and q.predict(q.features(0.0, 0.0, 0.0, 0.1, 20)) < 0.3
    assert q.snapshot()["accuracy"] > 0.9 and q.features(9.0, -1.0, 0.5, 3.0, None) == [2.0, 0.0, 0.5, 1.0, 0.0]
    assert q.score(0.2, 0.4, 0.6, 1.0, 0) == pytest.approx(q.predict(q.features(0.4, 0.4, 0.6, 1.0, 0)) * (1.0 + 0.6 + 0.2))
    c = P.ContextCluster.new(0b1010, 0.5, 0.5)
    c.update(0b1010, 0.3, 1.0, 0.9)
    assert c.total_gain == pytest.approx(0.75) and c.hits == 2 and c.momentum == pytest.approx(0.25 * 0.9 + 0.3) and c.signature == 0b1010


def test_engine_feeds_and_consults_the_policy_stack():
    from spiraltorch_b200.kdsl import Ctx
    src = "soft(radix, 2, 0.1, true);"
    ctx = Ctx(r=64, c=4096, k=16, sg=True)
    eng = SelfRewriteEngine().with_eta_floor(0.9).with_saga_depth(2).with_bandit_explore(0.3).enable_trace_mode(32)
    first = eng.tick(src, ctx, None, 0.1)
    assert first is not None and eng.generator_calls == 1
    key = eng.cached_keys()[0]
    assert eng.bandit_snapshots()[0]["key"] == key and eng.policy.last_key == key
    assert eng.policy.transitions.boost(None, key) > 0.0 and eng.saga_snapshots()[0]["to"] == key
    assert eng.chain_policy_snapshots()[0]["chain"] == key and eng.chain_feedback()[0]["uses"] == 1
    second = eng.tick(src, ctx, None, 0.1)                # the cached set is reused; its own transition now exists
    assert second is not None and eng.generator_calls == 1
    assert eng.transition_snapshots() and eng.transition_snapshots()[0]["from"] == key
    assert eng.policy.priority_multiplier(key) > 1.0 and eng.quality_model()["updates"] >= 2
    # stalled gains put the governor in debt and the next tick goes to the generator even though the cache could serve
    eng.policy.diversity.debt, eng.policy.diversity.cooldown_left = 2, 0
    third = eng.tick(src, ctx, None, 0.1)
    assert third is not None and eng.generator_calls == 2 and any(k == "DiversityForce" for k, _ in eng.take_trace())
