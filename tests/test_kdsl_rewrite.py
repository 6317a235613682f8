"""SpiralK rewrite helpers and the self-rewrite engine (reference behaviour: crates/st-kdsl/src/auto.rs and
src/self_mod.rs with their tests)."""
import math

import pytest

from spiraltorch_b200.kdsl import Ctx, WilsonMetrics
from spiraltorch_b200.kdsl_rewrite import (AiRewriteConfig, AiRewriteError, AiRewritePrompt, HeuristicHint,
                                           SelfRewriteEngine, context_affinity, ctx_signature, hint_key,
                                           rewrite_with_ai, rewrite_with_wilson, synthesize_program, template_generator)

CTX = Ctx(r=1024, c=16384, k=512, sg=True, sgc=256, kc=1024, tile_cols=128, radix=4, segments=2)


def test_synthesize_and_wilson_gate():
    hints = [HeuristicHint.new("radix", "radix", 0.8, "true")]
    script = synthesize_program("algo: 1", hints)
    assert script.startswith("algo: 1;") and "soft (radix, radix, 0.8, true);" in script
    low = WilsonMetrics(10.0, 9.9, 64, 128)
    out, src = rewrite_with_wilson("wg: 256;", CTX, low, hints, 0.02, 0.5)
    assert src == "wg: 256;" and not out.soft
    good = WilsonMetrics(10.0, 6.0, 96, 128)
    out, src = rewrite_with_wilson("wg: 256;", CTX, good, [HeuristicHint.new("tile_cols", "kc", 0.9, "c > 4096")], 0.05, 0.5)
    assert "tile_cols" in src and out.hard.get("wg") == 256 and out.soft and out.soft[0].value == 1024


def test_template_generator_and_ai_rewrite():
    cfg = AiRewriteConfig("template")
    prompt = AiRewritePrompt("wg: 128;", CTX, WilsonMetrics(10.0, 8.0, 90, 100), device_guard="sg")
    hints = template_generator(cfg, prompt)
    assert [h.field for h in hints] == ["tile_cols", "radix", "segments"]
    assert hints[0].value_expr == "max(128, 153)" and hints[1].value_expr == "4" and hints[2].value_expr == "4"
    out, script, used = rewrite_with_ai("wg: 128;", CTX, cfg, prompt)
    assert len(out.soft) == 3 and used == hints
    with pytest.raises(AiRewriteError) as e:
        rewrite_with_ai("wg: 128;", CTX, cfg, prompt, lambda c, p: [])
    assert e.value.kind == "Empty"
    with pytest.raises(AiRewriteError) as e:
        rewrite_with_ai("wg: 128;", CTX, AiRewriteConfig("m", max_hints=2), prompt)
    assert e.value.kind == "TooManyHints"
    with pytest.raises(AiRewriteError) as e:
        rewrite_with_ai("wg: 128;", CTX, cfg, prompt, lambda c, p: [HeuristicHint("radix", "((", "1.0")])
    assert e.value.kind == "Dsl"


def test_signature_and_affinity():
    assert ctx_signature(CTX) == ctx_signature(Ctx(**CTX.__dict__))
    other = Ctx(**{**CTX.__dict__, "c": 8192})
    assert ctx_signature(other) != ctx_signature(CTX)
    assert context_affinity(5, 5) == 1.0 and context_affinity(0, (1 << 64) - 1) == 0.0
    assert hint_key([HeuristicHint("a", "b", "c", "d"), HeuristicHint("e", "f", "g")]) == "a:b:c:d|e:f:g:true"


def test_engine_rewrites_below_floor_and_reuses_cache():
    calls = []

    def gen(cfg, prompt):
        calls.append(prompt.eta_bar)
        return [HeuristicHint.new("radix", 4, 0.9, "true")]
    eng = SelfRewriteEngine(gen, AiRewriteConfig("t", eta_floor=0.4)).enable_trace_mode(16)
    assert eng.tick("wg: 128;", CTX, None, 0.9) is None and not calls          # healthy: nothing to do
    ev = eng.tick("wg: 128;", CTX, None, 0.1)
    assert ev is not None and len(calls) == 1 and "soft (radix, 4" in ev.script and ev.eta_bar > 0.8
    assert eng.cached_keys() == [hint_key(ev.hints)]
    # the smoothed eta is healthy again, an observed dip alone still triggers; the cached hints are reused
    ev2 = eng.tick("wg: 128;", CTX, None, 0.2)
    assert ev2 is not None and len(calls) == 1 and ev2.script == ev.script
    st = eng.hint_statistics()[0]
    assert st.uses == 2 and st.best_gain > 0.6 and st.failures == 0
    kinds = [k for k, _ in eng.take_trace()]
    assert kinds == ["GeneratorSuccess", "CacheReuse"]
    # a very different context falls below the affinity threshold: the generator is asked again
    far = Ctx(r=3, c=7, k=1, sg=False, sgc=5, kc=9, tile_cols=11, radix=13, segments=17)
    eng.with_context_sensitivity(0.99)
    # the cluster opened by the two successes sits on CTX itself and bridges to any context at least half as close
    # as the sensitivity asks, so the cached hints would still be reused ...
    assert context_affinity(ctx_signature(CTX), ctx_signature(far)) < 0.99
    assert eng.cluster_bridge_affinity(ctx_signature(CTX), ctx_signature(far)) == 1.0
    # ... without it the direct affinity decides and the generator is asked again
    eng.clusters.clear()
    eng.tick("wg: 128;", far, None, 0.1)
    assert len(calls) == 2


def test_engine_freezes_hints_that_keep_failing_and_ages_the_cache():
    eng = SelfRewriteEngine(lambda c, p: [HeuristicHint.new("radix", 4, 0.05, "true")],
                            AiRewriteConfig("t", eta_floor=0.9)).with_anomaly_patience(2).with_max_staleness(3)
    ev = eng.tick("wg: 64;", CTX, None, 0.05)
    key = hint_key(ev.hints)
    # the cached hints score tanh(0.9 + 0.05) = 0.74: no help once the observed eta is already above that
    for _ in range(2):
        eng.tick("wg: 64;", CTX, None, 0.8)
    assert key in eng.frozen_hints() and eng.hint_statistics()[0].failures == 2
    eng.with_eta_floor(0.5)
    for _ in range(4):
        eng.tick("wg: 64;", CTX, None, 0.95)                                    # healthy ticks still age the cache
    assert eng.cached_keys() == []


def test_recombination_crosses_cached_hint_sets_before_asking_the_generator():
    assert SelfRewriteEngine.recombine_hints([], []) == [] and SelfRewriteEngine.recombine_hints([1], []) == [1]
    assert SelfRewriteEngine.recombine_hints([1, 2, 3], [4, 5, 6, 7]) == [1, 2, 6, 7]
    calls = []

    def gen(cfg, prompt):
        calls.append(1)
        return [HeuristicHint.new("radix", 8, 0.0, "true")]
    eng = SelfRewriteEngine(gen, AiRewriteConfig("t", eta_floor=0.97)).enable_trace_mode(32).with_recombination_trials(3)
    sig = ctx_signature(CTX)
    a = [HeuristicHint.new("radix", 4, 2.0, "true"), HeuristicHint.new("wg", 64, 0.0, "true")]
    b = [HeuristicHint.new("radix", 2, 0.0, "true"), HeuristicHint.new("wg", 256, 2.0, "true")]
    eng._push_cache(0.6, a, sig)                    # the higher stored eta ranks `a` first, so the cross tried is head(a) + tail(b)
    eng._push_cache(0.1, b, sig)
    # alone each set scores tanh(0.97 + 1.0) = 0.9618, under the observed 0.965; their cross keeps the two heavy rules
    # and scores tanh(0.97 + 2.0) = 0.9947, and is found without a generator call
    ev = eng.tick("wg: 128;", CTX, None, 0.965)
    kinds = [k for k, _ in eng.take_trace()]
    assert ev is not None and not calls and "RecombineSuccess" in kinds
    assert ev.eta_bar == pytest.approx(math.tanh(2.97), abs=1e-6)
    assert hint_key(ev.hints) in eng.cached_keys() and len(eng.cached_keys()) == 3
    assert eng.context_clusters()[0]["signature"] == sig


def test_context_clusters_follow_successes_and_fade():
    eng = SelfRewriteEngine(lambda c, p: [HeuristicHint.new("radix", 4, 0.9, "true")], AiRewriteConfig("t", eta_floor=0.4)).with_cluster_limit(2)
    sig = ctx_signature(CTX)
    eng.tick("wg: 128;", CTX, None, 0.1)
    (c,) = eng.context_clusters()
    assert c["signature"] == sig and c["hits"] == 1 and c["best_gain"] > 0.6
    assert eng.cluster_bridge_affinity(sig, sig) == 1.0
    assert eng.cluster_bridge_affinity(sig ^ ((1 << 40) - 1), sig) == 0.0          # 40 bits away from the cluster: under 0.4
    m0 = c["momentum"]
    for _ in range(3):
        eng.tick("wg: 128;", CTX, None, 0.95)                                       # healthy ticks: clusters only fade
    assert eng.context_clusters()[0]["momentum"] == pytest.approx(m0 * 0.9 ** 3)
    eng.with_cluster_decay(0.001)
    for _ in range(3):
        eng.tick("wg: 128;", CTX, None, 0.95)
    assert eng.context_clusters() == []
