"""SpiralK self-rewrite: hint generation, program synthesis and the engine that decides when to rewrite.

``synthesize_program`` appends ``soft(field, value, weight, condition)`` rules to a SpiralK program;
``rewrite_with_wilson`` does so only when the measured gain clears a threshold and its Wilson lower bound a
confidence; ``rewrite_with_ai`` asks a hint generator.  :class:`SelfRewriteEngine` watches the efficiency
``eta`` reported per tick: while the observed and smoothed ``eta`` stay at or above the floor nothing happens;
below it the engine first tries cached hint sets (ordered by their ``eta``, discounted by staleness and by how
far the current context is from the one they were learnt in), then asks the generator, evaluates the
synthesised program, scores it (``tanh(floor + mean soft weight)``), caches the hints under an FNV signature
of the context and keeps per-hint statistics; hint sets that fail repeatedly are frozen for a cool-down.

Restated from crates/st-kdsl/src/auto.rs (``WilsonMetrics``, ``HeuristicHint``, ``AiRewriteConfig``,
``AiRewritePrompt``, ``TemplateAiGenerator``, ``synthesize_program``, ``rewrite_with_wilson``,
``rewrite_with_ai``) and src/self_mod.rs (``SelfRewriteEngine`` :26, ``tick`` :1761, ``try_cached`` :1828,
``eta_from_out`` :2098, ``hint_key`` :2123, ``age_cache`` :2390, ``context_affinity`` / ``ctx_signature``
:2499-2521).  The reference's further layers (transition graph, sagas, chain policy, hint bandit) refine the
cache ordering and are not rebuilt; the ordering here uses eta, staleness, affinity and the hint's record.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from .kdsl import Ctx, KdslError, Out, Program, WilsonMetrics, should_rewrite

FNV_OFFSET_BASIS, FNV_PRIME, _MASK = 0xCBF29CE484222325, 0x100000001B3, (1 << 64) - 1


class AiRewriteError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass(frozen=True)
class HeuristicHint:
    field: str
    value_expr: str
    weight_expr: str
    condition_expr: str = "true"

    @classmethod
    def new(cls, field: str, value_expr, weight: float, condition_expr: str = "true") -> "HeuristicHint":
        return cls(field, str(value_expr), repr(float(weight)), condition_expr)


@dataclass
class AiRewriteConfig:
    model: str
    max_hints: int = 4
    default_weight: float = 0.72
    eta_floor: float = 0.35


@dataclass
class AiRewritePrompt:
    base_program: str
    ctx: Ctx
    metrics: Optional[WilsonMetrics] = None
    eta_bar: float = 0.5
    device_guard: Optional[str] = None
    notes: list = field(default_factory=list)


def eval_program(src: str, ctx: Ctx) -> Out:
    return Program.parse(src).evaluate(ctx)


def synthesize_program(base_src: str, hints) -> str:
    script = base_src.strip()
    if script and not script.endswith(";"):
        script += ";"
    for h in hints:
        script += f"\nsoft ({h.field}, {h.value_expr}, {h.weight_expr}, {h.condition_expr});"
    return script


def rewrite_with_wilson(base_src: str, ctx: Ctx, metrics: WilsonMetrics, hints, min_gain: float,
                        min_confidence: float) -> tuple:
    base_out = eval_program(base_src, ctx)
    if not should_rewrite(metrics, min_gain, min_confidence):
        return base_out, base_src
    script = synthesize_program(base_src, hints)
    return eval_program(script, ctx), script


def template_generator(config: AiRewriteConfig, prompt: AiRewritePrompt) -> list:
    """Deterministic hint generator: wider column tiles, radix 4 and more segments as the measured gain grows."""
    ctx = prompt.ctx
    gain = prompt.metrics.gain() if prompt.metrics is not None else 0.0
    tile_cols = max(ctx.tile_cols, 32)
    target = int(max(tile_cols * (1.0 + max(gain, 0.0)), tile_cols))
    guard = prompt.device_guard or "true"
    radix = 4 if gain > 0.08 else max(ctx.radix, 2)
    segments = max(ctx.segments, 1) * (2 if gain > 0.12 else 1)
    return [HeuristicHint.new("tile_cols", f"max({ctx.tile_cols}, {target})", config.default_weight, guard),
            HeuristicHint.new("radix", radix, config.default_weight, "true"),
            HeuristicHint.new("segments", segments, config.default_weight, guard)]


def _checked_hints(generator, config, prompt) -> list:
    try:
        hints = list(generator(config, prompt))
    except AiRewriteError:
        raise
    except Exception as exc:  # noqa: BLE001
        raise AiRewriteError("Generator", f"AI generator failed: {exc}") from exc
    if not hints:
        raise AiRewriteError("Empty", "AI generator returned empty hint set")
    if len(hints) > config.max_hints:
        raise AiRewriteError("TooManyHints", f"AI generator produced {len(hints)} hints exceeding the max allowed")
    return hints


def rewrite_with_ai(base_src: str, ctx: Ctx, config: AiRewriteConfig, prompt: AiRewritePrompt,
                    generator: Callable = template_generator) -> tuple:
    hints = _checked_hints(generator, config, prompt)
    script = synthesize_program(base_src, hints)
    try:
        out = eval_program(script, ctx)
    except KdslError as exc:
        raise AiRewriteError("Dsl", f"SpiralK evaluation failed: {exc}") from exc
    return out, script, hints


# ---- engine ----------------------------------------------------------------------------------------------------
@dataclass
class SelfRewriteEvent:
    script: str
    hints: list
    eta_bar: float
    out: Out


@dataclass
class HintStat:
    key: str
    uses: int = 0
    failures: int = 0
    total_gain: float = 0.0
    best_gain: float = 0.0
    last_eta: float = 0.0
    last_affinity: float = 0.0
    last_gain: float = 0.0

    def mean_gain(self) -> float:
        return self.total_gain / self.uses if self.uses else 0.0


@dataclass
class _Cached:
    key: str
    hints: list
    eta: float
    ctx_signature: int
    staleness: int = 0


def ctx_signature(ctx: Ctx) -> int:
    h = FNV_OFFSET_BASIS
    for v in (ctx.r, ctx.c, ctx.k, int(bool(ctx.sg)), ctx.sgc, ctx.kc, ctx.tile_cols, ctx.radix, ctx.segments):
        h = ((h ^ (int(v) & _MASK)) * FNV_PRIME) & _MASK
    return h


def context_affinity(cached: int, current: int) -> float:
    return max(0.0, min(1.0, 1.0 - bin(cached ^ current).count("1") / 64.0))


def hint_key(hints) -> str:
    return "|".join(f"{h.field}:{h.value_expr}:{h.weight_expr}:{h.condition_expr}" for h in hints)


class SelfRewriteEngine:
    def __init__(self, generator: Callable = template_generator, config: Optional[AiRewriteConfig] = None):
        self.generator = generator
        self.config = config or AiRewriteConfig("template")
        self.eta_floor = self.config.eta_floor
        self.max_history, self.cache_limit = 8, 6
        self.ctx_sensitivity, self.staleness_half_life, self.max_staleness = 0.5, 6, 24
        self.anomaly_patience, self.freeze_cooldown = 3, 8
        self.eta_history: deque = deque()
        self.cache: list = []
        self.stats: dict = {}
        self.frozen: dict = {}
        self.trace_limit = 0
        self.trace_log: deque = deque()
        self.generator_calls = 0
        from .kdsl_policy import HintPolicyStack
        self.policy = HintPolicyStack()
        self.recombination_trials = 2
        self.clusters: list = []                 # ContextCluster records of the contexts where hints paid off
        self.cluster_limit, self.cluster_decay = 6, 0.9

    # ---- configuration (builder style, like the reference) ----
    def with_eta_floor(self, v: float): self.eta_floor = v if v > 0 and math.isfinite(v) else self.eta_floor; return self   # noqa: E702
    def with_history(self, n: int): self.max_history = max(1, n); return self                      # noqa: E702
    def with_cache_limit(self, n: int): self.cache_limit = max(1, n); return self                  # noqa: E702
    def with_context_sensitivity(self, v: float): self.ctx_sensitivity = max(0.0, min(1.0, v)); return self    # noqa: E702
    def with_staleness_half_life(self, n: int): self.staleness_half_life = max(1, n); return self  # noqa: E702
    def with_max_staleness(self, n: int): self.max_staleness = max(1, n); return self              # noqa: E702
    def with_anomaly_patience(self, n: int): self.anomaly_patience = max(1, n); return self        # noqa: E702
    def enable_trace_mode(self, limit: int): self.trace_limit = max(1, limit); return self         # noqa: E702
    def with_recombination_trials(self, n: int): self.recombination_trials = max(1, n); return self   # noqa: E702
    def with_cluster_limit(self, n: int): self.cluster_limit = max(1, n); return self              # noqa: E702
    def with_cluster_decay(self, v: float): self.cluster_decay = min(v, 0.999) if v > 0 and math.isfinite(v) else self.cluster_decay; return self   # noqa: E702
    # the learning layers (bandit, chain policy, transition / saga graphs, diversity governor): crates/st-kdsl/src/self_mod.rs:1461-1612
    def with_diversity_window(self, n: int): self.policy.diversity.window = max(1, n); return self                      # noqa: E702
    def with_diversity_threshold(self, v: float): self.policy.diversity.threshold = v if v >= 0 and math.isfinite(v) else self.policy.diversity.threshold; return self   # noqa: E702
    def with_diversity_cooldown(self, n: int): self.policy.diversity.cooldown = max(1, n); return self                  # noqa: E702
    def with_transition_decay(self, v: float): self.policy.transitions.decay_rate = min(v, 0.999) if v > 0 and math.isfinite(v) else self.policy.transitions.decay_rate; return self   # noqa: E702
    def with_transition_fanout(self, n: int): self.policy.transitions.fanout = max(1, n); return self                   # noqa: E702
    def with_saga_depth(self, n: int): self.policy.saga.set_depth(max(0, n)); return self                               # noqa: E702
    def with_saga_decay(self, v: float): self.policy.saga.decay_rate = min(v, 0.999) if v > 0 and math.isfinite(v) else self.policy.saga.decay_rate; return self   # noqa: E702
    def with_saga_fanout(self, n: int): self.policy.saga.fanout = max(1, n); return self                                # noqa: E702
    def with_feedback_gamma(self, v: float): self.policy.feedback_gamma = max(0.01, min(1.0, v)); return self           # noqa: E702
    def with_chain_learning_rate(self, v: float): self.policy.chain_policy.lr = max(0.05, min(1.0, v)); return self     # noqa: E702
    def with_chain_discount(self, v: float): self.policy.chain_policy.discount = max(0.0, min(0.99, v)); return self    # noqa: E702
    def with_chain_explore_bonus(self, v: float): self.policy.chain_policy.explore_bonus = max(0.0, v); return self     # noqa: E702
    def with_chain_horizon(self, n: int): self.policy.chain_policy.horizon = max(1, n); return self                     # noqa: E702
    def with_bandit_explore(self, v: float): self.policy.bandit.explore = max(0.0, v); return self                      # noqa: E702
    def with_bandit_temperature(self, v: float): self.policy.bandit.temperature = max(0.1, v); return self              # noqa: E702
    def with_bandit_learning_rate(self, v: float): self.policy.bandit.learning_rate = max(0.05, min(1.0, v)); return self   # noqa: E702
    def with_bandit_decay(self, v: float): self.policy.bandit.decay_rate = min(v, 0.999) if v > 0 else self.policy.bandit.decay_rate; return self   # noqa: E702
    def with_bandit_min_pulls(self, n: int): self.policy.bandit.min_pulls = max(1, n); return self                      # noqa: E702
    def with_relation_decay(self, v: float): self.policy.relations.decay_rate = v; return self                          # noqa: E702
    def with_relation_fanout(self, n: int): self.policy.relations.max_neighbors = max(1, n); return self                # noqa: E702

    def transition_snapshots(self) -> list: return self.policy.transitions.snapshots()              # noqa: E704
    def saga_snapshots(self) -> list: return self.policy.saga.snapshots()                           # noqa: E704
    def chain_policy_snapshots(self) -> list: return self.policy.chain_policy.snapshots()           # noqa: E704
    def bandit_snapshots(self) -> list: return self.policy.bandit.snapshots()                       # noqa: E704
    def chain_feedback(self) -> list: return self.policy.snapshot()["chain_feedback"]              # noqa: E704
    def relation_graph(self) -> list: return self.policy.relations.snapshots()                      # noqa: E704
    def diversity_snapshot(self) -> dict: return self.policy.diversity.snapshot()                   # noqa: E704
    def quality_model(self) -> dict: return self.policy.quality.snapshot()                          # noqa: E704

    def context_clusters(self) -> list:
        return [{"signature": c.signature, "mean_gain": c.mean_gain(), "best_gain": c.best_gain, "momentum": c.momentum, "hits": c.hits}
                for c in sorted(self.clusters, key=lambda c: -c.best_gain)]

    # ---- introspection ----
    def smoothed_eta(self) -> Optional[float]:
        return sum(self.eta_history) / len(self.eta_history) if self.eta_history else None

    def hint_statistics(self) -> list:
        return sorted(self.stats.values(), key=lambda s: -s.best_gain)

    def frozen_hints(self) -> dict:
        return dict(self.frozen)

    def cached_keys(self) -> list:
        return [c.key for c in self.cache]

    def take_trace(self) -> list:
        out = list(self.trace_log)
        self.trace_log.clear()
        return out

    def _trace(self, kind: str, detail: str) -> None:
        if self.trace_limit:
            self.trace_log.append((kind, detail))
            while len(self.trace_log) > self.trace_limit:
                self.trace_log.popleft()

    # ---- core ----
    def eta_from_out(self, out: Out) -> float:
        if not out.soft:
            return max(self.eta_floor, 0.0)
        mean_w = sum(r.weight for r in out.soft) / len(out.soft)
        return abs(math.tanh(self.eta_floor + mean_w))

    def _eval(self, base_src: str, ctx: Ctx, hints) -> SelfRewriteEvent:
        script = synthesize_program(base_src, hints)
        try:
            out = eval_program(script, ctx)
        except KdslError as exc:
            raise AiRewriteError("Dsl", f"SpiralK evaluation failed: {exc}") from exc
        return SelfRewriteEvent(script, list(hints), self.eta_from_out(out), out)

    def _record_eta(self, eta: float) -> None:
        self.eta_history.append(eta)
        while len(self.eta_history) > self.max_history:
            self.eta_history.popleft()

    def _age(self) -> None:
        for c in self.cache:
            c.staleness += 1
        self.cache = [c for c in self.cache if c.staleness <= self.max_staleness]
        for k in list(self.frozen):
            self.frozen[k] -= 1
            if self.frozen[k] <= 0:
                del self.frozen[k]

    def _priority(self, c: _Cached, sig: int) -> float:
        decay = 0.5 ** (c.staleness / self.staleness_half_life)
        st = self.stats.get(c.key)
        record = 1.0 + (st.mean_gain() if st else 0.0) - 0.25 * (st.failures if st else 0)
        quality = self.policy.quality_score(st.last_gain, st.mean_gain(), st.best_gain, st.last_affinity, c.staleness) if st else 0.0
        return (c.eta + quality) * decay * context_affinity(c.ctx_signature, sig) * max(record, 0.05) * self.policy.priority_multiplier(c.key)

    def _penalize(self, key: str) -> None:
        st = self.stats.setdefault(key, HintStat(key))
        st.failures += 1
        self.policy.record_failure(key, st.mean_gain(), st.best_gain, st.last_affinity)
        if st.failures >= self.anomaly_patience and key not in self.frozen:
            self.frozen[key] = self.freeze_cooldown
            self._trace("Frozen", f"key={key} failures={st.failures}")

    def _success(self, key: str, observed: float, eta: float, affinity: float, fresh: bool = False, sig: Optional[int] = None) -> float:
        gain = max(0.0, eta - observed)
        st = self.stats.setdefault(key, HintStat(key))
        st.uses += 1
        st.total_gain += gain
        st.best_gain = max(st.best_gain, gain)
        st.last_eta, st.last_affinity, st.last_gain = eta, affinity, gain
        self.policy.record_success(key, gain, affinity, affinity, fresh, st.mean_gain(), st.best_gain)
        if sig is not None:
            self._promote_cluster(sig, gain, affinity)
        return gain

    # ---- context clusters (crates/st-kdsl/src/self_mod.rs:2419-2497) ----
    def _promote_cluster(self, sig: int, gain: float, affinity: float) -> None:
        """Fold a success into the nearest cluster of context signatures, or open a new one (the weakest goes when full)."""
        if not math.isfinite(gain):
            return
        from .kdsl_policy import ContextCluster
        near = max(self.clusters, key=lambda c: context_affinity(c.signature, sig), default=None)
        closeness = context_affinity(near.signature, sig) if near is not None else 0.0
        if closeness > 0.0:
            near.update(sig, gain, affinity * closeness, self.cluster_decay)
            return
        if len(self.clusters) >= self.cluster_limit:
            self.clusters.remove(min(self.clusters, key=lambda c: c.best_gain))
        self.clusters.append(ContextCluster.new(sig, gain, affinity))

    def _decay_clusters(self) -> None:
        for c in self.clusters:
            c.total_gain *= self.cluster_decay
            c.momentum *= self.cluster_decay
        self.clusters = [c for c in self.clusters if c.total_gain > 1e-4 or c.momentum > 1e-4]

    def cluster_bridge_affinity(self, cached: int, current: int) -> float:
        """Affinity of two contexts through a cluster close to both: sqrt(a_cached · a_current) times the cluster's
        energy min(1 + best gain + momentum/2, 1.6), capped at 1; clusters under 0.4 to the cached side or 0.2 to the
        current side do not bridge."""
        best = 0.0
        for c in self.clusters:
            to_cached, to_current = context_affinity(c.signature, cached), context_affinity(c.signature, current)
            if to_cached < 0.4 or to_current < 0.2:
                continue
            energy = min(1.0 + c.best_gain + c.momentum * 0.5, 1.6)
            best = max(best, min(min(math.sqrt(to_cached * to_current), 1.0) * energy, 1.0))
        return best

    def _effective_affinity(self, cached: int, current: int) -> float:
        """Direct affinity, lifted to the bridged one when the direct one is at least half the sensitivity."""
        aff = context_affinity(cached, current)
        return max(aff, self.cluster_bridge_affinity(cached, current)) if aff >= self.ctx_sensitivity * 0.5 else aff

    # ---- recombination (crates/st-kdsl/src/self_mod.rs:1902-1995, 2136-2152) ----
    @staticmethod
    def recombine_hints(a: list, b: list) -> list:
        """First half of `a` (rounded up) followed by the second half of `b`; an empty side yields the other."""
        if not a or not b:
            return list(a or b)
        return list(a[:(len(a) + 1) // 2]) + list(b[len(b) // 2:])

    def _try_recombined(self, base_src: str, ctx: Ctx, observed_eta: float, sig: int) -> Optional[SelfRewriteEvent]:
        """Cross the four best cached hint sets pairwise, at most `recombination_trials` evaluations per tick."""
        if len(self.cache) < 2 or self.recombination_trials == 0:
            return None
        pool = sorted(self.cache, key=lambda c: -self._priority(c, sig))[:4]
        attempts = 0
        for i, a in enumerate(pool):
            for b in pool[i + 1:]:
                if attempts >= self.recombination_trials:
                    return None
                if a.key == b.key:
                    continue
                combined = self.recombine_hints(a.hints, b.hints)
                key = hint_key(combined)
                if not combined or key in self.frozen or key in (a.key, b.key):
                    continue
                attempts += 1
                event = self._eval(base_src, ctx, combined)
                if event.eta_bar <= observed_eta:
                    self._trace("RecombineFailure", f"key={key} eta={event.eta_bar:.3f}")
                    st = self.stats.setdefault(key, HintStat(key))
                    st.uses += 1
                    st.last_eta = event.eta_bar
                    st.last_gain *= 0.5
                    st.last_affinity *= 0.5
                    st.total_gain *= 0.5
                    self._penalize(key)
                    continue
                aff = min(max((context_affinity(a.ctx_signature, sig) + context_affinity(b.ctx_signature, sig)) * 0.5, 0.1), 1.0)
                gain = self._success(key, observed_eta, event.eta_bar, aff, sig=sig)
                self._record_eta(event.eta_bar)
                self._push_cache(event.eta_bar, combined, sig)
                self._trace("RecombineSuccess", f"key={key} from=({a.key}, {b.key}) gain={gain:.3f} affinity={aff:.3f}")
                return event
        return None

    def _push_cache(self, eta: float, hints, sig: int) -> None:
        key = hint_key(hints)
        self.cache = [c for c in self.cache if c.key != key]
        self.cache.insert(0, _Cached(key, list(hints), eta, sig))
        del self.cache[self.cache_limit:]

    def tick(self, base_src: str, ctx: Ctx, metrics: Optional[WilsonMetrics], observed_eta: float) -> Optional[SelfRewriteEvent]:
        self._age()
        self.policy.advance()
        self._decay_clusters()
        smoothed = self.smoothed_eta()
        if observed_eta >= self.eta_floor and (observed_eta if smoothed is None else smoothed) >= self.eta_floor:
            return None
        sig = ctx_signature(ctx)
        force_fresh = self.policy.should_force_fresh()          # stalled gains: skip the cache and ask the generator
        if force_fresh:
            self._trace("DiversityForce", f"debt={self.policy.diversity.debt}")
        for c in ([] if force_fresh else sorted(self.cache, key=lambda c: -self._priority(c, sig))):
            if c.key in self.frozen:
                self._trace("CachePenalty", f"skip frozen key={c.key}")
                continue
            aff = self._effective_affinity(c.ctx_signature, sig)
            if aff < self.ctx_sensitivity or c.eta <= observed_eta:
                self._penalize(c.key)
                continue
            event = self._eval(base_src, ctx, c.hints)
            if event.eta_bar <= observed_eta:
                self._penalize(c.key)
                self._trace("CachePenalty", f"failed reuse key={c.key} eta={event.eta_bar:.3f}")
                continue
            gain = self._success(c.key, observed_eta, event.eta_bar, aff, sig=sig)
            c.eta, c.staleness, c.ctx_signature = event.eta_bar, 0, sig
            self._record_eta(event.eta_bar)
            self._trace("CacheReuse", f"key={c.key} gain={gain:.3f} affinity={aff:.3f}")
            return event
        if not force_fresh:
            event = self._try_recombined(base_src, ctx, observed_eta, sig)
            if event is not None:
                return event
        prompt = AiRewritePrompt(base_src, ctx, metrics, observed_eta if observed_eta > 0 and math.isfinite(observed_eta) else 0.5)
        self.generator_calls += 1
        hints = _checked_hints(self.generator, self.config, prompt)
        event = self._eval(base_src, ctx, hints)
        self._record_eta(event.eta_bar)
        self._push_cache(event.eta_bar, event.hints, sig)
        gain = self._success(hint_key(event.hints), observed_eta, event.eta_bar, 1.0, fresh=True, sig=sig)
        self._trace("GeneratorSuccess", f"key={hint_key(event.hints)} gain={gain:.3f} eta={event.eta_bar:.3f}")
        return event
