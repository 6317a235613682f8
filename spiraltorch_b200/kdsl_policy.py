"""Learning layers of the SpiralK self-rewrite engine: what it remembers about its hint sets beyond the cache itself.

* :class:`HintBandit` — a UCB-style arm per hint set (mean gain, exploration bonus, failure penalty);
* :class:`ChainFeedback` / :class:`ChainPolicyModel` — rewards of whole hint chains, and a temporal-difference value per
  chain signature truncated to a horizon;
* :class:`HintRelationGraph`, :class:`HintTransitionGraph`, :class:`HintSagaTracker` — which hint set tends to follow
  which: pairwise relations inside a chain, decayed first-order transitions with a fan-out cap, and multi-step prefixes
  ("sagas") up to a depth;
* :class:`DiversityGovernor` — asks for a fresh generation when the recent gains stall;
* :class:`HintQualityModel` — an online logistic model of "will this reuse succeed" on five features;
* :class:`ContextCluster` — running gain statistics of one context signature neighbourhood;
* :class:`HintPolicyStack` — the bundle the engine consults (`priority_multiplier`) and feeds (`record_success`,
  `record_failure`, `advance`).

Reference parity: crates/st-kdsl/src/self_mod.rs (`ChainFeedback` :84-126, `ChainPolicyModel` :173-463, `HintBandit`
:196-337, `HintRelationGraph` :452-568, `HintTransitionGraph` :754-875, `HintSagaTracker` :877-1025,
`DiversityGovernor` :1027-1121, `HintQualityModel` :1123-1246, `ContextCluster` :1248-1292, the way the bonuses
multiply in `cache_priority` :2041-2079).
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

ROOT = "__root__"


def _clamp(x: float, lo: float, hi: float) -> float:
    return min(max(x, lo), hi)


# ---------------------------------------------------------------------------------------------------------------
@dataclass
class BanditArm:
    pulls: int = 0
    failures: int = 0
    mean_gain: float = 0.0
    best_gain: float = 0.0
    last_gain: float = 0.0


class HintBandit:
    def __init__(self, explore: float = 0.55, temperature: float = 0.65, learning_rate: float = 0.35, decay: float = 0.97, min_pulls: int = 2):
        self.arms: Dict[str, BanditArm] = {}
        self.total_pulls = 0
        self.explore, self.temperature, self.learning_rate, self.decay_rate, self.min_pulls = explore, temperature, learning_rate, decay, min_pulls

    def observe_success(self, key: str, gain: float) -> None:
        if not math.isfinite(gain):
            return
        arm = self.arms.setdefault(key, BanditArm())
        arm.pulls += 1
        lr = _clamp(self.learning_rate, 0.05, 1.0)
        arm.mean_gain = gain if arm.pulls == 1 else arm.mean_gain * (1.0 - lr) + gain * lr
        arm.best_gain, arm.last_gain = max(arm.best_gain, gain), gain
        arm.failures -= arm.failures // 4
        self.total_pulls += 1

    def observe_failure(self, key: str) -> None:
        arm = self.arms.setdefault(key, BanditArm())
        arm.failures += 1
        arm.pulls += 1
        arm.mean_gain *= 0.5
        arm.last_gain *= 0.5
        self.total_pulls += 1

    def score(self, key: str) -> float:
        arm = self.arms.get(key)
        if arm is None:
            return max(self.explore, 0.0)
        pulls, total = max(arm.pulls, 1), max(self.total_pulls, 1)
        if pulls < max(self.min_pulls, 1):
            bonus = self.explore * 1.25
        elif self.explore <= 0.0:
            bonus = 0.0
        else:
            bonus = self.explore * math.sqrt(max(math.log1p(total) / pulls, 0.0))
        return arm.mean_gain + bonus - arm.failures * 0.05

    def multiplier(self, key: str) -> float:
        return _clamp(1.0 + self.score(key) / max(self.temperature, 0.1), 0.3, 4.0)

    def decay(self) -> None:
        d = _clamp(self.decay_rate, 0.5, 0.999)
        for arm in self.arms.values():
            arm.mean_gain *= d
            arm.last_gain *= d
            if abs(arm.mean_gain) < 1e-4 and arm.failures > 0:
                arm.failures -= 1
        self.total_pulls -= self.total_pulls // 16

    def snapshots(self) -> List[dict]:
        snaps = [{"key": k, "pulls": a.pulls, "failures": a.failures, "mean_gain": a.mean_gain, "best_gain": a.best_gain,
                  "last_gain": a.last_gain, "score": self.score(k)} for k, a in self.arms.items()]
        return sorted(snaps, key=lambda s: -s["score"])


# ---------------------------------------------------------------------------------------------------------------
@dataclass
class ChainFeedback:
    uses: int = 0
    successes: int = 0
    total_reward: float = 0.0
    ema_reward: float = 0.0
    last_reward: float = 0.0
    last_outcome: bool = True

    def reward(self, reward: float, success: bool, gamma: float) -> None:
        self.uses += 1
        self.successes += 1 if success else 0
        reward = max(reward, 0.0)
        self.total_reward += reward
        blend = _clamp(gamma, 0.01, 1.0)
        self.ema_reward = reward if self.uses == 1 else self.ema_reward * (1.0 - blend) + reward * blend
        self.last_reward, self.last_outcome = reward, success

    def score(self) -> float:
        if self.uses == 0:
            return 0.0
        return self.ema_reward * 0.6 + self.total_reward * 0.2 + (self.successes / self.uses) * 0.2


def chain_signature(chain: Sequence[str]) -> str:
    return " -> ".join(chain) if chain else "<empty>"


@dataclass
class _ChainValue:
    value: float = 0.0
    visits: int = 0
    last_reward: float = 0.0
    last_outcome: bool = True


class ChainPolicyModel:
    """V(chain) <- (1 - lr) V + lr (reward + discount V(chain without its first element))."""

    def __init__(self, lr: float = 0.35, discount: float = 0.55, decay: float = 0.96, explore_bonus: float = 0.35, horizon: int = 4):
        self.values: Dict[str, _ChainValue] = {}
        self.lr, self.discount, self.decay_rate, self.explore_bonus, self.horizon = lr, discount, decay, explore_bonus, max(horizon, 1)

    def _truncate(self, chain: Sequence[str]) -> Sequence[str]:
        return chain[-self.horizon:] if len(chain) > self.horizon else chain

    def observe(self, chain: Sequence[str], reward: float, success: bool) -> None:
        if not chain:
            return
        tr = self._truncate(chain)
        tail = self.values.get(chain_signature(tr[1:]), _ChainValue()).value if len(tr) > 1 else 0.0
        target = reward + self.discount * tail
        e = self.values.setdefault(chain_signature(tr), _ChainValue())
        e.visits += 1
        e.last_reward, e.last_outcome = reward, success
        e.value = target if e.visits == 1 else e.value * (1.0 - self.lr) + target * self.lr

    def score(self, chain: Sequence[str]) -> float:
        if not chain:
            return 0.0
        e = self.values.get(chain_signature(self._truncate(chain)))
        if e is None:
            return self.explore_bonus
        explore = self.explore_bonus / max(math.sqrt(max(e.visits, 1)), 1.0) if self.explore_bonus > 0.0 else 0.0
        return e.value + explore - (0.0 if e.last_outcome else self.explore_bonus * 0.5)

    def multiplier(self, chain: Sequence[str]) -> float:
        return _clamp(1.0 + self.score(chain) * 0.3, 0.25, 3.5)

    def decay(self) -> None:
        d = _clamp(self.decay_rate, 0.5, 0.999)
        for e in self.values.values():
            e.value *= d
            e.last_reward *= d

    def snapshots(self) -> List[dict]:
        return sorted(({"chain": k, "value": e.value, "visits": e.visits, "last_reward": e.last_reward, "last_outcome": e.last_outcome}
                       for k, e in self.values.items()), key=lambda s: -s["value"])


# ---------------------------------------------------------------------------------------------------------------
@dataclass
class _Edge:
    to: str
    strength: float          # weight / strength / synergy, depending on the graph
    total_gain: float
    best_gain: float = 0.0
    hits: int = 0

    def mean_gain(self) -> float:
        return self.total_gain / self.hits if self.hits else 0.0


class HintRelationGraph:
    """Pairwise "a was followed by b inside a rewarded chain" edges, strongest ``max_neighbors`` kept per node."""

    def __init__(self, max_neighbors: int = 6, decay: float = 0.94):
        self.adjacency: Dict[str, List[_Edge]] = {}
        self.max_neighbors, self.decay_rate = max(max_neighbors, 1), decay

    def observe_chain(self, chain: Sequence[str], reward: float) -> None:
        for a, b in zip(chain, chain[1:]):
            self.observe_edge(a, b, reward)

    def observe_edge(self, a: str, b: str, reward: float) -> None:
        reward = max(reward, 0.0)
        edges = self.adjacency.setdefault(a, [])
        e = next((x for x in edges if x.to == b), None)
        if e is None:
            edges.append(_Edge(b, 1.0, reward, reward, 1 if reward > 0.0 else 0))
        else:
            e.strength = min(e.strength + reward * 0.5, 16.0)
            e.total_gain += reward
            e.hits += 1 if reward > 0.0 else 0
        edges.sort(key=lambda x: -x.strength)
        del edges[self.max_neighbors:]

    def decay(self) -> None:
        d = _clamp(self.decay_rate, 0.5, 0.999)
        for edges in self.adjacency.values():
            edges[:] = [e for e in edges if e.strength > 1e-3 or e.total_gain > 1e-3]
            for e in edges:
                e.strength *= d
                e.total_gain *= d

    def snapshots(self) -> List[dict]:
        out = [{"from": a, "to": e.to, "weight": e.strength, "hits": e.hits, "mean_reward": e.mean_gain()} for a, es in self.adjacency.items() for e in es]
        return sorted(out, key=lambda s: -s["weight"])


class HintTransitionGraph:
    """First-order transitions with exponentially decayed strength; ``None`` as the source means the start of a run."""

    def __init__(self, decay: float = 0.88, fanout: int = 4):
        self.edges: Dict[str, List[_Edge]] = {}
        self.decay_rate, self.fanout = decay, max(fanout, 1)

    def observe(self, source: Optional[str], to: str, gain: float, affinity: float, ctx_affinity: float) -> None:
        gain = max(gain, 0.0)
        signal = (gain + 0.05) * (1.0 + affinity * 0.5 + ctx_affinity * 0.5)
        edges = self.edges.setdefault(source or ROOT, [])
        e = next((x for x in edges if x.to == to), None)
        if e is None:
            edges.append(_Edge(to, min(signal, 3.5), gain, gain, 1 if gain > 0.0 else 0))
        else:
            e.strength = min(e.strength * self.decay_rate + signal, 3.5)
            e.total_gain = e.total_gain * self.decay_rate + gain
            e.best_gain = max(e.best_gain, gain)
            e.hits += 1
        edges.sort(key=lambda x: -x.strength)
        del edges[self.fanout:]

    def boost(self, source: Optional[str], to: str) -> float:
        e = next((x for x in self.edges.get(source or ROOT, []) if x.to == to), None)
        return min(e.strength * (1.0 + min(e.mean_gain(), 1.5) * 0.35), 4.0) if e is not None else 0.0

    def penalize_target(self, target: str) -> None:
        for edges in self.edges.values():
            for e in edges:
                if e.to == target:
                    e.strength *= 0.5
                    e.total_gain *= self.decay_rate

    def decay(self) -> None:
        for k in list(self.edges):
            for e in self.edges[k]:
                e.strength *= self.decay_rate
                e.total_gain *= self.decay_rate
            self.edges[k] = [e for e in self.edges[k] if e.strength > 1e-4 or e.total_gain > 1e-4]
            if not self.edges[k]:
                del self.edges[k]

    def snapshots(self) -> List[dict]:
        out = [{"from": a, "to": e.to, "strength": e.strength, "hits": e.hits, "best_gain": e.best_gain, "mean_gain": e.mean_gain()}
               for a, es in self.edges.items() if a != ROOT for e in es]
        return sorted(out, key=lambda s: -s["strength"])


class HintSagaTracker:
    """Like the transition graph, but keyed by the last 0..depth hint sets, so a candidate that worked after this
    particular sequence outranks one that merely worked after the last step."""

    def __init__(self, depth: int = 3, decay: float = 0.9, fanout: int = 3):
        self.sequences: Dict[Tuple[str, ...], List[_Edge]] = {}
        self.depth, self.decay_rate, self.fanout = depth, decay, max(fanout, 1)

    def _prefixes(self, history: Sequence[str]):
        h = list(history)
        return [tuple(h[len(h) - n:]) for n in range(1, min(self.depth, len(h)) + 1)]

    def observe(self, history: Sequence[str], to: str, gain: float, affinity: float, ctx_affinity: float) -> None:
        if self.depth == 0:
            return
        gain = max(gain, 0.0)
        signal = (gain + 0.03) * (1.0 + _clamp(affinity, 0.0, 1.0) * 0.4 + _clamp(ctx_affinity, 0.0, 1.0) * 0.4)
        for prefix in [()] + self._prefixes(history):
            edges = self.sequences.setdefault(prefix, [])
            e = next((x for x in edges if x.to == to), None)
            if e is None:
                edges.append(_Edge(to, min(signal, 4.0), gain, gain, 1 if gain > 0.0 else 0))
            else:
                e.strength = min(e.strength * self.decay_rate + signal, 4.0)
                e.total_gain = e.total_gain * self.decay_rate + gain
                e.best_gain = max(e.best_gain, gain)
                e.hits += 1 if gain > 0.0 else 0
            edges.sort(key=lambda x: -x.strength)
            del edges[self.fanout:]

    def boost(self, history: Sequence[str], candidate: str) -> float:
        if self.depth == 0:
            return 0.0
        e = next((x for x in self.sequences.get((), []) if x.to == candidate), None)
        best = min(e.strength * (1.0 + min(e.mean_gain(), 1.5) * 0.3), 4.0) if e is not None else 0.0
        for prefix in self._prefixes(history):
            e = next((x for x in self.sequences.get(prefix, []) if x.to == candidate), None)
            if e is not None:
                best = max(best, min(e.strength * (1.0 + min(e.mean_gain(), 1.5) * 0.45 + len(prefix) * 0.1), 4.5))
        return best

    def penalize_target(self, target: str) -> None:
        for edges in self.sequences.values():
            for e in edges:
                if e.to == target:
                    e.strength *= 0.5
                    e.total_gain *= self.decay_rate

    def decay(self) -> None:
        for k in list(self.sequences):
            for e in self.sequences[k]:
                e.strength *= self.decay_rate
                e.total_gain *= self.decay_rate
            self.sequences[k] = [e for e in self.sequences[k] if e.strength > 1e-4 or e.total_gain > 1e-4]
            if not self.sequences[k]:
                del self.sequences[k]

    def set_depth(self, depth: int) -> None:
        self.depth = depth
        if depth == 0:
            self.sequences.clear()

    def snapshots(self) -> List[dict]:
        out = [{"prefix": list(p), "to": e.to, "synergy": e.strength, "hits": e.hits, "best_gain": e.best_gain, "mean_gain": e.mean_gain()}
               for p, es in self.sequences.items() for e in es]
        return sorted(out, key=lambda s: -s["synergy"])


# ---------------------------------------------------------------------------------------------------------------
class DiversityGovernor:
    def __init__(self, window: int = 4, threshold: float = 0.08, cooldown: int = 3):
        self.window, self.threshold, self.cooldown = max(window, 1), threshold, max(cooldown, 1)
        self.cooldown_left, self.debt = 0, 0
        self.history: Deque[float] = deque()

    def _push(self, gain: float) -> None:
        self.history.append(gain)
        while len(self.history) > self.window:
            self.history.popleft()

    def mean_gain(self) -> float:
        return sum(self.history) / len(self.history) if self.history else 0.0

    def record_success(self, gain: float, fresh: bool) -> None:
        gain = max(gain, 0.0)
        self._push(gain)
        mean = self.mean_gain()
        if mean < self.threshold and self.cooldown_left == 0:
            self.debt = max(self.debt, 1)
        elif mean >= self.threshold * 1.5:
            self.debt = max(self.debt - 1, 0)
        if fresh:
            if gain >= self.threshold:
                self.debt = max(self.debt - 1, 0)
            self.cooldown_left = max(self.cooldown, 1)
        elif gain >= self.threshold * 1.2:
            self.debt = max(self.debt - 1, 0)

    def record_failure(self) -> None:
        self._push(0.0)
        if self.cooldown_left == 0:
            self.debt = min(self.debt + 1, 4)

    def advance_cycle(self) -> None:
        self.cooldown_left = max(self.cooldown_left - 1, 0)

    def should_force_fresh(self) -> bool:
        return self.debt > 0 and self.cooldown_left == 0

    def snapshot(self) -> dict:
        return {"window": self.window, "threshold": self.threshold, "mean_gain": self.mean_gain(), "debt": self.debt,
                "cooldown": self.cooldown, "cooldown_left": self.cooldown_left}


class HintQualityModel:
    """sigmoid(w . (gain, mean gain, best gain, affinity, freshness) + b), trained online with momentum on the log loss."""

    def __init__(self, lr: float = 0.08, momentum: float = 0.2):
        self.weights, self.velocity = [0.0] * 5, [0.0] * 5
        self.bias = self.bias_velocity = 0.0
        self.lr, self.momentum, self.ema_accuracy, self.updates = lr, momentum, 0.5, 0

    @staticmethod
    def features(gain: float, mean: float, best: float, affinity: float, staleness: Optional[int]) -> List[float]:
        fresh = 0.0 if staleness is None else 1.0 / (1.0 + staleness)
        return [_clamp(gain, 0.0, 2.0), _clamp(mean, 0.0, 2.0), _clamp(best, 0.0, 2.0), _clamp(affinity, 0.0, 1.0), fresh]

    def predict(self, feats: Sequence[float]) -> float:
        x = self.bias + sum(w * f for w, f in zip(self.weights, feats))
        if x >= 0.0:
            return 1.0 / (1.0 + math.exp(-x))
        z = math.exp(x)
        return z / (1.0 + z)

    def score(self, last_gain: float, mean_gain: float, best_gain: float, last_affinity: float, staleness: Optional[int]) -> float:
        p = self.predict(self.features(max(last_gain, mean_gain), mean_gain, best_gain, last_affinity, staleness))
        return p * (1.0 + best_gain + mean_gain * 0.5)

    def observe(self, gain: float, mean: float, best: float, affinity: float, staleness: Optional[int], success: bool) -> None:
        if not math.isfinite(gain) and not math.isfinite(mean):
            return
        feats = self.features(gain, mean, best, affinity, staleness)
        pred = self.predict(feats)
        err = pred - (1.0 if success else 0.0)
        for i, f in enumerate(feats):
            self.velocity[i] = self.momentum * self.velocity[i] + (1.0 - self.momentum) * err * f
            self.weights[i] -= self.lr * self.velocity[i]
        self.bias_velocity = self.momentum * self.bias_velocity + (1.0 - self.momentum) * err
        self.bias -= self.lr * self.bias_velocity
        correct = pred >= 0.5 if success else pred < 0.5
        self.ema_accuracy = self.ema_accuracy * 0.9 + (0.1 if correct else 0.0)
        self.updates += 1

    def snapshot(self) -> dict:
        return {"weights": list(self.weights), "bias": self.bias, "accuracy": _clamp(self.ema_accuracy, 0.0, 1.0), "updates": self.updates,
                "learning_rate": self.lr}


@dataclass
class ContextCluster:
    signature: int
    total_gain: float = 0.0
    best_gain: float = 0.0
    momentum: float = 0.0
    hits: int = 0

    @classmethod
    def new(cls, signature: int, gain: float, affinity: float) -> "ContextCluster":
        gain = max(gain, 0.0)
        return cls(signature, gain, gain, gain * _clamp(affinity, 0.0, 1.0), 1 if gain > 0.0 else 0)

    def mean_gain(self) -> float:
        return self.total_gain / self.hits if self.hits else 0.0

    def update(self, signature: int, gain: float, affinity: float, decay: float) -> None:
        gain, affinity = max(gain, 0.0), _clamp(affinity, 0.0, 1.0)
        self.total_gain = self.total_gain * decay + gain
        self.best_gain = max(self.best_gain, gain)
        self.momentum = self.momentum * decay + gain * affinity
        self.hits += 1 if gain > 0.0 else 0
        if affinity > 0.0:                      # pull the stored signature towards the incoming one, bit pattern-wise
            self.signature ^= int(round((self.signature ^ signature) * affinity)) & 0xFFFFFFFFFFFFFFFF


# ---------------------------------------------------------------------------------------------------------------
class HintPolicyStack:
    """Everything above in one place, with the engine-facing calls."""

    def __init__(self, feedback_gamma: float = 0.35, chain_window: int = 4):
        self.bandit, self.chain_policy, self.relations = HintBandit(), ChainPolicyModel(), HintRelationGraph()
        self.transitions, self.saga, self.diversity, self.quality = HintTransitionGraph(), HintSagaTracker(), DiversityGovernor(), HintQualityModel()
        self.chain_feedback: Dict[str, ChainFeedback] = {}
        self.feedback_gamma, self.chain_window = feedback_gamma, max(chain_window, 1)
        self.last_key: Optional[str] = None
        self.history: Deque[str] = deque()

    def _chain_with(self, key: str) -> List[str]:
        return (list(self.history) + [key])[-self.chain_window:]

    def priority_multiplier(self, key: str) -> float:
        """transition x root x saga x chain-policy x bandit bonuses of a cached hint set, as the cache priority multiplies them."""
        return ((1.0 + self.transitions.boost(self.last_key, key) * 0.25) * (1.0 + self.transitions.boost(None, key) * 0.15)
                * (1.0 + self.saga.boost(self.history, key) * 0.2) * self.chain_policy.multiplier(self._chain_with(key)) * self.bandit.multiplier(key))

    def quality_score(self, last_gain: float, mean_gain: float, best_gain: float, last_affinity: float, staleness: Optional[int]) -> float:
        return self.quality.score(last_gain, mean_gain, best_gain, last_affinity, staleness)

    def should_force_fresh(self) -> bool:
        return self.diversity.should_force_fresh()

    def record_success(self, key: str, gain: float, affinity: float, ctx_affinity: float, fresh: bool, mean_gain: float = 0.0,
                       best_gain: float = 0.0, staleness: Optional[int] = 0) -> None:
        chain = self._chain_with(key)
        self.bandit.observe_success(key, gain)
        self.transitions.observe(self.last_key, key, gain, affinity, ctx_affinity)
        self.saga.observe(self.history, key, gain, affinity, ctx_affinity)
        self.relations.observe_chain(chain, gain)
        self.chain_policy.observe(chain, gain, True)
        self.chain_feedback.setdefault(chain_signature(chain), ChainFeedback()).reward(gain, True, self.feedback_gamma)
        self.diversity.record_success(gain, fresh)
        self.quality.observe(gain, mean_gain, max(best_gain, gain), affinity, staleness, True)
        self.last_key = key
        self.history.append(key)
        while len(self.history) > max(self.saga.depth, self.chain_window):
            self.history.popleft()

    def record_failure(self, key: str, mean_gain: float = 0.0, best_gain: float = 0.0, affinity: float = 0.0, staleness: Optional[int] = 0) -> None:
        chain = self._chain_with(key)
        self.bandit.observe_failure(key)
        self.transitions.penalize_target(key)
        self.saga.penalize_target(key)
        self.chain_policy.observe(chain, 0.0, False)
        self.chain_feedback.setdefault(chain_signature(chain), ChainFeedback()).reward(0.0, False, self.feedback_gamma)
        self.diversity.record_failure()
        self.quality.observe(0.0, mean_gain, best_gain, affinity, staleness, False)

    def advance(self) -> None:
        """One engine tick: every memory fades a little and the diversity cooldown runs down."""
        for layer in (self.bandit, self.chain_policy, self.relations, self.transitions, self.saga):
            layer.decay()
        self.diversity.advance_cycle()

    def snapshot(self) -> dict:
        return {"bandit": self.bandit.snapshots(), "chain_policy": self.chain_policy.snapshots(), "relations": self.relations.snapshots(),
                "transitions": self.transitions.snapshots(), "sagas": self.saga.snapshots(), "diversity": self.diversity.snapshot(),
                "quality": self.quality.snapshot(),
                "chain_feedback": sorted(({"chain": k, "uses": f.uses, "successes": f.successes, "score": f.score(), "ema_reward": f.ema_reward}
                                          for k, f in self.chain_feedback.items()), key=lambda s: -s["score"])}
