"""Deterministic hyper-parameter search: search spaces, random / exploit-and-jitter / population
strategies, a resource scheduler, trial bookkeeping with checkpoints, and tracker callbacks.

Restated from crates/spiral-hpo/src/lib.rs: ``ParamSpec`` / ``SearchSpace`` (:41-280),
``Objective`` (:284-320), strategies (:338-730), ``ResourceScheduler`` (:740-820), ``SearchLoop``
(:881-1145) and ``analysis.rs``.  Sampling is seeded: every suggestion draws from a generator keyed
by ``(seed, suggestion_count)``, so a loop restored from ``checkpoint()`` continues with the same
suggestions an uninterrupted loop would have produced.
"""
from __future__ import annotations

import copy
import math
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Optional

import numpy as np


class SearchError(ValueError):
    pass


@dataclass
class ParamSpec:
    kind: str                      # "float" | "int" | "categorical"
    name: str
    low: float = 0.0
    high: float = 0.0
    choices: tuple = ()

    @staticmethod
    def Float(name: str, low: float, high: float) -> "ParamSpec":
        return ParamSpec("float", name, float(low), float(high))

    @staticmethod
    def Int(name: str, low: int, high: int) -> "ParamSpec":
        return ParamSpec("int", name, int(low), int(high))

    @staticmethod
    def Categorical(name: str, choices) -> "ParamSpec":
        return ParamSpec("categorical", name, choices=tuple(choices))


class SearchSpace:
    def __init__(self, params: list[ParamSpec]):
        self.params = list(params)

    def __len__(self) -> int:
        return len(self.params)

    def is_empty(self) -> bool:
        return not self.params

    def validate(self) -> None:
        if not self.params:
            raise SearchError("search space must contain at least one parameter")
        seen = set()
        for p in self.params:
            if not p.name.strip():
                raise SearchError("parameter names must not be empty")
            if p.name in seen:
                raise SearchError(f"duplicate parameter '{p.name}'")
            seen.add(p.name)
            if p.kind in ("float", "int"):
                if not (math.isfinite(p.low) and math.isfinite(p.high)) or p.low > p.high:
                    raise SearchError(f"parameter '{p.name}' has an invalid range [{p.low}, {p.high}]")
            elif p.kind == "categorical":
                if not p.choices:
                    raise SearchError(f"categorical parameter '{p.name}' has no choices")
            else:
                raise SearchError(f"unknown parameter kind '{p.kind}'")

    def validate_suggestion(self, s: dict) -> None:
        for p in self.params:
            if p.name not in s:
                raise SearchError(f"suggestion lacks parameter '{p.name}'")
            v = s[p.name]
            if p.kind == "categorical":
                if v not in p.choices:
                    raise SearchError(f"'{v}' is not a choice of '{p.name}'")
            elif not (p.low <= v <= p.high):
                raise SearchError(f"value {v} of '{p.name}' is outside [{p.low}, {p.high}]")
        extra = set(s) - {p.name for p in self.params}
        if extra:
            raise SearchError(f"unknown parameters {sorted(extra)}")

    def draws_per_suggestion(self) -> int:
        return max(1, len(self.params))

    def sample(self, rng: np.random.Generator) -> dict:
        out = {}
        for p in self.params:
            raw = float(rng.random())
            if p.kind == "float":
                out[p.name] = p.low + (p.high - p.low) * raw
            elif p.kind == "int":
                span = int(p.high) - int(p.low) + 1
                out[p.name] = int(p.low) + min(span - 1, int(math.floor(raw * span)))
            else:
                out[p.name] = p.choices[min(len(p.choices) - 1, int(math.floor(raw * len(p.choices))))]
        return out

    def clamp(self, s: dict) -> None:
        for p in self.params:
            if p.name not in s:
                continue
            if p.kind == "float":
                s[p.name] = min(max(float(s[p.name]), p.low), p.high)
            elif p.kind == "int":
                s[p.name] = int(min(max(int(s[p.name]), int(p.low)), int(p.high)))
            elif s[p.name] not in p.choices:
                s[p.name] = p.choices[0]


class Objective:
    MINIMIZE, MAXIMIZE = "minimize", "maximize"

    def __init__(self, kind: str = "minimize"):
        if kind not in (self.MINIMIZE, self.MAXIMIZE):
            raise SearchError(f"unknown objective '{kind}'")
        self.kind = kind

    @staticmethod
    def from_maximize(maximize: bool) -> "Objective":
        return Objective(Objective.MAXIMIZE if maximize else Objective.MINIMIZE)

    def as_str(self) -> str:
        return self.kind

    def key(self, metric: float) -> float:
        """Sort key: smaller is better for both directions; NaN sorts last."""
        if math.isnan(metric):
            return math.inf
        return metric if self.kind == self.MINIMIZE else -metric

    def prefers(self, candidate: float, incumbent: float) -> bool:
        return self.key(candidate) < self.key(incumbent)


def _rng(seed: int, count: int) -> np.random.Generator:
    return np.random.default_rng([int(seed) & 0xFFFFFFFFFFFFFFFF, int(count)])


class RandomStrategy:
    name = "random"

    def __init__(self, seed: int):
        self.seed, self.suggestion_count = seed, 0

    def suggest(self, space: SearchSpace, objective: Objective) -> dict:
        s = space.sample(_rng(self.seed, self.suggestion_count))
        self.suggestion_count += 1
        return s

    def observe(self, suggestion: dict, metric: float, objective: Objective) -> None:
        pass

    def state(self) -> dict:
        return {"kind": "random", "seed": self.seed, "suggestion_count": self.suggestion_count}


class BayesianStrategy:
    """Explore with probability ``exploration``; otherwise jitter the best observation (Gaussian,
    sigma = 10 % of a float range, 25 % of an int span; categorical re-drawn with probability 1/4)."""

    name = "bayesian"

    def __init__(self, seed: int, exploration: float = 0.3):
        self.seed, self.exploration = seed, min(max(float(exploration), 0.0), 1.0)
        self.suggestion_count = 0
        self.observations: list[tuple[dict, float]] = []

    def suggest(self, space: SearchSpace, objective: Objective) -> dict:
        rng = _rng(self.seed, self.suggestion_count)
        s = space.sample(rng)
        self.suggestion_count += 1
        if not self.observations or float(rng.random()) < self.exploration:
            return s
        best = min(self.observations, key=lambda o: objective.key(o[1]))[0]
        s = dict(best)
        for p in space.params:
            if p.kind == "float":
                s[p.name] = s[p.name] + float(rng.standard_normal()) * abs(p.high - p.low) * 0.1
            elif p.kind == "int":
                span = max(1, int(p.high) - int(p.low))
                s[p.name] = int(s[p.name]) + int(round(float(rng.standard_normal()) * span * 0.25))
            else:
                idx = int(rng.integers(0, len(p.choices)))
                if float(rng.random()) < 0.25:
                    s[p.name] = p.choices[idx]
        space.clamp(s)
        return s

    def observe(self, suggestion: dict, metric: float, objective: Objective) -> None:
        self.observations.append((dict(suggestion), float(metric)))

    def state(self) -> dict:
        return {"kind": "bayesian", "seed": self.seed, "exploration": self.exploration,
                "suggestion_count": self.suggestion_count, "observations": copy.deepcopy(self.observations)}


class PopulationStrategy:
    """Keeps the ``population`` best observations; a suggestion mutates a random elite member."""

    name = "population"

    def __init__(self, seed: int, population: int = 8, elite: int = 2, mutation_rate: float = 0.3):
        if population < 1 or elite < 1 or elite > population:
            raise SearchError("population strategy needs 1 <= elite <= population")
        self.seed, self.population, self.elite = seed, population, elite
        self.mutation_rate = min(max(float(mutation_rate), 0.0), 1.0)
        self.suggestion_count = 0
        self.members: list[tuple[dict, float]] = []

    def suggest(self, space: SearchSpace, objective: Objective) -> dict:
        rng = _rng(self.seed, self.suggestion_count)
        fresh = space.sample(rng)
        self.suggestion_count += 1
        if len(self.members) < self.elite:
            return fresh
        elite = sorted(self.members, key=lambda m: objective.key(m[1]))[: self.elite]
        s = dict(elite[int(rng.integers(0, len(elite)))][0])
        for p in space.params:
            if float(rng.random()) < self.mutation_rate:
                s[p.name] = fresh[p.name]
        space.clamp(s)
        return s

    def observe(self, suggestion: dict, metric: float, objective: Objective) -> None:
        self.members.append((dict(suggestion), float(metric)))
        self.members.sort(key=lambda m: objective.key(m[1]))
        del self.members[self.population:]

    def state(self) -> dict:
        return {"kind": "population", "seed": self.seed, "population": self.population, "elite": self.elite,
                "mutation_rate": self.mutation_rate, "suggestion_count": self.suggestion_count,
                "members": copy.deepcopy(self.members)}


def restore_strategy(state: dict):
    k = state["kind"]
    if k == "random":
        s = RandomStrategy(state["seed"])
    elif k == "bayesian":
        s = BayesianStrategy(state["seed"], state["exploration"])
        s.observations = copy.deepcopy(state["observations"])
    elif k == "population":
        s = PopulationStrategy(state["seed"], state["population"], state["elite"], state["mutation_rate"])
        s.members = copy.deepcopy(state["members"])
    else:
        raise SearchError(f"unknown strategy '{k}'")
    s.suggestion_count = state["suggestion_count"]
    return s


@dataclass
class ResourceConfig:
    max_concurrent: int = 1
    min_interval_ms: Optional[int] = None

    def validate(self) -> None:
        if self.max_concurrent <= 0:
            raise SearchError("max_concurrent must be positive")


class ResourceScheduler:
    def __init__(self, config: ResourceConfig, state: Optional[dict] = None, clock: Callable[[], float] = time.time):
        self.config, self._clock = config, clock
        self.active_slots = 0 if state is None else state["active_slots"]
        self.last_scheduled_ms = None if state is None else state["last_scheduled_ms"]

    def try_reserve(self) -> bool:
        if self.active_slots >= self.config.max_concurrent:
            return False
        now = int(self._clock() * 1000)
        if self.config.min_interval_ms is not None and self.last_scheduled_ms is not None and \
                now < self.last_scheduled_ms + self.config.min_interval_ms:
            return False
        self.active_slots += 1
        self.last_scheduled_ms = now
        return True

    def release(self) -> None:
        self.active_slots = max(0, self.active_slots - 1)

    def state(self) -> dict:
        return {"active_slots": self.active_slots, "last_scheduled_ms": self.last_scheduled_ms}


@dataclass
class TrialRecord:
    id: int
    suggestion: dict
    metric: Optional[float] = None


@dataclass
class TrialSummary:
    completed: int
    pending: int
    objective: str
    best: Optional[TrialRecord] = None

    def has_best(self) -> bool:
        return self.best is not None


def best_trial(completed: list[TrialRecord], objective: Objective) -> Optional[TrialRecord]:
    done = [t for t in completed if t.metric is not None and not math.isnan(t.metric)]
    return min(done, key=lambda t: objective.key(t.metric)) if done else None


class ExperimentTracker:
    def on_suggest(self, trial: TrialRecord) -> None:
        pass

    def on_observe(self, trial: TrialRecord) -> None:
        pass

    def on_checkpoint(self, state: dict) -> None:
        pass


NoOpTracker = ExperimentTracker


class SearchLoop:
    def __init__(self, space: SearchSpace, strategy, objective: Objective = None, resources: ResourceConfig = None,
                 trackers: Optional[list[ExperimentTracker]] = None):
        space.validate()
        self._space, self._strategy = space, strategy
        self._objective = objective or Objective()
        self._resources = resources or ResourceConfig()
        self._resources.validate()
        self._scheduler = ResourceScheduler(self._resources)
        self._trackers = list(trackers or [])
        self._pending: list[TrialRecord] = []
        self._completed: list[TrialRecord] = []
        self._next_id = 0

    @classmethod
    def from_state(cls, space: SearchSpace, state: dict, trackers=None) -> "SearchLoop":
        loop = cls(space, restore_strategy(state["strategy"]), Objective(state["objective"]),
                   ResourceConfig(**state["resources"]), trackers)
        loop._scheduler = ResourceScheduler(loop._resources, state["scheduler"])
        loop._pending = [TrialRecord(**t) for t in state["pending"]]
        loop._completed = [TrialRecord(**t) for t in state["completed"]]
        loop._next_id = state["next_trial_id"]
        for t in loop._pending + loop._completed:
            space.validate_suggestion(t.suggestion)
        return loop

    def suggest(self) -> TrialRecord:
        if not self._scheduler.try_reserve():
            raise SearchError("no trial slot available (max_concurrent reached or min_interval not elapsed)")
        s = self._strategy.suggest(self._space, self._objective)
        self._space.validate_suggestion(s)
        t = TrialRecord(self._next_id, s)
        self._next_id += 1
        self._pending.append(t)
        for tr in self._trackers:
            tr.on_suggest(t)
        return t

    def observe(self, trial_id: int, metric: float) -> None:
        for i, t in enumerate(self._pending):
            if t.id == trial_id:
                break
        else:
            raise SearchError(f"unknown or already completed trial {trial_id}")
        t = self._pending.pop(i)
        t.metric = float(metric)
        self._completed.append(t)
        self._scheduler.release()
        self._strategy.observe(t.suggestion, t.metric, self._objective)
        for tr in self._trackers:
            tr.on_observe(t)

    def checkpoint(self) -> dict:
        state = {"strategy": self._strategy.state(), "objective": self._objective.kind,
                 "resources": asdict(self._resources), "scheduler": self._scheduler.state(),
                 "pending": [asdict(t) for t in self._pending], "completed": [asdict(t) for t in self._completed],
                 "next_trial_id": self._next_id}
        for tr in self._trackers:
            tr.on_checkpoint(state)
        return copy.deepcopy(state)

    def pending(self) -> list[TrialRecord]:
        return list(self._pending)

    def completed(self) -> list[TrialRecord]:
        return list(self._completed)

    def space(self) -> SearchSpace:
        return self._space

    def objective(self) -> Objective:
        return self._objective

    def best_trial(self) -> Optional[TrialRecord]:
        return best_trial(self._completed, self._objective)

    def summary(self) -> TrialSummary:
        return TrialSummary(len(self._completed), len(self._pending), self._objective.kind, self.best_trial())
