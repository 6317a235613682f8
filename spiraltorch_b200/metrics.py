"""Typed metric registry: evaluators are registered per input type and run over any value of that
type; an evaluator that raises is reported as a failure and never stops the others.

Restated from crates/st-metrics/src/registry.rs:53-230 (``MetricDescriptor``, ``MetricValue``
scalar / distribution, ``register_metric``, ``evaluate``, ``evaluate_report``, ``descriptors_for``).
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence, Union


@dataclass(frozen=True)
class MetricDescriptor:
    name: str
    description: str = ""
    unit: str = "unitless"          # "unitless" | "percent" | "probability" | "logit" | custom label
    tags: tuple = ()
    higher_is_better: Optional[bool] = None


MetricValue = Union[float, Sequence[float]]


def is_finite(value: MetricValue) -> bool:
    if isinstance(value, (int, float)):
        return math.isfinite(value)
    return all(math.isfinite(v) for v in value)


@dataclass
class MetricEvaluationFailure:
    descriptor: MetricDescriptor
    message: str


@dataclass
class MetricEvaluationReport:
    values: list = field(default_factory=list)
    failures: list = field(default_factory=list)

    def is_clean(self) -> bool:
        return not self.failures


_registry: list[tuple[type, MetricDescriptor, Callable[[Any], Optional[MetricValue]]]] = []
_lock = threading.Lock()


def register_metric(input_type: type, descriptor: MetricDescriptor, evaluator: Callable[[Any], Optional[MetricValue]]) -> None:
    with _lock:
        _registry.append((input_type, descriptor, evaluator))


def clear_registry() -> None:
    with _lock:
        _registry.clear()


def descriptors_for(input_type: type) -> list:
    with _lock:
        return [d for t, d, _ in _registry if issubclass(input_type, t)]


def evaluate_report(value: Any) -> MetricEvaluationReport:
    with _lock:
        entries = [(d, f) for t, d, f in _registry if isinstance(value, t)]
    rep = MetricEvaluationReport()
    for d, f in entries:
        try:
            out = f(value)
        except Exception as exc:  # noqa: BLE001 - isolate the failing evaluator
            rep.failures.append(MetricEvaluationFailure(d, f"{type(exc).__name__}: {exc}"))
            continue
        if out is not None:
            rep.values.append((d, float(out) if isinstance(out, (int, float)) else [float(v) for v in out]))
    return rep


def evaluate(value: Any) -> list:
    return evaluate_report(value).values
