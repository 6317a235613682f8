"""Hosted-LLM responses as Z-space observations.

No SDK is imported: callers pass a response mapping, an SDK response object, or an ``invoke``
callable that performs the request.  From the response text, usage counters, latency, finish reason
and probability-like fields the runtime derives the five canonical metrics ``speed, memory, stability,
frac, drs`` plus a metric-gradient vector, records a serialisable trace per call and keeps a fused
running estimate (bindings/st-py/spiraltorch/api_llm_runtime.py:861-1000 response parsing, :1084-1150
metric derivation, :1500-1600 partial / trace records).
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence

METRIC_KEYS = ("speed", "memory", "stability", "frac", "drs")
GRADIENT_BASIS = "spiraltorch.canonical_metric_gradient.v1"


def _get(source: Any, key: str, default: Any = None) -> Any:
    if source is None:
        return default
    if isinstance(source, Mapping):
        return source.get(key, default)
    return getattr(source, key, default)


def _as_float(v: Any) -> Optional[float]:
    if isinstance(v, bool) or v is None:
        return None
    try:
        f = float(v)
    except (TypeError, ValueError):
        return None
    return f if math.isfinite(f) else None


def _content_text(content: Any) -> str:
    """Text of a string, a ``{"text": ...}`` block, or a list of content blocks."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, Sequence) and not isinstance(content, (bytes, bytearray)):
        return "".join(_content_text(part) for part in content)
    for key in ("text", "content", "value"):
        inner = _get(content, key)
        if inner is not None and inner is not content:
            text = _content_text(inner)
            if text:
                return text
    return ""


def _first_choice(response: Any) -> Any:
    choices = _get(response, "choices")
    if isinstance(choices, Sequence) and not isinstance(choices, (str, bytes)) and choices:
        return choices[0]
    return None


def text_from_response(response: Any) -> str:
    """Primary text of OpenAI responses / chat-completions and Anthropic messages shapes."""
    if isinstance(response, str):
        return response
    text = _get(response, "output_text")
    if isinstance(text, str) and text:
        return text
    output = _get(response, "output")
    if isinstance(output, Sequence) and not isinstance(output, (str, bytes)):
        text = "".join(_content_text(_get(item, "content")) for item in output)
        if text:
            return text
    choice = _first_choice(response)
    if choice is not None:
        for cand in (_get(_get(choice, "message"), "content"), _get(choice, "text"), _get(choice, "content"),
                     _get(choice, "delta")):
            text = _content_text(cand)
            if text:
                return text
    for key in ("text", "content", "message"):
        text = _content_text(_get(response, key))
        if text:
            return text
    return ""


def usage_from_response(response: Any) -> Dict[str, float]:
    usage = _get(response, "usage")
    prompt = next((v for v in (_as_float(_get(usage, k)) for k in ("prompt_tokens", "input_tokens", "prompt")) if v is not None), None)
    completion = next((v for v in (_as_float(_get(usage, k)) for k in ("completion_tokens", "output_tokens", "completion")) if v is not None), None)
    total = next((v for v in (_as_float(_get(usage, k)) for k in ("total_tokens", "total")) if v is not None), None)
    if total is None:
        total = (prompt or 0.0) + (completion or 0.0)
    out: Dict[str, float] = {}
    if prompt is not None:
        out["prompt_tokens"] = prompt
    if completion is not None:
        out["completion_tokens"] = completion
    out["total_tokens"] = total
    return out


def finish_reason_from_response(response: Any) -> Optional[str]:
    for source in (_first_choice(response), response):
        for key in ("finish_reason", "stop_reason", "status"):
            v = _get(source, key)
            if v:
                return str(v)
    return None


def _to_probability(v: Any) -> Optional[float]:
    f = _as_float(v)
    if f is None:
        return None
    if 0.0 <= f <= 1.0:
        return f
    try:
        return max(0.0, min(1.0, math.exp(f)))
    except OverflowError:
        return None


def top_probability_from_response(response: Any) -> Optional[float]:
    for source in (response, _first_choice(response)):
        if source is None:
            continue
        for key in ("top_probability", "probability", "confidence"):
            p = _to_probability(_get(source, key))
            if p is not None:
                return p
        content = _get(_get(source, "logprobs"), "content")
        if isinstance(content, Sequence) and content:
            first = content[0]
            top = _get(first, "top_logprobs")
            if isinstance(top, Sequence) and top:
                vals = [p for p in (_to_probability(_get(t, "logprob")) for t in top) if p is not None]
                if vals:
                    return max(vals)
            p = _to_probability(_get(first, "logprob"))
            if p is not None:
                return p
    return None


def text_stats(text: str) -> Dict[str, float]:
    if not text:
        return {"chars": 0.0, "words": 0.0, "unique_chars": 0.0, "entropy": 0.0, "entropy_norm": 0.0}
    counts: Dict[str, int] = {}
    for ch in text:
        counts[ch] = counts.get(ch, 0) + 1
    entropy = -sum(c / len(text) * math.log2(c / len(text)) for c in counts.values())
    max_entropy = math.log2(max(2, len(counts)))
    return {"chars": float(len(text)), "words": float(len(text.split())), "unique_chars": float(len(counts)),
            "entropy": entropy, "entropy_norm": entropy / max_entropy}


def _estimate_tokens(text: str) -> float:
    return max(1.0, len(text) / 4.0) if text else 0.0


def runtime_metrics(*, prompt: Optional[str], text: str, usage: Mapping[str, float], latency_ms: Optional[float],
                    finish_reason: Optional[str], top_probability: Optional[float]):
    """``(metrics, telemetry)``: speed = tanh(tokens/s / 64), memory = tanh(total tokens / 2048),
    stability = 0.65·stop quality + 0.35·top probability, frac = normalised character entropy,
    drs = tanh((completion − prompt) / total)."""
    stats = text_stats(text)
    prompt_tokens = float(usage.get("prompt_tokens") or _estimate_tokens(prompt or ""))
    completion_tokens = float(usage.get("completion_tokens") or _estimate_tokens(text))
    total_tokens = float(usage.get("total_tokens") or prompt_tokens + completion_tokens)
    latency_s = max(0.0, float(latency_ms or 0.0) / 1000.0)
    tps = completion_tokens / max(latency_s, 1e-6) if latency_ms is not None else completion_tokens
    finish = (finish_reason or "").lower()
    if finish in {"stop", "completed", "complete", "success", "end_turn", "stop_sequence"}:
        stop = 0.95
    elif finish in {"length", "max_tokens", "incomplete"}:
        stop = 0.45
    elif finish in {"content_filter", "safety"}:
        stop = 0.15
    else:
        stop = 0.65
    prob = min(max(top_probability if top_probability is not None else 0.65, 0.0), 1.0)
    metrics = {"speed": math.tanh(tps / 64.0), "memory": math.tanh(total_tokens / 2048.0),
               "stability": min(max(0.65 * stop + 0.35 * prob, 0.0), 1.0),
               "frac": min(max(stats["entropy_norm"], 0.0), 1.0),
               "drs": math.tanh((completion_tokens - prompt_tokens) / max(1.0, total_tokens))}
    telemetry = {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens, "total_tokens": total_tokens,
                 "latency_ms": float(latency_ms) if latency_ms is not None else 0.0, "tokens_per_second": tps,
                 "response_chars": stats["chars"], "response_words": stats["words"],
                 "response_unique_chars": stats["unique_chars"], "response_entropy": stats["entropy"],
                 "response_entropy_norm": stats["entropy_norm"], "top_probability": prob}
    return metrics, telemetry


def metric_gradient_projection(metrics: Mapping[str, float], gradient_dim: int) -> Dict[str, Any]:
    """Centres the canonical metrics (speed, memory, stability, frac at 0.5; drs at 0) and folds them
    cyclically into ``gradient_dim`` components."""
    if gradient_dim < 1:
        raise ValueError("metric-gradient projection dimension must be positive")
    centred = [float(metrics.get(k, 0.5 if k != "drs" else 0.0)) - (0.5 if k != "drs" else 0.0) for k in METRIC_KEYS]
    grad = [0.0] * gradient_dim
    for i, v in enumerate(centred):
        grad[i % gradient_dim] += v
    return {"gradient": grad, "dimension": gradient_dim, "basis": GRADIENT_BASIS}


@dataclass
class ZSpacePartial:
    metrics: Dict[str, Any]
    weight: float = 1.0
    origin: Optional[str] = None
    telemetry: Dict[str, Any] = field(default_factory=dict)
    gradient_basis: Optional[str] = None


def partial_from_response(response: Any, *, prompt: Optional[str] = None, provider: Optional[str] = None,
                          model: Optional[str] = None, latency_ms: Optional[float] = None, bundle_weight: float = 1.0,
                          origin: Optional[str] = "api_llm", telemetry_prefix: str = "api_llm",
                          gradient_dim: int = 4) -> ZSpacePartial:
    text = text_from_response(response)
    finish = finish_reason_from_response(response)
    metrics, telemetry = runtime_metrics(prompt=prompt, text=text, usage=usage_from_response(response), latency_ms=latency_ms,
                                         finish_reason=finish, top_probability=top_probability_from_response(response))
    proj = metric_gradient_projection(metrics, gradient_dim)
    metrics["gradient"] = list(proj["gradient"])
    if provider:
        telemetry["provider_present"] = 1.0
    if model or _get(response, "model"):
        telemetry["model_present"] = 1.0
    if finish:
        telemetry["finish_reason_stop"] = 1.0 if finish.lower() == "stop" else 0.0
        telemetry["finish_reason_refusal"] = 1.0 if finish.lower() == "refusal" else 0.0
    telemetry["empty_text"] = 1.0 if not text.strip() else 0.0
    return ZSpacePartial(metrics, max(0.0, float(bundle_weight)), origin,
                         {f"{telemetry_prefix}.{k}": v for k, v in telemetry.items()}, proj["basis"])


@dataclass
class ApiLLMTrace:
    provider: Optional[str]
    model: Optional[str]
    prompt: Optional[str]
    text: str
    finish_reason: Optional[str]
    latency_ms: Optional[float]
    usage: Dict[str, float]
    metrics: Dict[str, Any]
    telemetry: Dict[str, Any]

    def as_dict(self) -> Dict[str, Any]:
        return {k: getattr(self, k) for k in self.__dataclass_fields__}


def trace_from_response(response: Any, *, prompt: Optional[str] = None, provider: Optional[str] = None,
                        model: Optional[str] = None, latency_ms: Optional[float] = None, gradient_dim: int = 4) -> ApiLLMTrace:
    part = partial_from_response(response, prompt=prompt, provider=provider, model=model, latency_ms=latency_ms,
                                 gradient_dim=gradient_dim)
    return ApiLLMTrace(provider, model or _get(response, "model"), prompt, text_from_response(response),
                       finish_reason_from_response(response), latency_ms, usage_from_response(response), part.metrics,
                       part.telemetry)


class ApiLLMZSpaceRuntime:
    """Calls ``invoke(prompt, **request)`` (any callable returning a response), times it, derives the trace
    and keeps an exponentially smoothed fused estimate of the canonical metrics."""

    def __init__(self, invoke: Callable[..., Any], *, provider: Optional[str] = None, model: Optional[str] = None,
                 smoothing: float = 0.35, gradient_dim: int = 4, trace_path: Optional[str] = None,
                 clock: Callable[[], float] = time.perf_counter):
        self.invoke, self.provider, self.model = invoke, provider, model
        self.smoothing = min(max(smoothing, 0.0), 1.0)
        self.gradient_dim, self.trace_path, self._clock = gradient_dim, trace_path, clock
        self.fused: Optional[Dict[str, float]] = None
        self.traces: List[ApiLLMTrace] = []

    def run(self, prompt: str, **request) -> ApiLLMTrace:
        t0 = self._clock()
        response = self.invoke(prompt, **request)
        latency_ms = (self._clock() - t0) * 1000.0
        trace = trace_from_response(response, prompt=prompt, provider=self.provider, model=self.model,
                                    latency_ms=latency_ms, gradient_dim=self.gradient_dim)
        a = self.smoothing
        cur = {k: float(trace.metrics[k]) for k in METRIC_KEYS}
        self.fused = cur if self.fused is None else {k: (1 - a) * self.fused[k] + a * cur[k] for k in METRIC_KEYS}
        self.traces.append(trace)
        if self.trace_path:
            with open(self.trace_path, "a", encoding="utf-8") as fh:
                fh.write(json.dumps(trace.as_dict(), sort_keys=True) + "\n")
        return trace

    def run_suite(self, prompts: Sequence[str], **request) -> Dict[str, Any]:
        traces = [self.run(p, **request) for p in prompts]
        return summarize_traces([t.as_dict() for t in traces])


def load_trace_events(path: str) -> List[Dict[str, Any]]:
    with open(path, encoding="utf-8") as fh:
        return [json.loads(line) for line in fh if line.strip()]


def summarize_traces(events: Sequence[Mapping[str, Any]]) -> Dict[str, Any]:
    n = len(events)
    if n == 0:
        return {"events": 0}
    mean = lambda xs: sum(xs) / len(xs) if xs else 0.0  # noqa: E731
    out: Dict[str, Any] = {"events": n,
                           "mean_latency_ms": mean([float(e.get("latency_ms") or 0.0) for e in events]),
                           "total_tokens": sum(float((e.get("usage") or {}).get("total_tokens", 0.0)) for e in events),
                           "empty_responses": sum(1 for e in events if not str(e.get("text", "")).strip()),
                           "finish_reasons": {}}
    for e in events:
        r = str(e.get("finish_reason") or "unknown")
        out["finish_reasons"][r] = out["finish_reasons"].get(r, 0) + 1
    for k in METRIC_KEYS:
        out[f"mean_{k}"] = mean([float((e.get("metrics") or {}).get(k, 0.0)) for e in events])
    return out


def compare_trace_runs(baseline: Sequence[Mapping[str, Any]], candidate: Sequence[Mapping[str, Any]]) -> Dict[str, Any]:
    a, b = summarize_traces(baseline), summarize_traces(candidate)
    keys = [k for k in a if k.startswith("mean_") and k in b]
    return {"baseline": a, "candidate": b, "delta": {k: b[k] - a[k] for k in keys}}
