"""Prompt / response policy evaluation with an audit log.

Restated from crates/spiral-safety/src/lib.rs: keyword terms per category and channel with
per-occurrence scores (:176-256), risk levels from the summed score (≥ 1.25 critical, ≥ 0.75 high,
≥ 0.4 medium; :124-167), refusal when the cumulative score reaches the threshold (:604-655),
conversation aggregation (:682-720), policy self-check (:725-745), reports (:747-790) and the
audit sink (:324-430).
"""
from __future__ import annotations

import threading
import time
from collections import Counter
from dataclasses import dataclass, field
from typing import Iterable, Optional, Sequence

PROMPT, RESPONSE = "prompt", "response"
TOXICITY, BIAS, SAFETY = "toxicity", "bias", "safety"
RISK_ORDER = {"low": 0, "medium": 1, "high": 2, "critical": 3}


class SafetyError(ValueError):
    pass


def _risk(score: float) -> str:
    if score >= 1.25:
        return "critical"
    if score >= 0.75:
        return "high"
    if score >= 0.4:
        return "medium"
    return "low"


@dataclass
class SafetyViolation:
    category: str
    offending_term: str
    score: float
    occurrences: int = 1
    guidance: Optional[str] = None
    risk: str = field(init=False)
    message: str = field(init=False)

    def __post_init__(self):
        per = self.score / self.occurrences if self.occurrences > 0 else self.score
        hits = f" ({self.occurrences} hits @ {per:.2f} ea)" if self.occurrences > 1 else ""
        self.message = (f"Detected {self.category} content triggered by '{self.offending_term}' with score "
                        f"{self.score:.2f}{hits}")
        self.risk = _risk(self.score)


@dataclass
class PolicyTerm:
    category: str
    keyword: str
    score: float
    channels: tuple = (PROMPT, RESPONSE)
    guidance: Optional[str] = None

    def for_channels(self, channels: Iterable[str]) -> "PolicyTerm":
        self.channels = tuple(channels)
        return self

    def with_guidance(self, guidance: str) -> "PolicyTerm":
        self.guidance = guidance
        return self

    def applies_to(self, channel: str) -> bool:
        return channel in self.channels

    def occurrence_count(self, lowercase: str) -> int:
        needle = self.keyword.lower()
        return lowercase.count(needle) if needle else 0


@dataclass
class KeywordRule:
    category: str
    term: str
    score: float

    def occurrence_count(self, lowercase: str) -> int:
        needle = self.term.lower()
        return lowercase.count(needle) if needle else 0


@dataclass
class SafetyVerdict:
    channel: str
    score: float
    violations: list
    allowed: bool

    def should_refuse(self) -> bool:
        return not self.allowed

    def dominant_risk(self) -> str:
        return max((v.risk for v in self.violations), key=RISK_ORDER.get, default="low")


@dataclass
class TurnVerdict:
    index: int
    verdict: SafetyVerdict


@dataclass
class ConversationVerdict:
    total_score: float
    highest_risk: str
    refused_turns: list
    turn_verdicts: list

    def should_refuse(self) -> bool:
        return bool(self.refused_turns)


@dataclass
class AuditEvent:
    channel: str
    content: str
    verdict: SafetyVerdict
    timestamp: float = field(default_factory=time.time)


@dataclass
class AuditSummary:
    total: int
    refused: int
    by_category: dict
    by_risk: dict


class AuditSink:
    def __init__(self):
        self._events: list[AuditEvent] = []
        self._lock = threading.Lock()

    def push(self, event: AuditEvent) -> None:
        with self._lock:
            self._events.append(event)

    def snapshot(self) -> list:
        with self._lock:
            return list(self._events)

    def clear(self) -> None:
        with self._lock:
            self._events.clear()

    def summarize(self) -> AuditSummary:
        ev = self.snapshot()
        cat, risk = Counter(), Counter()
        for e in ev:
            risk[e.verdict.dominant_risk()] += 1
            for v in e.verdict.violations:
                cat[v.category] += 1
        return AuditSummary(len(ev), sum(e.verdict.should_refuse() for e in ev), dict(cat), dict(risk))


def _default_terms() -> list:
    T = PolicyTerm
    return [
        T(TOXICITY, "hate", 0.6).with_guidance("De-escalate conversation and remind users of respectful conduct policies."),
        T(TOXICITY, "kill", 0.7).with_guidance("Escalate to human review if the user expresses intent to harm others."),
        T(TOXICITY, "die", 0.55), T(TOXICITY, "stupid", 0.4), T(TOXICITY, "idiot", 0.45),
        T(BIAS, "race", 0.5).with_guidance("Nudge the assistant toward inclusive, factual responses."),
        T(BIAS, "gender", 0.45), T(BIAS, "religion", 0.5), T(BIAS, "minority", 0.5), T(BIAS, "minorities", 0.5),
        T(SAFETY, "bomb", 0.7).with_guidance("Block instructions on weapon construction and alert moderators."),
        T(SAFETY, "suicide", 0.8).with_guidance("Redirect to crisis resources and provide supportive language."),
        T(SAFETY, "weapon", 0.65).for_channels([PROMPT]).with_guidance("Avoid providing facilitation for weapons acquisition."),
        T(SAFETY, "explosive", 0.65).for_channels([PROMPT]).with_guidance("Decline to detail explosive manufacturing guidance."),
        T(SAFETY, "self-harm", 0.75).with_guidance("Respond empathetically and surface well-being support options."),
    ]


class SafetyPolicy:
    def __init__(self, terms: Optional[Sequence[PolicyTerm]] = None, refusal_threshold: float = 0.5,
                 audit_sink: Optional[AuditSink] = None):
        self._terms = list(_default_terms() if terms is None else terms)
        self._threshold = refusal_threshold
        self._sink = audit_sink or AuditSink()
        self._rules: list[KeywordRule] = []

    @classmethod
    def with_default_terms(cls) -> "SafetyPolicy":
        return cls()

    @classmethod
    def from_terms(cls, terms, refusal_threshold: float, audit_sink: Optional[AuditSink] = None) -> "SafetyPolicy":
        return cls(terms, refusal_threshold, audit_sink)

    def audit_sink(self) -> AuditSink:
        return self._sink

    def with_audit_sink(self, sink: AuditSink) -> "SafetyPolicy":
        self._sink = sink
        return self

    def clear_audit_log(self) -> None:
        self._sink.clear()

    def terms(self) -> list:
        return list(self._terms)

    def with_term(self, term: PolicyTerm) -> "SafetyPolicy":
        self._terms.append(term)
        return self

    push_term = with_term

    def extend_terms(self, terms: Iterable[PolicyTerm]) -> None:
        self._terms.extend(terms)

    def refusal_threshold(self) -> float:
        return self._threshold

    def with_refusal_threshold(self, threshold: float) -> "SafetyPolicy":
        self._threshold = threshold
        return self

    def with_toxicity_terms(self, terms: Iterable[str], score: float = 0.5) -> "SafetyPolicy":
        self._terms.extend(PolicyTerm(TOXICITY, t, score) for t in terms)
        return self

    def with_bias_terms(self, terms: Iterable[str], score: float = 0.5) -> "SafetyPolicy":
        self._terms.extend(PolicyTerm(BIAS, t, score) for t in terms)
        return self

    def with_custom_rule(self, rule: KeywordRule) -> "SafetyPolicy":
        self._rules.append(rule)
        return self

    def custom_rules(self) -> list:
        return list(self._rules)

    def scan(self, content: str, channel: str) -> SafetyVerdict:
        low = content.lower()
        violations, total = [], 0.0
        for term in self._terms:
            if not term.applies_to(channel):
                continue
            n = term.occurrence_count(low)
            if n:
                v = SafetyViolation(term.category, term.keyword, term.score * n, n, term.guidance)
                total += v.score
                violations.append(v)
        for rule in self._rules:
            n = rule.occurrence_count(low)
            if n:
                v = SafetyViolation(rule.category, rule.term, rule.score * n, n)
                total += v.score
                violations.append(v)
        return SafetyVerdict(channel, total, violations, total < self._threshold)

    def evaluate(self, content: str, channel: str) -> SafetyVerdict:
        verdict = self.scan(content, channel)
        self._sink.push(AuditEvent(channel, content, verdict))
        return verdict

    def evaluate_batch(self, contents: Iterable[str], channel: str) -> list:
        return [self.evaluate(c, channel) for c in contents]

    def refusal_reason(self, verdict: SafetyVerdict) -> str:
        if not verdict.violations:
            return "Policy refusal triggered without explicit violation"
        return "Blocked due to " + ", ".join(f"{v.category} ({v.risk})" for v in verdict.violations)

    def evaluate_conversation(self, turns: Iterable[tuple]) -> ConversationVerdict:
        total, highest, refused, out = 0.0, "low", [], []
        for i, (channel, content) in enumerate(turns):
            v = self.evaluate(content, channel)
            total += v.score
            if RISK_ORDER[v.dominant_risk()] > RISK_ORDER[highest]:
                highest = v.dominant_risk()
            if v.should_refuse():
                refused.append(i)
            out.append(TurnVerdict(i, v))
        return ConversationVerdict(total, highest, refused, out)


def evaluate_policy_surface(policy: SafetyPolicy, dataset: Sequence[tuple]) -> None:
    """Raises when ``(content, should_pass)`` expectations do not hold for ``policy``."""
    for content, should_pass in dataset:
        v = policy.scan(content, PROMPT)
        if should_pass and v.should_refuse():
            raise SafetyError(f"content '{content}' expected to pass but was refused with score {v.score:.2f}")
        if not should_pass and not v.should_refuse():
            raise SafetyError(f"content '{content}' expected to be blocked but passed")


@dataclass
class PolicyReport:
    total: int
    refused: int
    allowed: int
    dominant_risk_counts: dict

    @classmethod
    def from_verdicts(cls, verdicts: Iterable[SafetyVerdict]) -> "PolicyReport":
        vs = list(verdicts)
        refused = sum(v.should_refuse() for v in vs)
        return cls(len(vs), refused, len(vs) - refused, dict(Counter(v.dominant_risk() for v in vs)))

    def refusal_rate(self) -> float:
        return self.refused / self.total if self.total else 0.0
