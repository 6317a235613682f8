"""Checkpoint of the state that lives beside a trainer: the desire trainer queue, the psi meter, the
accumulator synchroniser and the Autopilot's pending selection.  One JSON-serialisable document with a fixed
header, the list of components a deterministic resume requires, the captured payloads and the components that
could not be captured; ``validate`` checks every payload field by field and says whether a resume from the
document alone would replay the same run.

Restated from crates/st-core/src/runtime/trainer_external.rs: ``TrainerExternalStateCheckpoint`` :759,
``TrainerExternalCheckpointValidation`` :775, ``TrainerExternalCheckpointError`` :790,
``TrainerExternalCheckpointComponents`` :810, the desire-queue validation rules :150-230 (positive temperature,
non-negative entropy / penalty / weights, trigger tokens unique and paired with scores, positive sample count)
and the psi-meter checkpoint :231-420.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

KIND = "trainer_external_state"
CONTRACT_VERSION = "1"
SEMANTIC_OWNER = "spiraltorch_b200.runtime.trainer_external"
SEMANTIC_BACKEND = "python"
COMPONENTS = ("desire_trainer", "psi_meter", "accumulator_synchronizer", "autopilot")
MAX_SAFE_INTEGER = (1 << 53) - 1


class TrainerExternalCheckpointError(ValueError):
    def __init__(self, kind: str, field_name: str, message: str):
        super().__init__(f"invalid external checkpoint state at {field_name}: {message}" if kind == "InvalidState"
                         else f"external checkpoint {field_name} must be {message}")
        self.kind, self.field = kind, field_name


def _state(field_name: str, message: str) -> TrainerExternalCheckpointError:
    return TrainerExternalCheckpointError("InvalidState", field_name, message)


def _finite(field_name: str, v, *, positive: bool = False, non_negative: bool = False) -> None:
    if not isinstance(v, (int, float)) or not math.isfinite(v):
        raise _state(field_name, "must be finite")
    if positive and not v > 0:
        raise _state(field_name, "must be positive")
    if non_negative and v < 0:
        raise _state(field_name, "must be non-negative")


def validate_desire_trainer(events: list) -> None:
    for i, e in enumerate(events):
        pre = f"desire_trainer.events[{i}]"
        _finite(f"{pre}.timestamp", e.get("timestamp"), non_negative=True)
        if e.get("phase") not in ("observation", "injection", "integration"):
            raise _state(f"{pre}.phase", "must be observation, injection or integration")
        _finite(f"{pre}.temperature", e.get("temperature"), positive=True)
        _finite(f"{pre}.entropy", e.get("entropy"), non_negative=True)
        _finite(f"{pre}.hypergrad_penalty", e.get("hypergrad_penalty"), non_negative=True)
        w = e.get("weights") or {}
        for label in ("alpha", "beta", "gamma", "lam"):
            _finite(f"{pre}.weights.{label}", w.get(label), non_negative=True)
        t = e.get("trigger")
        if t is not None:
            tp = f"{pre}.trigger"
            rep = t.get("report") or {}
            toks, scores = rep.get("tokens", []), rep.get("scores", [])
            if len(toks) != len(scores):
                raise _state(f"{tp}.report_tokens", "must have the same length as report_scores")
            for j, tok in enumerate(toks):
                if not isinstance(tok, int) or tok < 0 or tok > MAX_SAFE_INTEGER:
                    raise _state(f"{tp}.report_tokens[{j}]", "must be an integer within the exact-integer limit")
                if tok in toks[:j]:
                    raise _state(f"{tp}.report_tokens[{j}]", "must be unique within the trigger report")
            for j, sc in enumerate(scores):
                _finite(f"{tp}.report_scores[{j}]", sc, non_negative=True)
            _finite(f"{tp}.mean_penalty", t.get("mean_penalty"), non_negative=True)
            _finite(f"{tp}.mean_entropy", t.get("mean_entropy"), non_negative=True)
            _finite(f"{tp}.temperature", t.get("temperature"), positive=True)
            if not isinstance(t.get("samples"), int) or not 0 < t["samples"] <= MAX_SAFE_INTEGER:
                raise _state(f"{tp}.samples", "must be a positive integer")


def validate_psi_meter(doc: dict) -> None:
    from ..psi import PsiMeter
    try:
        PsiMeter.from_checkpoint(doc)
    except (ValueError, KeyError, TypeError) as exc:
        raise _state("psi_meter", str(exc)) from exc
    if not 0.0 < float(doc["ema_alpha"]) < 1.0:
        raise _state("psi_meter.ema_alpha", "must be in (0, 1)")
    if int(doc["sample_rate"]) <= 0 or int(doc["step"]) < 0:
        raise _state("psi_meter.sample_rate", "sample_rate must be positive and step non-negative")


@dataclass
class TrainerExternalCheckpointValidation:
    required_components: list
    captured_components: list
    unresolved_components: list
    payload_complete: bool
    deterministic_resume_ready: bool
    kind: str = KIND
    contract_version: str = CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND


@dataclass
class TrainerExternalStateCheckpoint:
    required_components: list
    desire_trainer: Optional[list] = None
    psi_meter: Optional[dict] = None
    accumulator_synchronizer: Optional[dict] = None
    autopilot: Optional[dict] = None
    unresolved_components: list = field(default_factory=list)
    kind: str = KIND
    contract_version: str = CONTRACT_VERSION
    semantic_owner: str = SEMANTIC_OWNER
    semantic_backend: str = SEMANTIC_BACKEND

    def to_json(self) -> dict:
        return dict(self.__dict__)

    @classmethod
    def from_json(cls, doc: dict) -> "TrainerExternalStateCheckpoint":
        unknown = set(doc) - set(cls.__dataclass_fields__)
        if unknown:
            raise _state(sorted(unknown)[0], "unknown field")
        ckpt = cls(**doc)
        ckpt.validate()
        return ckpt

    def validate(self) -> TrainerExternalCheckpointValidation:
        for name, expected in (("kind", KIND), ("contract_version", CONTRACT_VERSION),
                               ("semantic_owner", SEMANTIC_OWNER), ("semantic_backend", SEMANTIC_BACKEND)):
            if getattr(self, name) != expected:
                raise TrainerExternalCheckpointError("InvalidMetadata", name, f"{expected}, got {getattr(self, name)}")
        for name in list(self.required_components) + list(self.unresolved_components):
            if name not in COMPONENTS:
                raise _state("required_components", f"unknown component '{name}'")
        if len(set(self.required_components)) != len(self.required_components):
            raise _state("required_components", "must not repeat a component")
        if self.desire_trainer is not None:
            validate_desire_trainer(self.desire_trainer)
        if self.psi_meter is not None:
            validate_psi_meter(self.psi_meter)
        if self.accumulator_synchronizer is not None and not isinstance(self.accumulator_synchronizer, dict):
            raise _state("accumulator_synchronizer", "must be an object")
        if self.autopilot is not None:
            if not isinstance(self.autopilot.get("picks", {}), dict) or not isinstance(self.autopilot.get("suggestion_ready"), bool):
                raise _state("autopilot", "needs picks (object) and suggestion_ready (bool)")
        captured = [c for c in COMPONENTS if getattr(self, c) is not None]
        for c in self.unresolved_components:
            if c in captured:
                raise _state("unresolved_components", f"'{c}' is both captured and unresolved")
        missing = [c for c in self.required_components if c not in captured]
        for c in missing:
            if c not in self.unresolved_components:
                raise _state("required_components", f"'{c}' is required but neither captured nor listed as unresolved")
        complete = not missing
        return TrainerExternalCheckpointValidation(list(self.required_components), captured,
                                                   list(self.unresolved_components), complete,
                                                   complete and not self.unresolved_components)


class TrainerExternalCheckpointComponents:
    """Builder: hand over whatever the trainer could capture; ``build`` records the rest as unresolved."""

    def __init__(self):
        self._parts: dict = {}
        self._required: list = []

    def require(self, *names: str) -> "TrainerExternalCheckpointComponents":
        for n in names:
            if n not in COMPONENTS:
                raise _state("required_components", f"unknown component '{n}'")
            if n not in self._required:
                self._required.append(n)
        return self

    def with_desire_trainer(self, state): self._parts["desire_trainer"] = state; return self                         # noqa: E702
    def with_psi_meter(self, state): self._parts["psi_meter"] = state; return self                                   # noqa: E702
    def with_accumulator_synchronizer(self, state): self._parts["accumulator_synchronizer"] = state; return self     # noqa: E702
    def with_autopilot(self, state): self._parts["autopilot"] = state; return self                                   # noqa: E702

    def build(self) -> TrainerExternalStateCheckpoint:
        parts = {k: v for k, v in self._parts.items() if v is not None}
        unresolved = [c for c in self._required if c not in parts]
        ckpt = TrainerExternalStateCheckpoint(list(self._required), unresolved_components=unresolved, **parts)
        ckpt.validate()
        return ckpt
