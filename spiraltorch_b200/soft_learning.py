"""Learned ranking of rank-k launch choices, and the A/B log the learner is trained from.

A linear model over launch-shape features (log sizes, workgroup / lane / tile ratios, merge kinds, backend one-hot)
gives each candidate a bonus ``tanh(w . f / temperature)`` on top of its heuristic score; the best of the top ``beam``
candidates wins.  The weights come from a JSON store (``SPIRALTORCH_SOFT_RANKER_PATH``, else ``~/.spiraltorch/
soft_ranker.json``, else the legacy ``soft_weights.json``), which is size-checked and validated before use.  Every
measured launch can be appended to a JSON-lines A/B log (``SPIRAL_ABLOG_PATH`` or ``~/.spiraltorch/ablog.jsonl``).

Reference parity: crates/st-core/src/heur/soft_learning.rs (`SoftRuleLearner` :24-154, `SoftContext::features`
:156-200, store paths and validation :202-420), crates/st-core/src/ability/ablog.rs (`ABEntry`, `record`,
`wilson_lower`).
"""
from __future__ import annotations

import json
import math
import os
import sys
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from .kdsl import wilson_lower_bound as wilson_lower  # noqa: F401  (the A/B log's acceptance bound)
from .unison import RankChoice

SOFT_RANKER_PATH_ENV = "SPIRALTORCH_SOFT_RANKER_PATH"
MAX_SOFT_RANKER_BYTES = 16 * 1024 * 1024
MAX_SOFT_RANKER_WEIGHTS = 100_000
MAX_SOFT_RANKER_KEY_BYTES = 4 * 1024
MAX_SOFT_RANKER_BEAM = 65_536
BACKENDS = ("wgpu", "mps", "cuda", "hip", "cpu")


class SoftRankerStoreError(ValueError):
    pass


def default_store_path() -> Path:
    return Path.home() / ".spiraltorch" / "soft_ranker.json"


def legacy_store_path() -> Path:
    return Path.home() / ".spiraltorch" / "soft_weights.json"


@dataclass
class SoftContext:
    rows: int
    cols: int
    k: int
    backend: str = "cuda"
    subgroup: bool = True

    def features(self, choice) -> List[Tuple[str, float]]:
        """``choice`` is a :class:`RankChoice` or any object with its fields; the merge kinds ``mk`` / ``mkd`` and the
        chunk ``ch`` of the reference's wider choice record count as 0 where the object has none."""
        if self.backend not in BACKENDS:
            raise ValueError(f"unknown backend {self.backend!r}; one of {BACKENDS}")
        mk, mkd, ch = (getattr(choice, n, 0) for n in ("mk", "mkd", "ch"))
        return [("bias", 1.0), ("rows_ln", math.log1p(max(self.rows, 1))), ("cols_ln", math.log1p(max(self.cols, 1))),
                ("k_ln", math.log1p(max(self.k, 1))), ("wg_ratio", choice.wg / 512.0), ("kl_ratio", choice.kl / 32.0),
                ("tile_ratio", choice.tile / 4096.0), ("ctile_ratio", choice.ctile / 4096.0), ("mk_kind", mk / 2.0),
                ("mkd_kind", mkd / 5.0), ("two_stage", 1.0 if choice.use_2ce else 0.0), ("ch_norm", ch / 8192.0),
                (f"backend_{self.backend}", 1.0), ("subgroup", 1.0 if self.subgroup else 0.0)]


def _load_store(path: Path) -> Optional[dict]:
    try:
        size = path.stat().st_size
    except FileNotFoundError:
        return None
    except OSError as exc:
        raise SoftRankerStoreError(f"cannot inspect {path}: {exc}") from exc
    if size > MAX_SOFT_RANKER_BYTES:
        raise SoftRankerStoreError(f"{path} holds {size} bytes, more than the {MAX_SOFT_RANKER_BYTES} allowed")
    try:
        value = json.loads(path.read_bytes())
    except (OSError, ValueError) as exc:
        raise SoftRankerStoreError(f"cannot read {path}: {exc}") from exc
    if not isinstance(value, dict) or not any(f in value for f in ("weights", "bias", "temperature", "beam")):
        raise SoftRankerStoreError(f"{path}: unrecognized schema")
    weights = value.get("weights", {})
    if not isinstance(weights, dict):
        raise SoftRankerStoreError(f"{path}: weights must be an object")
    if len(weights) > MAX_SOFT_RANKER_WEIGHTS:
        raise SoftRankerStoreError(f"{path}: {len(weights)} weights, more than the {MAX_SOFT_RANKER_WEIGHTS} allowed")
    for name, w in weights.items():
        if not name.strip() or len(name.encode()) > MAX_SOFT_RANKER_KEY_BYTES:
            raise SoftRankerStoreError(f"{path}: invalid weight name {name!r}")
        if not isinstance(w, (int, float)) or not math.isfinite(w):
            raise SoftRankerStoreError(f"{path}: non-finite value for {name!r}")
    bias, temperature, beam = value.get("bias", 0.0), value.get("temperature", 1.0), value.get("beam", 1)
    for name, v in (("bias", bias), ("temperature", temperature)):
        if not isinstance(v, (int, float)) or not math.isfinite(v):
            raise SoftRankerStoreError(f"{path}: non-finite value for {name!r}")
    if temperature <= 0.0:
        raise SoftRankerStoreError(f"{path}: temperature must be positive")
    if not isinstance(beam, int) or not 1 <= beam <= MAX_SOFT_RANKER_BEAM:
        raise SoftRankerStoreError(f"{path}: beam must lie in 1..{MAX_SOFT_RANKER_BEAM}")
    return {"weights": {k: float(v) for k, v in weights.items()}, "bias": float(bias), "temperature": float(temperature), "beam": beam}


class SoftRuleLearner:
    def __init__(self, weights: Optional[Dict[str, float]] = None, bias: float = 0.0, temperature: float = 1.0, beam: int = 1):
        self.weights, self.bias, self.temperature, self.beam = dict(weights or {}), bias, temperature, beam

    @classmethod
    def try_load_from(cls, path) -> Optional["SoftRuleLearner"]:
        stored = _load_store(Path(path))
        return cls(**stored) if stored is not None else None

    @classmethod
    def try_load(cls) -> Optional["SoftRuleLearner"]:
        """The store named by the environment, else the default store, else the legacy one (whose other schemas are
        ignored rather than reported)."""
        env = os.environ.get(SOFT_RANKER_PATH_ENV)
        if env:
            return cls.try_load_from(env)
        primary = cls.try_load_from(default_store_path())
        if primary is not None:
            return primary
        try:
            return cls.try_load_from(legacy_store_path())
        except SoftRankerStoreError as exc:
            if "unrecognized schema" in str(exc):
                return None
            raise

    @classmethod
    def maybe_load(cls) -> Optional["SoftRuleLearner"]:
        try:
            return cls.try_load()
        except SoftRankerStoreError as exc:
            print(f"[heur] {exc} (ignoring learned ranker)", file=sys.stderr)
            return None

    def learned_bonus(self, ctx: SoftContext, choice: RankChoice) -> float:
        dot = self.bias + sum(self.weights.get(name, 0.0) * value for name, value in ctx.features(choice))
        return math.tanh(dot / self.temperature)

    def rank(self, ctx: SoftContext, candidates: Sequence[Tuple[str, RankChoice, float]]) -> Tuple[int, List[float]]:
        """(index of the winner, score of every candidate); non-finite scores count as minus infinity."""
        scored = []
        for _, choice, base in candidates:
            s = base + self.learned_bonus(ctx, choice)
            scored.append(s if math.isfinite(s) else -math.inf)
        if not scored:
            return 0, scored
        order = sorted(range(len(scored)), key=lambda i: -scored[i])[:max(self.beam, 1)]
        return max(order, key=lambda i: scored[i]), scored


# ---------------------------------------------------------------------------------------------------------------
@dataclass
class ABEntry:
    """One measured launch: ``variant`` is "A" (soft rules), "B" (hard DSL) or "C" (generated table)."""
    rows: int
    cols: int
    k: int
    backend: str
    variant: str
    mk: int
    mkd: int
    tile: int
    ctile: int
    latency_ms: float
    ok: bool
    ts_ms: int = 0


def ablog_path() -> Path:
    env = os.environ.get("SPIRAL_ABLOG_PATH")
    return Path(env) if env else Path.home() / ".spiraltorch" / "ablog.jsonl"


def record(entry: ABEntry) -> None:
    """Appends the entry as one JSON line; a log that cannot be written is skipped silently, as logging must never fail a launch."""
    if not entry.ts_ms:
        entry.ts_ms = int(time.time() * 1000)
    path = ablog_path()
    try:
        path.parent.mkdir(parents=True, exist_ok=True)
        with open(path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(asdict(entry)) + "\n")
    except OSError:
        return
