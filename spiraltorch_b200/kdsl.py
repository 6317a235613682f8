"""SpiralK heuristics DSL, the autotune store / registry and Wilson-bound rewrite decisions.

Restated from crates/st-kdsl/src: ``Program::parse`` / ``evaluate`` (program.rs — hard assignments
``field: expr;``, ``soft(field, value, weight, condition);``, ``let`` / ``set`` variables, ``for i in
a..b { }``, ``if cond { } else { }``, functions ``sel log2 clamp min max abs``, context variables
``r c k sg sgc kc tile_cols radix segments``), ``autotune_store.rs`` (per-key buckets of at most 32
entries, numeric feature extraction from the context, relative feature distance for
``lookup_similar``, lower score wins for the same context), ``registry.rs`` (device / kernel profile
keys, bounded telemetry logs, best-by-TFLOP/s) and ``auto.rs:234-253`` (``wilson_lower_bound``,
``should_rewrite``).

On sm_100a the kernel choices are fixed at build time, so the DSL is not consulted on a hot path;
it is kept so that heuristic files written for the reference still parse and evaluate, and the
store is the place where the benchmark harness records the best launch parameters it measured.
"""
from __future__ import annotations

import json
import math
import os
import re
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

from .config import atomic_write

FIELDS = ("u2", "wg", "kl", "ch", "algo", "midk", "bottomk", "ctile", "tile_cols", "radix", "segments", "mk", "mkd", "tile")
CTX_VARS = ("r", "c", "k", "sg", "sgc", "kc", "tile_cols", "radix", "segments")


class KdslError(ValueError):
    pass


@dataclass
class Ctx:
    r: int = 0
    c: int = 0
    k: int = 0
    sg: bool = False
    sgc: int = 0
    kc: int = 0
    tile_cols: int = 0
    radix: int = 0
    segments: int = 0


@dataclass
class SoftRule:
    field: str
    value: float
    weight: float


@dataclass
class Out:
    hard: dict = field(default_factory=dict)
    soft: list = field(default_factory=list)


_TOKEN = re.compile(r"\s*(?:(\d+\.\d+|\d+)|([A-Za-z_][A-Za-z_0-9]*)|(\.\.|&&|\|\||==|!=|<=|>=|[-+*/%<>!(){};:,=]))")


def _tokenize(src: str) -> list:
    src = re.sub(r"#[^\n]*", "", src)
    out, pos = [], 0
    while pos < len(src):
        if src[pos:].strip() == "":
            break
        m = _TOKEN.match(src, pos)
        if not m:
            raise KdslError(f"unexpected character {src[pos:].strip()[:1]!r}")
        num, ident, op = m.groups()
        out.append(("num", float(num)) if num else ("id", ident) if ident else ("op", op))
        pos = m.end()
    return out


class Program:
    """Parsed SpiralK program; :meth:`evaluate` returns hard assignments and the soft rules whose
    condition held."""

    MAX_LOOP = 100_000

    def __init__(self, stmts: list):
        self._stmts = stmts

    # ---- parser -----------------------------------------------------------------------------------
    @classmethod
    def parse(cls, src: str) -> "Program":
        p = _Parser(_tokenize(src))
        stmts = []
        while not p.done():
            stmts.append(p.stmt())
        return cls(stmts)

    # ---- evaluator --------------------------------------------------------------------------------
    def evaluate(self, ctx: Ctx) -> Out:
        env = {k: (1.0 if v is True else 0.0 if v is False else float(v)) for k, v in vars(ctx).items()}
        out = Out()
        self._steps = 0
        self._run(self._stmts, env, out, set(vars(ctx)))
        return out

    def _run(self, stmts, env, out, readonly):
        for s in stmts:
            kind = s[0]
            if kind == "assign":
                v = self._eval(s[2], env)
                out.hard[s[1]] = bool(v) if s[1] == "u2" else int(round(v))
                env[s[1]] = float(v)
            elif kind == "soft":
                if self._eval(s[4], env) != 0.0:
                    out.soft.append(SoftRule(s[1], self._eval(s[2], env), self._eval(s[3], env)))
            elif kind == "let":
                env[s[1]] = self._eval(s[2], env)
            elif kind == "set":
                if s[1] not in env:
                    raise KdslError(f"set of undeclared variable '{s[1]}'")
                env[s[1]] = self._eval(s[2], env)
            elif kind == "if":
                self._run(s[2] if self._eval(s[1], env) != 0.0 else s[3], env, out, readonly)
            elif kind == "for":
                lo, hi = int(self._eval(s[2], env)), int(self._eval(s[3], env))
                for i in range(lo, hi):
                    self._steps += 1
                    if self._steps > self.MAX_LOOP:
                        raise KdslError("loop budget exceeded")
                    env[s[1]] = float(i)
                    self._run(s[4], env, out, readonly)
            elif kind == "while":
                while self._eval(s[1], env) != 0.0:
                    self._steps += 1
                    if self._steps > self.MAX_LOOP:
                        raise KdslError("loop budget exceeded")
                    self._run(s[2], env, out, readonly)

    def _eval(self, e, env) -> float:
        k = e[0]
        if k == "num":
            return e[1]
        if k == "var":
            if e[1] not in env:
                raise KdslError(f"unknown identifier '{e[1]}'")
            return env[e[1]]
        if k == "neg":
            return -self._eval(e[1], env)
        if k == "not":
            return 0.0 if self._eval(e[1], env) != 0.0 else 1.0
        if k == "call":
            a = [self._eval(x, env) for x in e[2]]
            f = e[1]
            try:
                if f == "sel":
                    return a[1] if a[0] != 0.0 else a[2]
                if f == "log2":
                    if a[0] <= 0:
                        raise KdslError("log2 of a non-positive value")
                    return math.log2(a[0])
                if f == "clamp":
                    return min(max(a[0], a[1]), a[2])
                if f == "min":
                    return min(a)
                if f == "max":
                    return max(a)
                if f == "abs":
                    return abs(a[0])
                if f == "floor":
                    return float(math.floor(a[0]))
                if f == "ceil":
                    return float(math.ceil(a[0]))
            except IndexError:
                raise KdslError(f"too few arguments for {f}()") from None
            raise KdslError(f"unknown function '{f}'")
        a, b = self._eval(e[1], env), None
        if k == "&&":
            return 1.0 if a != 0.0 and self._eval(e[2], env) != 0.0 else 0.0
        if k == "||":
            return 1.0 if a != 0.0 or self._eval(e[2], env) != 0.0 else 0.0
        b = self._eval(e[2], env)
        if k == "+":
            return a + b
        if k == "-":
            return a - b
        if k == "*":
            return a * b
        if k in ("/", "%"):
            if b == 0:
                raise KdslError("division by zero")
            return a / b if k == "/" else math.fmod(a, b)
        return 1.0 if {"==": a == b, "!=": a != b, "<": a < b, "<=": a <= b, ">": a > b, ">=": a >= b}[k] else 0.0


class _Parser:
    def __init__(self, toks: list):
        self.t, self.i = toks, 0

    def done(self) -> bool:
        return self.i >= len(self.t)

    def peek(self, k: int = 0):
        return self.t[self.i + k] if self.i + k < len(self.t) else (None, None)

    def next(self):
        if self.done():
            raise KdslError("unexpected end of program")
        tok = self.t[self.i]
        self.i += 1
        return tok

    def expect(self, op: str) -> None:
        tok = self.next()
        if tok != ("op", op):
            raise KdslError(f"expected '{op}', got {tok[1]!r}")

    def ident(self) -> str:
        kind, v = self.next()
        if kind != "id":
            raise KdslError(f"expected an identifier, got {v!r}")
        return v

    def block(self) -> list:
        self.expect("{")
        out = []
        while self.peek() != ("op", "}"):
            out.append(self.stmt())
        self.expect("}")
        return out

    def stmt(self):
        kind, v = self.peek()
        if kind == "id" and v == "soft" and self.peek(1) == ("op", "("):
            self.next(); self.expect("(")
            fld = self.ident()
            if fld not in FIELDS:
                raise KdslError(f"unknown field '{fld}'")
            self.expect(","); val = self.expr()
            self.expect(","); w = self.expr()
            self.expect(","); cond = self.expr()
            self.expect(")"); self.expect(";")
            return ("soft", fld, val, w, cond)
        if kind == "id" and v in ("let", "set"):
            self.next()
            name = self.ident()
            self.expect("=")
            e = self.expr()
            self.expect(";")
            return (v, name, e)
        if kind == "id" and v == "if":
            self.next()
            cond = self.expr()
            then = self.block()
            other = []
            if self.peek() == ("id", "else"):
                self.next()
                other = [self.stmt()] if self.peek() == ("id", "if") else self.block()
            return ("if", cond, then, other)
        if kind == "id" and v == "for":
            self.next()
            var = self.ident()
            if self.ident() != "in":
                raise KdslError("expected 'in' after the loop variable")
            lo = self.expr(); self.expect(".."); hi = self.expr()
            return ("for", var, lo, hi, self.block())
        if kind == "id" and v == "while":
            self.next()
            cond = self.expr()
            return ("while", cond, self.block())
        if kind == "id" and self.peek(1) == ("op", ":"):
            fld = self.ident()
            if fld not in FIELDS:
                raise KdslError(f"unknown field '{fld}'")
            self.expect(":")
            e = self.expr()
            self.expect(";")
            return ("assign", fld, e)
        raise KdslError(f"unexpected token {v!r}")

    # precedence: || < && < comparison < + - < * / % < unary
    def expr(self):
        return self._binary(0)

    _LEVELS = (("||",), ("&&",), ("==", "!=", "<", "<=", ">", ">="), ("+", "-"), ("*", "/", "%"))

    def _binary(self, level: int):
        if level == len(self._LEVELS):
            return self._unary()
        left = self._binary(level + 1)
        while self.peek()[0] == "op" and self.peek()[1] in self._LEVELS[level]:
            op = self.next()[1]
            left = (op, left, self._binary(level + 1))
        return left

    def _unary(self):
        if self.peek() == ("op", "-"):
            self.next()
            return ("neg", self._unary())
        if self.peek() == ("op", "!"):
            self.next()
            return ("not", self._unary())
        kind, v = self.next()
        if kind == "num":
            return ("num", v)
        if kind == "op" and v == "(":
            e = self.expr()
            self.expect(")")
            return e
        if kind == "id":
            if v in ("true", "false"):
                return ("num", 1.0 if v == "true" else 0.0)
            if self.peek() == ("op", "("):
                self.next()
                args = []
                if self.peek() != ("op", ")"):
                    args.append(self.expr())
                    while self.peek() == ("op", ","):
                        self.next()
                        args.append(self.expr())
                self.expect(")")
                return ("call", v, args)
            return ("var", v)
        raise KdslError(f"unexpected token {v!r}")


# ---- Wilson-bound rewrite decision -----------------------------------------------------------------
def wilson_lower_bound(wins: int, trials: int, z: float = 1.96) -> float:
    if trials == 0:
        return 0.0
    n = float(trials)
    p = wins / n
    denom = 1.0 + z * z / n
    centre = p + z * z / (2.0 * n)
    margin = z * math.sqrt((p * (1.0 - p) + z * z / (4.0 * n)) / n)
    return (centre - margin) / denom


@dataclass
class WilsonMetrics:
    baseline_latency: float
    candidate_latency: float
    wins: int
    trials: int

    def gain(self) -> float:
        return (self.baseline_latency - self.candidate_latency) / self.baseline_latency if self.baseline_latency > 0 else 0.0


def should_rewrite(metrics: WilsonMetrics, min_gain: float, min_confidence: float) -> bool:
    if metrics.trials == 0 or metrics.gain() < min_gain:
        return False
    return wilson_lower_bound(metrics.wins, metrics.trials) >= min_confidence


# ---- autotune store ---------------------------------------------------------------------------------
BUCKET_HISTORY_LIMIT = 32


def default_store_path() -> Path:
    return Path(os.environ.get("SPIRALTORCH_AUTOTUNE_STORE", str(Path.home() / ".spiraltorch" / "kernels.json")))


def _features(value: Any, path: str = "", out: Optional[list] = None) -> list:
    out = [] if out is None else out
    if isinstance(value, bool):
        out.append((path, 1.0 if value else 0.0))
    elif isinstance(value, (int, float)):
        out.append((path, float(value)))
    elif isinstance(value, (list, tuple)):
        for i, v in enumerate(value):
            _features(v, f"{path}.{i}" if path else str(i), out)
    elif isinstance(value, dict):
        for k, v in value.items():
            _features(v, f"{path}.{k}" if path else str(k), out)
    return sorted(out)


def _distance(a: list, b: list) -> float:
    da, db = dict(a), dict(b)
    d = 0.0
    for key in set(da) | set(db):
        if key in da and key in db:
            d += abs(da[key] - db[key]) / max(abs(da[key]), abs(db[key]), 1.0)
        else:
            d += abs(da.get(key, db.get(key)))
    return d


def load_store(path) -> dict:
    try:
        raw = json.loads(Path(path).read_text())
    except (OSError, ValueError):
        return {}
    out = {}
    for key, bucket in raw.items():
        if isinstance(bucket, dict) and "entries" in bucket:
            out[key] = bucket
        elif isinstance(bucket, dict) and "params" in bucket:          # legacy flat layout
            out[key] = {"entries": [{"updated_unix": bucket.get("updated_unix", 0), "score": bucket.get("score", 0.0),
                                     "params": bucket["params"], "context": None, "features": []}]}
    return out


def record_best(path, key: str, context: Any, score: float, params: Any) -> bool:
    """Keep ``params`` for ``(key, context)`` if ``score`` (lower is better) beats the stored one.
    Returns whether the entry was inserted or replaced."""
    store = load_store(path)
    entry = {"updated_unix": int(time.time()), "score": float(score), "params": params, "context": context,
             "features": [list(f) for f in _features(context)]}
    bucket = store.setdefault(key, {"entries": []})
    changed = True
    for i, e in enumerate(bucket["entries"]):
        if e["context"] == context:
            if score < e["score"]:
                bucket["entries"][i] = entry
            else:
                e["updated_unix"] = entry["updated_unix"]
                changed = False
            break
    else:
        bucket["entries"].append(entry)
    bucket["entries"].sort(key=lambda e: -e["updated_unix"])
    del bucket["entries"][BUCKET_HISTORY_LIMIT:]
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    atomic_write(path, json.dumps(store, indent=1, sort_keys=True))
    return changed


def lookup_similar(path, key: str, context: Any, limit: int = 4) -> list:
    """``[(entry, distance)]`` sorted by feature distance to ``context``, then by score."""
    bucket = load_store(path).get(key)
    if not bucket:
        return []
    feats = _features(context)
    matches = [(e, _distance(feats, [tuple(f) for f in e.get("features", [])])) for e in bucket["entries"]]
    matches.sort(key=lambda m: (m[1], m[0]["score"]))
    return matches[:limit]


def lookup_best(path, key: str, context: Any) -> Optional[dict]:
    m = lookup_similar(path, key, context, 1)
    return m[0][0] if m else None


# ---- registry -----------------------------------------------------------------------------------------
def _enc(v: str) -> str:
    return "".join(ch if (ch.isalnum() and ch.isascii()) or ch in "-_." else "-" if ch == " " else "_" for ch in v)


@dataclass(frozen=True)
class DeviceProfile:
    vendor: str
    device_id: int
    subgroup_size: int
    shared_kb: int
    driver: str

    def encode(self) -> str:
        return f"{_enc(self.vendor)}|{self.device_id:04x}|{self.subgroup_size}|{self.shared_kb}|{_enc(self.driver)}"

    @classmethod
    def current(cls) -> "DeviceProfile":
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            return cls("nvidia", p.major * 10 + p.minor, 32, 227, torch.version.cuda or "unknown")
        return cls("cpu", 0, 1, 0, "none")


@dataclass(frozen=True)
class KernelProfile:
    shader_revision: int
    op_signature: str

    def encode(self) -> str:
        return f"{self.shader_revision:016x}|{self.op_signature}"


@dataclass(frozen=True)
class AutotuneKey:
    device: DeviceProfile
    kernel: KernelProfile

    def encode(self) -> str:
        return f"{self.device.encode()}|{self.kernel.encode()}"

    __str__ = encode


@dataclass
class TelemetrySample:
    tflops: float
    bandwidth_gbps: float
    occupancy: float
    tile: Optional[dict] = None
    regress: bool = False

    def is_regression(self) -> bool:
        return self.regress


class TelemetryLog:
    def __init__(self):
        self._samples: list = []

    def push(self, sample: TelemetrySample) -> None:
        self._samples.append(sample)

    def push_bounded(self, sample: TelemetrySample, max_len: int) -> None:
        self._samples.append(sample)
        if max_len > 0 and len(self._samples) > max_len:
            del self._samples[: len(self._samples) - max_len]

    def __len__(self) -> int:
        return len(self._samples)

    def __iter__(self):
        return iter(self._samples)

    def best_by_tflops(self) -> Optional[TelemetrySample]:
        return max(self._samples, key=lambda s: s.tflops, default=None)

    def best_tile(self) -> Optional[dict]:
        b = self.best_by_tflops()
        return None if b is None else b.tile

    def summary(self) -> Optional[dict]:
        if not self._samples:
            return None
        n = len(self._samples)
        return {"samples": n, "mean_tflops": sum(s.tflops for s in self._samples) / n,
                "mean_bandwidth_gbps": sum(s.bandwidth_gbps for s in self._samples) / n,
                "mean_occupancy": sum(s.occupancy for s in self._samples) / n,
                "best_tflops": self.best_by_tflops().tflops, "regressions": sum(s.regress for s in self._samples)}

    def regression_rate(self) -> Optional[float]:
        return sum(s.regress for s in self._samples) / len(self._samples) if self._samples else None


class AutotuneRegistry:
    def __init__(self, capacity: int = 64):
        self._capacity, self._logs = max(1, capacity), {}

    @classmethod
    def with_capacity(cls, capacity: int) -> "AutotuneRegistry":
        return cls(capacity)

    def capacity(self) -> int:
        return self._capacity

    def set_capacity(self, capacity: int) -> None:
        self._capacity = max(1, capacity)
        for log in self._logs.values():
            del log._samples[: max(0, len(log) - self._capacity)]

    def record(self, key: AutotuneKey, sample: TelemetrySample) -> None:
        self._logs.setdefault(key.encode(), TelemetryLog()).push_bounded(sample, self._capacity)

    def log(self, key: AutotuneKey) -> Optional[TelemetryLog]:
        return self._logs.get(key.encode())

    def keys(self) -> list:
        return sorted(self._logs)
