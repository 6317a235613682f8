"""Two small companions of the SpiralK language: a query planner over tuner / telemetry rows, and a warp-level IR whose
statements emit CUDA warp intrinsics.

Parity: crates/st-kdsl/src/query.rs — `compile` (:138-250: ``SELECT cols WHERE col op number [AND ...] ORDER BY col
[ASC|DESC] LIMIT n``, case-insensitive, ``;`` ignored, the order defaults to descending), `QueryPlan::execute` (:50-85:
filters, then the sort with NaN last in either direction, then the limit, then the projection; a missing column reads
as 0), `Filter` (:105-136: equality within f64 epsilon); crates/st-kdsl/src/ir.rs — `ScalarType`, `Expr`, `SubgroupOp`,
`SubgroupStmt`, `SubgroupModule::{emit_function, emit_statements}`.  The reference's IR prints WGSL subgroup built-ins;
this one prints their sm_100a equivalents (``__shfl_xor_sync``, ``__ballot_sync``, ``__reduce_add_sync`` ...) as a
``__device__`` function body, which is what a generated kernel here would include.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .kdsl import KdslError

EPS = 2.220446049250313e-16
_OPS = {"=": lambda c, v: abs(c - v) <= EPS, "!=": lambda c, v: abs(c - v) > EPS, ">": lambda c, v: c > v, "<": lambda c, v: c < v,
        ">=": lambda c, v: c >= v, "<=": lambda c, v: c <= v}


@dataclass(frozen=True)
class Filter:
    column: str
    op: str
    value: float

    def matches(self, row: Dict[str, float]) -> bool:
        return _OPS[self.op](float(row.get(self.column, 0.0)), self.value)


@dataclass
class QueryPlan:
    selects: List[str] = field(default_factory=list)
    filters: List[Filter] = field(default_factory=list)
    order: Optional[Tuple[str, str]] = None          # (column, "asc" | "desc")
    limit: Optional[int] = None

    def execute(self, rows: Sequence[Dict[str, float]]) -> List[Dict[str, float]]:
        out = [dict(r) for r in rows if all(f.matches(r) for f in self.filters)]
        if self.order is not None:
            col, direction = self.order
            sign = 1.0 if direction == "asc" else -1.0

            def key(r):
                v = float(r.get(col, 0.0))
                return (1, 0.0) if math.isnan(v) else (0, sign * v)
            out.sort(key=key)                        # stable, NaN after every number in both directions
        if self.limit is not None:
            out = out[:self.limit]
        if not self.selects:
            return out
        return [{c: r[c] for c in self.selects if c in r} for r in out]


def _lex(src: str) -> List[Tuple[str, int]]:
    tokens, cur, start, i = [], "", 0, 0

    def flush():
        nonlocal cur
        if cur:
            tokens.append((cur.lower(), start))
            cur = ""
    while i < len(src):
        ch = src[i]
        if ch.isspace() or ch == ";":
            flush()
        elif ch in ",=!<>":
            flush()
            op = ch
            if i + 1 < len(src) and ch != "," and (src[i + 1] == "=" or (src[i + 1] == ">" and ch == "<")):
                op += src[i + 1]
                i += 1
            tokens.append((op, i - len(op) + 1))
        else:
            if not cur:
                start = i
            cur += ch
        i += 1
    flush()
    return tokens


def compile_query(src: str) -> QueryPlan:
    """Parses a query; a syntax error raises `KdslError` carrying the byte position of the offending token."""
    toks = _lex(src)
    plan = QueryPlan()
    if not toks:
        return plan
    cur = 0

    def fail():
        raise KdslError(f"query parse error at {toks[cur][1] if cur < len(toks) else len(src)}")

    def text(i):
        return toks[i][0]
    if text(0) != "select":
        fail()
    cur = 1
    while cur < len(toks):
        t = text(cur)
        if t == "where":
            cur += 1
            break
        if t in ("order", "limit"):
            break
        if t != ",":
            plan.selects.append(t)
        cur += 1
    while cur < len(toks):
        t = text(cur)
        if t in ("order", "limit"):
            break
        if t == "and":
            cur += 1
            continue
        column = t
        cur += 1
        if cur >= len(toks):
            fail()
        op = text(cur)
        cur += 1
        if cur >= len(toks):
            fail()
        try:
            value = float(text(cur))
        except ValueError:
            fail()
        cur += 1
        if op not in _OPS:
            fail()
        plan.filters.append(Filter(column, op, value))
    if cur < len(toks) and text(cur) == "order":
        cur += 1
        if cur >= len(toks) or text(cur) != "by":
            fail()
        cur += 1
        if cur >= len(toks):
            fail()
        column, direction = text(cur), "desc"
        cur += 1
        if cur < len(toks) and text(cur) in ("asc", "desc"):
            direction = text(cur)
            cur += 1
        plan.order = (column, direction)
    if cur < len(toks) and text(cur) == "limit":
        cur += 1
        if cur >= len(toks):
            fail()
        try:
            plan.limit = int(text(cur))
            if plan.limit < 0:
                raise ValueError
        except ValueError:
            fail()
    return plan


# ---- warp IR ---------------------------------------------------------------------------------------------------------------
SCALAR_TYPES = {"bool": "bool", "f16": "__half", "f32": "float", "i32": "int", "u32": "unsigned"}
FULL_MASK = "0xffffffffu"


@dataclass(frozen=True)
class WarpOp:
    """One warp-collective: ``kind`` in shuffle_xor / shuffle_up / shuffle_down / broadcast_first / ballot / all / any /
    reduce_add / reduce_min / reduce_max, ``value`` an expression, ``arg`` the lane mask or delta where one is needed."""
    kind: str
    value: str
    arg: Optional[str] = None

    def emit(self, ty: str) -> str:
        v, a = self.value, self.arg
        simple = {"shuffle_xor": f"__shfl_xor_sync({FULL_MASK}, {v}, {a})", "shuffle_up": f"__shfl_up_sync({FULL_MASK}, {v}, {a})",
                  "shuffle_down": f"__shfl_down_sync({FULL_MASK}, {v}, {a})", "broadcast_first": f"__shfl_sync({FULL_MASK}, {v}, 0)",
                  "ballot": f"__ballot_sync({FULL_MASK}, {v})", "all": f"(__all_sync({FULL_MASK}, {v}) != 0)",
                  "any": f"(__any_sync({FULL_MASK}, {v}) != 0)"}
        if self.kind in simple:
            if self.kind.startswith("shuffle") and a is None:
                raise KdslError(f"{self.kind} needs a lane mask or delta")
            return simple[self.kind]
        if self.kind in ("reduce_add", "reduce_min", "reduce_max"):
            op = self.kind.split("_")[1]
            if ty in ("i32", "u32"):                    # the hardware reduction exists for 32-bit integers only
                return f"__reduce_{op}_sync({FULL_MASK}, {v})"
            return f"warp_reduce_{op}({v})"             # a five-step butterfly of __shfl_xor_sync, emitted once per module
        raise KdslError(f"unknown warp op '{self.kind}'")


@dataclass(frozen=True)
class WarpStmt:
    name: str
    ty: str
    op: WarpOp

    def emit(self) -> str:
        if self.ty not in SCALAR_TYPES:
            raise KdslError(f"unknown scalar type '{self.ty}', expected one of {sorted(SCALAR_TYPES)}")
        return f"const {SCALAR_TYPES[self.ty]} {self.name} = {self.op.emit(self.ty)};"


_BUTTERFLY = """template <class T> __device__ __forceinline__ T warp_reduce_{op}(T v) {{
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {{ T o = __shfl_xor_sync({mask}, v, m); v = {expr}; }}
    return v;
}}
"""
_EXPR = {"add": "v + o", "min": "o < v ? o : v", "max": "o > v ? o : v"}


class WarpModule:
    def __init__(self):
        self.statements: List[WarpStmt] = []

    def push(self, stmt: WarpStmt) -> "WarpModule":
        self.statements.append(stmt)
        return self

    def emit_statements(self) -> str:
        return "".join(s.emit() + "\n" for s in self.statements)

    def helpers(self) -> str:
        need = sorted({s.op.kind.split("_")[1] for s in self.statements if s.op.kind.startswith("reduce_") and s.ty not in ("i32", "u32")})
        return "".join(_BUTTERFLY.format(op=o, mask=FULL_MASK, expr=_EXPR[o]) for o in need)

    def emit_function(self, name: str, params: str = "", tail: str = "") -> str:
        """``tail``: statements that use the declared names (the function returns nothing by itself)."""
        body = "".join("    " + s.emit() + "\n" for s in self.statements) + "".join("    " + line + "\n" for line in tail.splitlines())
        return f"{self.helpers()}__device__ __forceinline__ void {name}({params}) {{\n{body}}}\n"
