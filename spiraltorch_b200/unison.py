"""Three-voice chooser for rank-k launch parameters: a device-derived fallback, a SpiralK program from the
environment, a shared key/value record and a generated per-device table each propose a choice; every proposal is
refined against the fallback (aligned to whole warps, bounded by the device) and scored, and the best one wins.

Parity: crates/st-core/src/backend/unison_heuristics.rs — `fallback_with_scenario` (:1145-1240), `refine_choice`
(:1475-1595), `closeness` / `score_choice` (:1597-1688), `choose_unified_rank` (:1950-2045) — and the generated-table
voice of `wgpu_heuristics::choose` (crates/st-core/src/backend/wgpu_heuristics.rs).  The reference scores WGPU tile
knobs; here the same structure scores the knobs of the sm_100a rank kernels (`ops/rank.py`): whether to split into
per-chunk candidates + merge (`use_2ce`), the CTA size, lanes per key, the sweep tile and the compaction tile.

Voices:
  fallback   from `DeviceCaps` alone (`recommended_workgroup`, `default_lane_quota`, `recommended_tiles`,
             `prefers_two_stage`)
  kdsl_env   the SpiralK program in ``SPIRAL_HEUR_K`` evaluated on ``(r, c, k, sg)``; hard assignments override,
             soft rules with weight >= 0.5 nudge
  kdsl_kv    a `Choice` stored under ``SPIRAL_HEUR_KV_KEY`` (default ``spiral:heur:rank:<kind>:<bucket>``) in the store
             at ``SPIRAL_HEUR_KV_URL`` (``memory://...`` or ``redis://...``)
  generated  the nearest entry of the table shipped in ``data/rank_heuristics_b200.json`` (written by
             ``benchmarks/tune_rank.py`` from CUDA-event timings on the device)
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Dict, Optional

from . import kdsl
from .device_caps import DeviceCaps

KINDS = ("topk", "midk", "bottomk")
TABLE_PATH = Path(__file__).resolve().parent / "data" / "rank_heuristics_b200.json"


@dataclass(frozen=True)
class RankChoice:
    use_2ce: bool
    wg: int
    kl: int
    tile: int
    ctile: int
    subgroup: bool = True

    def as_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass
class UnifiedRankReport:
    choice: RankChoice
    source: str
    score: float
    baseline: RankChoice
    scores: Dict[str, float] = field(default_factory=dict)      # one entry per voice that spoke


def _check(rows: int, cols: int, k: int, kind: str) -> None:
    if kind not in KINDS:
        raise ValueError(f"unknown rank kind '{kind}', expected one of {KINDS}")
    if rows < 0 or cols <= 0 or k <= 0 or k > cols:
        raise ValueError(f"invalid rank problem rows={rows} cols={cols} k={k}")


def requires_compaction(kind: str) -> bool:
    return kind in ("midk", "bottomk")


def fallback(rows: int, cols: int, k: int, caps: DeviceCaps, kind: str = "topk") -> RankChoice:
    tile, ctile = caps.recommended_tiles(cols)
    if kind == "bottomk":                               # the compaction tile stays within half a sweep tile
        ctile = max(min(ctile, max(tile // 2, 128)), 128)
    return RankChoice(caps.prefers_two_stage(cols, k, rows), caps.recommended_workgroup(rows), caps.default_lane_quota(k), tile, ctile,
                      caps.subgroup)


def refine(choice: RankChoice, baseline: RankChoice, caps: DeviceCaps, cols: int) -> RankChoice:
    """Pulls a proposal into the device's domain: block size to whole warps within the limit, lanes to a power of two
    in [1, lane_width], tiles to warp multiples no larger than the padded row; zero fields inherit the baseline."""
    lanes = max(caps.lane_width, 1)
    wg = caps.align_workgroup(choice.wg) if choice.wg > 0 else baseline.wg
    kl = choice.kl if choice.kl > 0 else baseline.kl
    kl = min(1 << max(int(math.log2(max(kl, 1)) + 0.5), 0), lanes)
    padded = max(1 << max(cols - 1, 1).bit_length(), lanes)
    tile = choice.tile if choice.tile > 0 else baseline.tile
    tile = max(min(-(-tile // lanes) * lanes, padded), lanes)
    ctile = choice.ctile if choice.ctile > 0 else baseline.ctile
    ctile = max(min(-(-ctile // lanes) * lanes, tile), lanes)
    return RankChoice(bool(choice.use_2ce), wg, kl, tile, ctile, caps.subgroup)


def closeness(actual: int, target: int) -> float:
    if actual == 0 or target == 0:
        return 0.0
    return max(1.0 - min(abs(actual - target) / max(target, 1), 1.0), 0.0)


def score(choice: RankChoice, baseline: RankChoice, caps: DeviceCaps, rows: int, cols: int, k: int, kind: str,
          measured_gain: float = 0.0) -> float:
    """Agreement with the expected strategy (+0.25 / -0.1), closeness of block size, lanes and tiles to the baseline,
    and the device's occupancy score of the block size.  ``measured_gain`` (the fraction of the direct kernel's time a
    tuned entry saved on this device, in [0, 1]) replaces the strategy expectation when it is positive — the strategy
    that was timed faster *is* the expected one — and adds itself to the score: a measurement outranks shape rules."""
    if measured_gain > 0.0:
        s = 0.25 + min(measured_gain, 1.0)
    else:
        s = 0.25 if choice.use_2ce == caps.prefers_two_stage(cols, k, rows) else -0.1
    s += 0.2 * closeness(choice.wg, baseline.wg) + 0.2 * caps.occupancy_score(choice.wg)
    s += 0.15 * closeness(choice.kl, baseline.kl) + 0.1 * closeness(choice.tile, baseline.tile)
    if requires_compaction(kind):
        s += 0.1 * closeness(choice.ctile, baseline.ctile)
    return s


# ---- voices -------------------------------------------------------------------------------------------------------------
def _from_kdsl(src: str, rows: int, cols: int, k: int, caps: DeviceCaps, baseline: RankChoice) -> Optional[RankChoice]:
    try:
        out = kdsl.Program.parse(src).evaluate(kdsl.Ctx(r=rows, c=cols, k=k, sg=caps.subgroup))
    except kdsl.KdslError:
        return None
    fields = {"u2": "use_2ce", "use_2ce": "use_2ce", "wg": "wg", "kl": "kl", "tile": "tile", "tile_cols": "tile", "ctile": "ctile"}
    picked = {}
    for rule in out.soft:                              # soft rules first, so that hard assignments override them
        if rule.field in fields and rule.weight >= 0.5:
            picked[fields[rule.field]] = rule.value
    for name, value in out.hard.items():
        if name in fields:
            picked[fields[name]] = value
    if not picked:
        return None
    c = replace(baseline, **{f: (bool(v) if f == "use_2ce" else int(v)) for f, v in picked.items()})
    return c


def _bucket(n: int) -> int:
    return 1 << max(n - 1, 0).bit_length()


def kv_key(rows: int, cols: int, k: int, kind: str) -> str:
    return os.environ.get("SPIRAL_HEUR_KV_KEY") or f"spiral:heur:rank:{kind}:{_bucket(rows)}x{_bucket(cols)}k{_bucket(k)}"


def _from_kv(rows: int, cols: int, k: int, kind: str, baseline: RankChoice) -> Optional[RankChoice]:
    url = os.environ.get("SPIRAL_HEUR_KV_URL")
    if not url:
        return None
    from . import kv
    try:
        c = kv.connect(url).get_choice(kv_key(rows, cols, k, kind))
    except Exception:                                   # noqa: BLE001 - a store that is down must not stop a launch
        return None
    if c is None:
        return None
    return RankChoice(c.use_2ce, c.wg, c.kl, c.tile_cols or baseline.tile, c.ctile or baseline.ctile, baseline.subgroup)


_table_cache: Optional[list] = None


def load_table(path: Optional[Path] = None) -> list:
    """Entries ``{kind, rows, cols, k, use_2ce, wg, kl, tile, ctile, ms}``; an absent or unreadable file is an empty table."""
    global _table_cache
    if path is None and _table_cache is not None:
        return _table_cache
    try:
        entries = json.loads((path or TABLE_PATH).read_text()).get("entries", [])
    except (OSError, ValueError):
        entries = []
    if path is None:
        _table_cache = entries
    return entries


def _from_table(rows: int, cols: int, k: int, kind: str, baseline: RankChoice, table: Optional[list] = None):
    """``(choice, measured gain)`` of the nearest tuned shape, or ``None``."""
    best, best_d = None, None
    for e in (load_table() if table is None else table):
        if e.get("kind") != kind:
            continue
        d = sum(abs(math.log2(max(a, 1)) - math.log2(max(b, 1))) for a, b in ((rows, e["rows"]), (cols, e["cols"]), (k, e["k"])))
        if best_d is None or d < best_d:
            best, best_d = e, d
    if best is None or best_d > 3.0:                    # more than three octaves away in total: not a neighbour
        return None
    gain = 0.0
    if best.get("ms") and best.get("direct_ms"):
        gain = 1.0 - float(best["ms"]) / float(best["direct_ms"])
    return RankChoice(bool(best["use_2ce"]), int(best["wg"]), int(best["kl"]), int(best.get("tile") or baseline.tile),
                      int(best.get("ctile") or baseline.ctile), baseline.subgroup), gain


def choose_unified_rank(rows: int, cols: int, k: int, caps: Optional[DeviceCaps] = None, kind: str = "topk",
                        table: Optional[list] = None) -> UnifiedRankReport:
    _check(rows, cols, k, kind)
    caps = caps or DeviceCaps.probe()
    baseline = fallback(rows, cols, k, caps, kind)
    best, best_source = baseline, "fallback"
    best_score = score(baseline, baseline, caps, rows, cols, k, kind)
    scores = {"fallback": best_score}
    voices = []
    src = os.environ.get("SPIRAL_HEUR_K")
    if src:
        voices.append(("kdsl_env", _from_kdsl(src, rows, cols, k, caps, baseline)))
    voices.append(("kdsl_kv", _from_kv(rows, cols, k, kind, baseline)))
    if caps.backend == "cuda":
        voices.append(("generated", _from_table(rows, cols, k, kind, baseline, table)))
    for name, proposal in voices:
        if proposal is None:
            continue
        gain = 0.0
        if isinstance(proposal, tuple):
            proposal, gain = proposal
        refined = refine(proposal, baseline, caps, cols)
        s = score(refined, baseline, caps, rows, cols, k, kind, gain)
        scores[name] = s
        if s > best_score:
            best, best_score, best_source = refined, s, name
    return UnifiedRankReport(best, best_source, best_score, baseline, scores)
