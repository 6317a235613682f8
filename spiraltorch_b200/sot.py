"""SoT-3D-phi: a spiral plan of reasoning steps.  Steps sit on a golden-angle logarithmic spiral that climbs in height;
they are grouped into macro orbits of Fibonacci lengths, each orbit into meso chunks of Tribonacci lengths (roles
explore / structure / verify) and each chunk into micro chunks of Tetranacci lengths (roles diverge / ground / design /
test).  The last step of every group is a reflection point.

Parity: bindings/st-py/src/sot.rs — `fibonacci_orbits` (:110), `nacci_numbers` / `pack_with_sequence` (:133-175: the
largest admissible n-nacci number closest to half of what remains, the larger one on ties), `build_plan` (:185-330),
`build_plan_seeded` (:352-371, splitmix64 angle offset), the tensor exports (:643-758) and the module functions
`generate_plan`, `pack_tribonacci_chunks`, `pack_tetranacci_chunks`, `fibonacci_pacing`, `golden_angle`,
`golden_ratio` (:933-980).  The plan's columns are built as tensors in one pass (positions, features, roles,
reflections), so a plan of any length lands on a device as a single copy.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .tensor import Tensor

GOLDEN_ANGLE = 2.399963229728653          # pi (3 - sqrt 5)
GOLDEN_RATIO = 1.618033988749895
MESO_ROLES = ("explore", "structure", "verify")
MICRO_ROLES = ("diverge", "ground", "design", "test")
__all__ = ["generate_plan", "pack_tetranacci_chunks", "pack_tribonacci_chunks", "fibonacci_pacing", "golden_angle", "golden_ratio",
           "SoT3DPlan", "SoT3DStep", "MacroSummary"]


def golden_angle() -> float:
    return GOLDEN_ANGLE


def golden_ratio() -> float:
    return GOLDEN_RATIO


def _fibonacci_orbits(total: int) -> List[Tuple[int, int]]:
    """``(actual, ideal)`` lengths: 1, 1, 2, 3, 5, ... with the last orbit cut to what is left."""
    out, a, b = [], 1, 1
    while total > 0:
        take = min(a, total)
        out.append((take, a))
        total -= take
        a, b = b, a + b
    return out


def fibonacci_pacing(total_steps: int) -> List[int]:
    return [a for a, _ in _fibonacci_orbits(total_steps)]


def _nacci(order: int, seeds: Sequence[int], limit: int) -> List[int]:
    seq = list(seeds)
    while seq[-1] < limit:
        seq.append(sum(seq[-order:]))
    return sorted({v for v in seq if v <= limit}) or [1]


def _pack(length: int, order: int, seeds: Sequence[int]) -> List[int]:
    chunks, remaining = [], length
    while remaining > 0:
        target = remaining / 2.0
        best = min(_nacci(order, seeds, remaining), key=lambda c: (abs(c - target), -c))
        chunks.append(best)
        remaining -= best
    return chunks


def pack_tribonacci_chunks(length: int) -> List[int]:
    return _pack(length, 3, (1, 1, 2))


def pack_tetranacci_chunks(length: int) -> List[int]:
    return _pack(length, 4, (1, 1, 2, 4))


@dataclass
class SoT3DStep:
    index: int
    angle: float
    radius: float
    x: float
    y: float
    height: float
    z_track: float
    curvature: float
    macro_index: int
    macro_length: int
    macro_position: int
    macro_phase: float
    meso_index: int
    meso_length: int
    meso_position: int
    meso_phase: float
    meso_role: str
    meso_role_index: int
    micro_index: int
    micro_length: int
    micro_position: int
    micro_phase: float
    micro_role: str
    micro_role_index: int
    macro_reflection: bool
    meso_reflection: bool
    micro_reflection: bool

    @property
    def position(self) -> Tuple[float, float, float]:
        return self.x, self.y, self.height

    def as_dict(self) -> dict:
        return asdict(self)


@dataclass
class MacroSummary:
    index: int
    start: int
    length: int
    ideal_length: int
    reflection_step: Optional[int]
    height_gain: float
    mean_curvature: float

    def as_dict(self) -> dict:
        return asdict(self)


def _splitmix64(state: int) -> int:
    mask = (1 << 64) - 1
    z = (state + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    return z ^ (z >> 31)


class SoT3DPlan:
    def __init__(self, total_steps: int, base_radius: float, radial_growth: float, base_height: float, meso_gain: float, micro_gain: float,
                 angle_offset: float = 0.0):
        self.total_steps, self.base_radius, self.radial_growth = int(total_steps), float(base_radius), float(radial_growth)
        self.base_height, self.meso_gain, self.micro_gain = float(base_height), float(meso_gain), float(micro_gain)
        self._steps: List[SoT3DStep] = []
        self._macros: List[MacroSummary] = []
        self._build(angle_offset)

    def _build(self, offset: float) -> None:
        curv = math.sqrt(1.0 + self.radial_growth ** 2)
        z_track, step_i, meso_i, micro_i = 0.0, 0, 0, 0
        for macro_i, (macro_len, ideal) in enumerate(_fibonacci_orbits(self.total_steps)):
            start, dh, macro_pos, acc = step_i, self.base_height / GOLDEN_RATIO ** macro_i, 0, 0.0
            for meso_len in pack_tribonacci_chunks(macro_len):
                meso_pos = 0
                for micro_len in pack_tetranacci_chunks(meso_len):
                    for micro_pos in range(micro_len):
                        phase = lambda pos, n: pos / (n - 1) if n > 1 else 0.0          # noqa: E731
                        z_track += dh / macro_len
                        meso_phase, micro_phase = phase(meso_pos, meso_len), phase(micro_pos, micro_len)
                        angle = GOLDEN_ANGLE * step_i + offset
                        radius = self.base_radius * math.exp(self.radial_growth * step_i)
                        c = math.inf if abs(radius) <= 2.220446049250313e-16 else curv / abs(radius)
                        acc += c if math.isfinite(c) else 0.0
                        self._steps.append(SoT3DStep(
                            step_i, angle, radius, radius * math.cos(angle), radius * math.sin(angle),
                            z_track + self.meso_gain * (meso_phase - 0.5) + self.micro_gain * (micro_phase - 0.5), z_track, c,
                            macro_i, macro_len, macro_pos, phase(macro_pos, macro_len), meso_i, meso_len, meso_pos, meso_phase,
                            MESO_ROLES[meso_i % 3], meso_i % 3, micro_i, micro_len, micro_pos, micro_phase, MICRO_ROLES[micro_i % 4], micro_i % 4,
                            macro_pos + 1 == macro_len, meso_pos + 1 == meso_len, micro_pos + 1 == micro_len))
                        step_i, macro_pos, meso_pos = step_i + 1, macro_pos + 1, meso_pos + 1
                    micro_i += 1
                meso_i += 1
            self._macros.append(MacroSummary(macro_i, start, macro_len, ideal, start + macro_len - 1, dh, acc / macro_len))

    # ---- views -------------------------------------------------------------------------------------------------------------
    def steps(self) -> List[SoT3DStep]:
        return list(self._steps)

    def as_dicts(self) -> List[dict]:
        return [s.as_dict() for s in self._steps]

    def macro_summaries(self) -> List[MacroSummary]:
        return list(self._macros)

    @property
    def polyline(self) -> List[Tuple[float, float, float]]:
        return [s.position for s in self._steps]

    def reflection_points(self) -> List[Tuple[int, str]]:
        out = []
        for s in self._steps:
            out += [(s.index, name) for name, hit in (("micro", s.micro_reflection), ("meso", s.meso_reflection), ("macro", s.macro_reflection)) if hit]
        return out

    def _columns(self, fields: Sequence[str], width: int) -> torch.Tensor:
        if not self._steps:
            return torch.zeros(0, width, dtype=torch.float32)
        cols = []
        for f in fields:
            if f in ("meso_gain", "micro_gain"):
                cols.append([getattr(self, f)] * len(self._steps))
            else:
                cols.append([float(getattr(s, f)) for s in self._steps])
        return torch.tensor(cols, dtype=torch.float64).T.contiguous().to(torch.float32)

    _FEATURES = ("radius", "angle", "height", "curvature", "macro_phase", "meso_phase", "micro_phase", "meso_gain", "micro_gain")

    def as_tensor(self) -> Tensor:
        """``[steps, 3]``: x, y, height."""
        return Tensor._wrap(self._columns(("x", "y", "height"), 3))

    def feature_tensor(self) -> Tensor:
        """``[steps, 9]``: radius, angle, height, curvature, the three phases, meso gain, micro gain."""
        return Tensor._wrap(self._columns(self._FEATURES, 9))

    def role_tensor(self) -> Tensor:
        return Tensor._wrap(self._columns(("meso_role_index", "micro_role_index"), 2))

    def reflection_tensor(self) -> Tensor:
        return Tensor._wrap(self._columns(("macro_reflection", "meso_reflection", "micro_reflection"), 3))

    def macro_summary_tensor(self) -> Tensor:
        """``[orbits, 6]``: index, length, ideal length, height gain, mean curvature, reflection step (-1 when none)."""
        rows = [[m.index, m.length, m.ideal_length, m.height_gain, m.mean_curvature, -1.0 if m.reflection_step is None else m.reflection_step]
                for m in self._macros]
        return Tensor._wrap(torch.tensor(rows, dtype=torch.float32).reshape(len(rows), 6))

    def biome_tensor(self, include_reflections: bool = True, include_roles: bool = True) -> Tensor:
        fields = ("x", "y", "height", "radius", "angle", "curvature", "macro_phase", "meso_phase", "micro_phase", "meso_gain", "micro_gain")
        if include_roles:
            fields += ("meso_role_index", "micro_role_index")
        if include_reflections:
            fields += ("macro_reflection", "meso_reflection", "micro_reflection")
        return Tensor._wrap(self._columns(fields, len(fields)))

    def infuse_biome(self, biome, label_prefix: Optional[str] = None, include_reflections: bool = True, include_roles: bool = True) -> None:
        """Absorbs the plan's table into a tensor biome under ``<prefix>_plan`` with weight ``1 + meso gain + micro gain``."""
        biome.absorb_weighted(f"{label_prefix or 'sot'}_plan", self.biome_tensor(include_reflections, include_roles),
                              1.0 + self.meso_gain + self.micro_gain)

    def grow_biome(self, topos, label_prefix: Optional[str] = None, include_reflections: bool = True, include_roles: bool = True):
        from .topos import TensorBiome
        biome = TensorBiome(topos)
        self.infuse_biome(biome, label_prefix, include_reflections, include_roles)
        return biome

    def __repr__(self) -> str:
        return f"SoT3DPlan(steps={self.total_steps}, base_radius={self.base_radius:.3f}, growth={self.radial_growth:.3f})"


def generate_plan(total_steps: int, base_radius: float = 1.0, radial_growth: float = 0.05, base_height: float = 1.0, meso_gain: float = 0.2,
                  micro_gain: float = 0.05, seed: Optional[int] = None) -> SoT3DPlan:
    """``seed`` rotates the whole spiral by a reproducible angle (splitmix64 of the seed, scaled to one turn)."""
    if total_steps < 0:
        raise ValueError("total_steps must be non-negative")
    offset = 0.0 if seed is None else _splitmix64(int(seed) & ((1 << 64) - 1)) / float((1 << 64) - 1) * 2.0 * math.pi
    return SoT3DPlan(total_steps, base_radius, radial_growth, base_height, meso_gain, micro_gain, offset)
