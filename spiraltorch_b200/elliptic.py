"""Elliptic warp: reads an orientation vector as a point on a sphere of a given curvature radius and reports where it
sits — geodesic distance from the pole, the sheet of the azimuth, spin alignment, the rotation frame that carries the pole
onto it, and derived "heat" / "noise" scalars.  The microlocal lift uses it to split an interface's energy into leading
and trailing bands on positively curved charts.

Parity: crates/st-core/src/theory/microlocal/elliptic.rs — `LieFrame` (:15-167), `EllipticWarp::map_orientation*`
(:188-490), `EllipticTelemetry::{lerp, event_tags}` (:492-633), the soft-logic sample (:635-660), `EllipticAccumulator`
(:662-815), `compute_homology_index` (:848-864); Python surface bindings/st-py/src/elliptic.rs (`EllipticWarp`,
`EllipticTelemetry`).  The nine differentiable features are also available for a whole batch of orientations as one
tensor program (`EllipticWarp.features`), and the reference's hand-derived Jacobian is obtained from that program by
automatic differentiation.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import List, Optional, Sequence, Tuple

import torch

EPS = 1.1920929e-07
FEATURES = ("geodesic_radius", "normalized_radius", "spin_alignment", "sheet_position", "normal_bias", "resonance_heat", "rotor_x", "rotor_y", "rotor_z")


def _quat_to_matrix(q: Sequence[float]) -> List[float]:
    w, x, y, z = q
    return [1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w), 2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
            2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]


def _matrix_to_quat(m: Sequence[float]) -> List[float]:
    tr = m[0] + m[4] + m[8]
    if tr > 0.0:
        s = max(math.sqrt(tr + 1.0), EPS) * 2.0
        return [0.25 * s, (m[7] - m[5]) / s, (m[2] - m[6]) / s, (m[3] - m[1]) / s]
    if m[0] > m[4] and m[0] > m[8]:
        s = max(math.sqrt(1.0 + m[0] - m[4] - m[8]), EPS) * 2.0
        return [(m[7] - m[5]) / s, 0.25 * s, (m[1] + m[3]) / s, (m[2] + m[6]) / s]
    if m[4] > m[8]:
        s = max(math.sqrt(1.0 + m[4] - m[0] - m[8]), EPS) * 2.0
        return [(m[2] - m[6]) / s, (m[1] + m[3]) / s, 0.25 * s, (m[5] + m[7]) / s]
    s = max(math.sqrt(1.0 + m[8] - m[0] - m[4]), EPS) * 2.0
    return [(m[3] - m[1]) / s, (m[2] + m[6]) / s, (m[5] + m[7]) / s, 0.25 * s]


class LieFrame:
    """A rotation kept as a unit quaternion with non-negative scalar part and its 3x3 matrix (row-major)."""

    def __init__(self, quaternion: Sequence[float] = (1.0, 0.0, 0.0, 0.0)):
        q = [float(v) for v in quaternion]
        n = math.sqrt(sum(v * v for v in q))
        if n <= EPS:
            q = [1.0, 0.0, 0.0, 0.0]
        else:
            q = [v / n for v in q]
            if q[0] < 0.0:
                q = [-v for v in q]
        self.quaternion, self.rotation = q, _quat_to_matrix(q)

    identity = classmethod(lambda cls: cls())
    from_quaternion = classmethod(lambda cls, q: cls(q))

    @classmethod
    def from_axis_angle(cls, axis: Sequence[float], angle: float) -> "LieFrame":
        n = math.sqrt(sum(a * a for a in axis))
        if n <= EPS:
            return cls()
        s, c = math.sin(0.5 * angle), math.cos(0.5 * angle)
        return cls([c, axis[0] / n * s, axis[1] / n * s, axis[2] / n * s])

    @classmethod
    def from_matrix(cls, m: Sequence[float]) -> "LieFrame":
        return cls(_matrix_to_quat(m))

    def rotation_matrix(self) -> List[float]:
        return list(self.rotation)

    def apply(self, v: Sequence[float]) -> List[float]:
        r = self.rotation
        return [r[0] * v[0] + r[1] * v[1] + r[2] * v[2], r[3] * v[0] + r[4] * v[1] + r[5] * v[2], r[6] * v[0] + r[7] * v[1] + r[8] * v[2]]

    def apply_inverse(self, v: Sequence[float]) -> List[float]:
        r = self.rotation
        return [r[0] * v[0] + r[3] * v[1] + r[6] * v[2], r[1] * v[0] + r[4] * v[1] + r[7] * v[2], r[2] * v[0] + r[5] * v[1] + r[8] * v[2]]

    def inverse(self) -> "LieFrame":
        w, x, y, z = self.quaternion
        return LieFrame([w, -x, -y, -z])

    def compose(self, other: "LieFrame") -> "LieFrame":
        w1, x1, y1, z1 = self.quaternion
        w2, x2, y2, z2 = other.quaternion
        return LieFrame([w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2, w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2,
                         w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2, w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2])

    def relative_to(self, reference: "LieFrame") -> "LieFrame":
        return reference.inverse().compose(self)

    def log(self) -> List[float]:
        w, x, y, z = self.quaternion
        nv = math.sqrt(x * x + y * y + z * z)
        if nv <= EPS:
            return [0.0, 0.0, 0.0]
        k = 2.0 * math.atan2(nv, w) / nv
        return [x * k, y * k, z * k]

    @classmethod
    def exp(cls, tangent: Sequence[float]) -> "LieFrame":
        th = math.sqrt(sum(t * t for t in tangent))
        return cls() if th <= EPS else cls.from_axis_angle([t / th for t in tangent], th)

    def transport(self, vector: Sequence[float], target: "LieFrame") -> List[float]:
        return target.apply_inverse(self.apply(vector))


def homology_index(sheet_index: int, sheet_count: int, spin_alignment: float, normalized_radius: float) -> int:
    spin = (int(math.floor(min(max(spin_alignment, -1.0), 1.0) * 32767.0 + 0.5)) + 32768) & 0xFFFFFFFF
    radius = int(math.floor(min(max(normalized_radius, 0.0), 1.0) * 65535.0 + 0.5))
    return (((sheet_index & 0x3FF) << 22) ^ ((sheet_count & 0x3FF) << 12) ^ (spin << 1) ^ radius) & 0xFFFFFFFF


def _lerp(a: float, b: float, t: float) -> float:
    return a + (b - a) * t


@dataclass
class EllipticTelemetry:
    curvature_radius: float = 1.0
    geodesic_radius: float = 0.0
    normalized_radius: float = 0.0
    spin_alignment: float = 0.0
    sheet_index: int = 0
    sheet_position: float = 0.0
    normal_bias: float = 1.0
    sheet_count: int = 1
    topological_sector: int = 0
    homology_index: int = 0
    rotor_field: List[float] = field(default_factory=lambda: [0.0, 0.0, 0.0])
    flow_vector: List[float] = field(default_factory=lambda: [1.0, 0.0, 0.0])
    curvature_tensor: List[List[float]] = field(default_factory=lambda: [[0.0] * 3 for _ in range(3)])
    resonance_heat: float = 0.0
    noise_density: float = 0.0
    lie_frame: LieFrame = field(default_factory=LieFrame)
    lie_log: List[float] = field(default_factory=lambda: [0.0, 0.0, 0.0])
    rotor_transport: List[float] = field(default_factory=lambda: [0.0, 0.0, 0.0])

    def clamped_radius(self) -> float:
        return min(max(self.normalized_radius, 0.0), 1.0)

    def lie_quaternion(self) -> List[float]:
        return list(self.lie_frame.quaternion)

    def lie_rotation(self) -> List[float]:
        return self.lie_frame.rotation_matrix()

    def lerp(self, other: "EllipticTelemetry", t: float) -> "EllipticTelemetry":
        t = min(max(t, 0.0), 1.0)
        sheets = max(self.sheet_count, other.sheet_count, 1)
        pos = min(max(_lerp(self.sheet_position, other.sheet_position, t), 0.0), 1.0)
        mix3 = lambda a, b: [_lerp(x, y, t) for x, y in zip(a, b)]      # noqa: E731
        first = self if t < 0.5 else other
        return EllipticTelemetry(
            max(_lerp(self.curvature_radius, other.curvature_radius, t), EPS), max(_lerp(self.geodesic_radius, other.geodesic_radius, t), 0.0),
            min(max(_lerp(self.normalized_radius, other.normalized_radius, t), 0.0), 1.0),
            min(max(_lerp(self.spin_alignment, other.spin_alignment, t), -1.0), 1.0), min(int(math.floor(pos * sheets + 0.5)), sheets - 1), pos,
            min(max(_lerp(self.normal_bias, other.normal_bias, t), -1.0), 1.0), sheets, first.topological_sector, first.homology_index,
            mix3(self.rotor_field, other.rotor_field), mix3(self.flow_vector, other.flow_vector),
            [mix3(a, b) for a, b in zip(self.curvature_tensor, other.curvature_tensor)], _lerp(self.resonance_heat, other.resonance_heat, t),
            min(max(_lerp(self.noise_density, other.noise_density, t), 0.0), 1.0),
            LieFrame(mix3(self.lie_frame.quaternion, other.lie_frame.quaternion)), mix3(self.lie_log, other.lie_log),
            mix3(self.rotor_transport, other.rotor_transport))

    def event_tags(self) -> List[str]:
        return [f"elliptic.sheet:{self.sheet_index:02d}", f"elliptic.sector:{self.topological_sector:02d}",
                f"elliptic.radius:{self.clamped_radius():.4f}", f"elliptic.spin:{self.spin_alignment:.3f}", f"elliptic.heat:{self.resonance_heat:.3f}"]

    def as_dict(self) -> dict:
        """The record the soft-logic feedback and the atlas carry."""
        return {"curvature_radius": self.curvature_radius, "geodesic_radius": self.geodesic_radius, "normalized_radius": self.clamped_radius(),
                "spin_alignment": self.spin_alignment, "sheet_index": self.sheet_index, "sheet_position": self.sheet_position,
                "normal_bias": self.normal_bias, "sheet_count": self.sheet_count, "topological_sector": self.topological_sector,
                "homology_index": self.homology_index, "rotor_field": list(self.rotor_field), "flow_vector": list(self.flow_vector),
                "curvature_tensor": [list(r) for r in self.curvature_tensor], "resonance_heat": self.resonance_heat,
                "noise_density": self.noise_density, "quaternion": self.lie_quaternion(), "rotation": self.lie_rotation(),
                "lie_log": list(self.lie_log), "rotor_transport": list(self.rotor_transport)}


@dataclass
class EllipticDifferential:
    features: List[float]                    # in the order of `FEATURES`
    jacobian: List[List[float]]              # [9][3]: d feature / d orientation


class EllipticWarp:
    def __init__(self, curvature_radius: float, sheet_count: int = 2, spin_harmonics: int = 1):
        self._radius, self._sheets, self._harmonics = max(float(curvature_radius), EPS), max(int(sheet_count), 1), max(int(spin_harmonics), 1)

    def with_sheet_count(self, sheet_count: int) -> "EllipticWarp":
        self._sheets = max(int(sheet_count), 1)
        return self

    def with_spin_harmonics(self, harmonics: int) -> "EllipticWarp":
        self._harmonics = max(int(harmonics), 1)
        return self

    def configure(self, sheet_count: Optional[int] = None, spin_harmonics: Optional[int] = None) -> None:
        if sheet_count is not None:
            self.with_sheet_count(sheet_count)
        if spin_harmonics is not None:
            self.with_spin_harmonics(spin_harmonics)

    def clone(self) -> "EllipticWarp":
        return EllipticWarp(self._radius, self._sheets, self._harmonics)

    def curvature_radius(self) -> float:
        return self._radius

    def sheet_count(self) -> int:
        return self._sheets

    def spin_harmonics(self) -> int:
        return self._harmonics

    def max_geodesic(self) -> float:
        return self._radius * math.pi

    # ---- batched, differentiable ---------------------------------------------------------------------------------------------
    def features(self, orientations: torch.Tensor) -> torch.Tensor:
        """``[N, 3] -> [N, 9]`` (columns: `FEATURES`), differentiable with respect to the orientations.  Rows of zero
        length give NaN; callers filter them (the scalar form returns ``None`` for those)."""
        o = orientations.to(torch.float64)
        d = o / o.norm(dim=-1, keepdim=True)
        dz = d[..., 2].clamp(-1.0, 1.0)
        polar = torch.acos(dz)
        sin_t = torch.sqrt((1.0 - dz * dz).clamp(min=0.0))
        geodesic = polar * self._radius
        normalized = (geodesic / max(self._radius * math.pi, EPS)).clamp(0.0, 1.0)
        azimuth = torch.atan2(d[..., 1], d[..., 0])
        spin = torch.sin(azimuth / math.pi * self._harmonics)
        phase = torch.frac((azimuth + math.pi) / (2.0 * math.pi))
        sheet_pos = phase.clamp(0.0, 1.0) if self._sheets > 1 else torch.zeros_like(phase)
        heat = normalized * torch.sqrt(spin * spin + EPS)
        safe = sin_t.clamp(min=EPS)
        on = sin_t > EPS
        rx = torch.where(on, -d[..., 1] / safe * polar, torch.zeros_like(polar))
        ry = torch.where(on, d[..., 0] / safe * polar, torch.zeros_like(polar))
        return torch.stack([geodesic, normalized, spin, sheet_pos, dz, heat, rx, ry, torch.zeros_like(polar)], dim=-1)

    # ---- one orientation -----------------------------------------------------------------------------------------------------
    def map_orientation(self, orientation: Sequence[float]) -> Optional[EllipticTelemetry]:
        v = [float(x) for x in list(orientation)[:3]]
        if not v:
            return None
        v += [0.0] * (3 - len(v))
        n = math.sqrt(sum(x * x for x in v))
        if not math.isfinite(n) or n <= EPS:
            return None
        d = [x / n for x in v]
        dz = min(max(d[2], -1.0), 1.0)
        polar, sin_t = math.acos(dz), math.sqrt(max(1.0 - dz * dz, 0.0))
        geodesic = polar * self._radius
        normalized = min(max(geodesic / max(self._radius * math.pi, EPS), 0.0), 1.0)
        azimuth = math.atan2(d[1], d[0])
        spin = math.sin(azimuth / math.pi * self._harmonics)
        phase = math.modf((azimuth + math.pi) / (2.0 * math.pi))[0]
        sheet_index = min(int(math.floor(phase * self._sheets)), self._sheets - 1)
        sheet_pos = min(max(phase, 0.0), 1.0) if self._sheets > 1 else 0.0
        frame = LieFrame.from_axis_angle([-d[1], d[0], 0.0], polar)                  # z cross dir
        rotor_unit = [0.0, 0.0, 0.0] if sin_t <= EPS else [-d[1] / max(sin_t, EPS), d[0] / max(sin_t, EPS), 0.0]
        rotor = [u * polar for u in rotor_unit]
        rotor_norm = math.sqrt(sum(r * r for r in rotor))
        noise = 1.0 - rotor_norm / (polar + EPS)
        noise = min(max(noise if math.isfinite(noise) else 0.0, 0.0), 1.0)
        sector = (sheet_index << 1) | (0 if dz >= 0.0 else 1)
        inv = 1.0 / max(self._radius, EPS)
        return EllipticTelemetry(self._radius, geodesic, normalized, spin, sheet_index, sheet_pos, dz, self._sheets, sector,
                                 homology_index(sheet_index, self._sheets, spin, normalized), rotor, frame.apply([1.0, 0.0, 0.0]),
                                 [[d[i] * d[j] * inv for j in range(3)] for i in range(3)], normalized * math.sqrt(spin * spin + EPS), noise,
                                 frame, frame.log(), frame.apply_inverse(rotor))

    def map_orientation_differential(self, orientation: Sequence[float]) -> Optional[Tuple[EllipticTelemetry, EllipticDifferential]]:
        tel = self.map_orientation(orientation)
        if tel is None:
            return None
        v = torch.tensor(([float(x) for x in list(orientation)[:3]] + [0.0, 0.0, 0.0])[:3], dtype=torch.float64)
        jac = torch.autograd.functional.jacobian(lambda o: self.features(o[None])[0], v)
        jac = torch.where(torch.isfinite(jac), jac, torch.zeros_like(jac))
        return tel, EllipticDifferential(self.features(v[None])[0].tolist(), jac.tolist())

    map_orientation_with_differential = map_orientation_differential


class EllipticAccumulator:
    """Weighted mean of telemetry records (quaternions are averaged and re-normalised; sector and homology index follow
    the heaviest contribution)."""

    def __init__(self):
        self.weight, self.items = 0.0, []
        self.sector, self.sector_w, self.homology, self.homology_w = 0, 0.0, 0, 0.0

    def accumulate(self, t: EllipticTelemetry, weight: float) -> None:
        if not math.isfinite(weight) or weight <= 0.0:
            return
        self.items.append((t, weight))
        self.weight += weight
        if t.topological_sector == self.sector:
            self.sector_w += weight
        elif self.sector_w <= 0.0 or weight > self.sector_w:
            self.sector, self.sector_w = t.topological_sector, weight
        if t.homology_index == self.homology:
            self.homology_w += weight
        elif self.homology_w <= 0.0 or weight > self.homology_w:
            self.homology, self.homology_w = t.homology_index, weight

    def finish(self) -> Optional[EllipticTelemetry]:
        if self.weight <= 0.0:
            return None
        W = self.weight
        mean = lambda f: sum(f(t) * w for t, w in self.items) / W                     # noqa: E731
        mean3 = lambda f: [sum(f(t)[i] * w for t, w in self.items) / W for i in range(3)]   # noqa: E731
        sheets = max(max(t.sheet_count for t, _ in self.items), 1)
        pos = min(max(mean(lambda t: t.sheet_position), 0.0), 1.0)
        quat = [sum(t.lie_frame.quaternion[i] * w for t, w in self.items) / W for i in range(4)]
        return EllipticTelemetry(
            max(mean(lambda t: t.curvature_radius), EPS), max(mean(lambda t: t.geodesic_radius), 0.0),
            min(max(mean(lambda t: t.normalized_radius), 0.0), 1.0), min(max(mean(lambda t: t.spin_alignment), -1.0), 1.0),
            min(int(math.floor(pos * sheets + 0.5)), sheets - 1), pos, min(max(mean(lambda t: t.normal_bias), -1.0), 1.0), sheets, self.sector,
            self.homology, mean3(lambda t: t.rotor_field), mean3(lambda t: t.flow_vector),
            [[sum(t.curvature_tensor[i][j] * w for t, w in self.items) / W for j in range(3)] for i in range(3)],
            mean(lambda t: t.resonance_heat), min(max(mean(lambda t: t.noise_density), 0.0), 1.0), LieFrame(quat), mean3(lambda t: t.lie_log),
            mean3(lambda t: t.rotor_transport))
