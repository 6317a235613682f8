"""Z-space introspection: which region of the elliptic chart the latest soft-logic feedback sits in (spin band x
radius band), and readers of the telemetry hub's feedback slot.

Parity: crates/st-core/src/telemetry/zspace_region.rs — `ZSpaceSpinBand` (:16-52: leading above 0.33, trailing below
-0.33), `ZSpaceRadiusBand` (:55-91: core below 0.33, mantle below 0.66, else edge), `ZSpaceRegionKey` (:94-113),
`ZSpaceRegionDescriptor::from_elliptic` (:116-172); bindings/st-py/src/introspect.rs — `zspace_snapshot`,
`softlogic_feedback`, `clear_zspace_feedback`, `describe_zspace`, `softlogic_signal` and the aliases `snapshot`,
`feedback`, `clear`, `describe` (:537-672).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from . import hub, observability
from .hub import SoftlogicZFeedback

SPIN_BANDS = ("leading", "neutral", "trailing")
RADIUS_BANDS = ("core", "mantle", "edge")
__all__ = ["ZSpaceSpinBand", "ZSpaceRadiusBand", "ZSpaceRegionKey", "ZSpaceRegionDescriptor", "SoftlogicZFeedback", "zspace_snapshot",
           "softlogic_feedback", "clear_zspace_feedback", "describe_zspace", "snapshot", "feedback", "clear", "describe", "softlogic_signal"]


class ZSpaceSpinBand:
    values = SPIN_BANDS

    @staticmethod
    def classify(spin_alignment: float) -> str:
        return "leading" if spin_alignment > 0.33 else ("trailing" if spin_alignment < -0.33 else "neutral")

    @staticmethod
    def label(band: str) -> str:
        return f"spin.{band}"


class ZSpaceRadiusBand:
    values = RADIUS_BANDS

    @staticmethod
    def classify(normalized_radius: float) -> str:
        return "core" if normalized_radius < 0.33 else ("mantle" if normalized_radius < 0.66 else "edge")

    @staticmethod
    def label(band: str) -> str:
        return f"radius.{band}"


@dataclass(frozen=True)
class ZSpaceRegionKey:
    spin: str
    radius: str

    def label(self) -> str:
        return f"spin.{self.spin}.radius.{self.radius}"


@dataclass(frozen=True)
class ZSpaceRegionDescriptor:
    spin_alignment: float
    normalized_radius: float
    curvature_radius: float
    geodesic_radius: float
    sheet_index: int
    sheet_count: int
    topological_sector: int

    @classmethod
    def from_elliptic(cls, sample: dict) -> "ZSpaceRegionDescriptor":
        """``sample``: the elliptic record of a soft-logic feedback (`EllipticTelemetry.as_dict()`)."""
        d = cls(min(max(float(sample.get("spin_alignment", 0.0)), -1.0), 1.0), min(max(float(sample.get("normalized_radius", 0.0)), 0.0), 1.0),
                max(float(sample.get("curvature_radius", 0.0)), 0.0), max(float(sample.get("geodesic_radius", 0.0)), 0.0),
                int(sample.get("sheet_index", 0)), int(sample.get("sheet_count", 0)), int(sample.get("topological_sector", 0)))
        key = d.key()
        observability.emit_tensor_op("zspace_region_descriptor", (1,), (2,))
        observability.emit_tensor_op_meta("zspace_region_descriptor", lambda: {
            "backend": "host", "kind": "zspace_region_descriptor", "spin_alignment": d.spin_alignment, "normalized_radius": d.normalized_radius,
            "curvature_radius": d.curvature_radius, "geodesic_radius": d.geodesic_radius, "sheet_index": d.sheet_index,
            "sheet_count": d.sheet_count, "topological_sector": d.topological_sector, "spin_band": ZSpaceSpinBand.label(key.spin),
            "radius_band": ZSpaceRadiusBand.label(key.radius), "region_label": key.label()})
        return d

    def key(self) -> ZSpaceRegionKey:
        return ZSpaceRegionKey(ZSpaceSpinBand.classify(self.spin_alignment), ZSpaceRadiusBand.classify(self.normalized_radius))

    def label(self) -> str:
        return self.key().label()


def region_descriptor(feedback: SoftlogicZFeedback) -> Optional[ZSpaceRegionDescriptor]:
    return None if feedback.elliptic is None else ZSpaceRegionDescriptor.from_elliptic(feedback.elliptic)


def zspace_snapshot() -> Optional[ZSpaceRegionDescriptor]:
    fb = hub.get_softlogic_z()
    return None if fb is None else region_descriptor(fb)


def softlogic_feedback() -> Optional[SoftlogicZFeedback]:
    return hub.get_softlogic_z()


def clear_zspace_feedback() -> bool:
    return hub.clear_softlogic_z()


def describe_zspace(*, latest: bool = True, feedback: bool = False):
    """The latest feedback itself (``feedback=True``) or its region descriptor; ``None`` when nothing was published."""
    if not latest:
        raise RuntimeError("only the latest Z-space snapshot is currently available")
    fb = hub.get_softlogic_z()
    if fb is None:
        return None
    return fb if feedback else region_descriptor(fb)


def softlogic_signal() -> Optional[dict]:
    fb = hub.get_softlogic_z()
    if fb is None:
        return None
    above, here, beneath = fb.band_energy
    total = above + here + beneath
    out = {"psi_total": fb.psi_total, "weighted_loss": fb.weighted_loss, "band_energy": tuple(fb.band_energy),
           "band_energy_detail": {"above": above, "here": here, "beneath": beneath, "total": total, "drift": fb.drift},
           "drift": fb.drift, "z_signal": fb.z_signal, "scale": None if fb.scale is None else (fb.scale.physical_radius, fb.scale.log_radius),
           "events": list(fb.events), "attributions": [(s, w) for s, w in fb.attributions]}
    region = region_descriptor(fb)
    if region is not None:
        out["region"] = region
    return out


snapshot, feedback, clear, describe = zspace_snapshot, softlogic_feedback, clear_zspace_feedback, describe_zspace
