"""Observation accounting: how many distinct observation trees a branching process with symmetric child slots can
show at each depth (a Pólya / Burnside count), how an observed run compares with that bound, and the bridge that turns
one microlocal conductor report into such a run (interface -> active gauges -> scale slots -> matched macro drives ->
active pulses) together with the macro templates' merged feedback.

Reference parity: crates/st-core/src/theory/observation.rs (`ObservationCounts` :32-84, `GaugeSummary` / `PulseSummary`
:86-140, `ObservationBridge::ingest` :178-236, the telemetry record :238-440, the helper reductions :441-560).  The
counting side (`ObservabilityConfig`, `ObservationalCoalgebra`, `ObservabilityAssessment`) is written here from the
combinatorics the bridge needs: with R root symbols and b child slots acted on by a group G, the number of trees of
depth d + 1 is s_{d+1} = R * |Orb_G(s_d^b)|, the orbit count being the cycle-index evaluation for G.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from . import observability as _obs
from .hub import SoftlogicZFeedback
from .macro_model import MacroDrive, MacroTemplateBank
from .microlocal import InterfaceZReport, MicrolocalFeedback

_U128_MAX = (1 << 128) - 1
SLOT_SYMMETRIES = ("trivial", "symmetric", "cyclic", "dihedral")


def _phi(n: int) -> int:
    out, m, p = n, n, 2
    while p * p <= m:
        if m % p == 0:
            while m % p == 0:
                m //= p
            out -= out // p
        p += 1
    return out - out // m if m > 1 else out


def slot_orbits(symmetry: str, child_signatures: int, branching: int) -> int:
    """Number of orbits of ``child_signatures`` colours on ``branching`` slots under the slot group (saturating at
    2^128 - 1): ordered tuples, multisets, necklaces or bracelets."""
    c, b = max(int(child_signatures), 0), int(branching)
    if b <= 0:
        return 1
    if symmetry == "trivial":
        n = c ** b
    elif symmetry == "symmetric":
        n = math.comb(c + b - 1, b)
    elif symmetry in ("cyclic", "dihedral"):
        necklaces = sum(_phi(d) * c ** (b // d) for d in range(1, b + 1) if b % d == 0) // b
        if symmetry == "cyclic":
            n = necklaces
        elif b % 2 == 0:
            n = (2 * necklaces + c ** (b // 2 + 1) + c ** (b // 2)) // 4
        else:
            n = (necklaces + c ** ((b + 1) // 2)) // 2
    else:
        raise ValueError(f"unknown slot symmetry {symmetry!r}; one of {SLOT_SYMMETRIES}")
    return min(n, _U128_MAX)


@dataclass(frozen=True)
class ColorAction:
    """A group acting on the palette of root colours: ``trivial`` keeps every colour observable, a transitive action
    (``symmetric``, ``cyclic``, ``dihedral``) leaves a single observable class."""
    palette_size: int
    symmetry: str = "trivial"

    def observable_classes(self) -> int:
        if self.palette_size <= 0:
            return 0
        return self.palette_size if self.symmetry == "trivial" else 1

    def singleton_observable(self) -> bool:
        return self.symmetry == "trivial" or self.palette_size <= 1


@dataclass
class ObservabilityConfig:
    root_cardinality: int
    branching_factor: int
    slot_symmetry: str = "symmetric"
    color_action: Optional[ColorAction] = None

    def __post_init__(self):
        if self.slot_symmetry not in SLOT_SYMMETRIES:
            raise ValueError(f"unknown slot symmetry {self.slot_symmetry!r}; one of {SLOT_SYMMETRIES}")

    def with_color_action(self, action: ColorAction) -> "ObservabilityConfig":
        self.color_action = action
        return self

    def effective_roots(self) -> int:
        """Root symbols that remain distinguishable once the colour action is imposed."""
        base = max(int(self.root_cardinality), 0)
        return min(base, self.color_action.observable_classes()) if self.color_action is not None else base


@dataclass
class ObservabilityAssessment:
    expected: List[int]
    observed: List[int]
    efficiency: List[float]            # observed / expected per depth (0 where nothing is expected)

    def saturated_depths(self) -> List[int]:
        return [d for d, (o, e) in enumerate(zip(self.observed, self.expected)) if e > 0 and o >= e]

    def mean_efficiency(self) -> float:
        return sum(self.efficiency) / len(self.efficiency) if self.efficiency else 0.0


class ObservationalCoalgebra:
    """Unfolds the signature counts depth by depth and keeps them, so repeated assessments reuse the prefix."""

    def __init__(self, config: ObservabilityConfig):
        self.config = config
        self._levels: List[int] = []

    def unique_signatures(self, depth: int) -> int:
        return self.unfold(depth)[depth]

    def unfold(self, depth: int) -> List[int]:
        roots = self.config.effective_roots()
        while len(self._levels) <= depth:
            if not self._levels:
                self._levels.append(min(roots, _U128_MAX))
            else:
                orbits = slot_orbits(self.config.slot_symmetry, self._levels[-1], self.config.branching_factor)
                self._levels.append(min(roots * orbits, _U128_MAX))
        return self._levels[:depth + 1]

    def assess(self, observed: Sequence[int]) -> ObservabilityAssessment:
        obs = [max(int(o), 0) for o in observed]
        expected = self.unfold(max(len(obs) - 1, 0)) if obs else []
        eff = [(o / e if e > 0 else 0.0) for o, e in zip(obs, expected)]
        return ObservabilityAssessment(list(expected), obs, eff)


# ---------------------------------------------------------------------------------------------------------------
# the bridge from a conductor report
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class ObservationCounts:
    total_gauges: int = 0
    root_interfaces: int = 0
    active_gauges: int = 0
    active_scale_slots: int = 0
    matched_macro_drives: int = 0
    active_pulses: int = 0

    def depths(self) -> List[int]:
        return [self.root_interfaces, self.active_gauges, self.active_scale_slots, self.matched_macro_drives, self.active_pulses]

    def coverage(self) -> float:
        return self.active_gauges / self.total_gauges if self.total_gauges else 0.0

    def inactive_gauges(self) -> int:
        return max(self.total_gauges - self.active_gauges, 0)

    def pulse_activation_rate(self) -> float:
        return self.active_pulses / self.total_gauges if self.total_gauges else 0.0


@dataclass
class GaugeSummary:
    id: str
    active: bool
    radius: int
    physical_radius: float
    matched_template: bool
    pulse_support: Optional[float]
    z_bias: Optional[float]
    quality: Optional[float]

    def is_active(self) -> bool:
        return self.active


@dataclass
class PulseSummary:
    total: int = 0
    active: int = 0
    inactive: int = 0
    mean_support: float = 0.0
    max_support: float = 0.0
    mean_z_bias: float = 0.0

    def activation_rate(self) -> float:
        return self.active / self.total if self.total else 0.0


@dataclass
class ObservationBridgeSnapshot:
    counts: ObservationCounts
    depth_counts: List[int]
    assessment: ObservabilityAssessment
    microlocal_feedback: Optional[MicrolocalFeedback]
    drives: Dict[str, MacroDrive]
    softlogic_feedback: SoftlogicZFeedback
    gauges: List[GaugeSummary]
    pulses: PulseSummary

    def has_interface(self) -> bool:
        return self.counts.root_interfaces > 0

    def observed_counts(self) -> List[int]:
        return self.depth_counts


class ObservationBridge:
    def __init__(self, config: ObservabilityConfig, templates: Optional[MacroTemplateBank] = None):
        self.coalgebra = ObservationalCoalgebra(config)
        self.templates = templates if templates is not None else MacroTemplateBank()

    with_templates = classmethod(lambda cls, config, templates: cls(config, templates))

    def ingest(self, report: InterfaceZReport) -> ObservationBridgeSnapshot:
        drives = self.templates.drive_matched(report)
        gauges = _gauge_summaries(report, drives)
        active = [g for g in gauges if g.active]
        counts = ObservationCounts(total_gauges=len(gauges), root_interfaces=1 if report.has_interface() else 0, active_gauges=len(active),
                                   active_scale_slots=len({(g.id, g.radius, float(g.physical_radius)) for g in active}),
                                   matched_macro_drives=len(drives), active_pulses=sum(1 for p in report.pulses if not p.is_empty()))
        depth_counts = counts.depths()
        merged: Optional[MicrolocalFeedback] = None
        for d in drives.values():
            merged = d.feedback if merged is None else merged.merge(d.feedback)
        snap = ObservationBridgeSnapshot(counts, depth_counts, self.coalgebra.assess(depth_counts), merged, drives, report.feedback, gauges,
                                         _pulse_summary(report, gauges))
        _emit(snap)
        return snap


def _gauge_summaries(report: InterfaceZReport, drives: Dict[str, MacroDrive]) -> List[GaugeSummary]:
    out = []
    for i, sig in enumerate(report.signatures):
        gid = report.gauge_id(i) or f"gauge#{i}"
        pulse = report.pulses[i] if i < len(report.pulses) else None
        out.append(GaugeSummary(gid, sig.has_interface(), sig.radius, sig.physical_radius, gid in drives,
                                pulse.support if pulse is not None else None, pulse.z_bias if pulse is not None else None,
                                report.qualities[i] if i < len(report.qualities) else None))
    return out


def _pulse_summary(report: InterfaceZReport, gauges: Sequence[GaugeSummary]) -> PulseSummary:
    s = PulseSummary(total=len(report.pulses))
    supports, biases = [], []
    for i, pulse in enumerate(report.pulses):
        if pulse.is_empty():
            s.inactive += 1
        else:
            s.active += 1
        if i < len(gauges):
            if gauges[i].pulse_support is not None:
                supports.append(gauges[i].pulse_support)
            if gauges[i].z_bias is not None:
                biases.append(gauges[i].z_bias)
    if supports:
        s.mean_support, s.max_support = sum(supports) / len(supports), max(max(supports), 0.0)
    if biases:
        s.mean_z_bias = sum(biases) / len(biases)
    return s


def _emit(snap: ObservationBridgeSnapshot) -> None:
    _obs.emit_tensor_op("observation_bridge_ingest", [len(snap.gauges), len(snap.depth_counts)], [1, max(len(snap.depth_counts), 1)])

    def build():
        eff = [e if math.isfinite(e) else 0.0 for e in snap.assessment.efficiency]
        fb, sl, c, p = snap.microlocal_feedback, snap.softlogic_feedback, snap.counts, snap.pulses
        return {"backend": "cpu", "requested_backend": "auto", "kind": "st_core_observation_bridge_ingest",
                "has_interface": snap.has_interface(), "total_gauges": c.total_gauges, "active_gauges": c.active_gauges,
                "inactive_gauges": c.inactive_gauges(), "active_scale_slots": c.active_scale_slots,
                "matched_macro_drives": c.matched_macro_drives, "active_pulses": c.active_pulses, "coverage": c.coverage(),
                "pulse_activation_rate": c.pulse_activation_rate(), "depths": len(snap.depth_counts),
                "expected_depths": len(snap.assessment.expected), "efficiency_min": min(eff) if eff else 0.0,
                "efficiency_max": max(eff) if eff else 0.0, "efficiency_mean": sum(eff) / len(eff) if eff else 0.0,
                "gauges": len(snap.gauges), "matched_template_gauges": sum(1 for g in snap.gauges if g.matched_template),
                "quality_samples": sum(1 for g in snap.gauges if g.quality is not None), "pulse_total": p.total, "pulse_active": p.active,
                "pulse_inactive": p.inactive, "pulse_mean_support": p.mean_support, "pulse_max_support": p.max_support,
                "pulse_mean_z_bias": p.mean_z_bias, "softlogic_psi_total": sl.psi_total, "softlogic_weighted_loss": sl.weighted_loss,
                "softlogic_band_energy_total": sum(sl.band_energy), "softlogic_drift": sl.drift, "softlogic_z_signal": sl.z_signal,
                "softlogic_events": len(sl.events), "softlogic_attributions": len(sl.attributions), "has_softlogic_scale": sl.scale is not None,
                "has_elliptic": sl.elliptic is not None, "has_microlocal_feedback": fb is not None,
                "has_threshold_scale": fb is not None and fb.threshold_scale is not None,
                "threshold_scale": fb.threshold_scale if fb is not None and fb.threshold_scale is not None else 1.0,
                "has_bias_gain": fb is not None and fb.bias_gain is not None,
                "bias_gain": fb.bias_gain if fb is not None and fb.bias_gain is not None else 1.0}
    _obs.emit_tensor_op_meta("observation_bridge_ingest", build)
