"""Macro-scale interface templates: a sharp-interface energy, its kinetics, dimensionless audit numbers, an analysis
checklist and a numerical recipe bundled as one object, plus the bridge that turns a microlocal interface signature
into a front velocity and a feedback record for the gauges.

Reference parity: crates/st-core/src/theory/macro.rs (terms and constraints :27-292, kinetics :294-430, scales and
dimensionless groups :433-527, checklist and recipes :530-667, template bank :670-811, cards :822-987 and :1378-1440,
the Z bridge :990-1355).  The weighted averages over a signature's cells run as tensor reductions, so a signature on
the GPU is reduced there and only scalars come back.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Dict, Iterator, List, Optional, Sequence, Tuple, Union

import torch

from .microlocal import (InterfaceSignature, InterfaceZLift, InterfaceZPulse, InterfaceZReport, MicrolocalFeedback)

_EPS = 2.220446049250313e-16


# ---------------------------------------------------------------------------------------------------------------
# participants and energy terms
# ---------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class PhasePair:
    """The interface between phases ``i`` and ``j``."""
    i: str
    j: str


@dataclass(frozen=True)
class PhaseTriple:
    """A triple junction (two fluids and a solid, say)."""
    i: str
    j: str
    k: str


@dataclass
class Anisotropy:
    """Direction dependence of a surface tension: ``kind`` is ``isotropic``, ``fourier`` (``modes`` = (k, amplitude)
    pairs of ``1 + sum a_k cos(k theta)``), ``tabulated`` (``weights``) or ``custom`` (a note; never evaluated)."""
    kind: str = "isotropic"
    modes: Tuple[Tuple[int, float], ...] = ()
    weights: Tuple[float, ...] = ()
    note: str = ""

    @classmethod
    def isotropic(cls) -> "Anisotropy":
        return cls()

    @classmethod
    def fourier(cls, modes: Sequence[Tuple[int, float]]) -> "Anisotropy":
        return cls("fourier", modes=tuple((int(k), float(a)) for k, a in modes))

    @classmethod
    def tabulated(cls, weights: Sequence[float], description: str = "") -> "Anisotropy":
        return cls("tabulated", weights=tuple(float(w) for w in weights), note=description)

    @classmethod
    def custom(cls, note: str) -> "Anisotropy":
        return cls("custom", note=note)

    def evaluate(self, normal: Sequence[float]) -> Optional[float]:
        """gamma(n) / sigma for an averaged unit normal (first component = first grid axis); None where it cannot be
        evaluated."""
        if self.kind == "isotropic":
            return 1.0
        if self.kind == "fourier":
            if len(normal) < 2:
                return None
            nx, ny = normal[1], normal[0]
            if abs(nx) + abs(ny) <= 1e-12:
                return None
            theta = math.atan2(ny, nx)
            return max(1.0 + sum(a * math.cos(k * theta) for k, a in self.modes), 0.0)
        if self.kind == "tabulated":
            return max(sum(self.weights) / len(self.weights), 0.0) if self.weights else 1.0
        return None


@dataclass
class SurfaceTerm:
    pair: PhasePair
    sigma: float
    anisotropy: Anisotropy = field(default_factory=Anisotropy)

    def __post_init__(self):
        self.sigma = max(self.sigma, 0.0)


@dataclass
class BendingTerm:
    pair: PhasePair
    kappa: float
    spontaneous_curvature: Optional[float] = None

    def __post_init__(self):
        self.kappa = max(self.kappa, 0.0)


@dataclass
class LineTensionTerm:
    triple: PhaseTriple
    lam: float

    def __post_init__(self):
        self.lam = max(self.lam, 0.0)


@dataclass
class BulkPotential:
    """``kind``: ``constant`` (``value``), ``linear`` (``gradient``) or ``custom``."""
    phase: str
    kind: str = "constant"
    value: float = 0.0
    gradient: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    note: str = ""


@dataclass
class Kernel:
    """Non-local interaction kernel: ``gaussian`` (``param`` = length), ``power_law`` (``param`` = exponent), ``custom``."""
    kind: str
    strength: float
    param: float = 0.0
    note: str = ""


@dataclass
class NonlocalInteraction:
    phase: str
    kernel: Kernel


@dataclass
class PhaseConstraint:
    phase: str
    target: float

    def __post_init__(self):
        self.target = max(self.target, 0.0)


@dataclass
class InterfaceConstraint:
    pair: PhasePair
    target: float

    def __post_init__(self):
        self.target = max(self.target, 0.0)


@dataclass
class Constraints:
    volumes: List[PhaseConstraint] = field(default_factory=list)
    areas: List[InterfaceConstraint] = field(default_factory=list)
    topology: Optional[str] = None


@dataclass
class BoundaryCondition:
    """``kind`` ``young`` (``equilibrium_angle``) or ``cahn_hoffman`` (``anisotropy``) against ``solid``."""
    phase: str
    kind: str
    solid: str
    equilibrium_angle: float = 0.0
    anisotropy: Optional[Anisotropy] = None


@dataclass
class MacroInterfacialFunctional:
    surface_terms: List[SurfaceTerm] = field(default_factory=list)
    bending_terms: List[BendingTerm] = field(default_factory=list)
    line_tensions: List[LineTensionTerm] = field(default_factory=list)
    bulk_potentials: List[BulkPotential] = field(default_factory=list)
    nonlocal_terms: List[NonlocalInteraction] = field(default_factory=list)
    boundary_conditions: List[BoundaryCondition] = field(default_factory=list)
    constraints: Constraints = field(default_factory=Constraints)

    @classmethod
    def minimal(cls, pair: PhasePair, sigma: float) -> "MacroInterfacialFunctional":
        return cls(surface_terms=[SurfaceTerm(pair, sigma)])


# ---------------------------------------------------------------------------------------------------------------
# kinetics
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class ExternalForce:
    """``kind``: ``pressure_jump``, ``bulk_potential``, ``nonlocal``, ``custom`` (all contribute ``magnitude``) or
    ``contact_angle`` (contributes ``-friction * (z_bias - equilibrium)`` of the current pulse)."""
    kind: str
    magnitude: float = 0.0
    equilibrium: float = 0.0
    friction: float = 0.0
    note: str = ""


@dataclass
class CurvatureContributions:
    mean_curvature: float
    anisotropic_curvature: Optional[float] = None
    bending_operator: Optional[float] = None
    forcing: float = 0.0

    def with_anisotropy(self, value: float) -> "CurvatureContributions":
        return replace(self, anisotropic_curvature=value)

    def with_bending(self, value: float) -> "CurvatureContributions":
        return replace(self, bending_operator=value)


@dataclass
class MacroKinetics:
    """``flow``: ``non_conserved`` (Allen-Cahn like), ``conserved`` or ``surface_diffusion``."""
    flow: str
    mobility: float
    external_forces: List[ExternalForce] = field(default_factory=list)

    @classmethod
    def non_conserved(cls, mobility: float) -> "MacroKinetics":
        return cls("non_conserved", mobility)

    @classmethod
    def conserved(cls, mobility: float) -> "MacroKinetics":
        return cls("conserved", mobility)

    @classmethod
    def surface_diffusion(cls, surface_mobility: float) -> "MacroKinetics":
        return cls("surface_diffusion", surface_mobility)

    def with_force(self, force: ExternalForce) -> "MacroKinetics":
        self.external_forces.append(force)
        return self

    def forcing_from_pulse(self, pulse: Optional[InterfaceZPulse]) -> float:
        total = 0.0
        for f in self.external_forces:
            if f.kind == "contact_angle":
                total += -f.friction * (pulse.z_bias - f.equilibrium) if pulse is not None else 0.0
            else:
                total += f.magnitude
        return total

    def evaluate_velocity(self, c: CurvatureContributions) -> float:
        mobility = max(self.mobility, 0.0)
        if self.flow == "surface_diffusion":
            return -mobility * (c.bending_operator if c.bending_operator is not None else c.mean_curvature)
        curvature = c.anisotropic_curvature if c.anisotropic_curvature is not None else c.mean_curvature
        return mobility * (curvature - (c.bending_operator or 0.0) + c.forcing)


# ---------------------------------------------------------------------------------------------------------------
# scales, audit numbers, checklist, recipe
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class PhysicalScales:
    sigma: float
    reference_length: Optional[float] = None
    velocity_scale: Optional[float] = None
    viscosity: Optional[float] = None
    density_difference: Optional[float] = None
    gravity: Optional[float] = None
    interface_thickness: Optional[float] = None
    diffusion: Optional[float] = None
    bending_modulus: Optional[float] = None
    line_tension: Optional[float] = None
    mobility_ratio: Optional[float] = None


@dataclass
class DimensionlessGroups:
    capillary: Optional[float] = None
    bond: Optional[float] = None
    cahn: Optional[float] = None
    peclet: Optional[float] = None
    bending_length: Optional[float] = None
    line_tension_length: Optional[float] = None
    mobility_ratio: Optional[float] = None

    @classmethod
    def from_scales(cls, s: PhysicalScales) -> "DimensionlessGroups":
        sigma = max(s.sigma, _EPS)
        g = cls(mobility_ratio=s.mobility_ratio)
        if s.viscosity is not None and s.velocity_scale is not None:
            g.capillary = s.viscosity * s.velocity_scale / sigma
        if s.density_difference is not None and s.gravity is not None and s.reference_length is not None:
            g.bond = s.density_difference * s.gravity * s.reference_length ** 2 / sigma
        if s.interface_thickness is not None and s.reference_length is not None and s.reference_length > 0.0:
            g.cahn = abs(s.interface_thickness / s.reference_length)
        if s.velocity_scale is not None and s.reference_length is not None and s.diffusion is not None and s.diffusion > 0.0:
            g.peclet = s.velocity_scale * s.reference_length / s.diffusion
        if s.bending_modulus is not None and s.bending_modulus > 0.0 and s.sigma > 0.0:
            g.bending_length = math.sqrt(s.bending_modulus / sigma)
        if s.line_tension is not None and s.line_tension > 0.0 and s.sigma > 0.0:
            g.line_tension_length = s.line_tension / sigma
        return g

    def sharp_interface_ok(self) -> bool:
        """The sharp-interface description holds while the Cahn number stays below 0.1 (or is unknown)."""
        return self.cahn is None or self.cahn < 0.1


@dataclass
class AnalysisChecklist:
    existence: bool
    regularity: bool
    energy_decay: bool
    constraint_handling: bool
    notes: List[str] = field(default_factory=list)

    @classmethod
    def minimal_surface(cls) -> "AnalysisChecklist":
        return cls(True, False, True, True, ["perimeter is lower semicontinuous, so a volume-constrained minimiser exists",
                                             "mean-curvature flow keeps the energy decreasing under time splitting"])

    @classmethod
    def anisotropic(cls, strongly_convex: bool, bending_regulariser: bool) -> "AnalysisChecklist":
        notes = ["the Cahn-Hoffman vector carries the force balance on facets",
                 "a strongly convex gamma smooths facets: classical solutions" if strongly_convex
                 else "a non-convex gamma needs facet tracking or a small bending regulariser"]
        if bending_regulariser:
            notes.append("a small kappa suppresses facet pinning and stabilises the numerics")
        return cls(True, strongly_convex or bending_regulariser, True, True, notes)

    @classmethod
    def membrane(cls) -> "AnalysisChecklist":
        return cls(True, True, True, True, ["Willmore-Helfrich flow by operator splitting",
                                            "the surface Laplacian of the mean curvature needs C1 meshes or level-set regularisation"])

    @classmethod
    def pattern(cls) -> "AnalysisChecklist":
        return cls(True, False, True, False, ["non-local kernels need an FFT-friendly quadrature or a fast multipole sum",
                                              "convex splitting keeps sigma |Gamma| + K * chi decreasing"])

    @classmethod
    def contact_line(cls) -> "AnalysisChecklist":
        return cls(True, False, True, True, ["the dynamic contact-angle law needs the line friction calibrated",
                                             "line tension enters the Herring balance through lambda kappa_g"])


@dataclass
class NumericalRecipe:
    """``algorithm``: ``mbo`` (Merriman-Bence-Osher threshold dynamics), ``minimizing_movements`` or ``level_set``."""
    algorithm: str
    steps: List[str]

    @classmethod
    def mbo(cls, enforce_volume: bool) -> "NumericalRecipe":
        steps = ["diffuse the mask with the Gaussian kernel of width sqrt(2 dt)", "threshold back to a sharp interface"]
        if enforce_volume:
            steps.append("shift the threshold so that every phase volume stays fixed")
        return cls("mbo", steps)

    @classmethod
    def minimizing_movements(cls) -> "NumericalRecipe":
        return cls("minimizing_movements", ["solve argmin over Gamma of E[Gamma] + d(Gamma, Gamma_k)^2 / (2 dt)",
                                            "update the constraints through their Lagrange multipliers"])

    @classmethod
    def level_set(cls, split_biharmonic: bool) -> "NumericalRecipe":
        steps = ["advect phi with the curvature-dependent velocity", "reinitialise the signed distance to control stiffness"]
        if split_biharmonic:
            steps.append("split the bending operator into two diffusion passes")
        return cls("level_set", steps)


# ---------------------------------------------------------------------------------------------------------------
# cards: the five ready-made parameter sets
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class MinimalCardConfig:
    phase_pair: PhasePair
    sigma: float
    mobility: float
    volume: Optional[float] = None
    physical_scales: Optional[PhysicalScales] = None


@dataclass
class AnisotropicCardConfig:
    phase_pair: PhasePair
    sigma: float
    anisotropy: Anisotropy
    mobility: float
    volume: Optional[float] = None
    bending_regularisation: Optional[float] = None
    physical_scales: Optional[PhysicalScales] = None


@dataclass
class MembraneCardConfig:
    phase_pair: PhasePair
    sigma: float
    bending_modulus: float
    mobility: float
    spontaneous_curvature: Optional[float] = None
    pressure_jump: Optional[float] = None
    physical_scales: Optional[PhysicalScales] = None


@dataclass
class PatternCardConfig:
    phase: str
    sigma: float
    kernel: Kernel
    mobility: float
    physical_scales: Optional[PhysicalScales] = None


@dataclass
class ContactCardConfig:
    phase_pair: PhasePair
    sigma: float
    equilibrium_angle: float
    contact_friction: float
    mobility: float
    solid: str
    line_tension: Optional[float] = None
    physical_scales: Optional[PhysicalScales] = None


MacroCard = Union[MinimalCardConfig, AnisotropicCardConfig, MembraneCardConfig, PatternCardConfig, ContactCardConfig]


@dataclass
class MacroModelTemplate:
    functional: MacroInterfacialFunctional
    kinetics: MacroKinetics
    nondimensional: DimensionlessGroups
    analysis: AnalysisChecklist
    numerics: NumericalRecipe

    @classmethod
    def from_card(cls, card: MacroCard) -> "MacroModelTemplate":
        scales = replace(card.physical_scales) if card.physical_scales is not None else PhysicalScales(card.sigma)
        if isinstance(card, MinimalCardConfig):
            fn = MacroInterfacialFunctional.minimal(card.phase_pair, card.sigma)
            if card.volume is not None:
                fn.constraints.volumes.append(PhaseConstraint(card.phase_pair.i, card.volume))
            return cls(fn, MacroKinetics.non_conserved(card.mobility), DimensionlessGroups.from_scales(scales),
                       AnalysisChecklist.minimal_surface(), NumericalRecipe.mbo(card.volume is not None))
        if isinstance(card, AnisotropicCardConfig):
            fn = MacroInterfacialFunctional.minimal(card.phase_pair, card.sigma)
            fn.surface_terms[0].anisotropy = card.anisotropy
            if card.volume is not None:
                fn.constraints.volumes.append(PhaseConstraint(card.phase_pair.i, card.volume))
            if card.bending_regularisation is not None:
                fn.bending_terms.append(BendingTerm(card.phase_pair, card.bending_regularisation))
            return cls(fn, MacroKinetics.non_conserved(card.mobility), DimensionlessGroups.from_scales(scales),
                       AnalysisChecklist.anisotropic(card.anisotropy.kind in ("tabulated", "fourier"), card.bending_regularisation is not None),
                       NumericalRecipe.mbo(card.volume is not None))
        if isinstance(card, MembraneCardConfig):
            fn = MacroInterfacialFunctional.minimal(card.phase_pair, card.sigma)
            fn.bending_terms.append(BendingTerm(card.phase_pair, card.bending_modulus, card.spontaneous_curvature))
            kin = MacroKinetics.non_conserved(card.mobility).with_force(ExternalForce("bulk_potential", card.pressure_jump or 0.0))
            scales.bending_modulus = card.bending_modulus
            return cls(fn, kin, DimensionlessGroups.from_scales(scales), AnalysisChecklist.membrane(), NumericalRecipe.level_set(True))
        if isinstance(card, PatternCardConfig):
            fn = MacroInterfacialFunctional.minimal(PhasePair(card.phase + "_in", "out"), card.sigma)
            fn.nonlocal_terms.append(NonlocalInteraction(card.phase, card.kernel))
            kin = MacroKinetics.non_conserved(card.mobility).with_force(ExternalForce("nonlocal", card.kernel.strength))
            return cls(fn, kin, DimensionlessGroups.from_scales(scales), AnalysisChecklist.pattern(), NumericalRecipe.minimizing_movements())
        if isinstance(card, ContactCardConfig):
            fn = MacroInterfacialFunctional.minimal(card.phase_pair, card.sigma)
            fn.boundary_conditions.append(BoundaryCondition(card.phase_pair.i, "young", card.solid, card.equilibrium_angle))
            if card.line_tension is not None:
                fn.line_tensions.append(LineTensionTerm(PhaseTriple(card.phase_pair.i, card.phase_pair.j, card.solid), card.line_tension))
            kin = MacroKinetics.non_conserved(card.mobility).with_force(
                ExternalForce("contact_angle", equilibrium=card.equilibrium_angle, friction=card.contact_friction))
            scales.line_tension = card.line_tension
            return cls(fn, kin, DimensionlessGroups.from_scales(scales), AnalysisChecklist.contact_line(), NumericalRecipe.minimizing_movements())
        raise TypeError(f"unknown macro card {type(card).__name__}")

    def couple_with(self, lift: InterfaceZLift) -> "MacroZBridge":
        return MacroZBridge(self, lift)


# ---------------------------------------------------------------------------------------------------------------
# the bridge from a microlocal signature to a front velocity and gauge feedback
# ---------------------------------------------------------------------------------------------------------------
def _weighted_mean(values: torch.Tensor, weights: Optional[torch.Tensor]) -> float:
    """Mean of ``values`` over the cells of positive weight (plain mean when no cell has any)."""
    if values.numel() == 0:
        return 0.0
    v = values.to(torch.float64)
    if weights is not None:
        w = weights.to(torch.float64).clamp_min(0.0)
        total = w.sum()
        if float(total) > 0.0:
            return float((v * w).sum() / total)
    return float(v.mean())


def _average_normal(signature: InterfaceSignature, weights: Optional[torch.Tensor]) -> Optional[List[float]]:
    if signature.orientation is None or signature.orientation.shape[0] == 0:
        return None
    w = (weights if weights is not None else signature.r_machine).to(torch.float64).clamp_min(0.0)
    total = float(w.sum())
    if total <= 0.0:
        return None
    comp = (signature.orientation.to(torch.float64) * w.unsqueeze(0)).flatten(1).sum(dim=1) / total
    norm = float(comp.norm())
    return None if norm <= 1e-12 else (comp / norm).tolist()


@dataclass
class MacroDrive:
    pulse: InterfaceZPulse
    contributions: CurvatureContributions
    velocity: float
    dimensionless: DimensionlessGroups
    feedback: MicrolocalFeedback

    def sharp_interface_ok(self) -> bool:
        return self.dimensionless.sharp_interface_ok()

    def microlocal_feedback(self) -> MicrolocalFeedback:
        return self.feedback


class MacroZBridge:
    def __init__(self, template: MacroModelTemplate, lift: InterfaceZLift):
        self.template = template
        self.lift = lift

    def anisotropy_factor_for_normal(self, normal: Sequence[float]) -> Optional[float]:
        """Surface-tension-weighted gamma(n) / sigma over the functional's surface terms."""
        weighted = total = 0.0
        for term in self.template.functional.surface_terms:
            if term.sigma > 0.0:
                f = term.anisotropy.evaluate(normal)
                weighted += term.sigma * (1.0 if f is None else f)
                total += term.sigma
        return weighted / total if total > 0.0 else None

    def ingest_signature(self, signature: InterfaceSignature) -> MacroDrive:
        pulse = self.lift.project(signature)
        w = signature.perimeter_density
        mean_curv = _weighted_mean(signature.mean_curvature, w)
        signed = _weighted_mean(signature.signed_mean_curvature, w) if signature.signed_mean_curvature is not None else None
        normal = _average_normal(signature, w)
        factor = self.anisotropy_factor_for_normal(normal) if normal is not None else None
        if signed is not None:
            anis = signed * factor if factor is not None else signed
        else:
            anis = mean_curv * factor if factor is not None else None
        h0 = next((t.spontaneous_curvature for t in self.template.functional.bending_terms if t.spontaneous_curvature is not None), None)
        contributions = CurvatureContributions(mean_curv, anis, mean_curv - h0 if h0 is not None else None,
                                               self.template.kinetics.forcing_from_pulse(pulse))
        velocity = self.template.kinetics.evaluate_velocity(contributions)
        return MacroDrive(pulse, contributions, velocity, replace(self.template.nondimensional),
                          self.derive_feedback(contributions, velocity, pulse))

    def derive_feedback(self, c: CurvatureContributions, velocity: float, pulse: InterfaceZPulse) -> MicrolocalFeedback:
        nd = self.template.nondimensional
        clamp = lambda x, lo, hi: min(max(x, lo), hi)                               # noqa: E731
        threshold = 1.0
        if pulse.support < 1e-6:
            threshold *= 0.9
        if not nd.sharp_interface_ok():
            threshold *= 0.75
        if nd.cahn is not None:
            threshold *= 1.1 if nd.cahn < 0.02 else (0.8 if nd.cahn > 0.1 else 1.0)
        if c.anisotropic_curvature is not None:
            ratio = abs(c.anisotropic_curvature) / max(abs(c.mean_curvature), 1e-6)
            threshold *= 0.85 if ratio > 1.5 else (1.05 if ratio < 0.5 else 1.0)
        if nd.capillary is not None:
            cap = max(nd.capillary, 0.0)
            smoothing = clamp(cap / (1.0 + cap), 0.2, 0.8)
        else:
            smoothing = 0.6 if threshold < 1.0 else 0.3
        fluct = pulse.density_fluctuation()
        severity = clamp(fluct - 0.45, 0.0, 0.55)
        relief = clamp(0.25 - fluct, 0.0, 0.25)
        if fluct > 0.45:
            threshold = max(threshold * max(1.0 - severity * 0.3, 0.65), 0.25)
            smoothing = max(smoothing, 0.55 + severity * 0.5)
        elif fluct < 0.25:
            threshold *= 1.0 + relief * 0.5
            smoothing = clamp(smoothing * clamp(0.75 - relief * 0.2, 0.4, 0.9), 0.15, 0.8)
        if c.anisotropic_curvature is not None and abs(c.anisotropic_curvature) > abs(c.mean_curvature):
            smoothing = min(smoothing + 0.1, 0.9)
        vel = abs(velocity)
        gain = 1.0
        if nd.bond is not None:
            gain *= 0.8 if nd.bond > 1.0 else (1.1 if nd.bond < 0.1 else 1.0)
        if vel > 1.0:
            gain *= 1.0 + (min(vel, 5.0) - 1.0) * 0.15
        elif vel < 0.05:
            gain *= 0.85
        tempo = max(vel, 0.01)
        if fluct > 0.45:
            gain *= max(1.0 - severity * 0.25, 0.65)
            tempo = max(tempo, 0.45 + fluct * 0.9)
        elif fluct < 0.25:
            gain *= 1.0 + relief * 0.4
            tempo = max(tempo * (0.85 - relief * 0.2), 0.01)
        fb = MicrolocalFeedback().with_bias_gain(gain).with_smoothing(smoothing).with_tempo_hint(tempo)
        if abs(c.forcing) > 0.0:
            fb = fb.with_stderr_hint(abs(c.forcing))
        if abs(threshold - 1.0) > 1e-3:
            fb = fb.with_threshold_scale(threshold)
        t = pulse.elliptic
        if t is None:
            return fb
        # an elliptic chart rides on the pulse: steer its radius, sheet count and spin harmonics as well
        mc = abs(c.mean_curvature)
        if math.isfinite(mc) and mc > 1e-6:
            lo = max(t.curvature_radius * 0.5, 1e-4)
            fb = fb.with_elliptic_radius(clamp(1.0 / mc, lo, max(t.curvature_radius * 3.0, lo)))
        else:
            fb = fb.with_elliptic_radius(t.curvature_radius)
        anis_ratio = clamp(abs(c.anisotropic_curvature) / max(mc, 1e-6), 0.0, 4.0) if c.anisotropic_curvature is not None else 0.0
        sheets = int(clamp(round(anis_ratio * 4.0) + 2, 2, 16)) if anis_ratio > 0.0 else int(clamp(max(t.sheet_count, 1), 1, 8))
        sheets = max(sheets, int(clamp((t.topological_sector & 0x7) + 2, 2, 16)), int(clamp(round(t.resonance_heat * 6.0) + 2, 2, 16)))
        fb = fb.with_elliptic_sheet_count(sheets)
        spin = abs(t.spin_alignment)
        harmonics = 5 if spin > 0.75 else 3 if spin > 0.5 else 2 if spin > 0.25 else 1
        if t.resonance_heat > 0.45:
            harmonics = max(harmonics, 4)
        if t.resonance_heat > 0.8:
            harmonics = max(harmonics, 5)
        if t.noise_density > 0.6:
            harmonics = min(harmonics, 2)
        if t.topological_sector & 0x3 == 3:
            harmonics = max(harmonics, 4)
        fb = fb.with_elliptic_spin_harmonics(harmonics)
        fb = fb.with_smoothing(clamp(smoothing * clamp(1.0 - t.noise_density, 0.1, 0.95), 0.0, 1.0))
        fb = fb.with_bias_gain(gain * (1.0 + t.resonance_heat * 0.3) * (1.0 - t.noise_density * 0.5) * (1.0 + abs(t.rotor_field[2]) * 0.2))
        return fb.with_tempo_hint(max(max(vel, 0.01) + abs(t.flow_vector[2]) * 0.25 + t.resonance_heat * 0.2, 0.01))


class MacroTemplateBank:
    """Named templates, kept in registration order; couples all of them to a lift, or drives those whose id matches a
    gauge of a conductor report."""

    def __init__(self):
        self._entries: Dict[str, MacroModelTemplate] = {}

    def register(self, template_id: str, template: MacroModelTemplate) -> bool:
        if template_id in self._entries:
            return False
        self._entries[template_id] = template
        return True

    def register_card(self, template_id: str, card: MacroCard) -> bool:
        return self.register(template_id, MacroModelTemplate.from_card(card))

    def with_template(self, template_id: str, template: MacroModelTemplate) -> "MacroTemplateBank":
        self.register(template_id, template)
        return self

    def with_card(self, template_id: str, card: MacroCard) -> "MacroTemplateBank":
        self.register_card(template_id, card)
        return self

    def get(self, template_id: str) -> Optional[MacroModelTemplate]:
        return self._entries.get(template_id)

    def remove(self, template_id: str) -> Optional[MacroModelTemplate]:
        return self._entries.pop(template_id, None)

    def items(self) -> Iterator[Tuple[str, MacroModelTemplate]]:
        return iter(self._entries.items())

    def ids(self) -> List[str]:
        return list(self._entries)

    def __len__(self) -> int:
        return len(self._entries)

    def is_empty(self) -> bool:
        return not self._entries

    def to_vec(self) -> List[MacroModelTemplate]:
        return list(self._entries.values())

    def couple(self, template_id: str, lift: InterfaceZLift) -> Optional[MacroZBridge]:
        t = self.get(template_id)
        return t.couple_with(lift) if t is not None else None

    def couple_all(self, lift: InterfaceZLift) -> Dict[str, MacroZBridge]:
        return {k: t.couple_with(lift.clone()) for k, t in self._entries.items()}

    def drive_matched(self, report: InterfaceZReport) -> Dict[str, MacroDrive]:
        drives: Dict[str, MacroDrive] = {}
        for k, t in self._entries.items():
            sig = report.signature_for(k)
            if sig is not None:
                drives[k] = t.couple_with(report.lift.clone()).ingest_signature(sig)
        return drives

    def feedback_from_report(self, report: InterfaceZReport) -> Optional[MicrolocalFeedback]:
        combined: Optional[MicrolocalFeedback] = None
        for drive in self.drive_matched(report).values():
            combined = drive.feedback if combined is None else combined.merge(drive.feedback)
        return combined
