"""ψ meter: a weighted, exponentially smoothed health score of a training run.

Every sampled step the meter takes a :class:`PsiInput` (loss, gradient norm, update ratio, activation drift,
attention entropy, band energy, positive curvature), smooths each enabled component with an EMA, sums them
with the configured weights into ``total`` and emits a :class:`PsiEvent` whenever a smoothed component crosses
its threshold.  Steps that are not sampled return the previous smoothed values unchanged.

Restated from crates/st-core/src/telemetry/psi.rs: ``PsiComponent`` :38-160 (token aliases of ``parse_list``),
``PsiConfig`` :165-275 (``automated`` from a band hint, ``apply_spiral_tuning``), ``PsiMeter`` :500-690
(defaults filled in by ``new``, ``update``, checkpoint round trip), ``PsiAutomationHint`` :723.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Optional


class PsiComponent(enum.IntFlag):
    LOSS = 1 << 0
    GRAD_NORM = 1 << 1
    UPDATE_RATIO = 1 << 2
    ACT_DRIFT = 1 << 3
    ATTN_ENTROPY = 1 << 4
    BAND_ENERGY = 1 << 5
    POSITIVE_CURVATURE = 1 << 6

    @classmethod
    def defaults(cls) -> "PsiComponent":
        return cls.LOSS | cls.GRAD_NORM | cls.UPDATE_RATIO | cls.ACT_DRIFT | cls.POSITIVE_CURVATURE

    @classmethod
    def from_token(cls, token: str) -> "PsiComponent":
        t = token.strip().lower()
        table = {("loss",): cls.LOSS, ("grad", "grad_norm", "gradnorm"): cls.GRAD_NORM,
                 ("update", "update_ratio", "ratio"): cls.UPDATE_RATIO, ("act", "act_drift", "drift"): cls.ACT_DRIFT,
                 ("attn", "attn_entropy", "attention", "entropy"): cls.ATTN_ENTROPY,
                 ("band", "band_energy", "energy"): cls.BAND_ENERGY,
                 ("curv", "curvature", "positive_curvature", "pos_curv"): cls.POSITIVE_CURVATURE}
        for names, comp in table.items():
            if t in names:
                return comp
        raise ValueError(f"unknown psi component '{t}': expected one of Loss, Grad, Update, Act, Attn, Band, Curvature")

    @classmethod
    def parse_list(cls, spec: str) -> "PsiComponent":
        mask = cls(0)
        for seg in spec.replace("|", ",").replace(";", ",").split(","):
            for tok in seg.split():
                mask |= cls.from_token(tok)
        return mask

    @property
    def label(self) -> str:
        return (self.name or "unknown").lower()


ORDER = (PsiComponent.LOSS, PsiComponent.GRAD_NORM, PsiComponent.UPDATE_RATIO, PsiComponent.ACT_DRIFT,
         PsiComponent.ATTN_ENTROPY, PsiComponent.BAND_ENERGY, PsiComponent.POSITIVE_CURVATURE)


@dataclass
class PsiAutomationHint:
    above: int = 0
    here: int = 0
    beneath: int = 0
    band_focus: float = 0.0
    drift_weight: float = 0.0

    def depth(self) -> int:
        return self.above + self.here + self.beneath


@dataclass
class PsiSpiralTuning:
    """Adjustments derived from the spiral-dynamics advisory: components to force on, weight increments,
    threshold shifts and a stability score in [0, 1] that sets the sampling floor."""
    required_components: PsiComponent = PsiComponent(0)
    weight_increments: dict = field(default_factory=dict)
    threshold_shifts: dict = field(default_factory=dict)
    stability_score: float = 1.0

    def is_neutral(self) -> bool:
        return not self.required_components and not self.weight_increments and not self.threshold_shifts


@dataclass
class PsiConfig:
    enabled: bool = False
    components: PsiComponent = PsiComponent(0)
    weights: dict = field(default_factory=dict)
    ema_alpha: float = 0.0
    sample_rate: int = 0
    thresholds: dict = field(default_factory=dict)

    @classmethod
    def automated(cls, hint: PsiAutomationHint) -> "PsiConfig":
        depth = max(1, hint.depth())
        alpha = 0.28 if depth <= 24 else (0.22 if depth <= 96 else 0.16)
        rate = 1 if depth <= 48 else (2 if depth <= 128 else 4)
        cfg = cls(True, PsiComponent.defaults() | PsiComponent.BAND_ENERGY | PsiComponent.POSITIVE_CURVATURE, {},
                  alpha, max(1, rate), {})
        clamp = lambda v, lo, hi: max(lo, min(hi, v))       # noqa: E731
        cfg.weights[PsiComponent.LOSS] = 1.0
        cfg.weights[PsiComponent.GRAD_NORM] = 0.35
        cfg.weights[PsiComponent.UPDATE_RATIO] = clamp(math.sqrt(1.0 / depth), 0.2, 0.6)
        cfg.weights[PsiComponent.ACT_DRIFT] = clamp(hint.drift_weight, 0.1, 0.4)
        cfg.weights[PsiComponent.BAND_ENERGY] = clamp(hint.band_focus / depth, 0.1, 0.5)
        cfg.weights[PsiComponent.POSITIVE_CURVATURE] = clamp(max(hint.above, hint.beneath) / depth, 0.1, 0.6)
        return cfg

    def apply_spiral_tuning(self, tuning: PsiSpiralTuning) -> None:
        self.components |= tuning.required_components
        for comp, delta in tuning.weight_increments.items():
            self.weights[comp] = max(0.0, min(10.0, self.weights.get(comp, 0.0) + delta))
        for comp, shift in tuning.threshold_shifts.items():
            self.thresholds[comp] = self.thresholds.get(comp, 0.0) + shift
        floor = 1 if tuning.stability_score < 0.25 else (2 if tuning.stability_score < 0.6 else 3)
        self.sample_rate = max(self.sample_rate, floor)


@dataclass
class PsiInput:
    loss: float = 0.0
    grad_l2: float = 0.0
    update_ratio: float = 0.0
    act_drift: float = 0.0
    attn_entropy: float = 0.0
    band_energy: float = 0.0
    curvature_pos: float = 0.0

    def take(self, comp: PsiComponent) -> float:
        return {PsiComponent.LOSS: self.loss, PsiComponent.GRAD_NORM: self.grad_l2,
                PsiComponent.UPDATE_RATIO: self.update_ratio, PsiComponent.ACT_DRIFT: self.act_drift,
                PsiComponent.ATTN_ENTROPY: self.attn_entropy, PsiComponent.BAND_ENERGY: self.band_energy,
                PsiComponent.POSITIVE_CURVATURE: self.curvature_pos}.get(comp, 0.0)


@dataclass
class PsiReading:
    total: float
    breakdown: dict
    step: int


@dataclass
class PsiEvent:
    component: PsiComponent
    value: float
    threshold: float
    up: bool
    step: int

    def __str__(self) -> str:
        return (f"psi.threshold:{self.component.name}:{'up' if self.up else 'down'}:{self.value:.3f}:"
                f"{self.threshold:.3f}@{self.step}")


CHECKPOINT_KIND = "psi_meter"
CHECKPOINT_VERSION = 1


class PsiMeter:
    def __init__(self, cfg: Optional[PsiConfig] = None):
        cfg = cfg or PsiConfig(enabled=True)
        cfg = PsiConfig(cfg.enabled, cfg.components, dict(cfg.weights), cfg.ema_alpha, cfg.sample_rate, dict(cfg.thresholds))
        if not cfg.components:
            cfg.components = PsiComponent.defaults()
        if not cfg.weights:
            cfg.weights.update({PsiComponent.LOSS: 1.0, PsiComponent.GRAD_NORM: 0.3, PsiComponent.UPDATE_RATIO: 0.4,
                                PsiComponent.ACT_DRIFT: 0.2})
        cfg.weights.setdefault(PsiComponent.POSITIVE_CURVATURE, 0.25)
        if not 0.0 < cfg.ema_alpha < 1.0:
            cfg.ema_alpha = 0.2
        if cfg.sample_rate <= 0:
            cfg.sample_rate = 1
        self.cfg, self.ema, self.step = cfg, {}, 0

    def config(self) -> PsiConfig:
        return self.cfg

    def update(self, x: PsiInput) -> tuple:
        self.step += 1
        breakdown = dict(self.ema)
        if not self.cfg.enabled or self.step % self.cfg.sample_rate != 0:
            total = sum(w * breakdown.get(c, 0.0) for c, w in self.cfg.weights.items())
            return PsiReading(total, breakdown, self.step), []
        alpha, total, events = self.cfg.ema_alpha, 0.0, []
        for comp in ORDER:
            if not (self.cfg.components & comp):
                continue
            raw = float(x.take(comp))
            prev = self.ema.get(comp, raw)
            ema = alpha * raw + (1.0 - alpha) * prev
            self.ema[comp] = breakdown[comp] = ema
            total += self.cfg.weights.get(comp, 0.0) * ema
            thr = self.cfg.thresholds.get(comp)
            if thr is not None:
                up, down = ema > thr and prev <= thr, ema < thr and prev >= thr
                if up or down:
                    events.append(PsiEvent(comp, ema, thr, up, self.step))
        return PsiReading(total, breakdown, self.step), events

    # ---- checkpoint --------------------------------------------------------------------------------------
    def checkpoint(self) -> dict:
        def entries(m: dict) -> list:
            for c, v in m.items():
                if c not in ORDER or not math.isfinite(v):
                    raise ValueError("psi meter state contains an unknown component or a non-finite value")
            return [{"component": c.label, "value": float(m[c])} for c in sorted(m, key=lambda c: c.label)]
        return {"kind": CHECKPOINT_KIND, "contract_version": CHECKPOINT_VERSION, "enabled": self.cfg.enabled,
                "components": [c.label for c in sorted(ORDER, key=lambda c: c.label) if self.cfg.components & c],
                "weights": entries(self.cfg.weights), "thresholds": entries(self.cfg.thresholds),
                "ema": entries(self.ema), "ema_alpha": self.cfg.ema_alpha, "sample_rate": self.cfg.sample_rate,
                "step": self.step}

    @classmethod
    def from_checkpoint(cls, doc: dict) -> "PsiMeter":
        if doc.get("kind") != CHECKPOINT_KIND or doc.get("contract_version") != CHECKPOINT_VERSION:
            raise ValueError("not a psi meter checkpoint of this contract version")

        def table(items) -> dict:
            return {PsiComponent.from_token(e["component"]): float(e["value"]) for e in items}
        comps = PsiComponent(0)
        for label in doc["components"]:
            comps |= PsiComponent.from_token(label)
        meter = cls(PsiConfig(bool(doc["enabled"]), comps, table(doc["weights"]), float(doc["ema_alpha"]),
                              int(doc["sample_rate"]), table(doc["thresholds"])))
        meter.ema, meter.step = table(doc["ema"]), int(doc["step"])
        return meter
