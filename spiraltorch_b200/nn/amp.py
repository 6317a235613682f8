"""Mixed precision and optimiser control for ``st.nn`` modules.

Restated from crates/st-nn/src/mixed_precision.rs:14-206 (``AutocastGuard`` thread-local flag;
``GradScaler``: scale the loss gradient, unscale accumulators, skip the step and back off on a
non-finite accumulator norm, grow after ``growth_interval`` clean steps, limits [1, 65536]) and
crates/st-nn/src/optim/mod.rs (``OptimizerMode`` :398-445, ``ZSpaceParameterOptimizer`` :448-690,
``WarmupCosineScheduler`` :698-800, ``SpectralLrAdapter`` :35-150).
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass
from typing import Optional

import torch

from ..tensor import Tensor, TensorError
from .modules import Module

_autocast = threading.local()


def autocast_enabled() -> bool:
    return getattr(_autocast, "enabled", False)


class AutocastGuard:
    """``with AutocastGuard.enable():`` — modules consult :func:`autocast_enabled` to run their
    matrix products in bf16 (the CUDA GEMM path always does)."""

    def __init__(self, enabled: bool):
        self._enabled = enabled

    @classmethod
    def enable(cls) -> "AutocastGuard":
        return cls(True)

    @classmethod
    def disable(cls) -> "AutocastGuard":
        return cls(False)

    def __enter__(self):
        self._previous = autocast_enabled()
        _autocast.enabled = self._enabled
        return self

    def __exit__(self, *exc):
        _autocast.enabled = self._previous
        return False


@dataclass
class OptimizerMode:
    kind: str = "euclidean"
    curvature: float = -1.0
    learning_rate: float = 0.0

    @staticmethod
    def euclidean() -> "OptimizerMode":
        return OptimizerMode()

    @staticmethod
    def realgrad(learning_rate: float) -> "OptimizerMode":
        if not (learning_rate > 0 and math.isfinite(learning_rate)):
            raise TensorError(f"learning rate must be positive, got {learning_rate}")
        return OptimizerMode("realgrad", learning_rate=learning_rate)

    @staticmethod
    def hypergrad(curvature: float, learning_rate: float) -> "OptimizerMode":
        if not curvature < 0:
            raise TensorError(f"curvature must be negative, got {curvature}")
        if not (learning_rate > 0 and math.isfinite(learning_rate)):
            raise TensorError(f"learning rate must be positive, got {learning_rate}")
        return OptimizerMode("hypergrad", curvature, learning_rate)


class SpectralLrAdapter:
    """Per-parameter learning-rate multiplier from smoothed gradient statistics: energy (mean
    square), spin (mean sign agreement with the previous gradient) and a curvature proxy (ratio of
    the largest row norm to the mean row norm) compared with ``curvature_target``."""

    def __init__(self, smoothing: float = 0.9, curvature_target: float = 1.0, curvature_gain: float = 0.1,
                 spin_gain: float = 0.1, energy_gain: float = 0.05, min_scale: float = 0.25, max_scale: float = 4.0):
        self.smoothing, self.curvature_target = smoothing, curvature_target
        self.curvature_gain, self.spin_gain, self.energy_gain = curvature_gain, spin_gain, energy_gain
        self.min_scale, self.max_scale = min_scale, max_scale
        self.reset()

    def reset(self) -> None:
        self.avg_curvature, self.avg_spin, self.avg_energy = self.curvature_target, 0.0, 0.0
        self._prev: dict[str, torch.Tensor] = {}

    def set_curvature_target(self, curvature: float) -> None:
        self.curvature_target = abs(float(curvature))

    def state(self) -> dict:
        return {k: getattr(self, k) for k in ("smoothing", "curvature_target", "curvature_gain", "spin_gain",
                                              "energy_gain", "min_scale", "max_scale", "avg_curvature", "avg_spin",
                                              "avg_energy")}

    @classmethod
    def from_state(cls, state: dict) -> "SpectralLrAdapter":
        a = cls(**{k: state[k] for k in ("smoothing", "curvature_target", "curvature_gain", "spin_gain", "energy_gain",
                                         "min_scale", "max_scale")})
        a.avg_curvature, a.avg_spin, a.avg_energy = state["avg_curvature"], state["avg_spin"], state["avg_energy"]
        return a

    def scale_for(self, name: str, grad: torch.Tensor) -> float:
        g = grad.detach().float()
        rows = g.norm(dim=1)
        curv = float(rows.max() / rows.mean().clamp(min=1e-12))
        energy = float((g * g).mean())
        prev = self._prev.get(name)
        spin = 0.0 if prev is None or prev.shape != g.shape else float((torch.sign(prev) * torch.sign(g)).mean())
        self._prev[name] = g.clone()
        s = self.smoothing
        self.avg_curvature = s * self.avg_curvature + (1 - s) * curv
        self.avg_spin = s * self.avg_spin + (1 - s) * spin
        self.avg_energy = s * self.avg_energy + (1 - s) * energy
        scale = 1.0 - self.curvature_gain * (self.avg_curvature - self.curvature_target) \
            + self.spin_gain * self.avg_spin - self.energy_gain * math.log1p(self.avg_energy)
        return min(max(scale, self.min_scale), self.max_scale)


class ZSpaceParameterOptimizer:
    def __init__(self, fallback_lr: float):
        if not (fallback_lr > 0 and math.isfinite(fallback_lr)):
            raise TensorError(f"learning rate must be positive, got {fallback_lr}")
        self._fallback_lr = float(fallback_lr)
        self._mode = OptimizerMode.euclidean()
        self._adapter: Optional[SpectralLrAdapter] = None
        self._meta_scale = 1.0
        self._steps = 0

    def set_mode(self, mode: OptimizerMode) -> None:
        self._mode = mode

    def mode(self) -> OptimizerMode:
        return self._mode

    def fallback_learning_rate(self) -> float:
        return self._fallback_lr

    def meta_learning_rate_scale(self) -> float:
        return self._meta_scale

    def set_fallback_learning_rate(self, learning_rate: float) -> None:
        if not (learning_rate > 0 and math.isfinite(learning_rate)):
            raise TensorError(f"learning rate must be positive, got {learning_rate}")
        self._fallback_lr = float(learning_rate)

    def set_adapter(self, adapter: Optional[SpectralLrAdapter]) -> None:
        self._adapter = adapter

    def adapter(self) -> Optional[SpectralLrAdapter]:
        return self._adapter

    def state(self) -> dict:
        return {"fallback_lr": self._fallback_lr, "mode": vars(self._mode).copy(), "meta_scale": self._meta_scale,
                "steps": self._steps, "adapter": None if self._adapter is None else self._adapter.state()}

    def prepare_module(self, module: Module) -> None:
        if self._mode.kind == "realgrad":
            module.attach_realgrad(self._mode.learning_rate)
        elif self._mode.kind == "hypergrad":
            module.attach_hypergrad(self._mode.curvature, self._mode.learning_rate)

    def zero_grad(self, module: Module) -> None:
        module.zero_accumulators()

    def scale_learning_rate(self, module: Module, factor: float) -> None:
        if not (factor > 0 and math.isfinite(factor)):
            raise TensorError(f"learning-rate factor must be positive, got {factor}")
        self._fallback_lr *= factor
        for p in module.parameters():
            if p.hypergrad is not None:
                p.hypergrad.learning_rate *= factor
            if p.realgrad is not None:
                p.realgrad.learning_rate *= factor

    def step(self, module: Module) -> None:
        self._steps += 1
        if self._adapter is None:
            module.apply_step(self._fallback_lr)
            return
        for p in module.parameters():
            accs = p.accumulators()
            scale = self._adapter.scale_for(p.name, accs[0]) if accs else 1.0
            tapes = [t for t in (p.hypergrad, p.realgrad) if t is not None]
            for t in tapes:
                t.learning_rate *= scale
            p.apply_step(self._fallback_lr * scale)
            for t in tapes:
                t.learning_rate /= scale


class GradScaler:
    def __init__(self, scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000):
        if not (scale > 0 and math.isfinite(scale)):
            raise TensorError(f"grad scaler scale must be positive, got {scale}")
        if not (growth_factor > 1 and math.isfinite(growth_factor)):
            raise TensorError("grad_scaler_growth_factor must exceed 1")
        if not 0 < backoff_factor < 1:
            raise TensorError("grad_scaler_backoff_factor must lie in (0, 1)")
        if growth_interval <= 0:
            raise TensorError("grad_scaler_growth_interval must be positive")
        self._scale, self._growth, self._backoff = float(scale), growth_factor, backoff_factor
        self._interval, self._tracker = growth_interval, 0
        self._min, self._max = 1.0, 65536.0

    def with_limits(self, min_scale: float, max_scale: float) -> "GradScaler":
        if min_scale > 0 and math.isfinite(min_scale):
            self._min = min_scale
        if max_scale >= self._min and math.isfinite(max_scale):
            self._max = max_scale
        return self

    def scale(self) -> float:
        return self._scale

    def scale_loss(self, loss: float) -> float:
        return loss * self._scale

    def try_scale_loss(self, loss: float) -> float:
        if not math.isfinite(loss):
            raise TensorError("grad_scaler_loss is not finite")
        s = loss * self._scale
        if not math.isfinite(s) or abs(s) > 3.4028234e38:
            raise TensorError("grad_scaler_scaled_loss is not finite")
        return s

    def scale_tensor(self, tensor: Tensor) -> Tensor:
        return tensor.scale(self._scale)

    def unscale_module(self, module: Module) -> None:
        if self._scale != 1.0:
            for p in module.parameters():
                p.scale_accumulators(1.0 / self._scale)

    def has_overflow(self, module: Module) -> bool:
        for p in module.parameters():
            for a in p.accumulators():
                if not bool(torch.isfinite((a.float() ** 2).sum())):
                    return True
        return False

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self._scale = min(max(self._scale * self._backoff, self._min), self._max)
            self._tracker = 0
        else:
            self._tracker += 1
            if self._tracker >= self._interval:
                self._scale = min(max(self._scale * self._growth, self._min), self._max)
                self._tracker = 0

    def step(self, optimizer: ZSpaceParameterOptimizer, module: Module) -> bool:
        """Unscale, skip on overflow (accumulators cleared, scale backed off) or step; returns
        whether the optimiser stepped."""
        self.unscale_module(module)
        if self.has_overflow(module):
            self.update(True)
            module.zero_accumulators()
            return False
        optimizer.step(module)
        self.update(False)
        return True


class WarmupCosineScheduler:
    def __init__(self, base_lr: float, min_lr: float, warmup_steps: int, total_steps: int):
        if not (base_lr > 0 and math.isfinite(base_lr)):
            raise TensorError(f"learning rate must be positive, got {base_lr}")
        if not (min_lr >= 0 and math.isfinite(min_lr)):
            raise TensorError("scheduler_min_lr must be finite and non-negative")
        if total_steps <= 0 or warmup_steps > total_steps or warmup_steps < 0:
            raise TensorError(f"invalid schedule: warmup {warmup_steps}, total {total_steps}")
        self.base_lr, self.min_lr, self.warmup_steps, self.total_steps = base_lr, min_lr, warmup_steps, total_steps
        self._step = 0
        self.last_lr = min(min_lr, base_lr) if warmup_steps > 0 else base_lr

    def step(self) -> float:
        self._step += 1
        if self.warmup_steps > 0 and self._step <= self.warmup_steps:
            lr = self.min_lr + (self.base_lr - self.min_lr) * self._step / self.warmup_steps
        else:
            decay = max(1, self.total_steps - self.warmup_steps)
            progress = min(self._step - self.warmup_steps, decay) / decay
            lr = self.min_lr + (self.base_lr - self.min_lr) * 0.5 * (1.0 + math.cos(math.pi * progress))
        self.last_lr = max(lr, self.min_lr)
        return self.last_lr

    def step_optimizer(self, optimizer: ZSpaceParameterOptimizer, module: Module) -> float:
        lr = self.step() * optimizer.meta_learning_rate_scale()
        cur = optimizer.fallback_learning_rate()
        if cur > 0:
            optimizer.scale_learning_rate(module, lr / cur)
        else:
            optimizer.set_fallback_learning_rate(lr)
        return lr


_PRESSURE_MAX = 1.0e6


@dataclass(frozen=True)
class CurvatureDecision:
    """What one scheduler observation decided (crates/st-nn/src/trainer.rs:641-648); also readable by key."""
    raw_pressure: float
    smoothed_pressure: float
    curvature: float
    changed: bool

    def __getitem__(self, key: str):
        return getattr(self, key)

    def as_dict(self) -> dict:
        return {"raw_pressure": self.raw_pressure, "smoothed_pressure": self.smoothed_pressure, "curvature": self.curvature,
                "changed": self.changed}


class CurvatureScheduler:
    """Keeps the (negative) curvature of the hyperbolic optimiser near a target gradient pressure.

    ``observe_pressure(p)`` smooths ``p`` (EMA, ``smoothing``), and outside the tolerance band moves
    the curvature by ``clamp(kp · (1 + boost · stability) · error, ±step)`` where stability falls from
    1 to 0 as the relative variance of the pressure approaches ``stability_threshold``; inside the
    band, after ``dither_period`` stable steps, it dithers by ``±dither_strength · step``.
    Behaviour and defaults: crates/st-nn/src/trainer.rs:155-640; environment overrides
    ``SPIRAL_CURVATURE_{STEP,TOLERANCE,ALPHA,KP,STABILITY_THRESHOLD,STABILITY_BOOST,DITHER_STRENGTH,DITHER_PERIOD}``.
    """

    def __init__(self, initial: float, min_curvature: float, max_curvature: float, target_pressure: float):
        lo, hi = min(min_curvature, -1e-6), min(max_curvature, -1e-6)
        if lo > hi:
            lo, hi = hi, lo
        self.min_curvature, self.max_curvature = lo, hi
        self.current = min(min(max(initial, lo), hi), -1e-6)
        self.target_pressure = min(max(target_pressure, 0.0), _PRESSURE_MAX) if math.isfinite(target_pressure) else 0.0
        self.tolerance, self.step, self.kp, self.alpha = 0.05, 0.05, 1.0, 0.2
        self.ema_pressure: Optional[float] = None
        self.ema_pressure2: Optional[float] = None
        self.stability_threshold, self.stability_boost, self.stable_steps = 1.0e-3, 0.5, 0
        self.dither_strength, self.dither_period, self.dither_sign = 0.15, 8, 1.0

    # setters ignore values outside their domain, as the reference does
    def set_step(self, v: float):
        if math.isfinite(v) and v > 0:
            self.step = v

    def set_proportional_gain(self, v: float):
        if math.isfinite(v) and v >= 0:
            self.kp = v

    def set_tolerance(self, v: float):
        if math.isfinite(v) and v >= 0:
            self.tolerance = v

    def set_smoothing(self, v: float):
        if math.isfinite(v) and v > 0:
            self.alpha = min(max(v, 0.01), 1.0)

    def set_stability_threshold(self, v: float):
        if math.isfinite(v) and v > 0:
            self.stability_threshold = v

    def set_stability_boost(self, v: float):
        if math.isfinite(v) and v >= 0:
            self.stability_boost = v

    def set_dither(self, strength: float, period: int):
        if math.isfinite(strength) and strength >= 0:
            self.dither_strength = min(strength, 1.0)
        if period > 0:
            self.dither_period = int(period)

    def set_target_pressure(self, v: float):
        if math.isfinite(v):
            self.target_pressure = min(max(v, 0.0), _PRESSURE_MAX)

    def set_bounds(self, min_curvature: float, max_curvature: float):
        lo, hi = min(min_curvature, -1e-6), min(max_curvature, -1e-6)
        if lo > hi:
            lo, hi = hi, lo
        self.min_curvature, self.max_curvature = lo, hi
        self.current = min(min(max(self.current, lo), hi), -1e-6)

    def apply_env_overrides(self, env=None) -> "CurvatureScheduler":
        import os
        env = os.environ if env is None else env

        def num(key, cast=float):
            try:
                return cast(env[key])
            except (KeyError, ValueError):
                return None
        for key, setter in (("SPIRAL_CURVATURE_STEP", self.set_step), ("SPIRAL_CURVATURE_TOLERANCE", self.set_tolerance),
                            ("SPIRAL_CURVATURE_ALPHA", self.set_smoothing), ("SPIRAL_CURVATURE_KP", self.set_proportional_gain),
                            ("SPIRAL_CURVATURE_STABILITY_THRESHOLD", self.set_stability_threshold),
                            ("SPIRAL_CURVATURE_STABILITY_BOOST", self.set_stability_boost)):
            v = num(key)
            if v is not None:
                setter(v)
        s, p = num("SPIRAL_CURVATURE_DITHER_STRENGTH"), num("SPIRAL_CURVATURE_DITHER_PERIOD", int)
        if s is not None or p is not None:
            self.set_dither(self.dither_strength if s is None else s, self.dither_period if p is None else p)
        return self

    def sync(self, curvature: float) -> None:
        """Adopts an externally chosen curvature and forgets the pressure history."""
        self.current = min(min(max(curvature, self.min_curvature), self.max_curvature), -1e-6)
        self.ema_pressure = self.ema_pressure2 = None
        self.stable_steps, self.dither_sign = 0, 1.0

    def last_pressure_variance(self) -> Optional[float]:
        if self.ema_pressure is None or self.ema_pressure2 is None:
            return None
        return max(self.ema_pressure2 - self.ema_pressure ** 2, 0.0)

    def observe(self, gradient: torch.Tensor) -> "CurvatureDecision":
        """Pressure = mean absolute value of a gradient tensor."""
        return self.observe_pressure(float(gradient.detach().abs().mean()) if gradient.numel() else 0.0)

    def observe_pressure(self, raw_pressure: float) -> "CurvatureDecision":
        raw = min(max(raw_pressure, 0.0), _PRESSURE_MAX) if math.isfinite(raw_pressure) else 0.0
        a = self.alpha
        smoothed = raw if self.ema_pressure is None else self.ema_pressure + a * (raw - self.ema_pressure)
        smoothed = min(max(smoothed, 0.0), _PRESSURE_MAX)
        self.ema_pressure = smoothed
        sq = raw * raw
        self.ema_pressure2 = sq if self.ema_pressure2 is None else self.ema_pressure2 + a * (sq - self.ema_pressure2)
        variance = max(self.ema_pressure2 - smoothed * smoothed, 0.0)
        rel_var = variance / (smoothed * smoothed + 1.0e-6)
        error = smoothed - self.target_pressure
        within = abs(error) <= self.tolerance
        stable = within and rel_var <= self.stability_threshold
        self.stable_steps = self.stable_steps + 1 if stable else 0
        delta = 0.0
        if not within:
            stability = max(1.0 - min(max(rel_var / self.stability_threshold, 0.0), 1.0), 0.0)
            kp = self.kp * (1.0 + self.stability_boost * stability)
            delta = min(max(kp * error, -self.step), self.step)
        elif stable and self.dither_strength > 0 and self.stable_steps >= self.dither_period:
            delta = self.dither_sign * self.dither_strength * self.step
            self.dither_sign = -self.dither_sign
            self.stable_steps = 0
        changed = False
        if abs(delta) > 1.1920929e-07:
            nxt = min(min(max(self.current + delta, self.min_curvature), self.max_curvature), -1e-6)
            if abs(nxt - self.current) > 1.1920929e-07:
                self.current, changed = nxt, True
        return CurvatureDecision(raw, smoothed, self.current, changed)

    _FIELDS = ("min_curvature", "max_curvature", "target_pressure", "tolerance", "step", "kp", "alpha", "current",
               "ema_pressure", "ema_pressure2", "stability_threshold", "stability_boost", "stable_steps",
               "dither_strength", "dither_period", "dither_sign")

    def state(self) -> dict:
        d = {k: getattr(self, k) for k in self._FIELDS}
        d["proportional_gain"], d["smoothing"] = d.pop("kp"), d.pop("alpha")
        return d

    @classmethod
    def from_state(cls, state: dict) -> "CurvatureScheduler":
        s = dict(state)
        for key in ("min_curvature", "max_curvature", "current"):
            if not (math.isfinite(s[key]) and s[key] < 0):
                raise ValueError(f"curvature scheduler state: {key} must be negative and finite")
        if s["min_curvature"] > s["max_curvature"]:
            raise ValueError("curvature scheduler state: min_curvature exceeds max_curvature")
        sch = cls(s["current"], s["min_curvature"], s["max_curvature"], s["target_pressure"])
        s["kp"], s["alpha"] = s.pop("proportional_gain"), s.pop("smoothing")
        for k in cls._FIELDS:
            setattr(sch, k, s[k])
        return sch


# ---- coherence-driven learning-rate policy ------------------------------------------------------------------------------
@dataclass(frozen=True)
class CoherenceSignal:
    """The part of a sequencer's diagnostics the spectral policy consumes, re-derived through the coherence contract
    so every number agrees with the normalized weights (crates/st-nn/src/trainer.rs:668-985)."""
    dominant_channel: Optional[int]
    preserved_channels: int
    z_bias: float
    control: object                  # zspace_coherence.ControlPayload
    classification: object           # zspace_coherence.ClassificationPayload
    repaired_weights_total: int = 0
    pre_discard_repairs_total: int = 0

    @classmethod
    def from_diagnostics(cls, diagnostics) -> Optional["CoherenceSignal"]:
        from .. import zspace_coherence as zc
        try:
            proj = diagnostics.project_to_zspace_partial()
        except zc.CoherenceProjectionError:
            return None
        if proj.control is None or proj.classification is None:
            return None
        pre = diagnostics.pre_discard
        return cls(diagnostics.dominant_channel, diagnostics.preserved_channels(), diagnostics.z_bias, proj.control,
                   proj.classification, diagnostics.repaired_weights_total, 0 if pre is None else pre.repairs_total)

    @property
    def label(self) -> str:
        return self.classification.label

    @property
    def repairs_total(self) -> int:
        return self.repaired_weights_total + self.pre_discard_repairs_total


@dataclass
class SpectralAdjustment:
    band_scale: tuple          # smoothed (above, here, beneath) gradient-band multipliers
    lr_multiplier: float       # factor to apply to the current learning rate this step
    lr_scale: float            # resulting absolute scale against the base learning rate
    local_lr: tuple            # band scales divided by their mean, smoothed
    metrics: dict


class SpectralLearningRatePolicy:
    """Turns coherence diagnostics + the roundtable band energy into per-band gradient scales and a learning-rate
    multiplier (crates/st-nn/src/trainer.rs:4612-5216).

    Per observation: the dominant channel's position biases Above or Beneath (``sheet_gain``), the Z bias does the same
    (``spin_gain``), curvature and a flat spectrum (``1 - spectral_radius``) lift all bands; band energy shares tilt the
    bands by ``energy_gain``; the dominant channel's index mod 3 picks the band that gets the phase gain (larger while
    the dominant channel has not changed for a while — "stuck"); the coherence label scales the learning rate (cascade
    0.7, symmetric 0.9, diffuse 1.15) and flattens the side bands.  Everything is smoothed (faster when the label
    changed), clamped to the band / lr bounds, and the lr multiplier is limited to ``max_lr_step`` per observation."""

    _STATE = ("smoothing", "event_smoothing", "turnover_smoothing", "coherence_gain", "curvature_gain", "sheet_gain", "spin_gain",
              "radius_gain", "energy_gain", "phase_gain", "stuck_phase_gain", "max_phase_gain", "stuck_turnover_threshold",
              "dominant_turnover", "last_dominant", "last_label", "min_lr_scale", "max_lr_scale", "max_lr_step", "min_band_scale",
              "max_band_scale", "band_state", "lr_state", "applied_lr_scale", "local_lr_state")

    def __init__(self):
        self.smoothing, self.event_smoothing, self.turnover_smoothing = 0.2, 0.75, 0.15
        self.coherence_gain, self.curvature_gain, self.sheet_gain, self.spin_gain = 0.5, 0.15, 0.6, 0.4
        self.radius_gain, self.energy_gain = 0.35, 0.25
        self.phase_gain, self.stuck_phase_gain, self.max_phase_gain, self.stuck_turnover_threshold = 0.25, 0.35, 0.65, 0.12
        self.dominant_turnover, self.last_dominant, self.last_label = 0.0, None, None
        self.min_lr_scale, self.max_lr_scale, self.max_lr_step = 0.1, 6.0, 1.4
        self.min_band_scale, self.max_band_scale = 0.5, 2.75
        self.band_state, self.lr_state, self.applied_lr_scale, self.local_lr_state = [1.0, 1.0, 1.0], 1.0, 1.0, [1.0, 1.0, 1.0]

    # builders: values outside the domain are ignored
    def _set_smooth(self, name, v):
        if math.isfinite(v) and v > 0:
            setattr(self, name, min(max(v, 1.0e-3), 1.0))
        return self

    def _set_nonneg(self, name, v, clamp_low=False):
        if math.isfinite(v) and (clamp_low or v >= 0):
            setattr(self, name, max(v, 0.0))
        return self

    def with_smoothing(self, v): return self._set_smooth("smoothing", v)                       # noqa: E704
    def with_event_smoothing(self, v): return self._set_smooth("event_smoothing", v)           # noqa: E704
    def with_turnover_smoothing(self, v): return self._set_smooth("turnover_smoothing", v)     # noqa: E704
    def with_phase_gain(self, v): return self._set_nonneg("phase_gain", v)                     # noqa: E704
    def with_stuck_phase_gain(self, v): return self._set_nonneg("stuck_phase_gain", v)         # noqa: E704
    def with_stuck_turnover_threshold(self, v): return self._set_nonneg("stuck_turnover_threshold", v)   # noqa: E704
    def with_coherence_gain(self, v): return self._set_nonneg("coherence_gain", v, True)       # noqa: E704
    def with_sheet_gain(self, v): return self._set_nonneg("sheet_gain", v, True)               # noqa: E704
    def with_spin_gain(self, v): return self._set_nonneg("spin_gain", v, True)                 # noqa: E704
    def with_radius_gain(self, v): return self._set_nonneg("radius_gain", v, True)             # noqa: E704
    def with_energy_gain(self, v): return self._set_nonneg("energy_gain", v, True)             # noqa: E704

    def _clamp_state(self) -> None:
        cl = lambda v, lo, hi: min(max(v, lo), hi)                                             # noqa: E731
        self.band_state = [cl(v, self.min_band_scale, self.max_band_scale) for v in self.band_state]
        self.local_lr_state = [cl(v, self.min_band_scale, self.max_band_scale) for v in self.local_lr_state]
        self.lr_state = cl(self.lr_state, self.min_lr_scale, self.max_lr_scale)
        self.applied_lr_scale = cl(self.applied_lr_scale, self.min_lr_scale, self.max_lr_scale)

    def with_lr_bounds(self, lo, hi):
        if math.isfinite(lo) and math.isfinite(hi) and lo > 0 and hi > lo:
            self.min_lr_scale, self.max_lr_scale = lo, hi
            self._clamp_state()
        return self

    def with_band_bounds(self, lo, hi):
        if math.isfinite(lo) and math.isfinite(hi) and lo > 0 and hi > lo:
            self.min_band_scale, self.max_band_scale = lo, hi
            self._clamp_state()
        return self

    def with_max_lr_step(self, v):
        if math.isfinite(v) and v > 0:
            self.max_lr_step = max(v, 1.0)
        return self

    def apply_env_overrides(self, env=None) -> "SpectralLearningRatePolicy":
        """``SPIRAL_SPECTRAL_POLICY_{SMOOTHING,EVENT_SMOOTHING,TURNOVER_SMOOTHING,PHASE_GAIN,STUCK_PHASE_GAIN,MAX_PHASE_GAIN,
        STUCK_TURNOVER_THRESHOLD,LR_MIN,LR_MAX,BAND_MIN,BAND_MAX}``; unparsable or out-of-domain values are ignored."""
        import os
        env = os.environ if env is None else env

        def num(key):
            try:
                v = float(env["SPIRAL_SPECTRAL_POLICY_" + key])
                return v if math.isfinite(v) else None
            except (KeyError, ValueError):
                return None
        for key, fn in (("SMOOTHING", self.with_smoothing), ("EVENT_SMOOTHING", self.with_event_smoothing),
                        ("TURNOVER_SMOOTHING", self.with_turnover_smoothing), ("PHASE_GAIN", self.with_phase_gain),
                        ("STUCK_PHASE_GAIN", self.with_stuck_phase_gain)):
            v = num(key)
            if v is not None:
                fn(v)
        v = num("MAX_PHASE_GAIN")
        if v is not None and v >= 0:
            self.max_phase_gain = v
        v = num("STUCK_TURNOVER_THRESHOLD")
        if v is not None and v >= 0:
            self.stuck_turnover_threshold = min(v, 1.0)
        lo, hi = num("LR_MIN"), num("LR_MAX")
        if lo is not None and hi is not None:
            self.with_lr_bounds(lo, hi)
        lo, hi = num("BAND_MIN"), num("BAND_MAX")
        if lo is not None and hi is not None:
            self.with_band_bounds(lo, hi)
        self._clamp_state()
        return self

    with_env_overrides = apply_env_overrides

    def state(self) -> dict:
        return {k: (list(getattr(self, k)) if isinstance(getattr(self, k), list) else getattr(self, k)) for k in self._STATE}

    @classmethod
    def from_state(cls, state: dict) -> "SpectralLearningRatePolicy":
        p = cls()
        for k in cls._STATE:
            if k not in state:
                raise ValueError(f"spectral policy state is missing '{k}'")
            v = state[k]
            if k in ("band_state", "local_lr_state"):
                v = [float(x) for x in v]
                if len(v) != 3 or not all(math.isfinite(x) and x > 0 for x in v):
                    raise ValueError(f"spectral policy state '{k}' must hold three positive finite values")
            elif k not in ("last_dominant", "last_label") and not math.isfinite(float(v)):
                raise ValueError(f"spectral policy state '{k}' must be finite")
            setattr(p, k, v)
        if not (0 < p.min_lr_scale < p.max_lr_scale and 0 < p.min_band_scale < p.max_band_scale):
            raise ValueError("spectral policy bounds must satisfy 0 < min < max")
        if p.max_lr_step < 1.0:
            raise ValueError("spectral policy max_lr_step must be at least 1")
        inside = all(p.min_band_scale <= v <= p.max_band_scale for v in p.band_state + p.local_lr_state) and \
            all(p.min_lr_scale <= v <= p.max_lr_scale for v in (p.lr_state, p.applied_lr_scale))
        if not inside:
            raise ValueError("spectral policy state lies outside its own bounds")
        return p

    def last_coherence_label(self) -> Optional[str]:
        return self.last_label

    @staticmethod
    def _smooth(prev: float, target: float, alpha: float) -> float:
        return target if not math.isfinite(prev) else prev + (target - prev) * alpha

    def observe(self, diagnostics, curvature: float, band_energy) -> Optional[SpectralAdjustment]:
        signal = diagnostics if isinstance(diagnostics, CoherenceSignal) or diagnostics is None else CoherenceSignal.from_diagnostics(diagnostics)
        return self.observe_signal(signal, curvature, band_energy)

    def observe_signal(self, signal: Optional[CoherenceSignal], curvature: float, band_energy) -> Optional[SpectralAdjustment]:
        if signal is None:
            return None
        cl = lambda v, lo, hi: min(max(v, lo), hi)                                             # noqa: E731
        label, ctl = signal.label, signal.control
        sheets = max(ctl.channels, 1)
        dominant = min(signal.dominant_channel or 0, sheets - 1)
        changed = self.last_dominant is not None and self.last_dominant != dominant
        self.dominant_turnover = cl(self._smooth(self.dominant_turnover, 1.0 if changed else 0.0, self.turnover_smoothing), 0.0, 1.0)
        self.last_dominant = dominant
        label_changed = self.last_label is not None and self.last_label != label
        self.last_label = label
        smoothing = max(self.event_smoothing, self.smoothing) if label_changed else self.smoothing
        sheet_bias = ((dominant + 0.5) / sheets - 0.5) * self.sheet_gain
        spin = cl(signal.z_bias, -1.0, 1.0)
        spin_bias = spin * self.spin_gain
        curv = math.sqrt(-curvature) * self.curvature_gain if curvature < 0 else 0.0
        radius_bias = cl(1.0 - ctl.spectral_radius, 0.0, 1.0) * self.radius_gain
        base = (1.0 + max(sheet_bias, 0.0) + max(spin_bias, 0.0) + curv * 0.25 + radius_bias * 0.5,
                1.0 + max(1.0 - abs(sheet_bias), 0.0) * 0.5 * self.sheet_gain + curv * 0.5 + (1.0 - radius_bias) * 0.25,
                1.0 + max(-sheet_bias, 0.0) + max(-spin_bias, 0.0) + curv * 0.25 + radius_bias * 0.5)
        be = (band_energy.above, band_energy.here, band_energy.beneath)
        tot = max(sum(abs(v) for v in be), 1e-5)
        stuck = self.dominant_turnover < self.stuck_turnover_threshold
        lr_label = {"background": 1.05 if stuck else 1.0, "symmetric_pulse": 0.9, "cascade_imbalance": 0.7, "diffuse_drift": 1.15}[label]
        band_label = {"cascade_imbalance": (0.92, 1.15, 0.92), "symmetric_pulse": (0.96, 1.06, 0.96)}.get(label, (1.0, 1.0, 1.0))
        pg = {"diffuse_drift": self.phase_gain * 1.15, "cascade_imbalance": 0.0, "symmetric_pulse": self.phase_gain * 0.35,
              "background": self.phase_gain}[label]
        if stuck and label != "cascade_imbalance":
            pg += self.stuck_phase_gain
        pg = cl(pg, 0.0, self.max_phase_gain)
        phase_mul = [1.0 - 0.5 * pg] * 3
        phase_mul[dominant % 3] = 1.0 + pg
        lo, hi = self.min_band_scale, self.max_band_scale
        for i in range(3):
            t = cl(base[i] * (1.0 + cl(be[i] / tot, -1.0, 1.0) * self.energy_gain), lo, hi)
            t = cl(t * phase_mul[i] * band_label[i], lo, hi)
            self.band_state[i] = self._smooth(self.band_state[i], t, smoothing)
        band = tuple(self.band_state)
        mean_band = sum(band) / 3.0
        target_lr = cl(mean_band * (1.0 + ctl.spectral_pressure * self.coherence_gain) * lr_label, self.min_lr_scale, self.max_lr_scale)
        self.lr_state = self._smooth(self.lr_state, target_lr, smoothing)
        target_lr = cl(self.lr_state, self.min_lr_scale, self.max_lr_scale)
        for i in range(3):
            self.local_lr_state[i] = self._smooth(self.local_lr_state[i], cl(band[i] / mean_band, lo, hi), smoothing)
        local = tuple(self.local_lr_state)
        mult = 1.0
        if math.isfinite(self.applied_lr_scale) and self.applied_lr_scale > 0:
            step = self.max_lr_step * 1.25 if label_changed else self.max_lr_step
            mult = cl(target_lr / self.applied_lr_scale, 1.0 / step, step)
        self.applied_lr_scale = cl(self.applied_lr_scale * mult, self.min_lr_scale, self.max_lr_scale)
        metrics = {"absolute_lr_scale": self.applied_lr_scale, "sheet_index": signal.dominant_channel, "sheet_count": sheets,
                   "spin_alignment": spin, "raw_mean_coherence": ctl.raw_mean_coherence, "raw_coherence_entropy": ctl.raw_coherence_entropy,
                   "spectral_radius": ctl.spectral_radius, "spectral_entropy": ctl.spectral_entropy,
                   "spectral_pressure": ctl.spectral_pressure, "effective_channels": ctl.effective_channels,
                   "distribution_channels": ctl.channels, "energy_ratio": ctl.energy_ratio, "control_kind": ctl.kind,
                   "control_contract_version": ctl.contract_version, "classification_reason": signal.classification.reason,
                   "classification_contract_version": signal.classification.contract_version, "label": label,
                   "band_scale": band, "local_lr": local}
        return SpectralAdjustment(band, mult, self.applied_lr_scale, local, metrics)
