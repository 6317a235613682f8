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

    def observe(self, gradient: torch.Tensor) -> dict:
        """Pressure = mean absolute value of a gradient tensor."""
        return self.observe_pressure(float(gradient.detach().abs().mean()) if gradient.numel() else 0.0)

    def observe_pressure(self, raw_pressure: float) -> dict:
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
        return {"raw_pressure": raw, "smoothed_pressure": smoothed, "curvature": self.current, "changed": changed}

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
