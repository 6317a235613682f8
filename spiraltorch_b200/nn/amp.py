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
