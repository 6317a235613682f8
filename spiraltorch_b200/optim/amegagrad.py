"""Amegagrad: the hypergrad (Poincaré-ball) and realgrad (Euclidean) optimizer tapes.

Semantics restated from the reference (crates/st-tensor/src/pure.rs):
* ``AmegaHypergrad.accumulate_wave``  ``g ← sat(g + v / max(|1 − c·v²|, tol))``      (:10637-10815)
* ``AmegaHypergrad.accumulate_pair``  ``g ← sat(g + (prediction − target))``          (:10837-10858)
* ``AmegaHypergrad.apply``            ``w ← project(sat(w − lr / max(|1 − c·w²|, tol) · g))``, ``g ← 0``
  with the row-wise Poincaré projection ``row · tanh(‖row‖/√−c) / ‖row‖``             (:10585-10615, :7528)
* ``AmegaRealgrad``                   ``g ← g + v``; ``w ← w − lr·g``; ``g ← 0``          (:11315-11470)
* topos defaults ``tolerance 1e-6, saturation 1e6, porosity 0.2`` and the porous saturation
  ``sat`` (crates/st-tensor/src/pure/topos.rs:169-188, :3267-3317).

On CUDA tensors accumulate/apply are single fused kernels (``csrc/optim/optim.cu``).
``Amegagrad`` mirrors the Python class of the reference (bindings/st-py/spiraltorch/optim.py:105-573):
one hypergrad and one realgrad of the same shape, ``step(weights)`` applies the hypergrad
update + projection and then the realgrad update on the projected weights, atomically.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

import torch

from ..ops import optim as K


@dataclass
class Topos:
    """Open-cartesian topos guard parameters (crates/st-tensor/src/pure/topos.rs:3207)."""
    curvature: float = -1.0
    tolerance: float = 1e-6
    saturation: float = 1e6
    max_depth: int = 8
    max_volume: int = 1 << 30
    porosity: float = 0.2

    def saturate(self, x: torch.Tensor) -> torch.Tensor:
        return K.porous_mix(x, self.saturation, self.porosity)


def _as_torch(x) -> torch.Tensor:
    return x.torch() if hasattr(x, "torch") and callable(x.torch) else torch.as_tensor(x, dtype=torch.float32)


class AmegaHypergrad:
    def __init__(self, curvature: float, learning_rate: float, rows: int, cols: int, *,
                 topos: Optional[Topos] = None, device=None):
        if not curvature < 0:
            raise ValueError(f"hypergrad curvature must be negative, got {curvature}")
        if not learning_rate > 0:
            raise ValueError("hypergrad learning rate must be positive")
        self.curvature, self.learning_rate = float(curvature), float(learning_rate)
        self.rows, self.cols = int(rows), int(cols)
        self.topos = topos or Topos(curvature=curvature, max_volume=max(1, rows * cols))
        self.gradient = torch.zeros(rows, cols, dtype=torch.float32, device=device or "cpu")

    def shape(self) -> tuple[int, int]:
        return (self.rows, self.cols)

    def _check(self, t: torch.Tensor) -> torch.Tensor:
        t = _as_torch(t).to(self.gradient.device, torch.float32)
        if t.numel() != self.rows * self.cols:
            raise ValueError(f"shape mismatch: expected {self.shape()}, got {tuple(t.shape)}")
        return t.reshape(self.rows, self.cols).contiguous()

    def accumulate_wave(self, wave, scale: float = 1.0) -> None:
        K.hyper_accumulate(self.gradient, self._check(wave), self.curvature, self.topos.tolerance,
                           self.topos.saturation, self.topos.porosity, conformal=True, scale=scale)

    def accumulate_pair(self, prediction, target) -> None:
        diff = self._check(prediction) - self._check(target)
        K.hyper_accumulate(self.gradient, diff, self.curvature, self.topos.tolerance,
                           self.topos.saturation, self.topos.porosity, conformal=False)

    def accumulate_barycenter_path(self, intermediates) -> None:
        """Accumulate the first density of a barycenter path as a wave and every later one against its
        predecessor (crates/st-tensor/src/pure.rs:11104-11125)."""
        if not intermediates:
            raise ValueError("empty input: barycenter_intermediates")
        prev = intermediates[0].density
        self.accumulate_wave(prev)
        for stage in intermediates[1:]:
            self.accumulate_pair(stage.density, prev)
            prev = stage.density

    def accumulate_complex_wave(self, real, imag) -> None:
        """Interleaves real/imaginary parts into one wave of the tape's shape."""
        r, i = _as_torch(real).reshape(-1), _as_torch(imag).reshape(-1)
        wave = torch.stack([r, i], dim=1).reshape(-1)[: self.rows * self.cols]
        if wave.numel() < self.rows * self.cols:
            wave = torch.cat([wave, wave.new_zeros(self.rows * self.cols - wave.numel())])
        self.accumulate_wave(wave)

    def absorb_text(self, encoder, text: str) -> None:
        """Encode ``text`` with ``encoder.encode_z_space`` and accumulate it as a wave
        (crates/st-tensor/src/pure.rs:10824-10835)."""
        self.accumulate_wave(encoder.encode_z_space(text, self.rows, self.cols))

    def apply(self, weights: torch.Tensor, realgrad: Optional["AmegaRealgrad"] = None) -> None:
        """In-place update of ``weights`` (and of ``realgrad``'s step on the projected weights)."""
        w = _as_torch(weights)
        if tuple(w.shape) != self.shape():
            raise ValueError(f"shape mismatch: expected {self.shape()}, got {tuple(w.shape)}")
        self.to(w.device)                     # the tape follows its weights (a module may have been moved)
        if realgrad is not None:
            realgrad.to(w.device)
        K.hyper_apply(w, self.gradient, None if realgrad is None else realgrad.gradient,
                      curvature=self.curvature, lr=self.learning_rate,
                      lr_real=0.0 if realgrad is None else realgrad.learning_rate,
                      tol=self.topos.tolerance, saturation=self.topos.saturation, porosity=self.topos.porosity)

    def reset(self) -> None:
        self.gradient.zero_()

    def to(self, device) -> "AmegaHypergrad":
        if self.gradient.device != torch.device(device):
            self.gradient = self.gradient.to(device)
        return self

    def gradient_norm(self) -> float:
        return float(self.gradient.norm())

    def checkpoint(self) -> dict:
        return {"kind": "amega_hypergrad", "curvature": self.curvature, "learning_rate": self.learning_rate,
                "rows": self.rows, "cols": self.cols, "topos": asdict(self.topos),
                "gradient": self.gradient.cpu().reshape(-1).tolist()}

    @classmethod
    def from_checkpoint(cls, ck: dict, device=None) -> "AmegaHypergrad":
        tape = cls(ck["curvature"], ck["learning_rate"], ck["rows"], ck["cols"], topos=Topos(**ck["topos"]),
                   device=device)
        tape.gradient.copy_(torch.tensor(ck["gradient"]).reshape(ck["rows"], ck["cols"]))
        return tape


class AmegaRealgrad:
    def __init__(self, learning_rate: float, rows: int, cols: int, device=None):
        if not learning_rate > 0:
            raise ValueError("realgrad learning rate must be positive")
        self.learning_rate, self.rows, self.cols = float(learning_rate), int(rows), int(cols)
        self.gradient = torch.zeros(rows, cols, dtype=torch.float32, device=device or "cpu")

    def shape(self) -> tuple[int, int]:
        return (self.rows, self.cols)

    def accumulate(self, grad) -> None:
        g = _as_torch(grad).to(self.gradient.device, torch.float32).reshape(self.rows, self.cols)
        self.gradient.add_(g)

    def to(self, device) -> "AmegaRealgrad":
        if self.gradient.device != torch.device(device):
            self.gradient = self.gradient.to(device)
        return self

    accumulate_wave = accumulate

    def accumulate_pair(self, prediction, target) -> None:
        self.accumulate(_as_torch(prediction) - _as_torch(target))

    def apply(self, weights: torch.Tensor) -> None:
        w = _as_torch(weights)
        self.to(w.device)
        K.hyper_apply(w, None, self.gradient, curvature=-1.0, lr=0.0, lr_real=self.learning_rate,
                      tol=1e-6, saturation=1e6, porosity=0.2)

    def reset(self) -> None:
        self.gradient.zero_()

    def checkpoint(self) -> dict:
        return {"kind": "amega_realgrad", "learning_rate": self.learning_rate, "rows": self.rows,
                "cols": self.cols, "gradient": self.gradient.cpu().reshape(-1).tolist()}

    @classmethod
    def from_checkpoint(cls, ck: dict, device=None) -> "AmegaRealgrad":
        tape = cls(ck["learning_rate"], ck["rows"], ck["cols"], device=device)
        tape.gradient.copy_(torch.tensor(ck["gradient"]).reshape(ck["rows"], ck["cols"]))
        return tape


class DesireGradientControl:
    """Learning-rate scales derived from a 'desire' signal (reference: ``DesireGradientControl``)."""

    def __init__(self, hyper_rate_scale: float = 1.0, real_rate_scale: float = 1.0):
        self._h, self._r = hyper_rate_scale, real_rate_scale

    def hyper_rate_scale(self) -> float:
        return self._h

    def real_rate_scale(self) -> float:
        return self._r


class Amegagrad:
    """``Amegagrad(*shape, curvature, hyper_learning_rate, real_learning_rate, topos, gain)``."""

    def __init__(self, *shape: int, curvature: float = -1.0, hyper_learning_rate: float = 1e-2,
                 real_learning_rate: float = 1e-2, topos: Optional[Topos] = None, gain: float = 1.0,
                 topos_control_gain: float = 0.0, device=None):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if len(shape) != 2:
            raise TypeError("Amegagrad expects a (rows, cols) shape")
        self._shape = (int(shape[0]), int(shape[1]))
        self.hyper = AmegaHypergrad(curvature, hyper_learning_rate, *self._shape, topos=topos, device=device)
        self.real = AmegaRealgrad(real_learning_rate, *self._shape, device=device)
        self.base_hyper_lr, self.base_real_lr = hyper_learning_rate, real_learning_rate
        self.gain = gain
        self.topos_control_gain = topos_control_gain
        self._control: Optional[DesireGradientControl] = None

    def shape(self) -> tuple[int, int]:
        return self._shape

    def zero_grad(self) -> None:
        self.hyper.reset()
        self.real.reset()

    def accumulate_wave(self, wave) -> None:
        self.hyper.accumulate_wave(wave)
        self.real.accumulate(wave)

    def accumulate_complex_wave(self, real, imag) -> None:
        self.hyper.accumulate_complex_wave(real, imag)

    def accumulate_pair(self, prediction, target) -> None:
        self.hyper.accumulate_pair(prediction, target)
        self.real.accumulate_pair(prediction, target)

    def absorb_text(self, encoder, text: str) -> None:
        self.hyper.absorb_text(encoder, text)

    def desire_control(self, control: Optional[DesireGradientControl] = None) -> Optional[DesireGradientControl]:
        if control is not None:
            self._control = control
        return self._control

    def topos_control_signal(self) -> dict:
        g = self.hyper.gradient
        return {"gradient_norm": float(g.norm()), "saturation_ratio": float((g.abs() >= self.hyper.topos.saturation).float().mean())}

    def topos_training_hints(self) -> dict:
        sig = self.topos_control_signal()
        return {"suggested_lr_scale": 1.0 / (1.0 + self.topos_control_gain * sig["saturation_ratio"]), **sig}

    def topos_diagnostics(self) -> dict:
        from dataclasses import asdict as _asdict
        return {"topos": _asdict(self.hyper.topos), **self.topos_control_signal()}

    def tune(self, control: Optional[DesireGradientControl] = None, gain: Optional[float] = None) -> None:
        control = control or self._control
        gain = self.gain if gain is None else gain
        h = r = 1.0
        if control is not None:
            h, r = control.hyper_rate_scale(), control.real_rate_scale()
        if self.topos_control_gain > 0:
            s = self.topos_training_hints()["suggested_lr_scale"]
            h, r = h * s, r * s
        self.hyper.learning_rate = self.base_hyper_lr * (1 + gain * (h - 1))
        self.real.learning_rate = self.base_real_lr * (1 + gain * (r - 1))

    def step(self, weights, *, tune: bool = True, gain: Optional[float] = None, control=None,
             use_topos: Optional[bool] = None) -> None:
        """One combined step: hypergrad update + projection on ``weights``, realgrad update on the
        projected weights, both accumulators reset (crates/st-tensor/src/pure.rs:11549-11562)."""
        if tune:
            self.tune(control, gain)
        w = _as_torch(weights)
        self.hyper.apply(w, realgrad=self.real)


def amegagrad(*shape, **kwargs) -> Amegagrad:
    return Amegagrad(*shape, **kwargs)
