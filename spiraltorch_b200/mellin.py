"""Mellin transforms on a log-uniform lattice.  With ``x_n = exp(t0 + n h)`` the transform ``M[f](s) = ∫ f(x) x^{s-1} dx``
becomes ``h e^{s t0} Σ_n w_n f_n z^n`` with ``z = e^{s h}``: a weighted Z-transform evaluated at points of the ``s``
plane.  A `MellinEvalPlan` fixes the evaluation points (a list, a vertical line, a rectangular mesh); evaluating a
grid on a plan is one ``[points, samples]`` complex matrix-vector product on the device that holds the samples.

Parity: crates/st-frac/src/zspace.rs — `LogLatticeWindow` (:174-243), `trapezoidal_weights(_windowed)` (:245-291),
`mellin_log_lattice_prefactor` (:293-314), `prepare_weighted_series` / `evaluate_weighted_series*` (:360-470);
crates/st-frac/src/mellin.rs — `sample_log_uniform*` (:43-105), `MellinEvalPlan` (:144-415), `MellinLogGrid`
(:647-1430: evaluation, plans, `l2_loss_grad_plan_match_grid` :978, `train_step_l2_plan_match_grid` :1065,
`hilbert_inner_product` :1398), `mellin_transform` (:1471), `mellin_transform_log_samples` (:1512),
`mellin_l2_inner_product` (:1545).  The reference evaluates each point with a Horner loop (and an optional WGPU
pass per plan, mellin_wgpu.rs); here powers come from ``exp(n s h)`` so every point and sample is independent, and
the "stable" form factors the largest power out before summing.
"""
from __future__ import annotations

import cmath
import math
from typing import Callable, Optional, Sequence, Tuple

import torch

WINDOWS = ("rectangular", "hann", "tukey", "blackman")


class MellinError(ValueError):
    def __init__(self, kind: str, message: str, **details):
        super().__init__(message)
        self.kind, self.details = kind, details


def _check_lattice(log_start: float, log_step: float) -> None:
    if not (math.isfinite(log_step) and log_step > 0.0):
        raise MellinError("invalid_log_step", "log_step must be positive and finite")
    if not math.isfinite(log_start):
        raise MellinError("invalid_log_start", "log_start must be finite")


def _finite(t: torch.Tensor, quantity: str) -> torch.Tensor:
    ok = torch.isfinite(torch.view_as_real(t)).all(-1) if t.is_complex() else torch.isfinite(t)
    if not bool(ok.all()):
        index = int((~ok).reshape(-1).nonzero()[0])
        raise MellinError("non_finite_output", f"{quantity} is not finite at index {index}", quantity=quantity, index=index)
    return t


def apply_window(weights: torch.Tensor, window: str) -> torch.Tensor:
    """Hann / Tukey (alpha 0.5) / Blackman taper over the lattice; lattices of one or two points are left alone."""
    if window not in WINDOWS:
        raise MellinError("window", f"unknown window '{window}', expected one of {WINDOWS}")
    n = weights.shape[0]
    if window == "rectangular" or n <= 2:
        return weights
    x = torch.arange(n, dtype=weights.dtype, device=weights.device) / (n - 1)
    if window == "hann":
        return weights * 0.5 * (1.0 - torch.cos(2 * math.pi * x))
    if window == "blackman":
        return weights * (0.42 - 0.5 * torch.cos(2 * math.pi * x) + 0.08 * torch.cos(4 * math.pi * x))
    alpha = 0.5
    rise = 0.5 * (1.0 + torch.cos(math.pi * (2.0 * x / alpha - 1.0)))
    fall = 0.5 * (1.0 + torch.cos(math.pi * (2.0 * x / alpha - 2.0 / alpha + 1.0)))
    return weights * torch.where(x < alpha / 2, rise, torch.where(x <= 1.0 - alpha / 2, torch.ones_like(x), fall))


def trapezoidal_weights(n: int, window: str = "rectangular", preserve_sum: bool = False, dtype=torch.float64) -> torch.Tensor:
    if n <= 0:
        raise MellinError("empty_samples", "at least one sample is required")
    w = torch.ones(n, dtype=dtype)
    if n > 1:
        w[0] = w[-1] = 0.5
    if window == "rectangular" and not preserve_sum:
        return w
    base = float(w.sum())
    w = apply_window(w, window)
    if preserve_sum and float(w.sum()) > torch.finfo(dtype).eps:
        w = w * (base / float(w.sum()))
    return w


def mellin_log_lattice_prefactor(log_start: float, log_step: float, s: complex) -> Tuple[complex, complex]:
    """``(h e^{s t0}, e^{s h})``."""
    _check_lattice(log_start, log_step)
    s = complex(s)
    if not (math.isfinite(s.real) and math.isfinite(s.imag)):
        raise MellinError("non_finite_abscissa", f"s = {s} is not finite")
    try:
        return cmath.exp(s * log_start) * log_step, cmath.exp(s * log_step)
    except OverflowError:
        raise MellinError("non_finite_output", "Mellin prefactor is not finite", quantity="Mellin prefactor", index=0)


def _complex(x, device=None) -> torch.Tensor:
    if not isinstance(x, torch.Tensor):
        return torch.as_tensor(x, dtype=torch.complex128, device=device)
    x = x if device is None else x.to(device)
    return x.to(torch.complex128 if x.dtype in (torch.float64, torch.complex128) else torch.complex64)


def prepare_weighted_series(samples, weights) -> torch.Tensor:
    s = _complex(samples)
    w = torch.as_tensor(weights, device=s.device)
    if s.dim() != 1 or s.numel() == 0:
        raise MellinError("empty_samples", "samples must be a non-empty vector")
    if w.shape != s.shape:
        raise MellinError("weight_length_mismatch", f"{s.numel()} samples but {w.numel()} weights")
    if not bool(torch.isfinite(w).all()):
        raise MellinError("non_finite_weight", "weights must be finite")
    if not bool(torch.isfinite(torch.view_as_real(s)).all()):
        raise MellinError("non_finite_sample", "samples must be finite", index=int((~torch.isfinite(torch.view_as_real(s)).all(-1)).nonzero()[0]))
    return _finite(s * w.to(s.real.dtype), "weighted coefficient")


def _series(weighted: torch.Tensor, log_z: torch.Tensor, stable: bool, derivative: bool):
    """``Σ_n c_n z^n`` (and ``d/dz``) at ``z = exp(log_z)`` for every entry of ``log_z``."""
    n = torch.arange(weighted.shape[0], dtype=weighted.real.dtype, device=weighted.device)
    expo = log_z.reshape(-1, 1) * n                                      # [points, samples]
    if stable:        # log-sum-exp over the terms c_n z^n: no single power or coefficient has to be representable on its own
        def lse(coeff):
            live = coeff != 0
            logc = torch.log(torch.where(live, coeff, torch.ones_like(coeff)))
            terms = expo + logc
            real = torch.where(live, terms.real, torch.full_like(terms.real, -float("inf")))
            shift = real.amax(1, keepdim=True)
            shift = torch.where(torch.isfinite(shift), shift, torch.zeros_like(shift))
            body = torch.where(live, torch.exp(terms - shift), torch.zeros_like(terms)).sum(1)
            return body * torch.exp(shift.squeeze(1)).to(body.dtype)
        value = lse(weighted)
        deriv = lse(weighted * n) * torch.exp(-log_z.reshape(-1)) if derivative else None
    else:
        powers = torch.exp(expo)
        value = powers @ weighted
        deriv = (powers @ (weighted * n)) * torch.exp(-log_z.reshape(-1)) if derivative else None   # Σ n c_n z^{n-1}
    return value.reshape(log_z.shape), (None if deriv is None else deriv.reshape(log_z.shape))


def weighted_z_transform(samples, weights, z, *, derivative: bool = False):
    """``Σ_n w_n f_n z^n`` at one or many ``z`` (a tensor in, a tensor out; a scalar in, a complex out)."""
    weighted = prepare_weighted_series(samples, weights)
    zt = _complex(z, weighted.device).to(weighted.dtype)
    if not bool(torch.isfinite(torch.view_as_real(zt)).all()):
        raise MellinError("non_finite_z", "z must be finite")
    # z = 0 has no logarithm: the series is its constant term there
    safe = torch.where(zt == 0, torch.ones_like(zt), zt)
    value, deriv = _series(weighted, torch.log(safe), False, derivative)
    zero = zt == 0
    value = torch.where(zero, weighted[0], value)
    if derivative:
        deriv = torch.where(zero, weighted[1] if weighted.numel() > 1 else torch.zeros_like(weighted[0]), deriv)
    scalar = not isinstance(z, torch.Tensor) and zt.dim() == 0
    _finite(value, "series value")
    if derivative:
        _finite(deriv, "series derivative")
        return (complex(value), complex(deriv)) if scalar else (value, deriv)
    return complex(value) if scalar else value


class MellinEvalPlan:
    """Evaluation points of the ``s`` plane for one lattice, with their prefactors ``h e^{s t0}`` and ``log z = s h``."""

    def __init__(self, log_start: float, log_step: float, s_values: torch.Tensor, shape: Tuple[int, int]):
        _check_lattice(log_start, log_step)
        self.log_start, self.log_step, self.shape = float(log_start), float(log_step), shape
        self.s = s_values.reshape(-1).to(torch.complex128)
        if self.s.numel() and not bool(torch.isfinite(torch.view_as_real(self.s)).all()):
            raise MellinError("non_finite_abscissa", "evaluation points must be finite")
        self.log_z = self.s * self.log_step
        self.prefactors = _finite(torch.exp(self.s * self.log_start) * self.log_step, "Mellin prefactor") if self.s.numel() else self.s
        self.z_points = _finite(torch.exp(self.log_z), "Z-plane mapping") if self.s.numel() else self.s

    @classmethod
    def many(cls, log_start: float, log_step: float, s_values) -> "MellinEvalPlan":
        s = torch.as_tensor(s_values, dtype=torch.complex128).reshape(-1)
        return cls(log_start, log_step, s, (1, s.numel()) if s.numel() else (0, 0))

    @classmethod
    def vertical_line(cls, log_start: float, log_step: float, real: float, imag_values) -> "MellinEvalPlan":
        im = torch.as_tensor(imag_values, dtype=torch.float64).reshape(-1)
        return cls(log_start, log_step, torch.complex(torch.full_like(im, float(real)), im), (1, im.numel()) if im.numel() else (0, 0))

    @classmethod
    def mesh(cls, log_start: float, log_step: float, real_values, imag_values) -> "MellinEvalPlan":
        re = torch.as_tensor(real_values, dtype=torch.float64).reshape(-1)
        im = torch.as_tensor(imag_values, dtype=torch.float64).reshape(-1)
        if not re.numel() or not im.numel():
            return cls(log_start, log_step, torch.zeros(0, dtype=torch.complex128), (0, 0))
        return cls(log_start, log_step, torch.complex(re[:, None].expand(-1, im.numel()), im[None, :].expand(re.numel(), -1)), (re.numel(), im.numel()))

    def __len__(self) -> int:
        return self.s.numel()

    def is_empty(self) -> bool:
        return self.s.numel() == 0

    def _run(self, weighted: torch.Tensor, stable: bool, derivative: bool):
        if weighted.dim() != 1 or weighted.numel() == 0:
            raise MellinError("empty_series", "the weighted series is empty")
        w = weighted.to(torch.complex128)
        dev = w.device
        value, dz = _series(w, self.log_z.to(dev), stable, derivative)
        pre = self.prefactors.to(dev)
        out = _finite(value * pre, "Mellin value")
        if not derivative:
            return out, None
        # d/ds [h e^{s t0} P(e^{s h})] = prefactor (t0 P + h z P')
        return out, _finite(pre * (self.log_start * value + self.log_step * self.z_points.to(dev) * dz), "Mellin derivative")

    def evaluate(self, weighted: torch.Tensor) -> torch.Tensor:
        return self._run(weighted, False, False)[0] if len(self) else torch.zeros(0, dtype=torch.complex128)

    def evaluate_stable(self, weighted: torch.Tensor) -> torch.Tensor:
        return self._run(weighted, True, False)[0] if len(self) else torch.zeros(0, dtype=torch.complex128)

    def evaluate_with_derivative(self, weighted: torch.Tensor, stable: bool = False):
        if not len(self):
            z = torch.zeros(0, dtype=torch.complex128)
            return z, z
        return self._run(weighted, stable, True)

    def evaluate_magnitude(self, weighted: torch.Tensor) -> torch.Tensor:
        return self.evaluate(weighted).abs()

    def evaluate_log_magnitude(self, weighted: torch.Tensor, epsilon: float = 0.0) -> torch.Tensor:
        mag = self.evaluate_magnitude(weighted)
        return _finite(torch.log(mag + epsilon) if math.isfinite(epsilon) and epsilon > 0.0 else torch.log1p(mag), "Mellin log magnitude")


def sample_log_uniform(log_start: float, log_step: float, n: int, f: Callable) -> torch.Tensor:
    """``f`` at ``x_k = exp(log_start + k log_step)``; ``f`` takes the tensor of abscissae (or, failing that, one float)."""
    if n <= 0:
        raise MellinError("empty_samples", "at least one sample is required")
    _check_lattice(log_start, log_step)
    x = torch.exp(log_start + log_step * torch.arange(n, dtype=torch.float64))
    try:
        v = f(x)
        v = torch.as_tensor(v)
        if v.shape != x.shape:
            raise TypeError
    except (TypeError, ValueError, RuntimeError):
        v = torch.tensor([complex(f(float(xi))) for xi in x])
    v = v.to(torch.complex128)
    if not bool(torch.isfinite(torch.view_as_real(v)).all()):
        raise MellinError("non_finite_sample", "the sampled function is not finite", index=int((~torch.isfinite(torch.view_as_real(v)).all(-1)).nonzero()[0]))
    return v


def sample_log_uniform_exp_decay(log_start: float, log_step: float, n: int, rate: float = 1.0) -> torch.Tensor:
    if not (math.isfinite(rate) and rate > 0.0):
        raise MellinError("invalid_rate", "rate must be positive and finite")
    return sample_log_uniform(log_start, log_step, n, lambda x: torch.exp(-rate * x))


class MellinLogGrid:
    """Samples of a function on a log-uniform lattice with quadrature weights; the object the Mellin transform, the
    Hilbert inner product ``<f, g> = h Σ w conj(f) g`` and the plan-matching trainer act on."""

    def __init__(self, log_start: float, log_step: float, samples, window: str = "rectangular", preserve_sum: bool = False):
        _check_lattice(log_start, log_step)
        s = torch.as_tensor(samples)
        s = s.to(torch.complex128)
        if s.dim() != 1 or s.numel() == 0:
            raise MellinError("empty_samples", "at least one sample is required")
        self.log_start, self.log_step = float(log_start), float(log_step)
        self.samples = s
        self.weights = trapezoidal_weights(s.numel(), window, preserve_sum).to(s.device)
        self.weighted = prepare_weighted_series(s, self.weights)

    new_with_window = classmethod(lambda cls, log_start, log_step, samples, window, preserve_sum=False:
                                  cls(log_start, log_step, samples, window, preserve_sum))

    @classmethod
    def from_function(cls, log_start: float, log_step: float, n: int, f: Callable, window: str = "rectangular",
                      preserve_sum: bool = False) -> "MellinLogGrid":
        return cls(log_start, log_step, sample_log_uniform(log_start, log_step, n, f), window, preserve_sum)

    def to(self, device) -> "MellinLogGrid":
        self.samples, self.weights, self.weighted = self.samples.to(device), self.weights.to(device), self.weighted.to(device)
        return self

    def __len__(self) -> int:
        return self.samples.numel()

    def support(self) -> Tuple[float, float]:
        return math.exp(self.log_start), math.exp(self.log_start + self.log_step * (len(self) - 1))

    def weighted_series(self) -> torch.Tensor:
        return self.weighted.clone()

    # ---- plans ----------------------------------------------------------------------------------------------------------
    def plan_many(self, s_values) -> MellinEvalPlan:
        return MellinEvalPlan.many(self.log_start, self.log_step, s_values)

    def plan_vertical_line(self, real: float, imag_values) -> MellinEvalPlan:
        return MellinEvalPlan.vertical_line(self.log_start, self.log_step, real, imag_values)

    def plan_mesh(self, real_values, imag_values) -> MellinEvalPlan:
        return MellinEvalPlan.mesh(self.log_start, self.log_step, real_values, imag_values)

    def _check_plan(self, plan: MellinEvalPlan) -> None:
        if plan.log_start != self.log_start or plan.log_step != self.log_step:
            raise MellinError("lattice_mismatch", "the plan was built for another lattice")

    def evaluate_plan(self, plan: MellinEvalPlan, *, stable: bool = False) -> torch.Tensor:
        self._check_plan(plan)
        return plan.evaluate_stable(self.weighted) if stable else plan.evaluate(self.weighted)

    def evaluate_plan_with_derivative(self, plan: MellinEvalPlan, *, stable: bool = False):
        self._check_plan(plan)
        return plan.evaluate_with_derivative(self.weighted, stable)

    def evaluate_plan_magnitude(self, plan: MellinEvalPlan) -> torch.Tensor:
        self._check_plan(plan)
        return plan.evaluate_magnitude(self.weighted)

    def evaluate_plan_log_magnitude(self, plan: MellinEvalPlan, epsilon: float = 0.0) -> torch.Tensor:
        self._check_plan(plan)
        return plan.evaluate_log_magnitude(self.weighted, epsilon)

    # ---- point / list / line / mesh forms ---------------------------------------------------------------------------------
    def evaluate(self, s: complex, *, stable: bool = False) -> complex:
        return complex(self.evaluate_plan(self.plan_many([complex(s)]), stable=stable)[0])

    def evaluate_stable(self, s: complex) -> complex:
        return self.evaluate(s, stable=True)

    def evaluate_with_derivative(self, s: complex, *, stable: bool = False) -> Tuple[complex, complex]:
        v, d = self.evaluate_plan_with_derivative(self.plan_many([complex(s)]), stable=stable)
        return complex(v[0]), complex(d[0])

    def evaluate_many(self, s_values, *, stable: bool = False) -> torch.Tensor:
        return self.evaluate_plan(self.plan_many(s_values), stable=stable)

    def evaluate_many_with_derivative(self, s_values, *, stable: bool = False):
        return self.evaluate_plan_with_derivative(self.plan_many(s_values), stable=stable)

    def evaluate_magnitude(self, s: complex) -> float:
        return abs(self.evaluate(s))

    def evaluate_many_magnitude(self, s_values) -> torch.Tensor:
        return self.evaluate_many(s_values).abs()

    def evaluate_vertical_line(self, real: float, imag_values) -> torch.Tensor:
        return self.evaluate_plan(self.plan_vertical_line(real, imag_values))

    def evaluate_vertical_line_magnitude(self, real: float, imag_values) -> torch.Tensor:
        return self.evaluate_vertical_line(real, imag_values).abs()

    def evaluate_vertical_line_log_magnitude(self, real: float, imag_values, epsilon: float = 0.0) -> torch.Tensor:
        return self.evaluate_plan_log_magnitude(self.plan_vertical_line(real, imag_values), epsilon)

    def evaluate_mesh(self, real_values, imag_values) -> torch.Tensor:
        plan = self.plan_mesh(real_values, imag_values)
        return self.evaluate_plan(plan).reshape(plan.shape)

    def evaluate_mesh_magnitude(self, real_values, imag_values) -> torch.Tensor:
        return self.evaluate_mesh(real_values, imag_values).abs()

    def evaluate_mesh_log_magnitude(self, real_values, imag_values, epsilon: float = 0.0) -> torch.Tensor:
        plan = self.plan_mesh(real_values, imag_values)
        return self.evaluate_plan_log_magnitude(plan, epsilon).reshape(plan.shape)

    # ---- Hilbert structure --------------------------------------------------------------------------------------------------
    def _same_lattice(self, other: "MellinLogGrid") -> None:
        if self.log_start != other.log_start or self.log_step != other.log_step:
            raise MellinError("lattice_mismatch", "grids live on different lattices")
        if len(self) != len(other):
            raise MellinError("sample_length_mismatch", f"expected {len(self)} samples, got {len(other)}")

    def hilbert_inner_product(self, other: "MellinLogGrid") -> complex:
        self._same_lattice(other)
        return complex(_finite((self.samples.conj() * other.samples.to(self.samples.device) * self.weights).sum() * self.log_step,
                               "Hilbert inner product"))

    def hilbert_norm(self) -> float:
        ip = self.hilbert_inner_product(self)
        if ip.real < -1e-6:
            raise MellinError("negative_inner_product", f"<f, f> = {ip}")
        return math.sqrt(max(ip.real, 0.0))

    # ---- plan matching ------------------------------------------------------------------------------------------------------
    def l2_loss_grad_plan_match_grid(self, plan: MellinEvalPlan, target: "MellinLogGrid"):
        """Mean squared distance between this grid's and the target's transform over the plan's points, and its gradient
        with respect to the (complex) samples: ``2/P Σ_p conj(pref_p) err_p conj(z_p)^n w_n``."""
        self._check_plan(plan)
        self._same_lattice(target)
        n = len(self)
        if not len(plan):
            return 0.0, torch.zeros(n, dtype=torch.complex128, device=self.samples.device)
        dev = self.samples.device
        idx = torch.arange(n, dtype=torch.float64, device=dev)
        powers = torch.exp(plan.log_z.to(dev).reshape(-1, 1) * idx)                       # [P, n]
        err = _finite((powers @ (self.weighted - target.weighted.to(dev))) * plan.prefactors.to(dev), "Mellin training error")
        loss = float((err.abs() ** 2).sum()) / len(plan)
        grad = (powers.conj().T @ (err * plan.prefactors.to(dev).conj())) * self.weights * (2.0 / len(plan))
        if not math.isfinite(loss):
            raise MellinError("non_finite_output", "Mellin training loss is not finite", quantity="Mellin training loss", index=0)
        return loss, _finite(grad, "Mellin training gradient")

    def train_step_l2_plan_match_grid(self, plan: MellinEvalPlan, target: "MellinLogGrid", lr: float) -> float:
        if not (math.isfinite(lr) and lr > 0.0):
            raise MellinError("invalid_learning_rate", "learning rate must be positive and finite")
        loss, grad = self.l2_loss_grad_plan_match_grid(plan, target)
        nxt = _finite(self.samples - lr * grad, "Mellin training sample")
        self.samples, self.weighted = nxt, prepare_weighted_series(nxt, self.weights)
        return loss


def mellin_transform(f: Callable, s: complex, value_range: Tuple[float, float], steps: int) -> complex:
    """Trapezoid rule in ``t = log x`` with ``steps`` intervals over ``[a, b]``."""
    if steps < 2:
        raise MellinError("insufficient_samples", "at least two steps are required")
    a, b = value_range
    if not (a > 0.0 and b > a and math.isfinite(b)):
        raise MellinError("invalid_range", "the range must satisfy 0 < a < b < inf")
    h = (math.log(b) - math.log(a)) / steps
    grid = MellinLogGrid.from_function(math.log(a), h, steps + 1, f)
    return grid.evaluate(s)


def mellin_transform_log_samples(log_start: float, log_step: float, samples, s: complex) -> complex:
    if len(samples) < 2:
        raise MellinError("insufficient_samples" if len(samples) else "empty_samples", "at least two samples are required")
    return MellinLogGrid(log_start, log_step, samples).evaluate(s)


def mellin_l2_inner_product(f: Callable, g: Callable, value_range: Tuple[float, float], steps: int) -> complex:
    if steps < 2:
        raise MellinError("insufficient_samples", "at least two steps are required")
    a, b = value_range
    if not (a > 0.0 and b > a and math.isfinite(b)):
        raise MellinError("invalid_range", "the range must satisfy 0 < a < b < inf")
    h = (math.log(b) - math.log(a)) / steps
    return MellinLogGrid.from_function(math.log(a), h, steps + 1, f).hilbert_inner_product(MellinLogGrid.from_function(math.log(a), h, steps + 1, g))
