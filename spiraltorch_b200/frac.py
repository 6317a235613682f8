"""Fractional calculus helpers: Grünwald–Letnikov coefficients and stencil, spectral fractional
derivative, radix FFT front-end and Mellin log-grid transform.

Reference parity: crates/st-frac (``gl_coeffs``, ``fracdiff_gl_1d``, ``fft``, ``mellin``) and the
shaders ``frac_gl_1d.wgsl`` / ``wgpu_fracdiff_gl.wgsl`` / ``wgpu_frac_specmul.wgsl``.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .ops import native

launch_count = 0


def gl_coeffs(alpha: float, m: int) -> torch.Tensor:
    """w_0 = 1, w_k = w_{k-1} * (1 - (alpha + 1) / k) = (-1)^k C(alpha, k)."""
    w = [1.0]
    for k in range(1, m + 1):
        w.append(w[-1] * (1.0 - (alpha + 1.0) / k))
    return torch.tensor(w, dtype=torch.float32)


def fracdiff_gl(x: torch.Tensor, alpha: float, h: float = 1.0, m: int | None = None) -> torch.Tensor:
    """Row-wise GL fractional derivative: ``y[i] = sum_{k<=min(i,m)} w[k] x[i-k] / h^alpha``."""
    global launch_count
    squeeze = x.dim() == 1
    x2 = (x[None, :] if squeeze else x).float().contiguous()
    rows, n = x2.shape
    m = n - 1 if m is None else min(m, n - 1)
    w = gl_coeffs(alpha, m).to(x2.device)
    h_alpha = float(h) ** alpha
    if not native.use_native(x2) or m > 8191:
        idx = torch.arange(n, device=x2.device)
        y = torch.zeros_like(x2)
        for k in range(m + 1):
            y[:, k:] += w[k] * x2[:, : n - k]
        y = y / h_alpha
    else:
        y = torch.empty_like(x2)
        st = native.lib().st_frac_gl(native.ptr(x2), native.ptr(w), native.ptr(y), ctypes.c_int(rows), ctypes.c_int(n),
                                     ctypes.c_int(m), ctypes.c_float(h_alpha), native.stream_ptr(x2.device))
        native.check(st, "st_frac_gl")
        launch_count += 1
    return y[0] if squeeze else y


def fracdiff_spectral(x: torch.Tensor, alpha: float, h: float = 1.0) -> torch.Tensor:
    """Spectral fractional derivative: FFT, multiply the spectrum by ``(i·omega)^alpha``, inverse FFT.  On CUDA all
    three steps are this library's kernels (shared-memory FFT and the spectral multiplier)."""
    from .ops import spectral
    spec = spectral.specmul_frac_derivative(spectral.fft(x), alpha, h)
    return spectral.fft(spec, inverse=True).real


def fft(x: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    from .ops import spectral
    return spectral.fft(x, inverse=inverse)


def specmul_frac_laplace(spectrum: torch.Tensor, power: float) -> torch.Tensor:
    """Fractional-Laplacian frequency envelope ``min(col, cols - 1 - col)^power`` on an FFT's coefficients
    (crates/st-core/src/backend/wgpu_frac.rs:491-500)."""
    from .ops import spectral
    return spectral.specmul_frac_laplace(spectrum, power)


def mellin_log_grid(f: torch.Tensor, t_min: float, t_max: float, s: complex) -> complex:
    """Mellin transform ``∫ f(t) t^(s-1) dt`` of samples taken on a logarithmic grid
    (trapezoid rule in ``log t``; crates/st-frac/src/mellin.rs:647)."""
    n = f.shape[-1]
    logt = torch.linspace(math.log(t_min), math.log(t_max), n, dtype=torch.float64)
    integrand = f.to(torch.complex128) * torch.exp(torch.complex(logt * s.real, logt * s.imag))
    val = torch.trapezoid(integrand, logt)
    return complex(val)


# ----------------------------------------------------------------------------------------------
# Scale stacks: interface persistence of a field across neighbourhood radii
# (crates/st-frac/src/scale_stack.rs:144-365)
# ----------------------------------------------------------------------------------------------


def _ball_offsets(ndim: int, radius: int):
    import itertools
    return [o for o in itertools.product(range(-radius, radius + 1), repeat=ndim)
            if sum(d * d for d in o) <= radius * radius]


def _shifted(field: torch.Tensor, offset, fill: float) -> torch.Tensor:
    """``out[i] = field[i + offset]`` with ``fill`` where the neighbour falls outside the field."""
    out = torch.full_like(field, fill)
    src, dst = [], []
    for d, n in zip(offset, field.shape):
        if abs(d) >= n:
            return out
        dst.append(slice(max(0, -d), n - max(0, d)))
        src.append(slice(max(0, d), n - max(0, -d)))
    out[tuple(dst)] = field[tuple(src)]
    return out


def detect_interfaces(field: torch.Tensor, radius: int, threshold: float) -> torch.Tensor:
    """True where the field's range over the Euclidean ball of ``radius`` exceeds ``threshold``."""
    f = field.float()
    hi = torch.full_like(f, -math.inf)
    lo = torch.full_like(f, math.inf)
    for off in _ball_offsets(f.dim(), radius):
        hi = torch.maximum(hi, _shifted(f, off, -math.inf))
        lo = torch.minimum(lo, _shifted(f, off, math.inf))
    return (hi - lo) > threshold


def detect_semantic_interfaces(field: torch.Tensor, radius: int, threshold: float, feature_axis: int,
                               metric: str = "euclidean") -> torch.Tensor:
    """Interfaces of a vector-valued field: some neighbour in the ball differs from the centre by more
    than ``threshold`` under the metric (``euclidean`` distance or ``cosine`` distance)."""
    f = field.float().movedim(feature_axis, -1)
    spatial = f.shape[:-1]
    gate = torch.zeros(spatial, dtype=torch.bool, device=f.device)
    valid_src = torch.ones(spatial, device=f.device)
    for off in _ball_offsets(len(spatial), radius):
        if not any(off):
            continue
        nb = _shifted(f, tuple(off) + (0,), 0.0)
        inside = _shifted(valid_src, off, 0.0) > 0
        if metric == "cosine":
            dist = 1.0 - torch.nn.functional.cosine_similarity(f, nb, dim=-1, eps=1e-12)
        else:
            dist = (f - nb).norm(dim=-1)
        gate |= inside & (dist > threshold)
    return gate


class ScaleStack:
    """Monotone gate fraction per scale and the persistence measure derived from its increments."""

    def __init__(self, threshold: float, samples, mode: str = "scalar"):
        self.threshold, self.samples, self.mode = threshold, list(samples), mode

    @staticmethod
    def _check(scales, threshold):
        if not len(scales):
            raise ValueError("scale list is empty")
        if threshold < 0:
            raise ValueError("threshold must be non-negative")
        if any(s <= 0 for s in scales) or any(b <= a for a, b in zip(scales, scales[1:])):
            raise ValueError("scales must be positive and strictly increasing")

    @classmethod
    def from_scalar_field(cls, field: torch.Tensor, scales, threshold: float) -> "ScaleStack":
        cls._check(scales, threshold)
        samples, prev = [], 0.0
        for s in scales:
            gate = detect_interfaces(field, max(int(math.ceil(s)), 1), threshold)
            prev = max(float(gate.float().mean()) if gate.numel() else 0.0, prev)
            samples.append((float(s), prev))
        return cls(threshold, samples, "scalar")

    @classmethod
    def from_semantic_field(cls, field: torch.Tensor, scales, threshold: float, feature_axis: int,
                            metric: str = "euclidean") -> "ScaleStack":
        cls._check(scales, threshold)
        if not 0 <= feature_axis < field.dim():
            raise ValueError(f"feature axis {feature_axis} out of range for a {field.dim()}-d field")
        if field.shape[feature_axis] == 0:
            raise ValueError("feature axis is empty")
        samples, prev = [], 0.0
        for s in scales:
            gate = detect_semantic_interfaces(field, max(int(math.ceil(s)), 1), threshold, feature_axis, metric)
            prev = max(float(gate.float().mean()) if gate.numel() else 0.0, prev)
            samples.append((float(s), prev))
        return cls(threshold, samples, f"semantic[{feature_axis},{metric}]")

    def persistence_measure(self):
        """``(scale_low, scale_high, mass)`` for every scale interval over which the gate grew."""
        bins, ps, pg = [], 0.0, 0.0
        for s, g in self.samples:
            if g - pg > 0:
                bins.append((ps, s, g - pg))
            ps, pg = s, g
        return bins

    def interface_density(self):
        bins = self.persistence_measure()
        if not bins:
            return None
        lo, hi, mass = bins[0]
        return mass / max(hi - lo, 2.220446049250313e-16)

    def moment(self, order: int) -> float:
        return sum(m * ((0.5 * (hi + lo)) if hi > lo else hi) ** order for lo, hi, m in self.persistence_measure())

    def estimate_boundary_dimension(self, ambient_dim: float, window: int):
        """``ambient_dim − slope`` of log gate fraction against log scale over the first ``window`` samples."""
        if len(self.samples) < 2 or window < 2:
            return None
        eps = 2.220446049250313e-16
        xs, ys = [], []
        for s, g in self.samples[:window]:
            if g <= 0:
                continue
            if g >= 1.0:
                if len(xs) >= 2:
                    break
                g = 1.0 - eps
            xs.append(math.log(max(s, eps)))
            ys.append(math.log(max(g, eps)))
        if len(xs) < 2:
            return None
        mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
        den = sum((x - mx) ** 2 for x in xs)
        if den <= eps:
            return None
        return ambient_dim - sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den

    def coherence_break_scale(self, level: float):
        if not 0.0 <= level <= 1.0:
            return None
        return next((s for s, g in self.samples if g >= level), None)

    def coherence_profile(self, levels):
        return [self.coherence_break_scale(l) for l in levels]


class FractalFieldGenerator:
    """Octave sum of escape-time samples on a log lattice (crates/st-frac/src/fractal_field.rs:52-180):
    per octave ``c = exp(i·x·f)``, ``escape`` = normalised Mandelbrot escape count of ``c``, weight
    ``escape · exp(−(x·f)²/2) · amplitude``; frequencies grow by ``lacunarity``, amplitudes by ``gain``."""

    def __init__(self, octaves: int, lacunarity: float, gain: float, iterations: int):
        if octaves < 1:
            raise ValueError("octave count must be at least 1")
        if not (math.isfinite(lacunarity) and lacunarity > 1.0):
            raise ValueError("lacunarity must be > 1.0")
        if not (math.isfinite(gain) and gain > 0.0):
            raise ValueError("gain must be positive")
        if iterations < 1:
            raise ValueError("iteration count must be at least 1")
        self.octaves, self.lacunarity, self.gain, self.iterations = octaves, lacunarity, gain, iterations

    def branching_field(self, log_start: float, log_step: float, length: int, device=None) -> torch.Tensor:
        if not math.isfinite(log_start):
            raise ValueError("log_start must be finite")
        if not (math.isfinite(log_step) and log_step > 0):
            raise ValueError("log_step must be positive")
        if length < 1:
            raise ValueError("lattice is empty")
        coord = log_start + log_step * torch.arange(length, dtype=torch.float32, device=device)
        total = torch.zeros(length, dtype=torch.complex64, device=device)
        freq, amp, norm = 1.0, 1.0, 0.0
        for _ in range(self.octaves):
            angle = coord * freq
            c = torch.complex(torch.cos(angle), torch.sin(angle))
            z = torch.zeros_like(c)
            escape = torch.full((length,), float(self.iterations), device=device)
            alive = torch.ones(length, dtype=torch.bool, device=device)
            for it in range(self.iterations):
                z = torch.where(alive, z * z + c, z)
                out = alive & ((z.real ** 2 + z.imag ** 2) > 4.0)
                escape = torch.where(out, torch.full_like(escape, float(it + 1)), escape)
                alive = alive & ~out
            weight = escape / self.iterations * torch.exp(-0.5 * angle ** 2) * amp
            total = total + c * weight
            norm += amp
            freq *= self.lacunarity
            amp *= self.gain
        return total / norm if norm > 0 else total

    def weave(self, base: torch.Tensor, log_start: float, log_step: float) -> torch.Tensor:
        """Adds the branching field to samples already taken on the same log lattice."""
        return base.to(torch.complex64) + self.branching_field(log_start, log_step, base.shape[-1], base.device)


def gl_coeffs_adaptive(alpha: float, tol: float, max_len: int) -> torch.Tensor:
    """Coefficients up to the first index whose magnitude drops below ``tol`` (at most ``max_len``)."""
    w = [1.0]
    while len(w) < max_len:
        nxt = w[-1] * (1.0 - (alpha + 1.0) / len(w))
        w.append(nxt)
        if abs(nxt) < tol:
            break
    return torch.tensor(w, dtype=torch.float32)


def fracdiff_gl_nd(x: torch.Tensor, alpha: float, axis: int, h: float = 1.0, m: int | None = None) -> torch.Tensor:
    """GL fractional derivative along one axis of an n-d tensor."""
    moved = x.movedim(axis, -1)
    y = fracdiff_gl(moved.reshape(-1, moved.shape[-1]), alpha, h, m)
    return y.reshape(moved.shape).movedim(-1, axis)


def fracdiff_gl_vjp(grad_out: torch.Tensor, alpha: float, h: float = 1.0, m: int | None = None) -> torch.Tensor:
    """Adjoint of :func:`fracdiff_gl` (the anti-causal stencil): ``gx[j] = Σ_k w[k] gy[j+k] / h^α``."""
    return fracdiff_gl(grad_out.flip(-1), alpha, h, m).flip(-1)
