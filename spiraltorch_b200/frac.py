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
    """Spectral fractional derivative: multiply the spectrum by ``(i·omega)^alpha``."""
    n = x.shape[-1]
    omega = 2 * math.pi * torch.fft.fftfreq(n, d=h, device=x.device)
    mult = torch.pow(torch.complex(torch.zeros_like(omega), omega), alpha)
    mult[0] = 0 if alpha > 0 else mult[0]
    return torch.fft.ifft(torch.fft.fft(x.to(torch.complex64)) * mult).real


def fft(x: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    z = x if torch.is_complex(x) else x.to(torch.complex64)
    return torch.fft.ifft(z) if inverse else torch.fft.fft(z)


def mellin_log_grid(f: torch.Tensor, t_min: float, t_max: float, s: complex) -> complex:
    """Mellin transform ``∫ f(t) t^(s-1) dt`` of samples taken on a logarithmic grid
    (trapezoid rule in ``log t``; crates/st-frac/src/mellin.rs:647)."""
    n = f.shape[-1]
    logt = torch.linspace(math.log(t_min), math.log(t_max), n, dtype=torch.float64)
    integrand = f.to(torch.complex128) * torch.exp(torch.complex(logt * s.real, logt * s.imag))
    val = torch.trapezoid(integrand, logt)
    return complex(val)
