"""Spectral ops on the repo's own kernels (``csrc/spectral/spectral.cu``): batched 1-D FFT along any dimension,
spectral multipliers of the fractional operators, window tables and the temporal volume renderer.

Reference parity: `st_frac::fft::fft_inplace` (crates/st-frac/src/fft.rs:122-150: forward sign -1, inverse scaled by
1/n), the direct-DFT fallback for other lengths and the canvas windows (crates/st-tensor/src/pure/wasm_canvas.rs:
233-265, 2837-2870), `wgpu_frac_specmul.wgsl` (fractional-Laplacian envelope ``min(col, cols-1-col)^power``), and the
temporal renderer (crates/st-backend-wgpu/src/render/temporal.rs:252-360).

CUDA tensors take the kernels: a transform of length ``n`` (a power of two up to 8192, any other length up to 4096)
runs inside one CTA's shared memory, so a batch costs one read and one write of the data; strides are passed to the
kernel, so transforming along a non-innermost dimension or picking one channel of an interleaved field needs no
transposition pass.  CPU tensors (and lengths above the shared-memory capacity) use ``torch.fft`` with the same
conventions; that path is also the numerical oracle of the tests.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import native

launch_count = 0
WINDOWS = ("rectangular", "hann", "hamming", "blackman")


class _FftArgs(ctypes.Structure):
    _fields_ = [("inp", ctypes.c_void_p), ("out", ctypes.c_void_p), ("window", ctypes.c_void_p),
                ("in_b0", ctypes.c_longlong), ("in_b1", ctypes.c_longlong), ("in_i", ctypes.c_longlong),
                ("out_b0", ctypes.c_longlong), ("out_b1", ctypes.c_longlong), ("out_i", ctypes.c_longlong),
                ("n", ctypes.c_int), ("batch0", ctypes.c_int), ("batch1", ctypes.c_int),
                ("complex_in", ctypes.c_int), ("inverse", ctypes.c_int)]


def window_coefficients(kind: str, n: int, device=None) -> torch.Tensor:
    """``n`` window samples over ``ratio = i / (n - 1)``: Hann ``0.5 - 0.5 cos(2 pi r)``, Hamming ``0.54 - 0.46 cos``,
    Blackman ``0.42 - 0.5 cos(2 pi r) + 0.08 cos(4 pi r)``; length 0 / 1 windows are all ones."""
    kind = kind.lower()
    if kind not in WINDOWS:
        raise ValueError(f"unknown window '{kind}', expected one of {WINDOWS}")
    if n <= 1 or kind == "rectangular":
        return torch.ones(max(n, 0), device=device)
    r = torch.arange(n, dtype=torch.float32, device=device) / (n - 1)
    c = torch.cos(2 * math.pi * r)
    if kind == "hann":
        return 0.5 - 0.5 * c
    if kind == "hamming":
        return 0.54 - 0.46 * c
    return 0.42 - 0.5 * c + 0.08 * torch.cos(4 * math.pi * r)


def _supported(n: int) -> bool:
    pow2 = n & (n - 1) == 0
    return n <= (8192 if pow2 else 4096)


def _launch(inp, out, window, n, batch0, batch1, in_strides, out_strides, complex_in, inverse) -> None:
    global launch_count
    a = _FftArgs(native.ptr(inp).value, native.ptr(out).value, None if window is None else native.ptr(window).value,
                 in_strides[0], in_strides[1], in_strides[2], out_strides[0], out_strides[1], out_strides[2],
                 n, batch0, batch1, int(complex_in), int(inverse))
    native.check(native.lib().st_fft_1d(ctypes.byref(a), native.stream_ptr(inp.device)), "st_fft_1d")
    launch_count += 1


def fft(x: torch.Tensor, dim: int = -1, inverse: bool = False, window: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Complex FFT of ``x`` (real or complex) along ``dim``; forward uses ``exp(-2 pi i k n / N)``, the inverse is
    scaled by ``1/N``.  ``window`` (``N`` real samples) multiplies the input first."""
    dim = dim % x.dim()
    n = x.shape[dim]
    if n == 0:
        raise ValueError("fft of an empty dimension")
    if window is not None and window.numel() != n:
        raise ValueError(f"window has {window.numel()} samples, the transform has {n}")
    cplx = torch.is_complex(x)
    if not (x.is_cuda and native.available() and _supported(n)) or x.dtype in (torch.complex128, torch.float64):
        z = x if cplx else x.to(torch.complex64)
        if window is not None:
            shape = [1] * x.dim()
            shape[dim] = n
            z = z * window.to(z.real.dtype).reshape(shape)
        return torch.fft.ifft(z, dim=dim) if inverse else torch.fft.fft(z, dim=dim)
    src = x.to(torch.complex64) if cplx else x.float()
    src = src.movedim(dim, -1)
    lead = src.shape[:-1]
    src = src.reshape(-1, n).contiguous()                       # a view when dim is innermost; one gather otherwise
    raw = torch.view_as_real(src) if cplx else src
    out = torch.empty(src.shape[0], n, dtype=torch.complex64, device=x.device)
    step = 2 if cplx else 1
    w = None if window is None else window.to(x.device, torch.float32).contiguous()
    _launch(raw, torch.view_as_real(out), w, n, src.shape[0], 1, (n * step, 0, step), (2 * n, 0, 2), cplx, inverse)
    return out.reshape(*lead, n).movedim(-1, dim)


def fft_field_interleaved(field: torch.Tensor, axis: str, inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
    """Per-channel FFT of a real vector field ``[H, W, C]`` along its rows (``axis='row'``, over W) or columns
    (``'col'``, over H).  Returns ``[H, W, 2C]`` with ``(re, im)`` of channel ``c`` at ``2c, 2c + 1`` — the canvas
    layout.  The kernel reads each channel with the field's own strides and writes the interleaved layout directly."""
    if field.dim() != 3:
        raise ValueError(f"vector field must be [H, W, C], got {tuple(field.shape)}")
    if axis not in ("row", "col"):
        raise ValueError("axis is 'row' or 'col'")
    H, W, C = field.shape
    n = W if axis == "row" else H
    win = None if window is None else window_coefficients(window, n, field.device)
    f = field.float().contiguous()
    if not (f.is_cuda and native.available() and _supported(n)):
        z = f.to(torch.complex64)
        d = 1 if axis == "row" else 0
        if win is not None:
            z = z * (win.reshape(1, W, 1) if axis == "row" else win.reshape(H, 1, 1))
        z = torch.fft.ifft(z, dim=d) if inverse else torch.fft.fft(z, dim=d)
        return torch.view_as_real(z).reshape(H, W, 2 * C)
    out = torch.empty(H, W, 2 * C, device=f.device)
    if axis == "row":       # batch0 = row, batch1 = channel, element = column
        _launch(f, out, win, W, H, C, (W * C, 1, C), (W * 2 * C, 2, 2 * C), False, inverse)
    else:                   # batch0 = column, batch1 = channel, element = row
        _launch(f, out, win, H, W, C, (C, 1, W * C), (2 * C, 2, W * 2 * C), False, inverse)
    return out


def specmul_frac_laplace(spectrum: torch.Tensor, power: float) -> torch.Tensor:
    """Multiplies a ``[rows, cols]`` complex spectrum by ``min(col, cols - 1 - col) ** power``."""
    return _specmul(spectrum, power, 1.0, 0)


def specmul_frac_derivative(spectrum: torch.Tensor, alpha: float, h: float = 1.0) -> torch.Tensor:
    """Multiplies by ``(i omega) ** alpha`` with ``omega = 2 pi fftfreq(cols, h)``; the zero frequency becomes 0 for
    ``alpha > 0``."""
    if not h > 0:
        raise ValueError("sample spacing must be positive")
    return _specmul(spectrum, alpha, h, 1)


def _specmul(spectrum: torch.Tensor, power: float, h: float, mode: int) -> torch.Tensor:
    global launch_count
    if not math.isfinite(power):
        raise ValueError("spectral power must be finite")
    z = spectrum if torch.is_complex(spectrum) else spectrum.to(torch.complex64)
    cols = z.shape[-1]
    if z.numel() == 0:
        raise ValueError("empty spectrum")
    if not (z.is_cuda and native.available()) or z.dtype != torch.complex64:
        col = torch.arange(cols, device=z.device)
        if mode == 0:
            mult = torch.minimum(col, cols - 1 - col).clamp(min=0).to(z.real.dtype) ** power
            return z * mult
        omega = 2 * math.pi * torch.fft.fftfreq(cols, d=h, device=z.device).to(z.real.dtype)
        mult = torch.pow(torch.complex(torch.zeros_like(omega), omega), power)
        if power > 0:
            mult[0] = 0
        return z * mult
    zc = z.contiguous()
    out = torch.empty_like(zc)
    st = native.lib().st_specmul(native.ptr(torch.view_as_real(zc)), native.ptr(torch.view_as_real(out)),
                                 ctypes.c_longlong(zc.numel() // cols), ctypes.c_int(cols), ctypes.c_float(power),
                                 ctypes.c_float(h), ctypes.c_int(mode), native.stream_ptr(zc.device))
    native.check(st, "st_specmul")
    launch_count += 1
    return out


def temporal_render(voxels: torch.Tensor, harmonics: Optional[torch.Tensor], decay: torch.Tensor, frames: int = 16,
                    sample_rate_hz: float = 24.0) -> torch.Tensor:
    """``out[f, v] = (voxel[v] + sum_c harmonics[v, c] sin(2 pi (c + 1) t_f)) exp(-decay[v] t_f)`` with ``t_f = f /
    sample_rate_hz``; a non-finite decay counts as 1, a negative one as 0, and a zero decay silences the voxel.
    ``voxels`` / ``decay`` have any (equal) shape, ``harmonics`` adds a trailing channel axis (or is ``None``).
    Returns ``[frames, *voxels.shape]``."""
    global launch_count
    if frames <= 0:
        raise ValueError("temporal renderer needs at least one frame")
    if not (math.isfinite(sample_rate_hz) and sample_rate_hz > 0):
        raise ValueError(f"invalid sample rate {sample_rate_hz}")
    if decay.shape != voxels.shape:
        raise ValueError(f"resonance_decay has shape {tuple(decay.shape)}, the volume {tuple(voxels.shape)}")
    channels = 0
    if harmonics is not None and harmonics.numel():
        if harmonics.shape[:-1] != voxels.shape:
            raise ValueError(f"temporal_harmonics has shape {tuple(harmonics.shape)}, expected {tuple(voxels.shape)} + (channels,)")
        channels = harmonics.shape[-1]
    v, d = voxels.float().contiguous(), decay.float().contiguous()
    if v.numel() == 0:
        raise ValueError("empty volume")
    if not (v.is_cuda and native.available()):
        t = torch.arange(frames, dtype=torch.float32, device=v.device) / sample_rate_hz
        base = v.reshape(1, -1).expand(frames, -1).clone()
        if channels:
            h = harmonics.float().reshape(-1, channels)
            h = torch.where(h.abs() > 1.1920929e-07, h, torch.zeros_like(h))
            freq = torch.arange(1, channels + 1, dtype=torch.float32, device=v.device)
            base = base + torch.sin(2 * math.pi * t[:, None] * freq[None, :]) @ h.T
        dd = torch.where(torch.isfinite(d), d.clamp(min=0.0), torch.ones_like(d)).reshape(1, -1)
        out = torch.where(dd <= 1.1920929e-07, torch.zeros_like(base), base * torch.exp(-dd * t[:, None]))
        return out.reshape(frames, *voxels.shape)
    out = torch.empty(frames, v.numel(), device=v.device)
    hp = harmonics.float().contiguous() if channels else None
    st = native.lib().st_temporal_render(native.ptr(v), native.ptr(hp), native.ptr(d), native.ptr(out),
                                         ctypes.c_longlong(v.numel()), ctypes.c_int(channels), ctypes.c_int(frames),
                                         ctypes.c_float(sample_rate_hz), native.stream_ptr(v.device))
    native.check(st, "st_temporal_render")
    launch_count += 1
    return out.reshape(frames, *voxels.shape)
