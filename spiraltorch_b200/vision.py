"""Vision stack: image transforms, the fused classification preprocessing pipeline, NeRF volume
rendering and the canvas projector — CUDA kernels in ``csrc/vision/vision.cu`` with PyTorch CPU
statements of the same arithmetic (the test oracle).

Reference parity: ``TransformDispatcher`` (crates/st-backend-wgpu/src/transform.rs:281) and the CPU
transforms of ``st-vision``; ``nerf_raymarch.wgsl`` / ``nerf_volume_utils.wgsl`` and the CPU NeRF
trainer (crates/st-vision/src/nerf/trainer.rs); ``CanvasProjector`` (crates/st-tensor/src/pure/
wasm_canvas.rs).  Images are fp32 ``[B, C, H, W]`` (a 3-D ``[C, H, W]`` image is treated as B = 1);
outputs are headless device buffers.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .ops import native

launch_count = 0


class _PreArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("B", "C", "src_h", "src_w", "resize_h", "resize_w", "out_h", "out_w",
                                            "crop_y", "crop_x", "flip", "do_jitter")] + \
               [(n, ctypes.c_float) for n in ("brightness", "contrast", "saturation", "hue")] + \
               [("mean", ctypes.c_float * 4)]


@dataclass
class ColorJitter:
    brightness: float = 1.0
    contrast: float = 1.0
    saturation: float = 1.0
    hue: float = 0.0                      # radians
    means: Optional[Sequence[float]] = None   # per-channel means for the contrast step (image means if None)

    @staticmethod
    def balanced() -> "ColorJitter":
        return ColorJitter(1.1, 1.1, 1.1, 0.05)

    @staticmethod
    def vivid() -> "ColorJitter":
        return ColorJitter(1.25, 1.3, 1.5, 0.15)


def _as4d(img: torch.Tensor):
    if img.dim() == 3:
        return img.unsqueeze(0), True
    if img.dim() != 4:
        raise ValueError("images must be [C,H,W] or [B,C,H,W]")
    return img, False


def _bilinear_ref(img: torch.Tensor, rh: int, rw: int) -> torch.Tensor:
    B, C, sh, sw = img.shape
    sy = (torch.arange(rh, device=img.device, dtype=torch.float32) + 0.5) * (sh / rh) - 0.5
    sx = (torch.arange(rw, device=img.device, dtype=torch.float32) + 0.5) * (sw / rw) - 0.5
    y0 = sy.floor().clamp(0, sh - 1)
    x0 = sx.floor().clamp(0, sw - 1)
    y1 = (y0 + 1).clamp(max=sh - 1).long()
    x1 = (x0 + 1).clamp(max=sw - 1).long()
    ly, lx = (sy - y0)[:, None], (sx - x0)[None, :]
    y0, x0 = y0.long(), x0.long()
    tl, tr = img[:, :, y0][:, :, :, x0], img[:, :, y0][:, :, :, x1]
    bl, br = img[:, :, y1][:, :, :, x0], img[:, :, y1][:, :, :, x1]
    top = tl * (1 - lx) + tr * lx
    bot = bl * (1 - lx) + br * lx
    return top * (1 - ly) + bot * ly


def _jitter_ref(img: torch.Tensor, j: ColorJitter, means) -> torch.Tensor:
    C = img.shape[1]
    out = img * j.brightness
    if j.contrast != 1.0:
        m = torch.tensor([means[min(c, 3)] for c in range(C)], device=img.device).view(1, C, 1, 1)
        out = (out - m) * j.contrast + m
    if C >= 3:
        r, g, b = out[:, 0], out[:, 1], out[:, 2]
        if j.saturation != 1.0:
            gray = r * 0.29899597 + g * 0.587096 + b * 0.11390703
            r, g, b = [(ch - gray) * j.saturation + gray for ch in (r, g, b)]
        if j.hue != 0.0:
            ch, sh = math.cos(j.hue), math.sin(j.hue)
            y = 0.299 * r + 0.587 * g + 0.114 * b
            u = -0.14713 * r - 0.28886 * g + 0.436 * b
            v = 0.615 * r - 0.51499 * g - 0.10001 * b
            up, vp = u * ch - v * sh, u * sh + v * ch
            r, g, b = y + 1.13983 * vp, y - 0.39465 * up - 0.58060 * vp, y + 2.03211 * up
        out = torch.cat([torch.stack([r, g, b], 1), out[:, 3:]], 1)
    return out


def preprocess(img: torch.Tensor, *, resize: Optional[tuple[int, int]] = None, crop: Optional[tuple[int, int]] = None,
               jitter: Optional[ColorJitter] = None, flip: bool = False) -> torch.Tensor:
    """resize → centre crop → colour jitter → horizontal flip; one fused kernel launch on CUDA."""
    global launch_count
    x, squeeze = _as4d(img)
    x = x.float().contiguous()
    B, C, sh, sw = x.shape
    rh, rw = resize if resize else (sh, sw)
    oh, ow = crop if crop else (rh, rw)
    if oh > rh or ow > rw:
        raise ValueError("crop size exceeds the (resized) image")
    cy, cx = (rh - oh) // 2, (rw - ow) // 2
    means = [0.0] * 4
    if jitter is not None:
        if jitter.means is not None:
            means = list(jitter.means) + [0.0] * (4 - len(jitter.means))
        elif jitter.contrast != 1.0:
            mm = (x * jitter.brightness).mean(dim=(0, 2, 3)).tolist()
            means = (mm + [0.0] * 4)[:4]
    if not native.use_native(x):
        y = _bilinear_ref(x, rh, rw) if (rh, rw) != (sh, sw) else x
        y = y[:, :, cy:cy + oh, cx:cx + ow]
        if jitter is not None:
            y = _jitter_ref(y, jitter, means)
        if flip:
            y = y.flip(-1)
        y = y.contiguous()
    else:
        a = _PreArgs()
        a.B, a.C, a.src_h, a.src_w, a.resize_h, a.resize_w = B, C, sh, sw, rh, rw
        a.out_h, a.out_w, a.crop_y, a.crop_x, a.flip = oh, ow, cy, cx, int(flip)
        a.do_jitter = int(jitter is not None)
        j = jitter or ColorJitter()
        a.brightness, a.contrast, a.saturation, a.hue = j.brightness, j.contrast, j.saturation, j.hue
        for i in range(4):
            a.mean[i] = means[i]
        y = torch.empty((B, C, oh, ow), dtype=torch.float32, device=x.device)
        st = native.lib().st_preprocess(native.ptr(x), native.ptr(y), ctypes.byref(a), native.stream_ptr(x.device))
        native.check(st, "st_preprocess")
        launch_count += 1
    return y[0] if squeeze else y


def resize(img, height: int, width: int):
    return preprocess(img, resize=(height, width))


def center_crop(img, height: int, width: int):
    return preprocess(img, crop=(height, width))


def horizontal_flip(img):
    return preprocess(img, flip=True)


def color_jitter(img, jitter: ColorJitter):
    return preprocess(img, jitter=jitter)


def classification_pipeline(img, size: int = 224, resize_to: int = 256, jitter: Optional[ColorJitter] = None,
                            flip: bool = True):
    """The reference's classification preprocessing (docs/performance/transforms.md:59-64)."""
    return preprocess(img, resize=(resize_to, resize_to), crop=(size, size),
                      jitter=jitter or ColorJitter.balanced(), flip=flip)


# ---- NeRF ------------------------------------------------------------------------------------------
def nerf_sample(rays: torch.Tensor, samples: int, stratified: bool = False, seed: int = 0):
    """``rays [R, 8]`` (origin, direction, t_min, t_max) → ``(points [R,S,3], t [R,S], deltas [R,S])``."""
    global launch_count
    R = rays.shape[0]
    rays = rays.float().contiguous()
    if not native.use_native(rays):
        t_min, t_max = rays[:, 6:7], rays[:, 7:8]
        interval = (t_max - t_min).clamp(min=1e-3) / samples
        i = torch.arange(samples, device=rays.device, dtype=torch.float32)[None, :]
        if stratified:
            base = (torch.arange(R, dtype=torch.int64)[:, None] * 9781 + seed * 6271) & 0xFFFFFFFF
            step = (1103515245 * ((base + torch.arange(samples, dtype=torch.int64)[None, :]) & 0xFFFFFFFF) + 12345) & 0xFFFFFFFF
            off = (((step >> 9) & 0x7FFFFF).float() / float(0x7FFFFF)).to(rays.device)
        else:
            off = torch.full((R, samples), 0.5, device=rays.device)
        t = t_min + (i + off.clamp(0, 0.999)) * interval
        nxt = torch.cat([t_min + (i[:, 1:]) * interval, t_max], 1) if samples > 1 else t_max
        deltas = (nxt - t).clamp(min=1e-3)
        pts = rays[:, None, 0:3] + rays[:, None, 3:6] * t[..., None]
        return pts, t, deltas
    pts = torch.empty((R, samples, 3), dtype=torch.float32, device=rays.device)
    t = torch.empty((R, samples), dtype=torch.float32, device=rays.device)
    d = torch.empty_like(t)
    st = native.lib().st_nerf_sample(native.ptr(rays), native.ptr(pts), native.ptr(t), native.ptr(d), ctypes.c_int(R),
                                     ctypes.c_int(samples), ctypes.c_int(int(stratified)), ctypes.c_uint(seed),
                                     native.stream_ptr(rays.device))
    native.check(st, "st_nerf_sample")
    launch_count += 1
    return pts, t, d


def _composite_ref(sigma, rad, deltas, delta_scale):
    alpha = 1 - torch.exp(-sigma.clamp(min=0) * deltas * delta_scale)
    T = torch.cumprod(torch.cat([torch.ones_like(alpha[:, :1]), 1 - alpha[:, :-1]], 1), 1)
    w = T * alpha
    return torch.cat([(w[..., None] * rad).sum(1), w.sum(1, keepdim=True)], 1)


class _Composite(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sigma, rad, deltas, delta_scale):
        global launch_count
        R, S = sigma.shape
        accum = torch.empty((R, 4), dtype=torch.float32, device=sigma.device)
        st = native.lib().st_nerf_composite_fwd(native.ptr(sigma), native.ptr(rad), native.ptr(deltas),
                                                native.ptr(accum), ctypes.c_int(R), ctypes.c_int(S),
                                                ctypes.c_float(delta_scale), native.stream_ptr(sigma.device))
        native.check(st, "st_nerf_composite_fwd")
        launch_count += 1
        ctx.save_for_backward(sigma, rad, deltas, accum)
        ctx.delta_scale = delta_scale
        return accum

    @staticmethod
    def backward(ctx, d_accum):
        global launch_count
        sigma, rad, deltas, accum = ctx.saved_tensors
        R, S = sigma.shape
        ds, dr = torch.empty_like(sigma), torch.empty_like(rad)
        st = native.lib().st_nerf_composite_bwd(native.ptr(sigma), native.ptr(rad), native.ptr(deltas),
                                                native.ptr(accum), native.ptr(d_accum.contiguous().float()),
                                                native.ptr(ds), native.ptr(dr), ctypes.c_int(R), ctypes.c_int(S),
                                                ctypes.c_float(ctx.delta_scale), native.stream_ptr(sigma.device))
        native.check(st, "st_nerf_composite_bwd")
        launch_count += 1
        return ds, dr, None, None


def nerf_composite(sigma: torch.Tensor, radiance: torch.Tensor, deltas: torch.Tensor, delta_scale: float = 1.0):
    """Front-to-back compositing → ``[R, 4]`` (rgb, opacity); differentiable in sigma and radiance."""
    if not native.use_native(sigma):
        return _composite_ref(sigma.float(), radiance.float(), deltas.float(), delta_scale)
    return _Composite.apply(sigma.float().contiguous(), radiance.float().contiguous(), deltas.float().contiguous(),
                            float(delta_scale))


class NerfField(torch.nn.Module):
    """Small MLP radiance field with frequency encoding (crates/st-vision/src/nerf/field.rs)."""

    def __init__(self, hidden: int = 64, frequencies: int = 6, layers: int = 3):
        super().__init__()
        self.frequencies = frequencies
        dims = [3 + 6 * frequencies] + [hidden] * layers
        self.net = torch.nn.Sequential(*[m for a, b in zip(dims[:-1], dims[1:]) for m in (torch.nn.Linear(a, b), torch.nn.ReLU())])
        self.head = torch.nn.Linear(hidden, 4)

    def encode(self, p):
        feats = [p]
        for k in range(self.frequencies):
            feats += [torch.sin((2.0 ** k) * p), torch.cos((2.0 ** k) * p)]
        return torch.cat(feats, -1)

    def forward(self, points):
        out = self.head(self.net(self.encode(points)))
        return out[..., 0], torch.sigmoid(out[..., 1:4])


def nerf_render(field: NerfField, rays: torch.Tensor, samples: int = 32, stratified: bool = False, seed: int = 0):
    pts, _, deltas = nerf_sample(rays, samples, stratified, seed)
    sigma, rad = field(pts)
    return nerf_composite(sigma, rad, deltas)


# ---- canvas ------------------------------------------------------------------------------------------
PALETTES = {"grayscale": 0, "spiral": 1, "diverging": 2}


def canvas_paint(x: torch.Tensor, palette: str = "spiral", lo: Optional[float] = None, hi: Optional[float] = None):
    """Paint a 2-D tensor into an RGBA8 image ``[H, W, 4]`` (uint8), normalising to ``[lo, hi]``."""
    global launch_count
    xf = x.float().contiguous()
    lo = float(xf[torch.isfinite(xf)].min()) if lo is None else lo
    hi = float(xf[torch.isfinite(xf)].max()) if hi is None else hi
    pal = PALETTES[palette]
    if not native.use_native(xf):
        t = ((xf - lo) / (hi - lo) if hi > lo else torch.zeros_like(xf))
        t = torch.where(torch.isfinite(t), t.clamp(0, 1), torch.zeros_like(t))
        if pal == 0:
            r = g = b = t
        elif pal == 1:
            r, g, b = (1.6 * t).clamp(max=1), t * t, (0.35 + 0.9 * (1 - (2 * t - 1).abs())).clamp(max=1)
        else:
            r = torch.where(t < 0.5, 2 * t, torch.ones_like(t))
            b = torch.where(t < 0.5, torch.ones_like(t), 2 * (1 - t))
            g = 1 - (2 * t - 1).abs()
        rgba = torch.stack([r, g, b, torch.ones_like(t)], -1)
        return (rgba * 255 + 0.5).to(torch.uint8)
    out = torch.empty((*xf.shape, 4), dtype=torch.uint8, device=xf.device)
    st = native.lib().st_canvas_paint(native.ptr(xf), native.ptr(out), ctypes.c_longlong(xf.numel()),
                                      ctypes.c_float(lo), ctypes.c_float(hi), ctypes.c_int(pal),
                                      native.stream_ptr(xf.device))
    native.check(st, "st_canvas_paint")
    launch_count += 1
    return out


def canvas_fft(field: torch.Tensor, axis: str = "2d", inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
    """Row / column / 2-D FFT of a (complex or real) field on the shared-memory FFT kernel; ``window`` names a taper
    (``hann`` / ``hamming`` / ``blackman``) applied along each transformed axis."""
    from .ops import spectral
    if axis not in ("row", "col", "2d"):
        raise ValueError("axis is 'row', 'col' or '2d'")
    out = field
    if axis in ("row", "2d"):
        w = None if window is None else spectral.window_coefficients(window, field.shape[-1], field.device)
        out = spectral.fft(out, dim=-1, inverse=inverse, window=w)
    if axis in ("col", "2d"):
        w = None if window is None else spectral.window_coefficients(window, field.shape[-2], field.device)
        out = spectral.fft(out, dim=-2, inverse=inverse, window=w)
    return out


class ColorVectorField:
    """Canvas vector field ``[H, W, 4]``: normalised energy plus three chroma channels per pixel, with the spectral
    views of the canvas projector (crates/st-tensor/src/pure/wasm_canvas.rs:267-1100): per-channel row / column FFTs
    in the interleaved ``[H, W, 8]`` layout and their magnitude, power, dB and phase maps."""

    FFT_INTERLEAVED_STRIDE = 8
    POWER_DB_EPSILON = 1e-12
    POWER_DB_FLOOR = -160.0

    def __init__(self, vectors: torch.Tensor):
        if vectors.dim() != 3 or vectors.shape[-1] != 4:
            raise ValueError(f"vector field must be [H, W, 4], got {tuple(vectors.shape)}")
        if vectors.shape[0] == 0 or vectors.shape[1] == 0:
            raise ValueError("empty input: canvas_fft")
        self.vectors = vectors.float()

    height = property(lambda self: self.vectors.shape[0])
    width = property(lambda self: self.vectors.shape[1])

    @classmethod
    def from_energy(cls, energy: torch.Tensor, palette: str = "spiral") -> "ColorVectorField":
        """Energy normalised to [0, 1] with the palette's colour (scaled to [0, 1]) as chroma."""
        e = energy.float()
        lo, hi = float(e.min()), float(e.max())
        norm = (e - lo) / max(hi - lo, 1e-12)
        rgb = canvas_paint(e, palette)[..., :3].float() / 255.0
        return cls(torch.cat([norm[..., None], rgb.to(norm.device)], dim=-1))

    def energy_tensor(self) -> torch.Tensor:
        return self.vectors[..., 0]

    def as_tensor(self) -> torch.Tensor:
        return self.vectors.reshape(self.height, self.width * 4)

    def _spectrum(self, axis: str, inverse: bool, window: Optional[str]) -> torch.Tensor:
        from .ops import spectral
        return spectral.fft_field_interleaved(self.vectors, axis, inverse, window)

    def fft_rows_tensor(self, inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._spectrum("row", inverse, window).reshape(self.height, self.width * 8)

    def fft_cols_tensor(self, inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._spectrum("col", inverse, window).reshape(self.height, self.width * 8)

    def fft_2d_tensor(self, inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        """Rows then columns, per channel; ``[H, W * 8]`` interleaved."""
        from .ops import spectral
        rows = torch.view_as_complex(self._spectrum("row", inverse, window).reshape(self.height, self.width, 4, 2).contiguous())
        w = None if window is None else spectral.window_coefficients(window, self.height, rows.device)
        both = spectral.fft(rows, dim=0, inverse=inverse, window=w)
        return torch.view_as_real(both).reshape(self.height, self.width * 8)

    @staticmethod
    def _views(spectrum: torch.Tensor, height: int, width: int):
        z = spectrum.reshape(height, width, 4, 2)
        return z[..., 0], z[..., 1]

    def _derived(self, which: str, axis: str, inverse: bool, window: Optional[str]) -> torch.Tensor:
        spec = {"row": self.fft_rows_tensor, "col": self.fft_cols_tensor, "2d": self.fft_2d_tensor}[axis](inverse, window)
        re, im = self._views(spec, self.height, self.width)
        power = re * re + im * im
        if which == "magnitude":
            out = power.sqrt()
        elif which == "power":
            out = power
        elif which == "power_db":
            out = (10.0 * torch.log10(power.clamp(min=self.POWER_DB_EPSILON))).clamp(min=self.POWER_DB_FLOOR)
        else:
            out = torch.atan2(im, re)
        return out.reshape(self.height, self.width * 4)

    def fft_magnitude_tensor(self, axis: str = "row", inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._derived("magnitude", axis, inverse, window)

    def fft_power_tensor(self, axis: str = "row", inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._derived("power", axis, inverse, window)

    def fft_power_db_tensor(self, axis: str = "row", inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._derived("power_db", axis, inverse, window)

    def fft_phase_tensor(self, axis: str = "row", inverse: bool = False, window: Optional[str] = None) -> torch.Tensor:
        return self._derived("phase", axis, inverse, window)


def temporal_volume_render(volume: torch.Tensor, density_scale: float = 1.0) -> torch.Tensor:
    """Front-to-back compositing of a ``[D, H, W]`` (or ``[D, H, W, 3]``) Z volume along depth."""
    if volume.dim() == 3:
        volume = volume[..., None].expand(-1, -1, -1, 3)
    D, H, W, _ = volume.shape
    rad = volume.permute(1, 2, 0, 3).reshape(H * W, D, 3).float().contiguous()
    sigma = rad.mean(-1) * density_scale
    deltas = torch.ones_like(sigma)
    return nerf_composite(sigma, rad, deltas).reshape(H, W, 4)


@dataclass
class TemporalRenderOutput:
    frames: int
    depth: int
    height: int
    width: int
    times: list                 # seconds of each frame
    data: torch.Tensor          # [frames, depth, height, width]

    def frame(self, index: int) -> Optional[torch.Tensor]:
        return self.data[index] if 0 <= index < self.frames else None


class TemporalRenderer:
    """Plays a Z-space volume forward in time: every voxel is its base value plus its temporal harmonics
    ``sum_c a_c sin(2 pi (c + 1) t)``, damped by ``exp(-decay t)``, sampled at ``frames`` instants ``sample_rate_hz``
    apart (crates/st-backend-wgpu/src/render/temporal.rs:196-360).  One kernel launch renders all frames."""

    def __init__(self, frames: int = 16, sample_rate_hz: float = 24.0):
        self.frames, self.sample_rate_hz = int(frames), float(sample_rate_hz)

    def render(self, voxels: torch.Tensor, resonance_decay: torch.Tensor, temporal_harmonics: Optional[torch.Tensor] = None) -> TemporalRenderOutput:
        from .ops import spectral
        if voxels.dim() != 3:
            raise ValueError(f"volume must be [depth, height, width], got {tuple(voxels.shape)}")
        data = spectral.temporal_render(voxels, temporal_harmonics, resonance_decay, self.frames, self.sample_rate_hz)
        D, H, W = voxels.shape
        return TemporalRenderOutput(self.frames, D, H, W, [f / self.sample_rate_hz for f in range(self.frames)], data)


# ----------------------------------------------------------------------------------------------
# Video pipeline: decoded frames → Z-space volume with temporal smoothing and per-frame digests
# (crates/st-vision/src/video/mod.rs:66-560)
# ----------------------------------------------------------------------------------------------


class VideoPipelineConfig:
    def __init__(self, temporal_alpha: float = 0.35, resonance_decay: float = 0.25, motion_gain: float = 1.0,
                 digest_window: int = 16, quiescence_threshold: float = 0.05):
        self.temporal_alpha = min(max(temporal_alpha, 0.0), 1.0)
        self.resonance_decay = min(max(resonance_decay, 0.0), 1.0)
        self.motion_gain = max(motion_gain, 0.0) if math.isfinite(motion_gain) else 1.0
        self.digest_window = max(int(digest_window), 1)
        self.quiescence_threshold = max(quiescence_threshold, 0.0)


def _energy(t: torch.Tensor) -> float:
    return float(t.abs().mean()) if t.numel() else 0.0


def _digest(samples, threshold: float) -> dict:
    """Statistics of (timestamp, motion energy, resonance energy) samples."""
    if not samples:
        return {"frames": 0, "duration": 0.0, "mean_motion_energy": 0.0, "motion_std": 0.0,
                "mean_resonance_energy": 0.0, "resonance_std": 0.0, "mean_resonance_decay": 0.0,
                "min_resonance_energy": 0.0, "max_resonance_energy": 0.0, "peak_motion_energy": 0.0,
                "peak_motion_timestamp": 0.0, "peak_resonance_energy": 0.0, "peak_resonance_timestamp": 0.0,
                "quiescence_ratio": 0.0}
    ts = [s[0] for s in samples]
    mo = torch.tensor([s[1] for s in samples], dtype=torch.float64)
    en = torch.tensor([s[2] for s in samples], dtype=torch.float64)
    duration = sum(max(b - a, 0.0) for a, b in zip(ts, ts[1:]))
    decay = [(a - b) / abs(a) if abs(a) > 1.1920929e-07 else 0.0 for a, b in zip(en.tolist(), en.tolist()[1:])]
    pm, pr = int(torch.argmax(mo)), int(torch.argmax(en))
    return {"frames": len(samples), "duration": duration,
            "mean_motion_energy": float(mo.mean()), "motion_std": float(mo.std(unbiased=False)),
            "mean_resonance_energy": float(en.mean()), "resonance_std": float(en.std(unbiased=False)),
            "mean_resonance_decay": sum(decay) / len(samples),
            "min_resonance_energy": float(en.min()), "max_resonance_energy": float(en.max()),
            "peak_motion_energy": float(mo[pm]), "peak_motion_timestamp": ts[pm],
            "peak_resonance_energy": float(en[pr]), "peak_resonance_timestamp": ts[pr],
            "quiescence_ratio": float((mo <= threshold).double().mean())}


class VideoPipeline:
    """Consumes ``(timestamp, frame[H, W])`` pairs from any iterable decoder.  Each frame and its
    motion embedding (gain × difference to the previous frame) form a two-slice stream frame that is
    blended into the running Z-space volume with ``temporal_alpha``; the pipeline reports per-depth
    energies, their exponentially smoothed weights, the Hann-windowed depth spectrum, a resonance
    envelope (EMA of the volume) and running / windowed temporal digests, and keeps an atlas timeline.
    Frames stay on the device they arrive on."""

    def __init__(self, decoder, config: Optional[VideoPipelineConfig] = None):
        self.decoder = iter(decoder)
        self.config = config or VideoPipelineConfig()
        self.frame_index = 0
        self.volume: Optional[torch.Tensor] = None         # [depth, H, W]
        self._previous: Optional[torch.Tensor] = None
        self._weights: Optional[torch.Tensor] = None
        self._envelope: Optional[torch.Tensor] = None
        self._samples: list = []
        self.timeline: list = []

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        out = self.next_frame()
        if out is None:
            raise StopIteration
        return out

    def next_frame(self) -> Optional[dict]:
        try:
            timestamp, frame = next(self.decoder)
        except StopIteration:
            return None
        frame = frame.float()
        if frame.dim() != 2:
            raise ValueError(f"decoded frame must be [H, W], got {tuple(frame.shape)}")
        cfg = self.config
        motion = (torch.zeros_like(frame) if self._previous is None
                  else (frame - self._previous) * max(cfg.motion_gain, 1.1920929e-07))
        self._previous = frame
        stream = torch.stack([frame, motion])
        if self.volume is None or self.volume.shape != stream.shape:
            self.volume = stream.clone()
        else:
            self.volume = torch.lerp(self.volume, stream, cfg.temporal_alpha)
        per_depth = self.volume.abs().mean(dim=(1, 2))
        if not bool(torch.isfinite(per_depth).all()):
            raise ValueError("temporal_resonance_weight is not finite")
        if self._weights is None or self._weights.shape != per_depth.shape:
            self._weights = per_depth.clone()
        else:
            self._weights = torch.lerp(self._weights, per_depth, cfg.resonance_decay)
        depth = self.volume.shape[0]
        window = torch.hann_window(depth, periodic=False, device=frame.device) if depth > 1 else torch.ones(1, device=frame.device)
        spectral = torch.fft.rfft(per_depth * window).abs()
        flat = self.volume.reshape(depth, -1)
        self._envelope = flat.clone() if self._envelope is None or self._envelope.shape != flat.shape \
            else torch.lerp(self._envelope, flat, cfg.resonance_decay)
        motion_energy, resonance_energy = _energy(motion), _energy(self._envelope)
        self._samples.append((float(timestamp), motion_energy, resonance_energy))
        w = self._weights
        pos = w[w > 1.1920929e-07]
        p = pos / pos.sum() if pos.numel() else pos
        entropy = float(-(p * p.log()).sum()) if p.numel() else 0.0
        top = int(torch.argmax(w))
        atlas = {"timestamp": float(timestamp), "collapse_total": resonance_energy,
                 "z_signal": top / (depth - 1) if depth > 1 else float(w[0]),
                 "loop_support": max(motion_energy, 0.0),
                 "metrics": {"z.motion_energy": motion_energy, "z.resonance_energy": resonance_energy,
                             "z.weight_entropy": entropy},
                 "notes": ["video.pipeline.z_dynamics"]}
        self.timeline.append(atlas)
        self.frame_index += 1
        return {"frame_index": self.frame_index - 1, "atlas_frame": atlas, "volume": self.volume,
                "motion_embedding": motion, "resonance_envelope": self._envelope,
                "z_dynamics": {"smoothed_weights": w.tolist(), "per_depth_energy": per_depth.tolist(),
                               "spectral_response": spectral.tolist()},
                "temporal_digest": self.temporal_digest(),
                "window_digest": self.temporal_digest_window(cfg.digest_window)}

    def last_volume(self) -> Optional[torch.Tensor]:
        return self.volume

    def atlas_timeline(self) -> list:
        return list(self.timeline)

    def temporal_digest(self) -> dict:
        return _digest(self._samples, self.config.quiescence_threshold)

    def temporal_digest_window(self, window: int) -> dict:
        return _digest(self._samples[-window:] if window > 0 else [], self.config.quiescence_threshold)


# ------------------------------------------------------------------------------------------------------
# Transform pipeline (torchvision-like operations with a seeded RNG) and the multi-view dataset adapter.
# Reference: TransformOperation / TransformPipeline / standard_classification_pipeline
# (crates/st-vision/src/lib.rs:3404-3540,4170-4197), MultiViewFrame / MultiViewDatasetAdapter
# (crates/st-vision/src/datasets/mod.rs:12-135).  Every operation runs through `preprocess`, i.e. on the
# fused CUDA kernel for device tensors.
# ------------------------------------------------------------------------------------------------------
class Normalize:
    name = "Normalize"

    def __init__(self, mean: Sequence[float], std: Sequence[float]):
        if len(mean) != len(std) or not mean or any(s == 0 for s in std):
            raise ValueError("Normalize: mean/std must be non-empty, of equal length, with non-zero std")
        self.mean, self.std = list(map(float, mean)), list(map(float, std))

    def apply(self, img: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
        if img.shape[-3] != len(self.mean):
            raise ValueError(f"Normalize: expected {len(self.mean)} channels, got {img.shape[-3]}")
        m = torch.tensor(self.mean, device=img.device).view(-1, 1, 1)
        s = torch.tensor(self.std, device=img.device).view(-1, 1, 1)
        return (img - m) / s


class Resize:
    name = "Resize"

    def __init__(self, height: int, width: int):
        if height <= 0 or width <= 0:
            raise ValueError("Resize: dimensions must be > 0")
        self.height, self.width = height, width

    def apply(self, img, gen):
        return resize(img, self.height, self.width)


class CenterCrop:
    name = "CenterCrop"

    def __init__(self, height: int, width: int):
        if height <= 0 or width <= 0:
            raise ValueError("CenterCrop: dimensions must be > 0")
        self.height, self.width = height, width

    def apply(self, img, gen):
        return center_crop(img, self.height, self.width)


class RandomHorizontalFlip:
    name = "RandomHorizontalFlip"

    def __init__(self, probability: float = 0.5):
        if not 0.0 <= probability <= 1.0:
            raise ValueError("horizontal_flip_probability must be in [0, 1]")
        self.probability = probability

    def apply(self, img, gen):
        return horizontal_flip(img) if float(torch.rand((), generator=gen)) < self.probability else img


class RandomColorJitter:
    """Random factors ``1 ± amount`` for brightness / contrast / saturation and a hue rotation of up to
    ``hue * pi``, applied in a random order (crates/st-vision/src/lib.rs:4011-4165)."""
    name = "ColorJitter"

    def __init__(self, brightness: float = 0.0, contrast: float = 0.0, saturation: float = 0.0, hue: float = 0.0):
        if brightness < 0 or contrast < 0 or saturation < 0 or not 0.0 <= hue <= 0.5:
            raise ValueError("color jitter amounts must be >= 0 and hue in [0, 0.5]")
        self.brightness, self.contrast, self.saturation, self.hue = brightness, contrast, saturation, hue

    def apply(self, img, gen):
        def draw(amount):
            return float((torch.rand((), generator=gen) * 2 - 1) * amount)
        ops = []
        if self.brightness > 0:
            ops.append(ColorJitter(brightness=1.0 + draw(self.brightness)))
        if self.contrast > 0:
            ops.append(ColorJitter(contrast=1.0 + draw(self.contrast)))
        if self.saturation > 0 and img.shape[-3] >= 3:
            ops.append(ColorJitter(saturation=1.0 + draw(self.saturation)))
        if self.hue > 0 and img.shape[-3] >= 3:
            ops.append(ColorJitter(hue=draw(self.hue) * math.pi))
        for i in torch.randperm(len(ops), generator=gen).tolist():
            img = color_jitter(img, ops[i])
        return img


class TransformPipeline:
    """Ordered list of transform operations sharing one seeded generator."""

    def __init__(self, seed: Optional[int] = None):
        self._ops: list = []
        self._gen = torch.Generator()
        self._gen.manual_seed(0 if seed is None else int(seed) & 0x7FFFFFFFFFFFFFFF)

    @classmethod
    def with_seed(cls, seed: int) -> "TransformPipeline":
        return cls(seed)

    def add(self, op) -> "TransformPipeline":
        if not hasattr(op, "apply") or not hasattr(op, "name"):
            raise TypeError("a transform operation needs .name and .apply(image, generator)")
        self._ops.append(op)
        return self

    def operations(self) -> list:
        return list(self._ops)

    def __len__(self) -> int:
        return len(self._ops)

    def is_empty(self) -> bool:
        return not self._ops

    def apply(self, img: torch.Tensor) -> torch.Tensor:
        for op in self._ops:
            img = op.apply(img, self._gen)
        return img


def standard_classification_pipeline(image_size: int, seed: Optional[int] = None) -> TransformPipeline:
    """Resize(size+32) → CenterCrop(size) → RandomHorizontalFlip(0.5) → ImageNet Normalize."""
    return (TransformPipeline(seed)
            .add(Resize(image_size + 32, image_size + 32)).add(CenterCrop(image_size, image_size))
            .add(RandomHorizontalFlip(0.5)).add(Normalize([0.485, 0.456, 0.406], [0.229, 0.224, 0.225])))


class MultiViewFrame:
    """Rays of one camera view: origins / directions ``[rays, dims]``, colours ``[rays, 3]``, bounds ``[rays, 2]``."""

    def __init__(self, origins, directions, colors, bounds):
        o, d, c, b = (torch.as_tensor(t, dtype=torch.float32) for t in (origins, directions, colors, bounds))
        if o.dim() != 2 or o.shape[0] == 0:
            raise ValueError("multiview_rays: empty input")
        if not (d.shape[0] == c.shape[0] == b.shape[0] == o.shape[0]):
            raise ValueError("multiview frame: row counts differ")
        if d.shape[1] != o.shape[1] or c.shape[1] != 3 or b.shape[1] != 2:
            raise ValueError("multiview frame: directions must match origins, colours need 3 and bounds 2 columns")
        self.origins, self.directions, self.colors, self.bounds = o, d, c, b

    def __len__(self) -> int:
        return self.origins.shape[0]


class MultiViewDatasetAdapter:
    def __init__(self, frames: Sequence[MultiViewFrame]):
        frames = list(frames)
        if not frames:
            raise ValueError("multiview_frames: empty input")
        self.origin_dims = frames[0].origins.shape[1]
        if any(f.origins.shape[1] != self.origin_dims for f in frames):
            raise ValueError("multiview frames disagree on the origin dimension")
        self._frames = frames
        self.set_frame_weights([1.0] * len(frames))

    def num_frames(self) -> int:
        return len(self._frames)

    def frames(self) -> list:
        return self._frames

    def frame_weights(self) -> list:
        return list(self._weights)

    def set_frame_weights(self, weights: Sequence[float]) -> None:
        w = [float(x) for x in weights]
        if len(w) != len(self._frames):
            raise ValueError(f"frame_weights: expected {len(self._frames)} values, got {len(w)}")
        if any((not math.isfinite(x)) or x < 0 for x in w) or sum(w) <= 0:
            raise ValueError("frame_weights must be finite, non-negative and not all zero")
        self._weights = w

    def sample_batch(self, gen: torch.Generator, batch_size: int) -> dict:
        """``batch_size`` rays drawn frame-by-weight, then uniformly inside the frame."""
        if batch_size <= 0:
            raise ValueError("batch_size must be > 0")
        fidx = torch.multinomial(torch.tensor(self._weights), batch_size, replacement=True, generator=gen)
        cols = {"origins": [], "directions": [], "colors": [], "bounds": []}
        for f in fidx.tolist():
            fr = self._frames[f]
            r = int(torch.randint(0, len(fr), (), generator=gen))
            for k in cols:
                cols[k].append(getattr(fr, k)[r])
        return {k: torch.stack(v) for k, v in cols.items()}
