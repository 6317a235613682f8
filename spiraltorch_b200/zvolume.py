"""Z-space volumes and the vision projector: depth-stacked feature slices with per-voxel temporal harmonics and
resonance decay, slice statistics, depth interpolation / spatial upscaling, diffusion, EMA streaming, sequence blending
and resonance-driven collapse to one image.

Parity: crates/st-vision/src/lib.rs — `ZSpaceVolume` (:555-1222, accumulate / blend_sequence :2218-2368),
`ZSliceProfile` / `ZSpaceTelemetryReport` (:567-752), `SpectralWindow` (:1267-1368), `TemporalResonanceBuffer`
(:1371-1445), `ZDiffuser` (:1449-1537), `VisionProjector` (:2373-2700), `ZSpaceStreamFrame` / aggregator (:150-440).

The volume is a ``[D, H, W]`` fp32 tensor on any device; every operation is a whole-tensor op (reductions per slice,
one stencil per diffusion step, one weighted sum for a collapse), so a CUDA volume never visits the host except for
the depth-weight vector (``D`` floats), which is control data.  `TemporalRenderer` plays a volume through the
temporal-renderer kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .tensor import Tensor, TensorError

_EPS = 1.1920929e-07
INTERPOLATION = ("nearest", "linear", "cubic")


def _raw(x) -> torch.Tensor:
    return x.torch() if isinstance(x, Tensor) else torch.as_tensor(x, dtype=torch.float32)


def normalise_weights(w: Sequence[float]) -> List[float]:
    """Divide by the sum of the finite entries; uniform when that sum is not positive."""
    total = sum(v for v in w if math.isfinite(v))
    if not math.isfinite(total) or total <= _EPS:
        return [1.0 / max(len(w), 1)] * len(w)
    return [v / total for v in w]


@dataclass(frozen=True)
class ZSpaceTelemetryReport:
    depth: int
    mean_intensity: float
    mean_std: float
    mean_energy: float
    total_energy: float
    max_energy: float
    energy_entropy: float


class ZSliceProfile:
    """Mean, standard deviation (population) and mean square of every depth slice."""

    def __init__(self, means: Sequence[float], stds: Sequence[float], energies: Sequence[float]):
        if not (len(means) == len(stds) == len(energies)):
            raise TensorError(f"data length mismatch: {len(means)} means, {len(stds)} stds, {len(energies)} energies")
        if not means:
            raise TensorError("empty input: z_slice_profile")
        self.means, self.stds, self.energies = list(means), list(stds), list(energies)

    def depth(self) -> int:
        return len(self.means)

    def mean(self, i: int) -> float:
        return self.means[i] if 0 <= i < len(self.means) else 0.0

    def std(self, i: int) -> float:
        return self.stds[i] if 0 <= i < len(self.stds) else 0.0

    def energy(self, i: int) -> float:
        return self.energies[i] if 0 <= i < len(self.energies) else 0.0

    def average_mean(self) -> float:
        return sum(self.means) / len(self.means)

    def average_std(self) -> float:
        return sum(self.stds) / len(self.stds)

    def average_energy(self) -> float:
        return sum(self.energies) / len(self.energies)

    def total_energy(self) -> float:
        return sum(self.energies)

    def max_energy(self) -> float:
        return max([0.0] + self.energies)

    def energy_entropy(self) -> float:
        """Shannon entropy (bits) of the energy shares."""
        total = self.total_energy()
        if total <= _EPS:
            return 0.0
        return -sum((e / total) * math.log2(e / total) for e in self.energies if math.isfinite(e) and e > 0)

    def summarize(self) -> ZSpaceTelemetryReport:
        return ZSpaceTelemetryReport(self.depth(), self.average_mean(), self.average_std(), self.average_energy(),
                                     self.total_energy(), self.max_energy(), self.energy_entropy())


class SpectralWindow:
    """Depth taper, normalised to sum one: rectangular, Hann, Hamming, Blackman, or a Gaussian of relative width
    ``sigma`` around the middle slice."""

    def __init__(self, kind: str = "hann", sigma: float = 0.4):
        kind = kind.lower()
        if kind not in ("rectangular", "hann", "hamming", "blackman", "gaussian"):
            raise ValueError(f"unknown spectral window '{kind}'")
        self.kind = kind
        self.sigma = sigma if (math.isfinite(sigma) and sigma > 1e-3) else 0.4

    rectangular = classmethod(lambda cls: cls("rectangular"))
    hann = classmethod(lambda cls: cls("hann"))
    hamming = classmethod(lambda cls: cls("hamming"))
    blackman = classmethod(lambda cls: cls("blackman"))
    gaussian = classmethod(lambda cls, sigma: cls("gaussian", sigma))

    def weights(self, depth: int) -> List[float]:
        if depth <= 0:
            return []
        if depth == 1:
            return [1.0]
        n1 = depth - 1
        if self.kind == "rectangular":
            w = [1.0] * depth
        elif self.kind == "hann":
            w = [max(0.5 * (1.0 - math.cos(2 * math.pi * n / n1)), 0.0) for n in range(depth)]
        elif self.kind == "hamming":
            w = [max(0.54 - 0.46 * math.cos(2 * math.pi * n / n1), 0.0) for n in range(depth)]
        elif self.kind == "blackman":
            w = [max(0.42 - 0.5 * math.cos(2 * math.pi * n / n1) + 0.08 * math.cos(4 * math.pi * n / n1), 0.0) for n in range(depth)]
        else:
            centre = n1 / 2.0
            denom = max(2.0 * self.sigma ** 2 * (centre + 1.0) ** 2, 1e-6)
            w = [math.exp(-((n - centre) ** 2) / denom) for n in range(depth)]
        return normalise_weights(w)


class TemporalResonanceBuffer:
    """EMA of depth-weight vectors across frames (``decay`` is the weight of the incoming vector); the history is
    renormalised after every update and restarts when the depth changes."""

    def __init__(self, decay: float = 0.5):
        self.decay = min(max(decay, 0.0), 1.0) if math.isfinite(decay) else 0.5
        self.history: Optional[List[float]] = None
        self.frames = 0

    def frames_accumulated(self) -> int:
        return self.frames

    def clear(self) -> None:
        self.history, self.frames = None, 0

    def apply(self, weights: Sequence[float]) -> List[float]:
        for v in weights:
            if not math.isfinite(v):
                raise TensorError(f"non-finite value for temporal_resonance_weight: {v}")
        if len(weights) == 0:
            self.clear()
            return []
        if self.history is not None and len(self.history) == len(weights):
            a = self.decay
            self.history = normalise_weights([h * (1.0 - a) + w * a for h, w in zip(self.history, weights)])
            self.frames += 1
        else:
            self.history, self.frames = normalise_weights(list(weights)), 1
        return list(self.history)


class ZSpaceVolume:
    def __init__(self, voxels: torch.Tensor, temporal_harmonics: Optional[torch.Tensor] = None,
                 resonance_decay: Optional[torch.Tensor] = None):
        v = _raw(voxels).float()
        if v.dim() != 3 or 0 in v.shape:
            raise TensorError(f"invalid dimensions: a Z-space volume is [depth, height, width], got {tuple(v.shape)}")
        self.voxels = v
        self.temporal_harmonics = None
        if temporal_harmonics is not None and temporal_harmonics.numel():
            h = _raw(temporal_harmonics).float()
            if h.shape[:3] != v.shape or h.dim() != 4:
                raise TensorError(f"shape mismatch: harmonics {tuple(h.shape)} against volume {tuple(v.shape)}")
            self.temporal_harmonics = h
        self.resonance_decay = torch.ones_like(v) if resonance_decay is None else _raw(resonance_decay).float().to(v.device)
        if self.resonance_decay.shape != v.shape:
            raise TensorError(f"shape mismatch: decay {tuple(self.resonance_decay.shape)} against volume {tuple(v.shape)}")

    # -- constructors ---------------------------------------------------------------------------------------------
    @classmethod
    def zeros(cls, depth: int, height: int, width: int, harmonic_channels: int = 0, device=None) -> "ZSpaceVolume":
        if depth <= 0 or height <= 0 or width <= 0:
            raise TensorError(f"invalid dimensions ({depth}, {height * width})")
        h = torch.zeros(depth, height, width, harmonic_channels, device=device) if harmonic_channels else None
        return cls(torch.zeros(depth, height, width, device=device), h)

    zeros_with_temporal = zeros

    @classmethod
    def from_voxels(cls, depth: int, height: int, width: int, voxels) -> "ZSpaceVolume":
        if depth <= 0 or height <= 0 or width <= 0:
            raise TensorError(f"invalid dimensions ({depth}, {height * width})")
        v = torch.as_tensor(voxels, dtype=torch.float32)
        if v.numel() != depth * height * width:
            raise TensorError(f"data length mismatch: expected {depth * height * width}, got {v.numel()}")
        return cls(v.reshape(depth, height, width))

    @classmethod
    def from_slices(cls, slices: Sequence) -> "ZSpaceVolume":
        if len(slices) == 0:
            raise TensorError("empty input: z_space_volume_slices")
        ts = [_raw(s).float() for s in slices]
        for t in ts:
            if t.shape != ts[0].shape or t.dim() != 2:
                raise TensorError(f"shape mismatch: slice {tuple(t.shape)} against {tuple(ts[0].shape)}")
        return cls(torch.stack(ts))

    # -- accessors ------------------------------------------------------------------------------------------------
    depth = property(lambda self: self.voxels.shape[0])
    height = property(lambda self: self.voxels.shape[1])
    width = property(lambda self: self.voxels.shape[2])
    harmonic_channels = property(lambda self: 0 if self.temporal_harmonics is None else self.temporal_harmonics.shape[-1])
    device = property(lambda self: self.voxels.device)

    def voxel_count(self) -> int:
        return self.voxels.numel()

    def to(self, device) -> "ZSpaceVolume":
        return ZSpaceVolume(self.voxels.to(device), None if self.temporal_harmonics is None else self.temporal_harmonics.to(device),
                            self.resonance_decay.to(device))

    def clone(self) -> "ZSpaceVolume":
        return ZSpaceVolume(self.voxels.clone(), None if self.temporal_harmonics is None else self.temporal_harmonics.clone(),
                            self.resonance_decay.clone())

    def ensure_harmonic_channels(self, channels: int) -> None:
        """Pads with zero channels or truncates to ``channels``."""
        cur = self.harmonic_channels
        if cur == channels:
            return
        if channels == 0:
            self.temporal_harmonics = None
            return
        h = torch.zeros(*self.voxels.shape, channels, device=self.device)
        if cur:
            h[..., :min(cur, channels)] = self.temporal_harmonics[..., :min(cur, channels)]
        self.temporal_harmonics = h

    def slice(self, index: int) -> Tensor:
        if not 0 <= index < self.depth:
            raise TensorError("invalid value: z_slice_index")
        return Tensor._wrap(self.voxels[index].clone())

    # -- statistics -----------------------------------------------------------------------------------------------
    def profile(self) -> ZSliceProfile:
        flat = self.voxels.reshape(self.depth, -1)
        mean = flat.mean(1)
        std = (flat - mean[:, None]).pow(2).mean(1).clamp(min=0).sqrt()
        stats = torch.stack([mean, std, flat.pow(2).mean(1)]).tolist()       # one host read for all three
        return ZSliceProfile(*stats)

    def telemetry_report(self) -> ZSpaceTelemetryReport:
        return self.profile().summarize()

    # -- collapse -------------------------------------------------------------------------------------------------
    def collapse_with_weights(self, weights: Sequence[float]) -> Tensor:
        if len(weights) != self.depth:
            raise TensorError(f"data length mismatch: expected {self.depth}, got {len(weights)}")
        for w in weights:
            if not math.isfinite(w):
                raise TensorError(f"non-finite value for z_space_weight: {w}")
        w = torch.tensor(list(weights), dtype=torch.float32, device=self.device)
        return Tensor._wrap(torch.tensordot(w, self.voxels, dims=1))

    def resonance_weights(self, resonance) -> List[float]:
        """Depth weights from a differential resonance: ``(|energy| + 1e-6) (1 + tanh objective) (1 + tanh homotopy)``
        with each field read cyclically along depth, normalised."""
        e, o, h = (_raw(t).reshape(-1) for t in (resonance.infinity_energy, resonance.recursive_objective, resonance.homotopy_flow))
        if e.numel() == 0 or o.numel() == 0:
            raise TensorError("empty input: differential_resonance")
        idx = torch.arange(self.depth)
        w = (e.cpu()[idx % e.numel()].abs() + 1e-6) * (1.0 + torch.tanh(o.cpu()[idx % o.numel()]))
        if h.numel():
            w = w * (1.0 + torch.tanh(h.cpu()[idx % h.numel()]))
        return normalise_weights(w.clamp(min=0).tolist())

    def project_resonance(self, resonance) -> Tensor:
        return self.collapse_with_weights(self.resonance_weights(resonance))

    # -- resampling -----------------------------------------------------------------------------------------------
    def interpolate(self, method: str = "linear") -> "ZSpaceVolume":
        """Inserts one slice between every pair of neighbours (``2D - 1`` slices): a copy of the nearer one, their
        mean, or the Catmull-Rom midpoint ``(-p0 + 9 p1 + 9 p2 - p3) / 16`` with the ends repeated."""
        method = method.lower()
        if method not in INTERPOLATION:
            raise ValueError(f"unknown interpolation '{method}', expected one of {INTERPOLATION}")
        if self.depth <= 1:
            return self.clone()
        v = self.voxels
        cur, nxt = v[:-1], v[1:]
        if method == "nearest":
            mid = cur
        elif method == "linear":
            mid = 0.5 * (cur + nxt)
        else:
            prev = torch.cat([v[:1], v[:-2]]) if self.depth > 2 else v[:1]
            ahead = torch.cat([v[2:], v[-1:]])
            mid = (-prev + 9.0 * cur + 9.0 * nxt - ahead) / 16.0
        out = torch.empty(2 * self.depth - 1, self.height, self.width, device=self.device)
        out[0::2], out[1::2] = v, mid
        return ZSpaceVolume(out)

    def upscale(self, factor: int) -> "ZSpaceVolume":
        """Bilinear resampling of every slice to ``factor`` times the size, corners aligned."""
        if factor <= 0:
            raise TensorError("invalid value: z_upscale_factor")
        if factor == 1:
            return self.clone()
        up = torch.nn.functional.interpolate(self.voxels[:, None], size=(self.height * factor, self.width * factor),
                                             mode="bilinear", align_corners=True)[:, 0]
        return ZSpaceVolume(up)

    # -- streaming ------------------------------------------------------------------------------------------------
    def accumulate(self, nxt: "ZSpaceVolume", alpha: float) -> None:
        """In-place EMA ``self <- (1 - alpha) self + alpha next`` over voxels, harmonics (the narrower side is padded
        with zero channels) and decay."""
        if self.voxels.shape != nxt.voxels.shape:
            raise TensorError(f"shape mismatch: {tuple(self.voxels.shape)} against {tuple(nxt.voxels.shape)}")
        if not (math.isfinite(alpha) and 0.0 <= alpha <= 1.0):
            raise TensorError("invalid value: temporal_alpha")
        self.voxels = torch.lerp(self.voxels, nxt.voxels.to(self.device), alpha)
        channels = max(self.harmonic_channels, nxt.harmonic_channels)
        if channels:
            self.ensure_harmonic_channels(channels)
            other = torch.zeros_like(self.temporal_harmonics)
            if nxt.harmonic_channels:
                other[..., :nxt.harmonic_channels] = nxt.temporal_harmonics.to(self.device)
            self.temporal_harmonics = torch.lerp(self.temporal_harmonics, other, alpha)
        self.resonance_decay = torch.lerp(self.resonance_decay, nxt.resonance_decay.to(self.device), alpha)

    def accumulated(self, nxt: "ZSpaceVolume", alpha: float) -> "ZSpaceVolume":
        out = self.clone()
        out.accumulate(nxt, alpha)
        return out

    @staticmethod
    def blend_sequence(sequence: Sequence["ZSpaceVolume"], weights: Sequence[float]) -> "ZSpaceVolume":
        """Weighted mean of volumes (voxels, harmonics, decay), divided by the weight sum when that is positive."""
        if len(sequence) == 0:
            raise TensorError("empty input: z_space_sequence")
        if len(weights) != len(sequence):
            raise TensorError(f"data length mismatch: expected {len(sequence)}, got {len(weights)}")
        base = sequence[0]
        channels = max(v.harmonic_channels for v in sequence)
        out = ZSpaceVolume.zeros(base.depth, base.height, base.width, channels, device=base.device)
        out.resonance_decay.zero_()
        total = 0.0
        for vol, w in zip(sequence, weights):
            if vol.voxels.shape != base.voxels.shape:
                raise TensorError(f"shape mismatch: {tuple(base.voxels.shape)} against {tuple(vol.voxels.shape)}")
            if not math.isfinite(w):
                raise TensorError(f"non-finite value for temporal_weight: {w}")
            total += w
            out.voxels += vol.voxels.to(base.device) * w
            out.resonance_decay += vol.resonance_decay.to(base.device) * w
            if vol.harmonic_channels and channels:
                out.temporal_harmonics[..., :vol.harmonic_channels] += vol.temporal_harmonics.to(base.device) * w
        if total > 0:
            out.voxels /= total
            out.resonance_decay /= total
            if channels:
                out.temporal_harmonics /= total
        return out

    def render_temporal(self, frames: int = 16, sample_rate_hz: float = 24.0):
        """Plays the volume through the temporal renderer: ``[frames, D, H, W]`` plus frame times."""
        from .vision import TemporalRenderer
        return TemporalRenderer(frames, sample_rate_hz).render(self.voxels, self.resonance_decay, self.temporal_harmonics)


class ZDiffuser:
    """``iterations`` steps of ``v <- (1 - rate) v + rate * mean(6-neighbourhood)``; neighbours outside the volume are
    left out of the mean (a voxel without neighbours stays)."""

    def __init__(self, iterations: int = 1, rate: float = 0.25):
        self.iterations = max(int(iterations), 0)
        self.rate = min(max(rate, 0.0), 1.0) if math.isfinite(rate) else 0.25

    def diffuse(self, volume: ZSpaceVolume) -> ZSpaceVolume:
        v = volume.voxels
        ones = torch.ones_like(v)
        for _ in range(self.iterations):
            s, c = torch.zeros_like(v), torch.zeros_like(v)
            for dim in range(3):
                n = v.shape[dim]
                if n < 2:
                    continue
                lo, hi = [slice(None)] * 3, [slice(None)] * 3
                lo[dim], hi[dim] = slice(0, n - 1), slice(1, n)
                s[tuple(hi)] += v[tuple(lo)]          # neighbour at index - 1
                c[tuple(hi)] += ones[tuple(lo)]
                s[tuple(lo)] += v[tuple(hi)]          # neighbour at index + 1
                c[tuple(lo)] += ones[tuple(hi)]
            avg = s / c.clamp(min=1.0)
            v = torch.where(c > 0, v * (1.0 - self.rate) + avg * self.rate, v)
        return ZSpaceVolume(v)


class VisionProjector:
    """Collapses a volume along depth with weights that combine the resonance weights, a Gaussian around a focus
    depth, an energy bias and a spectral window; also weights frames of a sequence with a Gaussian in time."""

    def __init__(self, focus: float = 0.5, spread: float = 0.35, energy_bias: float = 0.0, window: Optional[SpectralWindow] = None):
        self.focus = min(max(focus, 0.0), 1.0)
        self.spread = spread if (math.isfinite(spread) and spread > 1e-3) else 0.35
        self.energy_bias = energy_bias if math.isfinite(energy_bias) else 0.0
        self.window = window or SpectralWindow.hann()
        self.temporal_focus, self.temporal_decay = 1.0, 0.35

    def with_spectral_window(self, window: SpectralWindow) -> "VisionProjector":
        self.window = window
        return self

    @classmethod
    def from_summary(cls, summary) -> "VisionProjector":
        """Focus at the relative position of the mean energy between its extremes, spread from the relative energy
        deviation (narrower under drift), bias from the mean decay."""
        span = max(abs(summary.max_energy - summary.min_energy), 1e-3)
        focus = min(max((summary.mean_energy - summary.min_energy) / span, 0.0), 1.0)
        spread = min(max(summary.energy_std / span, 0.05), 1.0)
        drift = summary.mean_abs_drift
        if math.isfinite(drift):
            spread /= 1.0 + abs(drift)
        p = cls(focus, spread, summary.mean_decay)
        if math.isfinite(drift):
            p.temporal_decay = min(max(1.0 / (1.0 + abs(drift)), 0.05), 1.0)
        return p

    def calibrate_from_atlas(self, frame) -> None:
        z = getattr(frame, "z_signal", None)
        if z is not None and math.isfinite(z):
            self.focus = min(max(z, 0.0), 1.0)
        pressure = getattr(frame, "suggested_pressure", None)
        if pressure is not None and math.isfinite(pressure):
            self.spread = max(min(max(abs(pressure / 32.0), 0.05), 2.0), 0.05)
        total = getattr(frame, "collapse_total", None)
        if total is not None and math.isfinite(total):
            self.energy_bias = math.tanh(total)
        districts = getattr(frame, "districts", {}) or {}
        for name, value in (getattr(frame, "metrics", {}) or {}).items():
            if name in ("temporal_focus", "z_temporal_focus"):
                self.temporal_focus = min(max(value, 0.0), 1.0)
            elif name in ("temporal_decay", "z_temporal_decay") and math.isfinite(value):
                self.temporal_decay = min(max(abs(value), 0.05), 1.0)
            if str(districts.get(name, "")).lower() == "temporal" and math.isfinite(value):
                self.temporal_decay = min(max(abs(value), 0.05), 1.0)

    def depth_weights(self, volume: ZSpaceVolume, resonance) -> List[float]:
        w = volume.resonance_weights(resonance)
        window = self.window.weights(volume.depth)
        mod = max(1.0 + math.tanh(self.energy_bias), 0.1)
        if volume.depth > 1:
            spread, denom = max(self.spread, 1e-3), volume.depth - 1
            w = [v * max(math.exp(-0.5 * ((i / denom - self.focus) / spread) ** 2), 1e-6) * mod * max(window[i], 1e-6)
                 for i, v in enumerate(w)]
        else:
            w = [v * mod * max(window[0], 1e-6) for v in w]
        return normalise_weights(w)

    def depth_weights_with_temporal(self, volume, resonance, buffer: TemporalResonanceBuffer) -> List[float]:
        return buffer.apply(self.depth_weights(volume, resonance))

    def project(self, volume: ZSpaceVolume, resonance) -> Tensor:
        return volume.collapse_with_weights(self.depth_weights(volume, resonance))

    def project_with_temporal(self, volume, resonance, buffer: TemporalResonanceBuffer) -> Tensor:
        return volume.collapse_with_weights(self.depth_weights_with_temporal(volume, resonance, buffer))

    def temporal_weights(self, frames: int) -> List[float]:
        if frames <= 0:
            return []
        if frames == 1:
            return [1.0]
        focus, decay = min(max(self.temporal_focus, 0.0), 1.0), max(self.temporal_decay, 1e-3)
        w = [max(math.exp(-0.5 * ((i / (frames - 1) - focus) / decay) ** 2), 1e-6) for i in range(frames)]
        total = sum(w)
        return [1.0 / frames] * frames if (total <= _EPS or not math.isfinite(total)) else [v / total for v in w]

    def streaming_alpha(self) -> float:
        return min(max(1.0 - min(max(self.temporal_decay, 0.0), 0.99), 0.05), 0.95)

    def accumulate_temporal(self, state: ZSpaceVolume, nxt: ZSpaceVolume) -> None:
        state.accumulate(nxt, self.streaming_alpha())

    def fuse_sequence(self, sequence: Sequence[ZSpaceVolume]) -> ZSpaceVolume:
        if len(sequence) == 0:
            raise TensorError("empty input: z_space_sequence")
        return ZSpaceVolume.blend_sequence(sequence, self.temporal_weights(len(sequence)))


class ZSpaceStreamFrame:
    """Depth slices arriving together, optionally with the atlas frame and chrono snapshot of their instant."""

    def __init__(self, slices: Sequence, atlas_frame=None, chrono_snapshot=None):
        self.volume = ZSpaceVolume.from_slices(slices)
        self.atlas_frame, self.chrono_snapshot = atlas_frame, chrono_snapshot

    def depth(self) -> int:
        return self.volume.depth

    def slice_shape(self) -> tuple:
        return (self.volume.height, self.volume.width)

    def profile(self) -> ZSliceProfile:
        return self.volume.profile()

    def telemetry_report(self) -> ZSpaceTelemetryReport:
        return self.volume.telemetry_report()


class ZSpaceStreamFrameAggregator:
    """Concatenates stream frames along depth, keeping at most ``max_depth`` of the newest slices."""

    def __init__(self, max_depth: Optional[int] = None):
        self._slices: List[torch.Tensor] = []
        self.atlas_frame = None
        self.chrono_snapshot = None
        self.max_depth = None
        self.set_max_depth(max_depth)

    def set_max_depth(self, max_depth: Optional[int]) -> None:
        if max_depth is not None and max_depth <= 0:
            raise TensorError("invalid value: z_stream_max_depth")
        self.max_depth = max_depth
        if max_depth is not None:
            self.prune_oldest(max_depth)

    def __len__(self) -> int:
        return len(self._slices)

    def is_empty(self) -> bool:
        return not self._slices

    def slice_shape(self) -> Optional[tuple]:
        return tuple(self._slices[0].shape) if self._slices else None

    def extend(self, frame: ZSpaceStreamFrame) -> None:
        if self._slices and tuple(self._slices[0].shape) != frame.slice_shape():
            raise TensorError(f"shape mismatch: slices {frame.slice_shape()} against {tuple(self._slices[0].shape)}")
        self._slices.extend(frame.volume.voxels.unbind(0))
        if frame.atlas_frame is not None:
            self.atlas_frame = frame.atlas_frame
        if frame.chrono_snapshot is not None:
            self.chrono_snapshot = frame.chrono_snapshot
        if self.max_depth is not None:
            self.prune_oldest(self.max_depth)

    def prune_oldest(self, keep: int) -> None:
        if len(self._slices) > keep:
            self._slices = self._slices[len(self._slices) - keep:]

    def clear(self) -> None:
        self._slices, self.atlas_frame, self.chrono_snapshot = [], None, None

    def as_frame(self) -> Optional[ZSpaceStreamFrame]:
        return ZSpaceStreamFrame(self._slices, self.atlas_frame, self.chrono_snapshot) if self._slices else None

    def telemetry_report(self) -> Optional[ZSpaceTelemetryReport]:
        f = self.as_frame()
        return None if f is None else f.telemetry_report()
