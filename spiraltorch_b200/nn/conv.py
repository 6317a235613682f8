"""N-dimensional convolutions and pooling on channel-major flattened rows.

Every layer takes ``(batch, C·spatial)`` rows (NCHW-style flattening), stores its weight as
``(OC, IC·prod(kernel))`` and its bias as ``(1, OC)`` under ``{name}::weight`` / ``{name}::bias``, and
computes ``im2col → GEMM → +bias`` — the same decomposition as the reference
(crates/st-nn/src/layers/conv.rs:607 Conv2d, :1017 Conv3d, :1580 Conv4d, :2242 Conv6da,
:2750 MaxPool2d, :3074 AvgPool2d; crates/st-nn/src/layers/wave_scan.rs:179 WaveScan).  The GEMM goes
through the framework's matmul, i.e. the tcgen05 kernel on CUDA and PyTorch on CPU; the im2col
gather is a strided view (``unfold``) so nothing is materialised twice.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn.functional as F

from ..tensor import TensorError
from .fields import Conv1d
from .modules import Module, WaveGate, _mm


def _tup(v, n: int, what: str) -> tuple:
    t = (v,) * n if isinstance(v, int) else tuple(int(x) for x in v)
    if len(t) != n:
        raise TensorError(f"{what} needs {n} values, got {len(t)}")
    return t


class _ConvNd(Module):
    ND = 2

    def __init__(self, name: str, in_channels: int, out_channels: int, kernel, stride, padding, dilation, input_dims):
        super().__init__()
        n = self.ND
        self.name, self.ic, self.oc = name, int(in_channels), int(out_channels)
        self.kernel, self.stride = _tup(kernel, n, "kernel"), _tup(stride, n, "stride")
        self.padding, self.dilation = _tup(padding, n, "padding"), _tup(dilation, n, "dilation")
        self.input_dims = _tup(input_dims, n, "input dims")
        if min(self.ic, self.oc, *self.kernel, *self.stride, *self.dilation, *self.input_dims) < 1:
            raise TensorError(f"{name}: channels, kernel, stride, dilation and input dims must be positive")
        self.output_dims = tuple((d + 2 * p - dl * (k - 1) - 1) // s + 1 for d, p, dl, k, s in
                                 zip(self.input_dims, self.padding, self.dilation, self.kernel, self.stride))
        if min(self.output_dims) < 1:
            raise TensorError(f"{name}: kernel does not fit the padded input")
        span = self.ic * math.prod(self.kernel)
        count = self.oc * span
        # deterministic ramp 0.01, 0.02, … scaled so that the largest weight stays below one
        w = torch.arange(1, count + 1, dtype=torch.float32) * (0.01 / max(1.0, count * 0.01))
        self._register(f"{name}::weight", w.reshape(self.oc, span))
        self._register(f"{name}::bias", torch.zeros(1, self.oc))

    def output_shape(self) -> tuple:
        return (self.oc,) + self.output_dims

    def _cols(self, x: torch.Tensor) -> torch.Tensor:
        """im2col: ``[B·prod(out), IC·prod(kernel)]`` built from strided windows."""
        b = x.shape[0]
        img = x.reshape(b, self.ic, *self.input_dims)
        pad = []
        for p in reversed(self.padding):
            pad += [p, p]
        img = F.pad(img, pad)
        for axis, (k, s, dl) in enumerate(zip(self.kernel, self.stride, self.dilation)):
            span = dl * (k - 1) + 1
            win = img.unfold(2 + axis, span, s)                      # [..., out_axis, ..., span]
            img = win[..., ::dl]                                     # keep the k dilated taps
        # img: [B, IC, out..., k...] → [B, out..., IC, k...]
        n = self.ND
        perm = [0] + list(range(2, 2 + n)) + [1] + list(range(2 + n, 2 + 2 * n))
        return img.permute(perm).reshape(b * math.prod(self.output_dims), self.ic * math.prod(self.kernel))

    def _fwd(self, x, p):
        expect = self.ic * math.prod(self.input_dims)
        if x.shape[1] != expect:
            raise TensorError(f"{self.name}: expected {expect} columns, got {x.shape[1]}")
        b = x.shape[0]
        y = _mm(self._cols(x), p[f"{self.name}::weight"].t().contiguous()) + p[f"{self.name}::bias"]
        return y.reshape(b, math.prod(self.output_dims), self.oc).permute(0, 2, 1).reshape(b, -1)


class Conv2d(_ConvNd):
    ND = 2

    def __init__(self, name, in_channels, out_channels, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                 input_hw=(1, 1)):
        super().__init__(name, in_channels, out_channels, kernel, stride, padding, dilation, input_hw)


class Conv3d(_ConvNd):
    ND = 3

    def __init__(self, name, in_channels, out_channels, kernel, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1),
                 input_dhw=(1, 1, 1)):
        super().__init__(name, in_channels, out_channels, kernel, stride, padding, dilation, input_dhw)


class Conv4d(_ConvNd):
    ND = 4

    def __init__(self, name, in_channels, out_channels, kernel, stride=(1, 1, 1, 1), padding=(0, 0, 0, 0),
                 dilation=(1, 1, 1, 1), input_dims=(1, 1, 1, 1)):
        super().__init__(name, in_channels, out_channels, kernel, stride, padding, dilation, input_dims)


_LEECH_PACKING_DENSITY = math.pi ** 12 / math.factorial(12)
DEFAULT_CONV6DA_OFFSETS = ((0, 0, 0), (1, 0, 0), (-1, 0, 0), (0, 1, 0), (0, -1, 0), (0, 0, 1), (0, 0, -1))


def ramanujan_pi(order: int) -> float:
    """Partial sum of Ramanujan's 1/π series with ``order`` terms."""
    s = 0.0
    for k in range(max(order, 1)):
        s += math.factorial(4 * k) * (1103 + 26390 * k) / (math.factorial(k) ** 4 * 396 ** (4 * k))
    return 9801.0 / (2.0 * math.sqrt(2.0) * s)


class Conv6da(Module):
    """Six-neighbour (plus centre) adjacency convolution on a ``(D, H, W)`` grid with a Leech-lattice
    density term: per cell, the neighbour values of every input channel are gathered (zeros outside
    the grid), ``density = weight · Λ₂₄ packing density · ‖neighbours‖₂ · √rank`` is added to every
    output channel together with the bias, and the gathered vector is multiplied by the
    ``(OC, IC·neighbours)`` weight.  As in the reference's backward, the density term is treated as
    a constant of the input."""

    def __init__(self, name: str, in_channels: int, out_channels: int, grid: Sequence[int], leech_rank: int = 24,
                 leech_weight: float = 0.0, offsets: Sequence[Sequence[int]] = DEFAULT_CONV6DA_OFFSETS):
        super().__init__()
        self.name, self.ic, self.oc = name, int(in_channels), int(out_channels)
        self.grid = _tup(grid, 3, "grid")
        self.offsets = tuple(tuple(int(v) for v in o) for o in offsets)
        if min(self.ic, self.oc, *self.grid) < 1:
            raise TensorError(f"{name}: channels and grid dims must be positive")
        if not self.offsets:
            raise TensorError("conv6da_neighbors is empty")
        self.leech_scale = max(float(leech_weight), 0.0) * _LEECH_PACKING_DENSITY * math.sqrt(max(int(leech_rank), 1))
        self.pi_delta = ramanujan_pi(6) - math.pi
        span = self.ic * len(self.offsets)
        vals, seed = [], 0.01
        for _ in range(self.oc * span):
            vals.append(seed)
            seed = max((seed * 1.31) % 0.2, 1e-3)
        self._register(f"{name}::weight", torch.tensor(vals, dtype=torch.float32).reshape(self.oc, span))
        self._register(f"{name}::bias", torch.zeros(1, self.oc))

    def neighbor_count(self) -> int:
        return len(self.offsets)

    def _gather(self, x: torch.Tensor) -> torch.Tensor:
        """``[B, cells, neighbours·IC]`` with neighbour-major, channel-minor ordering."""
        b = x.shape[0]
        d, h, w = self.grid
        vol = x.reshape(b, self.ic, d, h, w)
        outs = []
        for od, oh, ow in self.offsets:
            shifted = torch.zeros_like(vol)
            sd = slice(max(0, -od), d - max(0, od)), slice(max(0, od), d - max(0, -od))
            sh = slice(max(0, -oh), h - max(0, oh)), slice(max(0, oh), h - max(0, -oh))
            sw = slice(max(0, -ow), w - max(0, ow)), slice(max(0, ow), w - max(0, -ow))
            if abs(od) < d and abs(oh) < h and abs(ow) < w:
                shifted[:, :, sd[0], sh[0], sw[0]] = vol[:, :, sd[1], sh[1], sw[1]]
            outs.append(shifted.reshape(b, self.ic, -1).transpose(1, 2))         # [B, cells, IC]
        return torch.cat(outs, dim=2)

    def _fwd(self, x, p):
        cells = math.prod(self.grid)
        if x.shape[1] != self.ic * cells:
            raise TensorError(f"{self.name}: expected {self.ic * cells} columns, got {x.shape[1]}")
        b = x.shape[0]
        nb = self._gather(x)
        geodesic = nb.detach().double().norm(dim=2)
        density = torch.where(geodesic > 2.220446049250313e-16, geodesic * self.leech_scale,
                              torch.zeros_like(geodesic)).float() if self.leech_scale > 2.220446049250313e-16 \
            else torch.zeros(b, cells, device=x.device)
        y = _mm(nb.reshape(b * cells, -1), p[f"{self.name}::weight"].t().contiguous()) + p[f"{self.name}::bias"]
        y = y.reshape(b, cells, self.oc) + (density + self.pi_delta).unsqueeze(-1)
        return y.permute(0, 2, 1).reshape(b, -1)


ZConv6DA = Conv6da


class _Pool2d(Module):
    MODE = "max"

    def __init__(self, channels: int, kernel, stride=None, padding=(0, 0), input_hw=(1, 1)):
        super().__init__()
        self.c = int(channels)
        self.kernel = _tup(kernel, 2, "kernel")
        self.stride = _tup(stride if stride else kernel, 2, "stride")
        self.padding, self.input_hw = _tup(padding, 2, "padding"), _tup(input_hw, 2, "input_hw")
        self.output_hw = tuple((d + 2 * p - k) // s + 1 for d, p, k, s in
                               zip(self.input_hw, self.padding, self.kernel, self.stride))
        if self.c < 1 or min(self.output_hw) < 1:
            raise TensorError("pooling window does not fit the input")

    def _fwd(self, x, p):
        if x.shape[1] != self.c * math.prod(self.input_hw):
            raise TensorError(f"pool: expected {self.c * math.prod(self.input_hw)} columns, got {x.shape[1]}")
        img = x.reshape(x.shape[0], self.c, *self.input_hw)
        if self.MODE == "max":
            y = F.max_pool2d(img, self.kernel, self.stride, self.padding)
        else:
            y = F.avg_pool2d(img, self.kernel, self.stride, self.padding, count_include_pad=True)
        return y.reshape(x.shape[0], -1)


class MaxPool2d(_Pool2d):
    MODE = "max"


class AvgPool2d(_Pool2d):
    MODE = "avg"


class WaveScan(Module):
    """``Conv1d`` over the step axis → ``WaveGate`` per step → the last step's features.

    Input rows are ``(batch, in_channels·steps)``; the output is ``(batch, features)``."""

    def __init__(self, name: str, in_channels: int, features: int, kernel_size: int, steps: int, *, stride: int = 1,
                 padding: int = 0, curvature: float = -1.0, temperature: float = 1.0):
        super().__init__()
        if in_channels < 1 or features < 1:
            raise TensorError("WaveScan needs positive in_channels and features")
        self.name, self.ic, self.features, self.steps = name, in_channels, features, steps
        self.conv = Conv1d(f"{name}::conv", in_channels, features, kernel_size, steps, stride=stride, padding=padding)
        self.gate = WaveGate(f"{name}::gate", features, curvature, temperature)
        self._params.extend(self.conv.parameters() + self.gate.parameters())

    def _fwd(self, x, p):
        b = x.shape[0]
        seq = self.conv._fwd(x, p).reshape(b, self.features, -1)            # [B, F, out_steps]
        out_steps = seq.shape[2]
        gated = self.gate._fwd(seq.permute(0, 2, 1).reshape(b * out_steps, self.features), p)
        return gated.reshape(b, out_steps, self.features)[:, -1]
