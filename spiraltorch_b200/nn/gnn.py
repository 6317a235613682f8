"""Graph layers: normalised-adjacency context, Z-space graph convolution with multi-hop
aggregation, a stacked network, graph read-outs and a batched regressor.

Restated from crates/st-nn/src/gnn: ``GraphContext`` (context.rs:10-160 — self loops, symmetric
``D^-1/2 A D^-1/2`` or row ``D^-1 A`` normalisation, ``propagate``), ``ZSpaceGraphConvolution``
(layer.rs:174-520 — weights initialised 0.01, 0.02, ...; support = Σ_h w_h · Â^h X with optional
self term, attenuation and sum / mean reducer; output = support · W + b), ``GraphReadout`` and the
regressors (readout.rs:20-700).  Propagation and the kernel product run on the GEMM for CUDA tensors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..tensor import Tensor, TensorError
from .modules import Module, _mm, _t


class GraphContext:
    def __init__(self, adjacency, self_loop_weight: float = 1.0, normalisation: str = "symmetric"):
        a = _t(adjacency).float()
        if a.dim() != 2 or a.shape[0] != a.shape[1] or a.shape[0] == 0:
            raise TensorError(f"adjacency must be a non-empty square matrix, got {tuple(a.shape)}")
        if not bool(torch.isfinite(a).all()) or bool((a < 0).any()):
            raise TensorError("adjacency weights must be finite and non-negative")
        if normalisation not in ("symmetric", "row"):
            raise TensorError(f"unknown normalisation '{normalisation}'")
        a = a + self_loop_weight * torch.eye(a.shape[0], device=a.device)
        deg = a.sum(1).clamp(min=1e-12)
        if normalisation == "symmetric":
            d = deg.rsqrt()
            self.norm_adjacency = d[:, None] * a * d[None, :]
        else:
            self.norm_adjacency = a / deg[:, None]
        self.normalisation = normalisation
        self._row_sums = self.norm_adjacency.sum(1)

    @classmethod
    def from_adjacency(cls, adjacency) -> "GraphContext":
        return cls(adjacency)

    @classmethod
    def with_self_loops(cls, adjacency, self_loop_weight: float) -> "GraphContext":
        return cls(adjacency, self_loop_weight)

    def node_count(self) -> int:
        return self.norm_adjacency.shape[0]

    def row_sums(self) -> list:
        return self._row_sums.tolist()

    def to(self, device) -> "GraphContext":
        self.norm_adjacency = self.norm_adjacency.to(device)
        self._row_sums = self._row_sums.to(device)
        return self

    def propagate_t(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[0] != self.node_count():
            raise TensorError(f"features have {x.shape[0]} rows, the graph has {self.node_count()} nodes")
        return _mm(self.norm_adjacency.to(x.device), x)

    def propagate(self, features: Tensor) -> Tensor:
        return Tensor._wrap(self.propagate_t(_t(features)))

    def measure_flows(self, features: Tensor) -> list:
        f = _t(features)
        return [{"node_index": i, "incoming_weight": float(self._row_sums[i]), "aggregated_norm": float(f[i].abs().sum())}
                for i in range(self.node_count())]


@dataclass
class NeighborhoodAggregation:
    hops: int = 1
    include_self: bool = False
    attenuation: float = 1.0
    reducer: str = "sum"            # "sum" | "mean"
    single: bool = True

    @classmethod
    def multi_hop_sum(cls, hops: int) -> "NeighborhoodAggregation":
        return cls(hops, True, 1.0, "sum", False)

    @classmethod
    def multi_hop_mean(cls, hops: int) -> "NeighborhoodAggregation":
        return cls(hops, True, 1.0, "mean", False)

    def validate(self) -> None:
        if self.hops < 1:
            raise TensorError("aggregation needs at least one hop")
        if not (self.attenuation > 0 and self.attenuation == self.attenuation):
            raise TensorError("attenuation must be positive and finite")
        if self.reducer not in ("sum", "mean"):
            raise TensorError(f"unknown reducer '{self.reducer}'")

    def weights(self) -> list:
        """Coefficient of Â^h X for h = 0 .. hops."""
        if self.single:
            return [0.0, 1.0]
        w = [1.0 if self.include_self else 0.0] + [self.attenuation ** (h - 1) for h in range(1, self.hops + 1)]
        if self.reducer == "mean":
            mass = sum(abs(v) for v in w) or 1.0
            w = [v / mass for v in w]
        return w


# ---- roundtable influence on message passing -------------------------------------------------------------------------
GNN_ROUNDTABLE_MAX_HISTORY_SIGNALS = 4096
_F32_MAX = 3.4028234663852886e38


class RoundtableBandSignal:
    """One roundtable observation for graph modules: band energies (+ drift and an optional spectral sample of the
    gradient) and the schedule's band sizes (crates/st-nn/src/gnn/mod.rs:44-230)."""

    def __init__(self, above: float, here: float, beneath: float, band_sizes, drift: float = 0.0, spectral=None,
                 issued_at: Optional[float] = None):
        import time
        from .zrba import SpectralFeatureSample
        self.above, self.here, self.beneath, self.drift = float(above), float(here), float(beneath), float(drift)
        self.band_sizes = tuple(int(v) for v in band_sizes)
        self.spectral = spectral or SpectralFeatureSample()
        self.issued_at = time.time() if issued_at is None else float(issued_at)
        self.validate()

    @classmethod
    def from_schedule(cls, schedule, energy, drift: float = 0.0, spectral=None) -> "RoundtableBandSignal":
        """``schedule``: a ``RoundtableSchedule``; ``energy``: its ``band_energy`` dict or an object with the three fields."""
        get = (lambda k: energy[k]) if isinstance(energy, dict) else (lambda k: getattr(energy, k))
        n = schedule.rows * schedule.cols
        sizes = (schedule.top_k, n - schedule.top_k - schedule.bottom_k, schedule.bottom_k)
        return cls(get("above"), get("here"), get("beneath"), sizes, drift, spectral)

    def validate(self) -> None:
        sp = self.spectral
        for name, v in (("band_energy.above", self.above), ("band_energy.here", self.here), ("band_energy.beneath", self.beneath),
                        ("spectral.energy", sp.energy)):
            if not math.isfinite(v):
                raise TensorError(f"GNN roundtable field '{name}' must be finite")
            if v < 0:
                raise TensorError(f"GNN roundtable field '{name}' must be non-negative")
            if v > _F32_MAX:
                raise TensorError(f"GNN roundtable field '{name}' must be in [-f32::MAX, f32::MAX]")
        if not math.isfinite(self.drift) or abs(self.drift) > _F32_MAX:
            raise TensorError("GNN roundtable field 'band_energy.drift' must be finite")
        for name, v, lo, hi in (("spectral.sheet_confidence", sp.sheet_confidence, 0.0, 1.0), ("spectral.curvature", sp.curvature, 0.0, 4.0),
                                ("spectral.spin", sp.spin, -1.0, 1.0)):
            if not math.isfinite(v) or not lo <= v <= hi:
                raise TensorError(f"GNN roundtable field '{name}' must be in [{lo}, {hi}]")
        if len(self.band_sizes) != 3 or any(v <= 0 for v in self.band_sizes):
            raise TensorError("GNN roundtable field 'band_sizes' must hold three positive sizes")
        if not math.isfinite(self.issued_at) or self.issued_at < 0:
            raise TensorError("GNN roundtable signal timestamp must be a finite, non-negative epoch time")

    def depth(self) -> int:
        return sum(self.band_sizes)

    def as_dict(self) -> dict:
        sp = self.spectral
        return {"band_energy": {"above": self.above, "here": self.here, "beneath": self.beneath, "drift": self.drift},
                "band_sizes": {"above": self.band_sizes[0], "here": self.band_sizes[1], "beneath": self.band_sizes[2]},
                "spectral": {"sheet_index": sp.sheet_index, "sheet_confidence": sp.sheet_confidence, "curvature": sp.curvature,
                             "spin": sp.spin, "energy": sp.energy}, "issued_at": self.issued_at}

    @classmethod
    def from_dict(cls, d: dict) -> "RoundtableBandSignal":
        from .zrba import SpectralFeatureSample
        e, z = d["band_energy"], d["band_sizes"]
        return cls(e["above"], e["here"], e["beneath"], (z["above"], z["here"], z["beneath"]), e.get("drift", 0.0),
                   SpectralFeatureSample(**d.get("spectral", {})), d.get("issued_at"))


def _cl(v, lo, hi):
    return min(max(v, lo), hi)


class RoundtableBandInfluence:
    """Band multipliers and a drift bias derived from a signal, and from them one scale per message-passing hop
    (crates/st-core/src/inference/gnn_roundtable.rs:70-255): hop 0 follows the Here multiplier, hop 1 the Above
    multiplier times the drift bias, deeper hops the Beneath multiplier over the drift bias with a 5 %-per-hop decay.

    The occupancy of each band mixes its energy share with its share of the schedule (more weight on energy when the
    spectral sample is confident or the energy is lopsided); the direction combines the occupancy asymmetry with the
    spectral spin; curvature pulls weight to the Here band; lopsided energy lifts both edge bands."""

    def __init__(self, signal: RoundtableBandSignal):
        signal.validate()
        self.signal = signal
        sp = signal.spectral
        total = max(signal.above + signal.here + signal.beneath, 1.0e-6)
        bary = [_cl(v / total, 0.0, 1.0) for v in (signal.above, signal.here, signal.beneath)]
        share = [v / signal.depth() for v in signal.band_sizes]
        focus = sp.sheet_confidence
        curv = _cl(sp.curvature / 4.0, 0.0, 1.0)
        stability = _cl(abs(sp.spin) * (1.0 - curv), 0.0, 1.0)
        e_rel = _cl(0.5 + 0.35 * focus + 0.25 * _cl(abs(bary[0] - bary[2]), 0.0, 1.0), 0.55, 0.9)
        occ = [e_rel * b + (1.0 - e_rel) * s_ for b, s_ in zip(bary, share)]
        direction = _cl(0.6 * _cl(occ[0] - occ[2], -1.0, 1.0) + 0.4 * focus * sp.spin, -1.0, 1.0)
        pull = _cl(focus * curv, 0.0, 1.0)
        edge_bias = max(max(bary[0], bary[2]) - bary[1], 0.0)
        edge = _cl(0.5 * edge_bias + 0.5 * abs(direction) * focus, 0.0, 1.0)
        edge_lift, center = _cl(1.0 + 0.18 * edge, 1.0, 1.35), _cl(1.0 - 0.24 * edge, 0.72, 1.0)
        lift = _cl(0.92 + 0.16 * stability + 0.10 * edge_bias, 0.85, 1.2)
        neutrality = _cl((occ[1] + stability + pull) / 3.0, 0.0, 1.0)
        relax = _cl(1.0 - pull, 0.65, 1.0)
        m = [(0.72 + 0.62 * occ[0]) * (1.0 + 0.26 * max(direction, 0.0) + 0.12 * edge_bias) * relax * edge_lift,
             (0.78 + 0.52 * occ[1]) * (1.0 + 0.18 * pull + 0.12 * neutrality) * (1.0 + 0.07 * (1.0 - focus)) * center,
             (0.72 + 0.62 * occ[2]) * (1.0 + 0.26 * max(-direction, 0.0) + 0.12 * edge_bias) * relax * edge_lift]
        m[0 if direction > 0 else 2 if direction < 0 else 1] *= lift
        self._multipliers = tuple(_cl(v, 0.35, 1.75) for v in m)
        dbias = _cl(0.55 * math.tanh(signal.drift) + 0.45 * direction, -1.0, 1.0)
        self._drift_bias = _cl((1.0 + 0.22 * dbias) * (1.0 + 0.08 * edge) * (1.0 - 0.12 * pull) * (1.0 - 0.06 * neutrality * stability),
                               0.55, 1.45)

    from_signal = classmethod(lambda cls, signal: cls(signal))

    def multipliers(self) -> tuple:
        return self._multipliers

    def drift_bias(self) -> float:
        return self._drift_bias

    def scale_for_step(self, step: int) -> float:
        a, h, b = self._multipliers
        if step == 0:
            s = h
        elif step == 1:
            s = a * self._drift_bias
        else:
            s = b / max(self._drift_bias, 0.5)
            if step > 2:
                s *= max(1.0 - min(step - 2, 8) * 0.05, 0.6)
        return _cl(s, 0.25, 2.0)

    def band_pass_scale_for_step(self, band: str, step: int, intensity: float) -> float:
        """Extra scale while the trainer back-propagates one band (``above`` / ``here`` / ``beneath``) at a time: the hop
        that matches the band (1 / 0 / >= 2) is lifted, the others damped, in proportion to ``intensity`` in [0, 1]."""
        if not (math.isfinite(intensity) and 0.0 <= intensity <= 1.0):
            raise TensorError("GNN roundtable field 'band_pass.intensity' must be in [0, 1]")
        band = band.lower()
        if band not in ("above", "here", "beneath"):
            raise TensorError(f"unknown roundtable band '{band}'")
        avg = max(sum(self._multipliers) / 3.0, 0.35)
        focus = intensity * _cl(self._multipliers[("above", "here", "beneath").index(band)] / avg, 0.8, 1.35)
        k = min(step, 2)
        if band == "above":
            s = 1.0 + (-0.10, 0.24, -0.14)[k] * focus
        elif band == "here":
            s = 1.0 + (0.20, -0.07, -0.10)[k] * focus
        elif k < 2:
            s = 1.0 + (-0.12, -0.08)[k] * focus
        else:
            s = 1.0 + 0.24 * focus * _cl(1.0 - min(max(step - 2, 0), 3) * 0.06, 0.82, 1.0)
        return _cl(s, 0.7, 1.35)


class RoundtableGnnBridge:
    """Shares roundtable band signals with graph modules: the trainer publishes one per step, graph networks read
    the latest; a bounded history keeps the last ``history_limit`` (crates/st-nn/src/roundtable.rs:165-290)."""

    def __init__(self, history_limit: int = 64):
        import threading
        self._lock = threading.Lock()
        self._latest: Optional[RoundtableBandSignal] = None
        self._history: list = []
        self._limit = 64
        self.set_history_limit(history_limit)

    def set_history_limit(self, limit: int) -> None:
        if not 1 <= limit <= GNN_ROUNDTABLE_MAX_HISTORY_SIGNALS:
            raise TensorError("invalid value: roundtable GNN history limit")
        with self._lock:
            self._limit = int(limit)
            del self._history[:max(len(self._history) - self._limit, 0)]

    def history_limit(self) -> int:
        return self._limit

    def publish(self, signal: RoundtableBandSignal) -> RoundtableBandSignal:
        signal.validate()
        with self._lock:
            self._latest = signal
            self._history.append(signal)
            del self._history[:max(len(self._history) - self._limit, 0)]
        return signal

    def record(self, schedule, energy, drift: float = 0.0, spectral=None) -> RoundtableBandSignal:
        return self.publish(RoundtableBandSignal.from_schedule(schedule, energy, drift, spectral))

    def latest(self) -> Optional[RoundtableBandSignal]:
        return self._latest

    def drain(self) -> list:
        with self._lock:
            out, self._history = self._history, []
        return out

    def __len__(self) -> int:
        return len(self._history)

    def is_empty(self) -> bool:
        return not self._history

    def snapshot_state(self) -> dict:
        with self._lock:
            return {"latest": None if self._latest is None else self._latest.as_dict(), "history": [s.as_dict() for s in self._history],
                    "history_limit": self._limit}

    def restore_state(self, state: dict) -> None:
        latest = None if state.get("latest") is None else RoundtableBandSignal.from_dict(state["latest"])
        history = [RoundtableBandSignal.from_dict(d) for d in state.get("history", ())]
        limit = int(state.get("history_limit", 64))
        if not 1 <= limit <= GNN_ROUNDTABLE_MAX_HISTORY_SIGNALS or len(history) > limit:
            raise TensorError("invalid value: roundtable GNN bridge state")
        with self._lock:
            self._latest, self._history, self._limit = latest, history, limit


class ZSpaceGraphConvolution(Module):
    def __init__(self, name: str, context: GraphContext, input_dim: int, output_dim: int, curvature: float = -1.0,
                 learning_rate: float = 1e-2):
        super().__init__()
        if input_dim <= 0 or output_dim <= 0:
            raise TensorError(f"invalid dimensions ({input_dim}, {output_dim})")
        self.name, self.context, self.curvature = name, context, curvature
        n = input_dim * output_dim
        self.weight = self._register(f"{name}::weight", (torch.arange(1, n + 1, dtype=torch.float32) * 0.01)
                                     .reshape(input_dim, output_dim))
        self.bias = self._register(f"{name}::bias", torch.zeros(1, output_dim))
        self.attach_hypergrad(curvature, learning_rate)
        self.aggregation = NeighborhoodAggregation()
        self.last_flows: Optional[list] = None
        self.roundtable: Optional[RoundtableBandInfluence] = None
        self.active_band_pass: Optional[tuple] = None       # (band, intensity) while one band is back-propagated
        self.last_step_scales: list = []

    def set_roundtable_influence(self, influence: Optional["RoundtableBandInfluence"]) -> None:
        self.roundtable = influence

    def set_active_band_pass(self, band: Optional[str], intensity: float = 1.0) -> None:
        self.active_band_pass = None if band is None else (band, float(intensity))

    def set_aggregation(self, aggregation: NeighborhoodAggregation) -> None:
        aggregation.validate()
        self.aggregation = aggregation

    def with_aggregation(self, aggregation: NeighborhoodAggregation) -> "ZSpaceGraphConvolution":
        self.set_aggregation(aggregation)
        return self

    def _support(self, x: torch.Tensor) -> torch.Tensor:
        cur, support = x, torch.zeros_like(x)
        scales = []
        for h, w in enumerate(self.aggregation.weights()):
            if h > 0:
                cur = self.context.propagate_t(cur)
            scale = 1.0
            if self.roundtable is not None:
                scale = self.roundtable.scale_for_step(h)
                if self.active_band_pass is not None:
                    scale *= self.roundtable.band_pass_scale_for_step(self.active_band_pass[0], h, self.active_band_pass[1])
            scales.append(scale)
            if abs(w * scale) > 1.1920929e-07:
                support = support + (w * scale) * cur
        self.last_step_scales = scales
        return support

    def _fwd(self, x, params):
        if x.shape[0] != self.context.node_count():
            raise TensorError(f"input has {x.shape[0]} rows, the graph has {self.context.node_count()} nodes")
        return _mm(self._support(x), params[f"{self.name}::weight"]) + params[f"{self.name}::bias"]


class ZSpaceGraphNetwork(Module):
    """Graph convolutions with ReLU between them (none after the last)."""

    def __init__(self, name: str, context: GraphContext, dims: Sequence[int], curvature: float = -1.0,
                 learning_rate: float = 1e-2):
        super().__init__()
        if len(dims) < 2:
            raise TensorError("a graph network needs at least an input and an output width")
        self.layers = [ZSpaceGraphConvolution(f"{name}.{i}", context, a, b, curvature, learning_rate)
                       for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))]
        for layer in self.layers:
            self._params.extend(layer.parameters())

    def _fwd(self, x, params):
        for i, layer in enumerate(self.layers):
            x = layer._fwd(x, params)
            if i + 1 < len(self.layers):
                x = torch.relu(x)
        return x

    def apply_roundtable_band(self, signal: RoundtableBandSignal) -> RoundtableBandInfluence:
        influence = RoundtableBandInfluence(signal)
        for layer in self.layers:
            layer.set_roundtable_influence(influence)
        return influence

    def clear_roundtable_band(self) -> None:
        for layer in self.layers:
            layer.set_roundtable_influence(None)

    def attach_roundtable_bridge(self, bridge: RoundtableGnnBridge) -> None:
        """Every ``refresh_roundtable()`` (the trainer calls it before a step) adopts the bridge's latest signal."""
        self._roundtable_bridge = bridge

    def refresh_roundtable(self) -> bool:
        bridge = getattr(self, "_roundtable_bridge", None)
        signal = None if bridge is None else bridge.latest()
        if signal is None:
            return False
        self.apply_roundtable_band(signal)
        return True


class GraphReadout:
    def __init__(self, kind: str = "mean"):
        if kind not in ("mean", "sum", "max"):
            raise TensorError(f"unknown readout '{kind}'")
        self.kind = kind

    @classmethod
    def mean(cls):
        return cls("mean")

    @classmethod
    def sum(cls):
        return cls("sum")

    @classmethod
    def max(cls):
        return cls("max")

    def as_str(self) -> str:
        return self.kind

    def pool(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[0] == 0:
            raise TensorError("cannot pool an empty graph")
        if self.kind == "mean":
            return x.mean(0, keepdim=True)
        if self.kind == "sum":
            return x.sum(0, keepdim=True)
        return x.max(0, keepdim=True).values

    def forward(self, node_features: Tensor) -> Tensor:
        return Tensor._wrap(self.pool(_t(node_features)))


class ZSpaceGraphRegressor(Module):
    """Network + read-out: node features ``(nodes, in)`` → one graph embedding ``(1, out)``."""

    def __init__(self, network: ZSpaceGraphNetwork, readout: GraphReadout):
        super().__init__()
        self.network, self.readout = network, readout
        self._params.extend(network.parameters())

    def _fwd(self, x, params):
        return self.readout.pool(self.network._fwd(x, params))


@dataclass
class GraphBatch:
    """Graphs stacked along the node axis of one block-diagonal context: ``sizes[i]`` nodes each."""
    sizes: list

    def validate(self, total_nodes: int) -> None:
        if not self.sizes or any(s <= 0 for s in self.sizes):
            raise TensorError("every graph of a batch needs at least one node")
        if sum(self.sizes) != total_nodes:
            raise TensorError(f"batch sizes sum to {sum(self.sizes)}, the input has {total_nodes} nodes")


class ZSpaceGraphBatchRegressor(Module):
    def __init__(self, network: ZSpaceGraphNetwork, readout: GraphReadout, batch: GraphBatch):
        super().__init__()
        self.network, self.readout, self.batch = network, readout, batch
        self._params.extend(network.parameters())

    def _fwd(self, x, params):
        self.batch.validate(x.shape[0])
        h = self.network._fwd(x, params)
        return torch.cat([self.readout.pool(part) for part in torch.split(h, self.batch.sizes, 0)], 0)

    def forward_batch(self, x: Tensor, batch: GraphBatch) -> Tensor:
        self.batch = batch
        return self.forward(x)
