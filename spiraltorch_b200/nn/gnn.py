"""Graph layers: normalised-adjacency context, Z-space graph convolution with multi-hop
aggregation, a stacked network, graph read-outs and a batched regressor.

Restated from crates/st-nn/src/gnn: ``GraphContext`` (context.rs:10-160 — self loops, symmetric
``D^-1/2 A D^-1/2`` or row ``D^-1 A`` normalisation, ``propagate``), ``ZSpaceGraphConvolution``
(layer.rs:174-520 — weights initialised 0.01, 0.02, ...; support = Σ_h w_h · Â^h X with optional
self term, attenuation and sum / mean reducer; output = support · W + b), ``GraphReadout`` and the
regressors (readout.rs:20-700).  Propagation and the kernel product run on the GEMM for CUDA tensors.
"""
from __future__ import annotations

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

    def set_aggregation(self, aggregation: NeighborhoodAggregation) -> None:
        aggregation.validate()
        self.aggregation = aggregation

    def with_aggregation(self, aggregation: NeighborhoodAggregation) -> "ZSpaceGraphConvolution":
        self.set_aggregation(aggregation)
        return self

    def _support(self, x: torch.Tensor) -> torch.Tensor:
        cur, support = x, torch.zeros_like(x)
        for h, w in enumerate(self.aggregation.weights()):
            if h > 0:
                cur = self.context.propagate_t(cur)
            if abs(w) > 1.1920929e-07:
                support = support + w * cur
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
