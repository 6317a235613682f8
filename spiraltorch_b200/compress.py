"""Model compression helpers on flat weight tensors: a quantisation-aware-training observer,
structured (block) pruning and a combined report.

Restated from crates/spiral-opt/src/quantization.rs:6-140 (EMA min/max observer; symmetric or
asymmetric levels; in-place fake quantisation with an MSE audit), pruning.rs:8-146 (zero the
``floor(blocks * target_sparsity)`` blocks of smallest L2 norm, plus every block under
``min_l2_keep``) and report.rs.  Works on CPU and CUDA tensors alike (plain PyTorch ops; none of
this is on a training hot path).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


class OptimisationError(ValueError):
    pass


@dataclass
class QatConfig:
    bit_width: int = 8
    ema_decay: float = 0.9
    clamp_value: Optional[float] = 6.0
    epsilon: float = 1e-6


@dataclass
class QuantizationReport:
    bit_width: int
    min_value: float
    max_value: float
    scale: float
    zero_point: float
    quant_error: float
    observed_steps: int


class QatObserver:
    def __init__(self, config: Optional[QatConfig] = None, leveling: str = "symmetric"):
        if leveling not in ("symmetric", "asymmetric"):
            raise OptimisationError(f"unknown leveling '{leveling}'")
        self.config, self.leveling = config or QatConfig(), leveling
        self.running_min, self.running_max, self.steps = math.inf, -math.inf, 0

    def observe(self, weights: torch.Tensor) -> None:
        if weights.numel() == 0:
            return
        lo, hi = float(weights.min()), float(weights.max())
        if self.steps == 0:
            self.running_min, self.running_max = lo, hi
        else:
            d = min(max(self.config.ema_decay, 0.0), 1.0)
            self.running_min = d * min(self.running_min, lo) + (1 - d) * lo
            self.running_max = d * max(self.running_max, hi) + (1 - d) * hi
        self.steps += 1

    def quantize(self, weights: torch.Tensor) -> QuantizationReport:
        """Fake-quantise ``weights`` in place and report the levels used."""
        c = self.config
        if weights.numel() == 0:
            return QuantizationReport(c.bit_width, 0.0, 0.0, 0.0, 0.0, 0.0, self.steps)
        if c.clamp_value is not None:
            weights.clamp_(-c.clamp_value, c.clamp_value)
        if self.leveling == "symmetric":
            m = max(abs(self.running_min), abs(self.running_max), c.epsilon)
            lo, hi = -m, m
        else:
            lo, hi = min(self.running_min, -c.epsilon), max(self.running_max, c.epsilon)
        levels = float(max(2 ** c.bit_width - 1, 1))
        scale = max(hi - lo, c.epsilon) / levels
        zero_point = round(-lo / scale) if self.leveling == "asymmetric" else 0.0
        deq = torch.round((weights.clamp(lo, hi) - lo) / scale) * scale + lo
        mse = float(((weights - deq) ** 2).mean())
        weights.copy_(deq)
        return QuantizationReport(c.bit_width, lo, hi, scale, float(zero_point), mse, self.steps)


@dataclass
class StructuredPruningConfig:
    block_size: int = 32
    target_sparsity: float = 0.5
    min_l2_keep: float = 1e-4


@dataclass
class StructuredPruningReport:
    target_sparsity: float
    achieved_sparsity: float
    block_size: int
    pruned_blocks: int
    kept_blocks: int
    l2_error: float


class StructuredPruner:
    def apply(self, weights: torch.Tensor, config: Optional[StructuredPruningConfig] = None) -> StructuredPruningReport:
        """Zero whole blocks of the flattened ``weights`` in place."""
        cfg = config or StructuredPruningConfig()
        if cfg.block_size <= 0:
            raise OptimisationError("block size must be positive")
        if not 0.0 <= cfg.target_sparsity <= 1.0:
            raise OptimisationError(f"target sparsity {cfg.target_sparsity} is outside [0, 1]")
        flat = weights.reshape(-1)
        n = flat.numel()
        if n == 0:
            return StructuredPruningReport(cfg.target_sparsity, 0.0, cfg.block_size, 0, 0, 0.0)
        blocks = -(-n // cfg.block_size)
        padded = torch.zeros(blocks * cfg.block_size, dtype=torch.float32, device=flat.device)
        padded[:n] = flat.float()
        norms = (padded.view(blocks, cfg.block_size) ** 2).sum(1)
        target = int(math.floor(blocks * cfg.target_sparsity))
        prune = norms < cfg.min_l2_keep ** 2
        if target >= blocks:
            prune[:] = True
        elif target > 0:
            idx = torch.topk(norms, target, largest=False, sorted=False).indices
            prune[idx] = True
        l2 = float(norms[prune].sum().sqrt())
        mask = (~prune).repeat_interleave(cfg.block_size)[:n]
        flat.mul_(mask.to(flat.dtype))
        pruned = int(prune.sum())
        return StructuredPruningReport(cfg.target_sparsity, pruned / blocks, cfg.block_size, pruned, blocks - pruned, l2)


@dataclass
class CompressionReport:
    original_params: int
    remaining_params: int
    quantization: Optional[QuantizationReport] = None
    pruning: Optional[StructuredPruningReport] = None
    estimated_latency_reduction: float = 0.0


def compress(weights: torch.Tensor, *, qat: Optional[QatObserver] = None,
             pruning: Optional[StructuredPruningConfig] = None) -> CompressionReport:
    """Prune, then fake-quantise ``weights`` in place; the latency estimate is the removed share."""
    n = weights.numel()
    prep = StructuredPruner().apply(weights, pruning) if pruning is not None else None
    remaining = int((weights != 0).sum())       # counted before quantisation: a symmetric grid with an
    qrep = None                                 # even number of steps has no exact zero
    if qat is not None:
        qat.observe(weights)
        qrep = qat.quantize(weights)
    return CompressionReport(n, remaining, qrep, prep, 1.0 - remaining / n if n else 0.0)
