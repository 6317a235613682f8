"""Z-RBA block: RBF attention + Beta-distributed residual gate + covariance head, with
uncertainty metrics.

Parity: crates/st-nn/src/z_rba/mod.rs:104-260 (`ZRBAConfig`, `ZRBA::forward`),
beta_residual.rs:60-280 (`BetaGate`), cov_head.rs:88-260 (`CovHead`), telemetry.rs:43-420
(`ZRBAMetrics`, `ZTelemetryBundle`).  The attention itself lives in `nn/zspace.py`.

Everything here is small dense algebra on (rows, d_model) tensors: the eigen-decompositions run
through `torch.linalg.eigh` on whichever device the inputs live on; the metrics use the exact
normal quantile / CDF (`torch.special.ndtri`, `erf`) where the reference carries rational
approximations of them.
"""
from __future__ import annotations

import math
from collections import Counter
from dataclasses import dataclass, field, asdict
from typing import Optional, Sequence

import torch

from ..tensor import Tensor, TensorError
from .modules import _t
from .zspace import AttentionTelemetry, ZFrame, ZIndex, ZMetricWeights, ZRBFAttention, ZTensor


@dataclass
class SpectralFeatureSample:
    """Summary of a gradient spectrum (crates/st-core/src/ops/zspace_round.rs:11-22)."""
    sheet_index: int = 0
    sheet_confidence: float = 0.0
    curvature: float = 0.0
    spin: float = 0.0
    energy: float = 0.0


def _finite(label: str, value: float) -> float:
    if not math.isfinite(value):
        raise TensorError(f"non-finite value for {label}: {value}")
    return value


# ----------------------------------------------------------------------------------------------
# Beta gate
# ----------------------------------------------------------------------------------------------
@dataclass
class BetaGateSample:
    sample: float
    alpha: float
    beta: float
    expected: float
    variance: float
    features: list
    applied: float

    def expected_value(self) -> float:
        return self.expected


@dataclass
class BetaGateConfig:
    momentum: float = 0.05
    seed: int = 42


def _dominant(values: Sequence[int]) -> float:
    """Most frequent value; ties go to the smaller one; 0 for an empty list."""
    if not values:
        return 0.0
    counts = Counter(values)
    best = max(counts.items(), key=lambda kv: (kv[1], -kv[0]))
    return float(best[0])


class BetaGate:
    """Maps seven spectral / index features to a Beta(alpha, beta) and draws the residual gate.

    Weights are the deterministic `tanh(0.05 cos(i) + 0.02 sin(i))` table; the exponential moving
    averages of the expected gate and its variance are only updated by successful draws.
    """

    def __init__(self, config: Optional[BetaGateConfig] = None):
        config = config or BetaGateConfig()
        i = torch.arange(14, dtype=torch.float64)
        self.weights = torch.tanh(torch.cos(i) * 0.05 + torch.sin(i) * 0.02).reshape(2, 7)
        self.bias = torch.tensor([0.1, 0.2], dtype=torch.float64)
        m = config.momentum
        self.momentum = min(max(m, 1e-4), 1.0) if math.isfinite(m) else BetaGateConfig().momentum
        self._gen = torch.Generator(device="cpu").manual_seed(int(config.seed))
        self._ema_mean, self._ema_var = 0.5, 0.25

    def ema(self) -> tuple:
        return self._ema_mean, self._ema_var

    def _features(self, stats: SpectralFeatureSample, indices: Sequence[ZIndex]) -> list:
        return [float(stats.sheet_confidence), float(stats.curvature), float(stats.spin), float(stats.energy),
                _dominant([i.band for i in indices]), float(stats.sheet_index), _dominant([i.echo for i in indices])]

    def try_forward(self, stats: SpectralFeatureSample, indices: Sequence[ZIndex]) -> BetaGateSample:
        feats = self._features(stats, indices)
        for f in feats:
            _finite("beta_gate_feature", f)
        raw = self.weights @ torch.tensor(feats, dtype=torch.float64) + self.bias
        alpha = _finite("beta_gate_alpha", float(torch.nn.functional.softplus(raw[0])) + 1e-3)
        beta = _finite("beta_gate_beta", float(torch.nn.functional.softplus(raw[1])) + 1e-3)
        conc = alpha + beta
        expected = alpha / conc
        variance = _finite("beta_gate_variance", alpha * beta / (conc * conc * (conc + 1.0)))
        # Beta(a, b) as a ratio of two Gamma draws from the gate's own generator.
        ga = torch._standard_gamma(torch.tensor([alpha, beta], dtype=torch.float64), generator=self._gen)
        sample = _finite("beta_gate_sample", float(ga[0] / ga.sum().clamp(min=1e-300)))
        out = BetaGateSample(sample, alpha, beta, expected, variance, feats, sample)
        m = self.momentum
        self._ema_mean = (1 - m) * self._ema_mean + m * expected
        self._ema_var = max((1 - m) * self._ema_var + m * variance, 1e-6)
        return out

    def forward(self, stats: SpectralFeatureSample, indices: Sequence[ZIndex]) -> BetaGateSample:
        """Like `try_forward`, but non-finite features yield the neutral Beta(1, 1) sample."""
        try:
            return self.try_forward(stats, indices)
        except TensorError:
            feats = [f if math.isfinite(f) else 0.0 for f in self._features(stats, indices)]
            return BetaGateSample(0.5, 1.0, 1.0, 0.5, 1.0 / 12.0, feats, 0.5)


# ----------------------------------------------------------------------------------------------
# Covariance head
# ----------------------------------------------------------------------------------------------
@dataclass
class CovHeadTelemetry:
    min_eigenvalue: float
    max_eigenvalue: float
    condition_number: float
    stabiliser: float


@dataclass
class CovHeadOutput:
    covariance: Tensor
    telemetry: CovHeadTelemetry


class CovHead:
    """Covariance of the rows of `mu`, truncated to `rank` eigen-directions, plus the mean diagonal
    variance, floored to a positive-definite matrix."""

    def __init__(self, rank: int, stabiliser: float = 1e-4):
        self.rank, self.stabiliser = max(1, int(rank)), float(stabiliser)

    def forward(self, mu, sigma_diag) -> CovHeadOutput:
        m, s = _t(mu).float(), _t(sigma_diag).float()
        if m.shape != s.shape:
            raise TensorError(f"shape mismatch: {tuple(s.shape)} vs {tuple(m.shape)}")
        if m.shape[0] == 0:
            raise TensorError("empty input: cov_head::forward")
        if not bool(torch.isfinite(m).all() and torch.isfinite(s).all()):
            raise TensorError("zrba_cov input is not finite")
        with torch.no_grad():
            rows = m.shape[0]
            c = (m - m.mean(0, keepdim=True)).double()
            sample = c.T @ c / rows
            w, v = torch.linalg.eigh(sample)
            k = min(self.rank, w.numel())
            top_w, top_v = w[-k:].clamp(min=0.0), v[:, -k:]
            combined = (top_v * top_w) @ top_v.T + torch.diag(s.double().mean(0).clamp(min=1e-6))
            w2, v2 = torch.linalg.eigh(0.5 * (combined + combined.T))
            adj = w2.clamp(min=self.stabiliser)
            psd = ((v2 * adj) @ v2.T).float()
            lo, hi = float(adj.min()), float(adj.max())
        tel = CovHeadTelemetry(_finite("zrba_cov_min_eigenvalue", lo), _finite("zrba_cov_max_eigenvalue", hi),
                               _finite("zrba_cov_condition_number", hi / lo if lo > 0 else math.inf), self.stabiliser)
        return CovHeadOutput(Tensor._wrap(psd), tel)


# ----------------------------------------------------------------------------------------------
# Metrics
# ----------------------------------------------------------------------------------------------
@dataclass
class ReliabilityBin:
    band: int
    expected: float
    observed: float


def _ranks(x: torch.Tensor) -> torch.Tensor:
    """Average ranks (ties share the mean of their positions)."""
    order = torch.argsort(x, stable=True)
    r = torch.empty_like(x, dtype=torch.float64)
    r[order] = torch.arange(x.numel(), dtype=torch.float64, device=x.device)
    uniq, inv = torch.unique(x, return_inverse=True)
    sums = torch.zeros(uniq.numel(), dtype=torch.float64, device=x.device).index_add_(0, inv, r)
    cnt = torch.zeros_like(sums).index_add_(0, inv, torch.ones_like(r))
    return (sums / cnt)[inv]


def spearman_rank_correlation(x, y) -> float:
    x, y = torch.as_tensor(x, dtype=torch.float64), torch.as_tensor(y, dtype=torch.float64)
    if x.numel() != y.numel() or x.numel() == 0:
        return 0.0
    rx, ry = _ranks(x), _ranks(y)
    rx, ry = rx - rx.mean(), ry - ry.mean()
    den = float(rx.norm() * ry.norm())
    return float((rx * ry).sum()) / den if den > 0 else 0.0


@dataclass
class ZRBAMetrics:
    """Interval coverage (PICP), mean interval width (PINAW), Gaussian NLL, CRPS, per-band
    reliability, and the Spearman correlation between |error| and predicted variance."""
    pin: float
    picp: float
    pinaw: float
    nll: float
    crps: float
    reliability_by_band: list = field(default_factory=list)
    ood_spearman: float = 0.0

    @classmethod
    def compute(cls, predictions, variances, targets, pin: float, indices: Sequence[ZIndex]) -> "ZRBAMetrics":
        p, v = _t(predictions).double(), _t(variances).double()
        t = torch.as_tensor(targets, dtype=torch.float64, device=p.device)
        if p.shape != v.shape:
            raise TensorError(f"shape mismatch: {tuple(v.shape)} vs {tuple(p.shape)}")
        rows, cols = p.shape
        if t.numel() != rows or len(indices) != rows:
            raise TensorError(f"data length mismatch: expected {rows}")
        if rows == 0:
            raise TensorError("empty input: zrba::metrics")
        if cols == 0:
            raise TensorError("invalid dimensions")
        pin = min(max(_finite("zrba_metrics_pin", float(pin)), 0.0), 1.0)
        q = float(torch.special.ndtri(torch.tensor(min(max(0.5 + pin / 2, 1e-6), 1 - 1e-6), dtype=torch.float64)))
        mean, var = p.mean(1), v.clamp(min=1e-6).mean(1)
        std = var.sqrt()
        lo, hi = mean - q * std, mean + q * std
        inside = (t >= lo) & (t <= hi)
        diff = t - mean
        z = diff / std
        pdf = torch.exp(-0.5 * z * z) / math.sqrt(2 * math.pi)
        cdf = 0.5 * (1 + torch.erf(z / math.sqrt(2)))
        crps = std.clamp(min=1e-6) * (z * (2 * cdf - 1) + 2 * pdf - 1 / math.sqrt(math.pi))
        nll = 0.5 * (torch.log(2 * math.pi * var) + diff * diff / var)
        bands = torch.tensor([i.band for i in indices], device=p.device)
        bins = [ReliabilityBin(int(b), pin, float(inside[bands == b].double().mean())) for b in sorted(set(bands.tolist()))]
        out = cls(pin, float(inside.double().mean()), float((hi - lo).mean()), float(nll.mean()), float(crps.mean()),
                  bins, spearman_rank_correlation(diff.abs(), var))
        for name in ("picp", "pinaw", "nll", "crps", "ood_spearman"):
            _finite("zrba_metrics_" + name, getattr(out, name))
        return out


@dataclass
class ZTelemetryBundle:
    metrics: ZRBAMetrics
    gate_mean: float
    gate_variance: float
    min_eigenvalue: float
    condition_number: float

    def to_json(self) -> dict:
        return {"metrics": asdict(self.metrics),
                "gate": {"mean": self.gate_mean, "variance": self.gate_variance},
                "covariance": {"min_eigenvalue": self.min_eigenvalue, "condition_number": self.condition_number}}


@dataclass
class ZRBATelemetry:
    attention: AttentionTelemetry
    gate: BetaGateSample
    covariance: CovHeadTelemetry

    def bundle_metrics(self, metrics: ZRBAMetrics) -> ZTelemetryBundle:
        return ZTelemetryBundle(metrics, self.gate.expected, self.gate.variance,
                                self.covariance.min_eigenvalue, self.covariance.condition_number)

    def metrics(self, predictions, variances, targets, pin: float, indices) -> ZRBAMetrics:
        return ZRBAMetrics.compute(predictions, variances, targets, pin, indices)


# ----------------------------------------------------------------------------------------------
# The block
# ----------------------------------------------------------------------------------------------
@dataclass
class ZCov:
    covariance: Tensor
    gate: BetaGateSample
    attention: AttentionTelemetry
    covariance_stats: CovHeadTelemetry


@dataclass
class ZRBAConfig:
    d_model: int = 128
    n_heads: int = 4
    metric: ZMetricWeights = field(default_factory=ZMetricWeights)
    ard: bool = True
    cov_rank: int = 8
    gate_momentum: float = 0.05
    gate_seed: int = 42
    gate_use_expected: bool = True


class ZRBA:
    """`mu' = g*mu + attn_mean`, `sigma' = g^2*sigma + attn_var`, then the covariance head on both."""

    def __init__(self, config: Optional[ZRBAConfig] = None, device="cpu"):
        config = config or ZRBAConfig()
        self.attn = ZRBFAttention(config.d_model, config.n_heads, config.metric, config.ard, device=device)
        self.gate = BetaGate(BetaGateConfig(config.gate_momentum, config.gate_seed))
        self.cov = CovHead(config.cov_rank)
        self.use_expected_gate = config.gate_use_expected

    def attention(self) -> ZRBFAttention:
        return self.attn

    def forward(self, inp: ZTensor, frame: ZFrame, stats: SpectralFeatureSample) -> tuple:
        if len(inp.indices) == 0:
            raise TensorError("empty input: zrba::forward")
        a = self.attn.forward(inp, frame)
        gate = self.gate.try_forward(stats, inp.indices)
        g = gate.expected if self.use_expected_gate else gate.sample
        gate.applied = g
        mu = _t(inp.mu).float() * g + _t(a.mean)
        sigma = _t(inp.sigma).float() * (g * g) + _t(a.variance)
        if not bool(torch.isfinite(mu).all() and torch.isfinite(sigma).all()):
            raise TensorError("zrba_output is not finite")
        cov = self.cov.forward(mu, sigma)
        out = ZTensor(Tensor._wrap(mu), Tensor._wrap(sigma), list(inp.indices))
        return (out, ZCov(cov.covariance, gate, a.telemetry, cov.telemetry),
                ZRBATelemetry(a.telemetry, gate, cov.telemetry))
