"""``SpiralLightning``: a session-bound training harness with staged plans, including the
self-supervised (InfoNCE) plan.

Restated from crates/st-nn/src/lightning.rs:63-700 (``LightningConfig`` + builder,
``LightningStage`` / ``LightningEpoch``, stage and plan reports with ``best_epoch`` /
``best_stage_index``, ``SpiralLightning::{train_epoch, fit_epochs, fit_plan, fit_selfsup_plan}``)
and crates/st-nn/src/trainer/selfsup.rs:590-720 (``InfoNCELoss`` as a ``Loss`` over a batch whose
first half are anchors and second half positives; per-batch metrics collected for the epoch).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Iterable, Optional, Sequence

import torch

from .. import plugin, selfsup
from ..tensor import Tensor, TensorError
from .losses import Loss
from .modules import Module
from .trainer import EpochStats, ModuleTrainer, RoundtableConfig, RoundtableSchedule


@dataclass
class LightningConfig:
    rows: int
    cols: int
    roundtable: RoundtableConfig = field(default_factory=RoundtableConfig)
    auto_prepare: bool = True

    @classmethod
    def builder(cls, rows: int, cols: int) -> "LightningConfigBuilder":
        return LightningConfigBuilder(rows, cols)

    def with_roundtable(self, roundtable: RoundtableConfig) -> "LightningConfig":
        return replace(self, roundtable=roundtable)

    def with_output_shape(self, rows: int, cols: int) -> "LightningConfig":
        return replace(self, rows=max(1, rows), cols=max(1, cols))

    def with_auto_prepare(self, auto_prepare: bool) -> "LightningConfig":
        return replace(self, auto_prepare=auto_prepare)

    def clamp_shape(self) -> None:
        self.rows, self.cols = max(1, self.rows), max(1, self.cols)


class LightningConfigBuilder:
    def __init__(self, rows: int, cols: int):
        self._cfg = LightningConfig(rows, cols)

    def output_shape(self, rows: int, cols: int) -> "LightningConfigBuilder":
        self._cfg = self._cfg.with_output_shape(rows, cols)
        return self

    def roundtable(self, roundtable: RoundtableConfig) -> "LightningConfigBuilder":
        self._cfg = self._cfg.with_roundtable(roundtable)
        return self

    def auto_prepare(self, auto_prepare: bool) -> "LightningConfigBuilder":
        self._cfg = self._cfg.with_auto_prepare(auto_prepare)
        return self

    def build(self) -> LightningConfig:
        self._cfg.clamp_shape()
        return self._cfg


@dataclass
class LightningStage:
    config: LightningConfig
    epochs: list = field(default_factory=list)       # each epoch: an iterable of (x, y) batches or a DataLoader
    label: Optional[str] = None

    def with_label(self, label: str) -> "LightningStage":
        self.label = label
        return self

    def add_epoch(self, batches) -> "LightningStage":
        self.epochs.append(batches)
        return self

    push_epoch = add_epoch


def _best(stats: Iterable[EpochStats]) -> Optional[EpochStats]:
    stats = [s for s in stats if s.batches > 0]
    return min(stats, key=lambda s: s.average_loss) if stats else None


@dataclass
class LightningStageReport:
    config: LightningConfig
    label: Optional[str]
    epochs: list

    def total_batches(self) -> int:
        return sum(e.batches for e in self.epochs)

    def best_epoch(self) -> Optional[EpochStats]:
        return _best(self.epochs)


@dataclass
class LightningReport:
    stages: list

    def epochs(self):
        return [e for s in self.stages for e in s.epochs]

    def total_epochs(self) -> int:
        return len(self.epochs())

    def total_batches(self) -> int:
        return sum(s.total_batches() for s in self.stages)

    def best_epoch(self) -> Optional[EpochStats]:
        return _best(self.epochs())

    def best_stage_index(self) -> Optional[int]:
        best = [(s.best_epoch().average_loss, i) for i, s in enumerate(self.stages) if s.best_epoch() is not None]
        return min(best)[1] if best else None


# ---- self-supervised plan ---------------------------------------------------------------------------
class InfoNCELoss(Loss):
    """Rows ``[0, B)`` of the prediction are anchors, rows ``[B, 2B)`` their positives; the target is
    ignored.  CUDA batches run the similarity GEMM on the tcgen05 kernel."""

    def __init__(self, temperature: float = 0.1, normalize: bool = True):
        self.temperature = temperature if (temperature > 0 and temperature == temperature) else 0.1
        self.normalize = normalize
        self._epoch_metrics: list = []

    def take_epoch_metrics(self) -> list:
        out, self._epoch_metrics = self._epoch_metrics, []
        return out

    def _split(self, pred: Tensor):
        p = pred.torch()
        if p.shape[0] % 2 != 0:
            raise TensorError(f"InfoNCELoss needs an even number of rows (anchors then positives), got {p.shape[0]}")
        b = p.shape[0] // 2
        return p[:b], p[b:]

    def forward(self, pred: Tensor, target: Tensor = None) -> Tensor:
        a, p = self._split(pred)
        res = selfsup.info_nce(a.detach(), p.detach(), self.temperature, self.normalize)
        res.logits = None
        self._epoch_metrics.append(res)
        return Tensor._wrap(torch.tensor([[res.loss]], device=a.device))

    __call__ = forward

    def backward(self, pred: Tensor, target: Tensor = None) -> Tensor:
        x = pred.torch().detach().clone().requires_grad_(True)
        b = x.shape[0] // 2
        with torch.enable_grad():
            loss, _ = selfsup.info_nce_torch(x[:b], x[b:], self.temperature, self.normalize)
            (g,) = torch.autograd.grad(loss, x)
        return Tensor._wrap(g)


@dataclass
class InfoNCEEpochMetrics:
    batches: int
    mean_loss: float
    mean_accuracy: float

    @classmethod
    def from_batches(cls, results: Sequence) -> Optional["InfoNCEEpochMetrics"]:
        if not results:
            return None
        losses = [float(r.loss) for r in results]
        accs = [float(r.top1_accuracy) for r in results]
        return cls(len(results), sum(losses) / len(losses), sum(accs) / len(accs))


@dataclass
class SelfSupStage:
    config: LightningConfig
    epochs: list = field(default_factory=list)        # each epoch: iterable of (anchors, positives) Tensor pairs
    temperature: float = 0.1
    normalize: bool = True
    label: Optional[str] = None


@dataclass
class SelfSupEpochReport:
    stats: EpochStats
    telemetry: Optional[InfoNCEEpochMetrics]


@dataclass
class SelfSupStageReport:
    config: LightningConfig
    label: Optional[str]
    epochs: list


@dataclass
class SelfSupPlanReport:
    stages: list

    def total_epochs(self) -> int:
        return sum(len(s.epochs) for s in self.stages)


class SpiralLightning:
    def __init__(self, session, rows: int = 1, cols: int = 1, config: Optional[LightningConfig] = None):
        self._session = session
        self._config = config or LightningConfig(rows, cols)
        self._config.clamp_shape()
        self._trainer: ModuleTrainer = session.trainer()
        self._schedule = self._trainer.roundtable(self._config.rows, self._config.cols, self._config.roundtable)
        self._prepared: set = set()

    @classmethod
    def with_config(cls, session, config: LightningConfig) -> "SpiralLightning":
        return cls(session, config=config)

    def session(self):
        return self._session

    def trainer(self) -> ModuleTrainer:
        return self._trainer

    def schedule(self) -> RoundtableSchedule:
        return self._schedule

    def config(self) -> LightningConfig:
        return self._config

    def set_auto_prepare(self, auto_prepare: bool) -> None:
        self._config.auto_prepare = auto_prepare

    def reconfigure(self, config: LightningConfig) -> None:
        config.clamp_shape()
        self._config = config
        self._schedule = self._trainer.roundtable(config.rows, config.cols, config.roundtable)

    def prepare_module(self, module: Module) -> None:
        self._trainer.prepare(module)
        self._prepared.add(id(module))

    def _ensure_prepared(self, module: Module) -> None:
        if self._config.auto_prepare and id(module) not in self._prepared:
            self.prepare_module(module)

    def train_epoch(self, module: Module, loss: Loss, batches) -> EpochStats:
        self._ensure_prepared(module)
        return self._trainer.train_epoch(module, loss, batches, self._schedule)

    def fit_epochs(self, module: Module, loss: Loss, epochs: Iterable) -> list:
        return [self.train_epoch(module, loss, batches) for batches in epochs]

    def fit_training_run(self, module: Module, loss: Loss, train_batches, validation_batches=None, **run_config) -> dict:
        self._ensure_prepared(module)
        return self._trainer.train_epochs(module, loss, train_batches, self._schedule,
                                          validation_batches=validation_batches, **run_config)

    def fit_plan(self, module: Module, loss: Loss, stages: Iterable[LightningStage]) -> LightningReport:
        reports = []
        for stage in stages:
            self.reconfigure(stage.config)
            stats = [self.train_epoch(module, loss, ep) for ep in stage.epochs]
            reports.append(LightningStageReport(stage.config, stage.label, stats))
        return LightningReport(reports)

    def fit_selfsup_plan(self, module: Module, stages: Iterable[SelfSupStage]) -> SelfSupPlanReport:
        out = []
        for stage in stages:
            self.reconfigure(stage.config)
            loss = InfoNCELoss(stage.temperature, stage.normalize)
            reps = []
            for epoch in stage.epochs:
                batches = []
                for anchors, positives in epoch:
                    if anchors.shape() != positives.shape():
                        raise TensorError(f"anchor / positive shape mismatch: {anchors.shape()} vs {positives.shape()}")
                    combined = anchors.cat_rows(positives)
                    batches.append((combined, Tensor.zeros(combined.shape()[0], self._config.cols, device=combined.device)))
                stats = self.train_epoch(module, loss, batches)
                tel = InfoNCEEpochMetrics.from_batches(loss.take_epoch_metrics())
                if tel is not None:
                    plugin.publish("Telemetry", {"selfsup": "info_nce", "stage": stage.label, "mean_loss": tel.mean_loss,
                                                 "mean_accuracy": tel.mean_accuracy, "batches": tel.batches})
                reps.append(SelfSupEpochReport(stats, tel))
            out.append(SelfSupStageReport(stage.config, stage.label, reps))
        return SelfSupPlanReport(out)
