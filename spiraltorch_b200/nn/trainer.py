"""``ModuleTrainer`` and the roundtable schedule of the public API.

Per batch (crates/st-nn/src/trainer.rs:7307-8566): forward → loss → output gradient → band
energy / split of the output gradient into Above / Here / Beneath (roundtable) → backward (one
pass per non-empty band when band mode is on, a single pass otherwise — the passes are linear in
the output gradient, so the accumulated result is the same) → finite checks → ``step``:
synchronise accumulators over the training device (data-parallel all-reduce **mean**), clip the
global gradient norm, apply the step → ``TrainerStep`` event.  ``EpochStart`` / ``EpochEnd``
events are published on :mod:`spiraltorch_b200.plugin`.

Roundtable split (crates/st-core/src/ops/zspace_round.rs:398-500): entries of the output
gradient are ranked by magnitude; the ``top_k`` largest form *Above*, the ``bottom_k`` smallest
non-negligible ones form *Beneath*, the rest (and everything within ``here_tolerance`` of zero)
is *Here*.  The three bands add up to the gradient.
"""
from __future__ import annotations

import copy
import hashlib
import json
import math
import time
from dataclasses import dataclass, field, asdict
from typing import Iterable, Optional, Sequence

import torch

from .. import plugin
from ..ops import native
from ..tensor import Tensor, TensorError
from .modules import Module


@dataclass
class RoundtableConfig:
    top_k: int = 8
    mid_k: int = 8
    bottom_k: int = 8
    here_tolerance: float = 1e-5
    psi_enabled: bool = False


@dataclass
class SoftLogicConfig:
    inertia: float = 0.5
    drift_gain: float = 0.0
    band_floor: float = 0.0


class RoundtableSchedule:
    def __init__(self, rows: int, cols: int, config: RoundtableConfig):
        self.rows, self.cols, self.config = rows, cols, config
        n = rows * cols
        self.top_k = max(0, min(config.top_k, n))
        self.bottom_k = max(0, min(config.bottom_k, n - self.top_k))

    def _masks(self, grad: torch.Tensor):
        flat = grad.reshape(-1)
        mag = flat.abs()
        live = mag > self.config.here_tolerance
        above = torch.zeros_like(live)
        beneath = torch.zeros_like(live)
        if self.top_k > 0 and live.any():
            k = min(self.top_k, int(live.sum()))
            idx = torch.topk(torch.where(live, mag, torch.full_like(mag, -1.0)), k).indices
            above[idx] = True
        rest = live & ~above
        if self.bottom_k > 0 and rest.any():
            k = min(self.bottom_k, int(rest.sum()))
            idx = torch.topk(torch.where(rest, -mag, torch.full_like(mag, -float("inf"))), k).indices
            beneath[idx] = True
        here = ~(above | beneath)
        return above, here, beneath

    def split(self, grad: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        g = grad.torch()
        if g.numel() != self.rows * self.cols:
            raise TensorError(f"roundtable schedule is for {self.rows}x{self.cols}, got {grad.shape()}")
        masks = self._masks(g)
        return tuple(Tensor._wrap((g.reshape(-1) * m).reshape(g.shape)) for m in masks)  # type: ignore

    def band_energy(self, grad: Tensor) -> dict:
        g = grad.torch()
        a, h, b = self._masks(g)
        sq = g.reshape(-1).pow(2)
        return {"above": float((sq * a).sum()), "here": float((sq * h).sum()), "beneath": float((sq * b).sum())}

    def describe(self) -> dict:
        return {"rows": self.rows, "cols": self.cols, **asdict(self.config)}


@dataclass
class EpochStats:
    batches: int = 0
    total_loss: float = 0.0
    average_loss: float = 0.0
    tensor_backend: dict = field(default_factory=dict)

    def as_dict(self) -> dict:
        return asdict(self)

    def __repr__(self) -> str:
        return f"EpochStats(batches={self.batches}, total_loss={self.total_loss:.6f}, average_loss={self.average_loss:.6f})"


@dataclass
class StepMetrics:
    step_time_ms: float = 0.0
    mem_peak_mb: float = 0.0
    retry_rate: float = 0.0
    extra: dict = field(default_factory=dict)


def _signal_from_trace_record(record):
    """A coherence signal from a stable ``Aggregated`` trace record; ``None`` unless the record carries a complete
    distribution witness whose re-derived summary agrees with the numbers written beside it."""
    from .. import zspace_coherence as zc
    from .amp import CoherenceSignal
    if not isinstance(record, dict) or record.get("kind") != "Aggregated":
        return None
    d = (record.get("payload") or {}).get("diagnostics") or {}
    wit = d.get("distribution_witness")
    try:
        witness = zc.DistributionWitness(**wit)
        dist = zc.validate_distribution_witness(witness)
        close = lambda a, b: a is not None and abs(a - b) <= 8 * 1.1920929e-07 * max(abs(b), 1.0)      # noqa: E731
        if d.get("distribution_channels") != dist.channels or not close(d.get("entropy"), dist.weight_entropy) \
                or not close(d.get("normalized_entropy"), dist.normalized_entropy) or not close(d.get("concentration"), dist.concentration):
            return None
        proj = zc.project(zc.DiagnosticsInput(d["mean_coherence"], d["entropy"], d["energy_ratio"], d["z_bias"], d["fractional_order"],
                                              list(witness.normalized_weights), d["preserved_channels"], d["discarded_channels"],
                                              d.get("dominant_channel")))
    except (TypeError, KeyError, zc.CoherenceProjectionError):
        return None
    if proj.control is None or proj.classification is None or proj.classification.label != d.get("classification_kind"):
        return None
    pre = d.get("pre_discard") or {}
    return CoherenceSignal(d.get("dominant_channel"), d["preserved_channels"], d["z_bias"], proj.control, proj.classification,
                           int(d.get("repaired_weights_total", 0)), int(pre.get("repairs_total", 0)))


class ModuleTrainer:
    def __init__(self, *, backend: str = "cpu", curvature: float = -1.0, hyper_learning_rate: float = 1e-2,
                 fallback_learning_rate: float = 1e-2, lane_width: Optional[int] = None,
                 subgroup: Optional[bool] = None, max_workgroup: Optional[int] = None,
                 shared_mem_per_workgroup: Optional[int] = None, band_backward: bool = False):
        if backend not in ("cpu", "cuda", "auto", "wgpu", "hip", "mps"):
            raise ValueError(f"unknown backend '{backend}'")
        if backend == "auto":
            backend = "cuda" if torch.cuda.is_available() else "cpu"
        if backend in ("wgpu", "hip", "mps"):
            raise RuntimeError(f"backend '{backend}' is not available in this build (cpu and cuda are)")
        if backend == "cuda" and not torch.cuda.is_available():
            raise RuntimeError("backend 'cuda' requested but no CUDA device is present")
        self.backend = backend
        self.device = torch.device("cuda" if backend == "cuda" else "cpu")
        self.curvature, self.hyper_learning_rate = curvature, hyper_learning_rate
        self.fallback_learning_rate = fallback_learning_rate
        self.band_backward = band_backward
        self.grad_clip_max_norm: Optional[float] = None
        self.realgrad_lr: Optional[float] = None
        self.training_device = None
        self._last_sync = {"enabled": False, "rank": 0, "world_size": 1, "buffers": 0, "values": 0}
        self.monitor = None
        self.steps = 0
        self.epoch = 0
        self.last_band_energy: Optional[dict] = None
        self.runtime_execution_plan: Optional[dict] = None

    # ---- configuration ---------------------------------------------------------------------
    def roundtable(self, rows: int, cols: int, config: Optional[RoundtableConfig] = None) -> RoundtableSchedule:
        sched = RoundtableSchedule(rows, cols, config or RoundtableConfig())
        plugin.publish("RoundtablePlanned", sched.describe())
        return sched

    def set_grad_clip_max_norm(self, max_norm: Optional[float]) -> None:
        if max_norm is not None and not max_norm > 0:
            raise ValueError("max_norm must be positive")
        self.grad_clip_max_norm = max_norm

    def enable_realgrad(self, learning_rate: float) -> None:
        self.realgrad_lr = learning_rate

    def bind_runtime_execution_plan(self, plan: dict) -> "ModuleTrainer":
        self.runtime_execution_plan = plan
        return self

    def set_training_device(self, device) -> None:
        self.training_device = device

    def clear_training_device(self) -> None:
        self.training_device = None

    def last_accumulator_sync(self) -> dict:
        return dict(self._last_sync)

    def prepare(self, module: Module) -> None:
        """Move the module to the trainer's device and attach the configured tapes."""
        module.to(self.device)
        if self.realgrad_lr is not None:
            module.attach_realgrad(self.realgrad_lr)

    def zero(self, module: Module) -> None:
        module.zero_accumulators()

    # ---- the step ---------------------------------------------------------------------------
    def _synchronize(self, module: Module) -> None:
        dev = self.training_device
        if dev is None or dev.world_size() == 1:
            self._last_sync = {"enabled": dev is not None, "rank": 0 if dev is None else dev.rank(),
                               "world_size": 1, "buffers": 0, "values": 0}
            return
        buffers = values = 0
        for p in module.parameters():
            for acc in p.accumulators():
                dev.synchronize_gradients(acc)      # all-reduce mean, in place, all-or-nothing
                buffers += 1
                values += acc.numel()
        self._last_sync = {"enabled": True, "rank": dev.rank(), "world_size": dev.world_size(),
                           "buffers": buffers, "values": values}

    def _clip(self, module: Module) -> Optional[float]:
        if self.grad_clip_max_norm is None:
            return None
        accs = [a for p in module.parameters() for a in p.accumulators()]
        if not accs:
            return 0.0
        total = math.sqrt(sum(float(a.pow(2).sum()) for a in accs))
        if total > self.grad_clip_max_norm:
            s = self.grad_clip_max_norm / (total + 1e-6)
            for a in accs:
                a.mul_(s)
        return total

    def step(self, module: Module) -> None:
        self._synchronize(module)
        self._clip(module)
        module.apply_step(self.fallback_learning_rate)
        self.steps += 1
        native.poll()     # a kernel that gave up a bounded wait left its outputs unwritten: stop training on them

    def _batches(self, batches) -> list[tuple[Tensor, Tensor]]:
        out = []
        for b in batches:
            x, y = b
            out.append((x.to(self.device) if x.device != self.device else x,
                        y.to(self.device) if y.device != self.device else y))
        return out

    def train_epoch(self, module: Module, loss, batches, schedule: Optional[RoundtableSchedule] = None) -> EpochStats:
        batches = self._batches(batches)
        self.epoch += 1
        plugin.publish("EpochStart", {"epoch": self.epoch})
        self.zero(module)
        module.train()
        stats = EpochStats(tensor_backend={"backend": self.backend, "ops_total": 0})
        from ..observability import TensorOpStepCollector
        collector = TensorOpStepCollector()
        collector.__enter__()                     # tensor-op events of this thread are folded into the epoch stats
        try:
            self._train_batches(module, loss, batches, schedule, stats)
        finally:
            collector.__exit__(None, None, None)
        stats.tensor_backend.update({k: v for k, v in collector.stats.as_dict().items() if k != "ops_total"})
        stats.tensor_backend["tensor_ops"] = collector.stats.ops_total
        stats.average_loss = stats.total_loss / max(1, stats.batches)
        plugin.publish("EpochEnd", {"epoch": self.epoch, "loss": stats.average_loss})
        return stats

    # ---- coherence-driven learning rate (crates/st-nn/src/trainer.rs:5667-5700, 7488-7545) ----------------------------
    def enable_spectral_learning_rate(self, policy=None) -> None:
        """Per step, a pending coherence signal (pushed diagnostics, or the latest ``Aggregated`` record a sequencer's
        trace recorder published on the plugin bus) is turned into roundtable band weights and a learning-rate
        multiplier; needs a roundtable schedule in ``train_epoch``."""
        from .amp import SpectralLearningRatePolicy
        self.spectral_policy = (policy or SpectralLearningRatePolicy()).apply_env_overrides()
        self.last_spectral_metrics = None
        self.enable_zspace_trace_coherence_bridge()

    def disable_spectral_learning_rate(self) -> None:
        self.spectral_policy = None
        self.last_spectral_metrics = None

    def push_coherence_diagnostics(self, diagnostics) -> bool:
        from .amp import CoherenceSignal
        self.pending_coherence = CoherenceSignal.from_diagnostics(diagnostics)
        return self.pending_coherence is not None

    def enable_zspace_trace_coherence_bridge(self) -> None:
        if getattr(self, "_coherence_bridge", None) is None:
            self._bridge_latest = None

            def on_trace(event: dict) -> None:
                sig = _signal_from_trace_record(event.get("record"))
                if sig is not None:
                    self._bridge_latest = sig
            self._coherence_bridge = plugin.subscribe("ZSpaceTrace", on_trace)

    def disable_zspace_trace_coherence_bridge(self) -> None:
        sid = getattr(self, "_coherence_bridge", None)
        if sid is not None:
            plugin.unsubscribe("ZSpaceTrace", sid)
            self._coherence_bridge = None
            self._bridge_latest = None

    def scale_learning_rates(self, module: Module, factor: float) -> None:
        if not (math.isfinite(factor) and factor > 0):
            raise TensorError(f"learning-rate factor must be positive and finite, got {factor}")
        self.fallback_learning_rate *= factor
        self.hyper_learning_rate *= factor
        if self.realgrad_lr is not None:
            self.realgrad_lr *= factor
        for p in module.parameters():
            for tape in (p.hypergrad, p.realgrad):
                if tape is not None:
                    tape.learning_rate *= factor

    def _spectral_band_weights(self, module: Module):
        policy = getattr(self, "spectral_policy", None)
        if policy is None:
            return None
        if getattr(self, "pending_coherence", None) is None and getattr(self, "_bridge_latest", None) is not None:
            self.pending_coherence, self._bridge_latest = self._bridge_latest, None
        signal, self.pending_coherence = getattr(self, "pending_coherence", None), None
        from ..inference import BandEnergy
        adj = policy.observe_signal(signal, self.curvature, BandEnergy(**self.last_band_energy))
        if adj is None:
            return None
        if math.isfinite(adj.lr_multiplier) and abs(adj.lr_multiplier - 1.0) > 1.0e-3:
            self.scale_learning_rates(module, adj.lr_multiplier)
        self.last_spectral_metrics = adj.metrics
        for w in adj.band_scale:
            if not (math.isfinite(w) and w >= 0):
                raise TensorError(f"band weight must be finite and non-negative, got {w}")
        return adj.band_scale

    def enable_autopilot(self, autopilot, apply_picks=None, device_load=None) -> None:
        """Couples an :class:`spiraltorch_b200.runtime.autopilot.Autopilot` to the step loop: before every
        batch the trainer builds the context (batch rows, feature columns, parameter count, device load), asks
        for a suggestion and hands the picks to ``apply_picks(dict)``; after the step it reports the step's
        :class:`StepMetrics` so that the bandit is credited and the device profile committed
        (the per-step hooks of crates/st-nn/src/trainer.rs:8100-8500)."""
        self.autopilot, self._apply_picks, self._device_load = autopilot, apply_picks, device_load
        self.last_autopilot_picks: dict = {}

    def enable_psi(self, meter) -> None:
        """Feeds a :class:`spiraltorch_b200.psi.PsiMeter` after every step (loss, global gradient norm, band
        energy when a roundtable schedule is active) and publishes ``PsiReading`` / ``PsiThresholdCross`` events;
        the latest reading is kept in ``last_psi``."""
        self.psi_meter, self.last_psi = meter, None

    def _psi_after(self, module, loss_value: float, grad_norm: float) -> None:
        meter = getattr(self, "psi_meter", None)
        if meter is None:
            return
        from ..psi import PsiInput
        band = sum(abs(v) for v in (self.last_band_energy or {}).values()) if getattr(self, "last_band_energy", None) else 0.0
        reading, events = meter.update(PsiInput(loss=loss_value, grad_l2=grad_norm, band_energy=band,
                                                update_ratio=self.fallback_learning_rate * grad_norm))
        self.last_psi = reading
        if plugin.has_listeners("PsiReading"):
            plugin.publish("PsiReading", {"step": reading.step, "total": reading.total,
                                          "breakdown": {c.label: v for c, v in reading.breakdown.items()}})
        for ev in events:
            plugin.publish("PsiThresholdCross", {"component": ev.component.label, "value": ev.value,
                                                 "threshold": ev.threshold, "up": ev.up, "step": ev.step})

    def attach_desire_bridge(self, bridge) -> None:
        """A :class:`spiraltorch_b200.desire_pipeline.DesireTrainerBridge` whose queued events belong to this
        trainer's resumable state."""
        self.desire_bridge = bridge

    def external_state_checkpoint(self):
        """State kept beside the module and its accumulators - psi meter, desire trainer queue, the Autopilot's
        pending selection - as one validated document (see :mod:`spiraltorch_b200.runtime.trainer_external`)."""
        from ..runtime.trainer_external import TrainerExternalCheckpointComponents
        b = TrainerExternalCheckpointComponents()
        meter = getattr(self, "psi_meter", None)
        if meter is not None:
            b.require("psi_meter").with_psi_meter(meter.checkpoint())
        bridge = getattr(self, "desire_bridge", None)
        if bridge is not None:
            b.require("desire_trainer").with_desire_trainer(bridge.checkpoint())
        ap = getattr(self, "autopilot", None)
        if ap is not None:
            b.require("autopilot").with_autopilot({"picks": dict(ap.picks), "suggestion_ready": bool(ap.suggestion_ready),
                                                   "profile_key": ap.profile_key})
        return b.build()

    def restore_external_state(self, checkpoint) -> None:
        """Inverse of :meth:`external_state_checkpoint` for the components attached to this trainer; a pending
        Autopilot suggestion cannot be revived (its bandit selection is gone) and is dropped."""
        checkpoint.validate()
        if checkpoint.psi_meter is not None and getattr(self, "psi_meter", None) is not None:
            from ..psi import PsiMeter
            self.psi_meter = PsiMeter.from_checkpoint(checkpoint.psi_meter)
        if checkpoint.desire_trainer is not None and getattr(self, "desire_bridge", None) is not None:
            self.desire_bridge.restore_checkpoint(checkpoint.desire_trainer)
        ap = getattr(self, "autopilot", None)
        if ap is not None and ap.suggestion_ready:
            ap.abandon_suggestion()

    def _autopilot_before(self, module, x) -> None:
        ap = getattr(self, "autopilot", None)
        if ap is None:
            return
        rows, cols = x.shape()
        load = float(self._device_load()) if self._device_load is not None else 0.0
        extras = [(n, 0.0) for n in ap.extra_features]
        ctx = ap.build_context(max(1, rows), max(1, cols), max(1, len(module.parameters())), load, extras)
        self.last_autopilot_picks = dict(ap.suggest(ctx)) if ctx else {}
        if self._apply_picks is not None and self.last_autopilot_picks:
            self._apply_picks(self.last_autopilot_picks)

    def _train_batches(self, module, loss, batches, schedule, stats) -> None:
        for x, y in batches:
            t0 = time.perf_counter()
            self._autopilot_before(module, x)
            pred = module.forward(x)
            value = loss.forward(pred, y)
            grad = loss.backward(pred, y)
            if schedule is not None:
                self.last_band_energy = schedule.band_energy(grad)
            weights = self._spectral_band_weights(module) if schedule is not None else None
            if schedule is not None and (self.band_backward or weights is not None):
                bands = schedule.split(grad)
                if weights is not None:
                    bands = tuple(Tensor._wrap(b.torch() * w) for b, w in zip(bands, weights))
                if self.band_backward:
                    for band in bands:
                        if float(band.torch().abs().max()) > 0.0:
                            module.backward(x, band)
                else:                                   # backward is linear in the gradient: one pass over the weighted sum
                    module.backward(x, Tensor._wrap(bands[0].torch() + bands[1].torch() + bands[2].torch()))
            else:
                module.backward(x, grad)
            for p in module.parameters():
                for a in p.accumulators():
                    if not torch.isfinite(a).all():
                        module.zero_accumulators()
                        raise TensorError(f"non-finite gradient in '{p.name}'; accumulators were cleared")
            gnorm = 0.0
            if getattr(self, "psi_meter", None) is not None:
                gnorm = math.sqrt(sum(float(a.pow(2).sum()) for p in module.parameters() for a in p.accumulators()))
            self.step(module)
            lv = float(value.torch().reshape(-1)[0])
            self._psi_after(module, lv, gnorm)
            stats.batches += 1
            stats.total_loss += lv
            stats.tensor_backend["ops_total"] += 1
            metrics = StepMetrics(step_time_ms=(time.perf_counter() - t0) * 1e3,
                                  mem_peak_mb=(torch.cuda.max_memory_allocated() / 2 ** 20) if self.device.type == "cuda" else 0.0,
                                  extra={"loss": lv, **({f"band_{k}": v for k, v in (self.last_band_energy or {}).items()})})
            if self.monitor is not None:
                self.monitor.observe(metrics)
            if getattr(self, "autopilot", None) is not None and self.autopilot.suggestion_ready:
                self.autopilot.report(metrics)
            plugin.publish("TrainerStep", {"step": self.steps, "epoch": self.epoch, "loss": lv,
                                           "step_time_ms": metrics.step_time_ms})

    def evaluate_epoch(self, module: Module, loss, batches) -> EpochStats:
        module.eval()
        stats = EpochStats(tensor_backend={"backend": self.backend})
        for x, y in self._batches(batches):
            stats.total_loss += float(loss.forward(module.forward(x), y).torch().reshape(-1)[0])
            stats.batches += 1
        stats.average_loss = stats.total_loss / max(1, stats.batches)
        module.train()
        return stats

    def train_epochs(self, module: Module, loss, batches, schedule=None, *, epochs: int = 1,
                     validation_batches=None, patience: Optional[int] = None, min_delta: float = 0.0,
                     shuffle_seed: Optional[int] = None, restore_best: bool = False) -> dict:
        batches = list(batches)
        history, best, best_state, bad = [], float("inf"), None, 0
        stopped_early = False
        for e in range(epochs):
            order = list(range(len(batches)))
            if shuffle_seed is not None:
                g = torch.Generator().manual_seed(shuffle_seed + e)
                order = torch.randperm(len(batches), generator=g).tolist()
            st = self.train_epoch(module, loss, [batches[i] for i in order], schedule)
            rec = {"epoch": e + 1, "batches": st.batches, "average_loss": st.average_loss}
            metric = st.average_loss
            if validation_batches is not None:
                vs = self.evaluate_epoch(module, loss, validation_batches)
                rec["validation"] = {"batches": vs.batches, "average_loss": vs.average_loss}
                metric = vs.average_loss
            history.append(rec)
            if metric < best - min_delta:
                best, bad = metric, 0
                if restore_best:
                    best_state = [(n, t.clone()) for n, t in module.state_dict()]
            else:
                bad += 1
                if patience is not None and bad >= patience:
                    stopped_early = True
                    break
        if restore_best and best_state is not None:
            module.load_state_dict(best_state)
        return {"epochs": history, "best_metric": best, "stopped_early": stopped_early,
                "epochs_run": len(history)}

    # ---- checkpoints ---------------------------------------------------------------------------
    def optimizer_checkpoint(self, module: Module) -> dict:
        """Per-parameter accumulator state with a fingerprint of the parameter value
        (crates/st-nn/src/module.rs:115-129)."""
        entries = []
        for p in module.parameters():
            entries.append({
                "name": p.name, "rows": p.value.shape[0], "cols": p.value.shape[1],
                "value_fingerprint": hashlib.sha256(p.value.cpu().numpy().tobytes()).hexdigest(),
                "euclidean_gradient": None if p.gradient is None else p.gradient.cpu().reshape(-1).tolist(),
                "hypergrad": None if p.hypergrad is None else p.hypergrad.checkpoint(),
                "realgrad": None if p.realgrad is None else p.realgrad.checkpoint(),
            })
        return {"kind": "spiraltorch.trainer_optimizer", "contract_version": "v2", "steps": self.steps,
                "epoch": self.epoch, "parameters": entries}

    def restore_optimizer_checkpoint(self, module: Module, ck: dict) -> None:
        """Prepare-all-then-commit; refuses a parameter whose value fingerprint changed
        (crates/st-nn/src/module.rs:131-185)."""
        from ..optim.amegagrad import AmegaHypergrad, AmegaRealgrad
        by_name = {p.name: p for p in module.parameters()}
        staged = []
        for e in ck["parameters"]:
            p = by_name.get(e["name"])
            if p is None:
                raise KeyError(f"checkpoint has unknown parameter '{e['name']}'")
            if tuple(p.value.shape) != (e["rows"], e["cols"]):
                raise TensorError(f"shape mismatch for '{e['name']}'")
            fp = hashlib.sha256(p.value.cpu().numpy().tobytes()).hexdigest()
            if fp != e["value_fingerprint"]:
                raise ValueError(f"parameter '{e['name']}' changed since the checkpoint (fingerprint mismatch)")
            staged.append((p, e))
        for p, e in staged:
            dev = p.value.device
            p.gradient = None if e["euclidean_gradient"] is None else \
                torch.tensor(e["euclidean_gradient"], device=dev).reshape(p.value.shape)
            p.hypergrad = None if e["hypergrad"] is None else AmegaHypergrad.from_checkpoint(e["hypergrad"], dev)
            p.realgrad = None if e["realgrad"] is None else AmegaRealgrad.from_checkpoint(e["realgrad"], dev)
        self.steps, self.epoch = ck.get("steps", self.steps), ck.get("epoch", self.epoch)

    def runtime_checkpoint_bundle(self, module: Module) -> dict:
        """``TrainerRuntimeCheckpointBundle`` (crates/st-core/src/runtime/trainer_checkpoint.rs:23-48):
        optimizer state + external resources (training-device identity), each with a sha256."""
        opt = self.optimizer_checkpoint(module)
        external = {"training_device": None if self.training_device is None else self.training_device.checkpoint(),
                    "grad_clip_max_norm": self.grad_clip_max_norm, "backend": self.backend}
        enc = lambda d: hashlib.sha256(json.dumps(d, sort_keys=True).encode()).hexdigest()  # noqa: E731
        return {"kind": "spiraltorch.trainer_runtime_bundle", "contract_version": "spiraltorch.trainer_runtime.v2",
                "resume_scope": "parameter values are external; re-attach concrete resources before commit",
                "optimizer_sha256": enc(opt), "external_sha256": enc(external),
                "optimizer": opt, "external": external}

    def restore_runtime_checkpoint_bundle(self, module: Module, bundle: dict) -> None:
        enc = lambda d: hashlib.sha256(json.dumps(d, sort_keys=True).encode()).hexdigest()  # noqa: E731
        if enc(bundle["optimizer"]) != bundle["optimizer_sha256"] or enc(bundle["external"]) != bundle["external_sha256"]:
            raise ValueError("runtime checkpoint bundle failed its integrity check")
        self.restore_optimizer_checkpoint(module, bundle["optimizer"])
        self.grad_clip_max_norm = bundle["external"].get("grad_clip_max_norm")
