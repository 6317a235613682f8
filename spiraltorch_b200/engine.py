"""Engine extension points: gradient / partition hook slots, a custom-operator registry and the
thread-local backend policy guard.

Restated from crates/st-core/src/engine/hook_points.rs:41-130 (``register_onebit_allreduce`` /
``register_zero_partition`` slots; calling an empty slot is a no-op / identity),
crates/st-core/src/ops/operator_registry.rs (named operators with arity checks and metadata) and
crates/st-core/src/backend/execution.rs:27-84 (``push_backend_policy`` RAII guard: per-op backend
labels that nest and restore).  Every call publishes a ``TensorOp`` event when someone listens.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch

from . import plugin
from .tensor import Tensor, TensorError

_lock = threading.Lock()
_grad_hook: Optional[Callable] = None
_part_hook: Optional[Callable] = None


def register_onebit_allreduce(hook: Optional[Callable[[torch.Tensor, int], None]]) -> None:
    """``hook(grad, world)`` mutates the flat gradient in place (e.g. sign compression + all-reduce)."""
    global _grad_hook
    with _lock:
        _grad_hook = hook


def register_zero_partition(hook: Optional[Callable[[torch.Tensor, int, int], torch.Tensor]]) -> None:
    """``hook(params, rank, world)`` returns the slice of the flat parameters this rank owns."""
    global _part_hook
    with _lock:
        _part_hook = hook


def call_onebit_allreduce(grad: torch.Tensor, world: int) -> bool:
    with _lock:
        hook = _grad_hook
    before = float(grad.norm()) if plugin.has_listeners("TensorOp") else 0.0
    if hook is not None:
        hook(grad, world)
    if plugin.has_listeners("TensorOp"):
        plugin.publish("TensorOp", {"op": "onebit_allreduce_hook", "registered": hook is not None, "world": world,
                                    "gradient_len": grad.numel(), "gradient_l2_before": before,
                                    "gradient_l2_after": float(grad.norm())})
    return hook is not None


def call_zero_partition(params: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    with _lock:
        hook = _part_hook
    out = hook(params, rank, world) if hook is not None else params
    if plugin.has_listeners("TensorOp"):
        plugin.publish("TensorOp", {"op": "zero_partition_hook", "registered": hook is not None, "rank": rank,
                                    "world": world, "input_len": params.numel(), "output_len": out.numel()})
    return out


def default_zero_partition(params: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous equal shards (the last one takes the remainder) — the layout of the fused
    data-parallel step, which keeps optimizer state only for the shard a rank owns."""
    n = params.numel()
    per = -(-n // world)
    return params.reshape(-1)[rank * per: min(n, (rank + 1) * per)]


# ---- operator registry ---------------------------------------------------------------------------------
@dataclass
class OperatorSpec:
    name: str
    arity: int
    forward: Callable
    backward: Optional[Callable] = None
    description: str = ""
    metadata: dict = field(default_factory=dict)


class OperatorRegistry:
    def __init__(self):
        self._ops: dict[str, OperatorSpec] = {}
        self._lock = threading.Lock()

    def register(self, spec: OperatorSpec, replace: bool = False) -> None:
        if not spec.name or spec.arity < 0:
            raise TensorError("operator needs a name and a non-negative arity")
        with self._lock:
            if spec.name in self._ops and not replace:
                raise TensorError(f"operator '{spec.name}' is already registered")
            self._ops[spec.name] = spec

    def unregister(self, name: str) -> bool:
        with self._lock:
            return self._ops.pop(name, None) is not None

    def names(self) -> list:
        with self._lock:
            return sorted(self._ops)

    def get(self, name: str) -> OperatorSpec:
        with self._lock:
            if name not in self._ops:
                raise TensorError(f"unknown operator '{name}'")
            return self._ops[name]

    def call(self, name: str, *inputs: Tensor) -> Tensor:
        spec = self.get(name)
        if len(inputs) != spec.arity:
            raise TensorError(f"operator '{name}' takes {spec.arity} inputs, got {len(inputs)}")
        out = spec.forward(*inputs)
        if not isinstance(out, Tensor):
            out = Tensor._wrap(torch.as_tensor(out, dtype=torch.float32))
        if plugin.has_listeners("TensorOp"):
            plugin.publish("TensorOp", {"op": f"custom::{name}", "inputs": [t.shape() for t in inputs], "output": out.shape()})
        return out

    def call_backward(self, name: str, inputs: Sequence[Tensor], grad_output: Tensor) -> list:
        spec = self.get(name)
        if spec.backward is None:
            raise TensorError(f"operator '{name}' has no backward")
        grads = spec.backward(*inputs, grad_output)
        grads = list(grads) if isinstance(grads, (list, tuple)) else [grads]
        if len(grads) != spec.arity:
            raise TensorError(f"backward of '{name}' returned {len(grads)} gradients for {spec.arity} inputs")
        return grads


_global_registry = OperatorRegistry()


def global_operator_registry() -> OperatorRegistry:
    return _global_registry


# ---- backend policy --------------------------------------------------------------------------------------
POLICY_OPS = ("matmul", "prepacked_matmul", "layer_norm", "attention", "softmax", "tensor_util")
_policy = threading.local()


@dataclass
class BackendPolicy:
    """Per-op backend labels; ``None`` leaves the op on the session default.  This build has two
    backends: ``cpu`` and ``cuda`` (the sm_100a kernels)."""
    matmul: Optional[str] = None
    prepacked_matmul: Optional[str] = None
    layer_norm: Optional[str] = None
    attention: Optional[str] = None
    softmax: Optional[str] = None
    tensor_util: Optional[str] = None

    def validate(self) -> None:
        for op in POLICY_OPS:
            v = getattr(self, op)
            if v is not None and v not in ("cpu", "cuda", "auto"):
                raise TensorError(f"backend '{v}' for {op} is not available in this build (cpu, cuda, auto)")


class push_backend_policy:
    """``with push_backend_policy(BackendPolicy(matmul="cpu")):`` — nests; the previous policy is
    restored on exit, also when the body raises."""

    def __init__(self, policy: BackendPolicy):
        policy.validate()
        self._policy = policy

    def __enter__(self):
        stack = getattr(_policy, "stack", None)
        if stack is None:
            stack = _policy.stack = []
        stack.append(self._policy)
        return self._policy

    def __exit__(self, *exc):
        _policy.stack.pop()
        return False


def current_backend_policy() -> BackendPolicy:
    """The effective policy of this thread: inner guards override outer ones per op."""
    eff = BackendPolicy()
    for pol in getattr(_policy, "stack", []):
        for op in POLICY_OPS:
            v = getattr(pol, op)
            if v is not None:
                setattr(eff, op, v)
    return eff


def backend_for(op: str, default: str = "auto") -> str:
    if op not in POLICY_OPS:
        raise TensorError(f"unknown policy op '{op}'")
    return getattr(current_backend_policy(), op) or default


# ----------------------------------------------------------------------------------------------
# Collapse drive (crates/st-core/src/engine/collapse_drive.rs:27-305)
# ----------------------------------------------------------------------------------------------
import math as _math


@dataclass
class CollapseConfig:
    """Thresholds of the psi-driven collapse / bloom controller.  `trend_*` and `*_deviation_*`
    triggers are off while their thresholds are infinite."""
    enabled: bool = False
    hi: float = 2.0
    lo: float = 0.3
    hysteresis: float = 0.1
    warmup_steps: int = 50
    cooldown_steps: int = 10
    collapse_scale: float = 0.2
    collapse_max_norm: Optional[float] = 1.0
    collapse_lr_decay: Optional[float] = 0.1
    bloom_lr_mul: float = 1.2
    trend_alpha: float = 0.0
    collapse_trend_threshold: float = _math.inf
    bloom_trend_threshold: float = -_math.inf
    baseline_alpha: float = 0.0
    collapse_deviation_threshold: float = _math.inf
    bloom_deviation_threshold: float = _math.inf

    @classmethod
    def automated(cls, depth: int, band_focus: float = 0.0, drift_weight: float = 0.0) -> "CollapseConfig":
        """Thresholds derived from a model's depth and the psi meter's band focus / drift weight."""
        d = float(max(depth, 1))
        cl = lambda x, lo, hi: min(max(x, lo), hi)
        return cls(True, cl(1.4 + _math.log1p(d) * 0.6, 1.8, 4.5), cl(0.18 + 0.4 / _math.sqrt(d), 0.2, 0.6),
                   0.08 + 0.02 * _math.log1p(d), int(cl(depth * 2, 20, 240)), int(cl(round(d / 8.0), 2, 12)),
                   cl(0.18 + 0.9 / _math.sqrt(d), 0.1, 0.4), 1.0, 0.12, cl(1.05 + band_focus / d, 1.05, 1.6),
                   cl(0.18 + 1.2 / _math.sqrt(d), 0.2, 0.65), cl(0.08 + band_focus / (d + 4.0), 0.06, 0.25),
                   -(0.06 + cl(drift_weight, 0.05, 0.6)), cl(0.04 + 1.5 / (d + 6.0), 0.05, 0.3),
                   cl(0.12 + 0.35 / _math.sqrt(d) + band_focus * 0.02, 0.12, 0.35), cl(0.1 + drift_weight * 0.3, 0.1, 0.35))


@dataclass(frozen=True)
class DriveCmd:
    """`kind` is "none", "collapse" (scale gradients by `grad_scale`, clip to `max_norm`, decay the
    learning rate by `lr_decay`) or "bloom" (multiply the learning rate by `lr_mul`)."""
    kind: str = "none"
    grad_scale: Optional[float] = None
    max_norm: Optional[float] = None
    lr_decay: Optional[float] = None
    lr_mul: Optional[float] = None
    due_to_trend: bool = False
    due_to_deviation: bool = False


_DRIVE_SCALARS = {"warmup": 0.0, "stable": 1.0, "collapse": 2.0, "bloom": 3.0}


class CollapseDrive:
    """State machine warmup -> stable <-> collapse / bloom over the total psi reading.

    From warmup / stable: psi >= hi (or a rising trend / positive deviation from the moving baseline)
    issues a collapse, psi <= lo (or the mirrored triggers) a bloom; either starts a cool-down of
    `cooldown_steps` silent updates.  A collapse ends once psi <= hi - hysteresis, a bloom once
    psi >= lo + hysteresis."""

    def __init__(self, cfg: Optional[CollapseConfig] = None):
        self.cfg = cfg or CollapseConfig()
        self.state, self.cooldown, self.last_step = "warmup", 0, 0
        self.prev_total: Optional[float] = None
        self.trend, self.baseline = 0.0, None

    def enabled(self) -> bool:
        return self.cfg.enabled

    def diagnostics(self) -> dict:
        return {"state": self.state, "state_scalar": _DRIVE_SCALARS[self.state], "trend": self.trend,
                "baseline": self.baseline, "cooldown": self.cooldown}

    def update(self, total: float, step: int) -> DriveCmd:
        c = self.cfg
        self.last_step = step
        if not c.enabled:
            return DriveCmd()
        if step < c.warmup_steps:
            self.state = "warmup"
            return DriveCmd()
        if self.state == "warmup":
            self.state = "stable"
        if self.cooldown > 0:
            self.cooldown -= 1
            return DriveCmd()
        ct = cd = bt = bd = False
        if self.prev_total is not None:
            delta = total - self.prev_total
            a = min(max(c.trend_alpha, 0.0), 1.0)
            self.trend = a * delta + (1 - a) * self.trend if a > 0 else delta
            b = min(max(c.baseline_alpha, 0.0), 1.0)
            if b > 0:
                base = self.prev_total if self.baseline is None else self.baseline
                self.baseline = (1 - b) * base + b * total
                dev = total - self.baseline
                cd = _math.isfinite(c.collapse_deviation_threshold) and dev >= c.collapse_deviation_threshold
                bd = _math.isfinite(c.bloom_deviation_threshold) and dev <= -c.bloom_deviation_threshold
            else:
                self.baseline = total
            ct = _math.isfinite(c.collapse_trend_threshold) and self.trend >= c.collapse_trend_threshold
            bt = _math.isfinite(c.bloom_trend_threshold) and self.trend <= c.bloom_trend_threshold
        else:
            self.baseline, self.trend = total, 0.0
        self.prev_total = total
        if self.state in ("warmup", "stable"):
            if total >= c.hi or ct or cd:
                self.state, self.cooldown = "collapse", c.cooldown_steps
                return DriveCmd("collapse", c.collapse_scale, c.collapse_max_norm, c.collapse_lr_decay, None, ct, cd)
            if total <= c.lo or bt or bd:
                self.state, self.cooldown = "bloom", c.cooldown_steps
                return DriveCmd("bloom", lr_mul=c.bloom_lr_mul, due_to_trend=bt, due_to_deviation=bd)
        elif self.state == "collapse":
            if total <= c.hi - c.hysteresis:
                self.state = "stable"
        elif self.state == "bloom":
            if total >= c.lo + c.hysteresis:
                self.state = "stable"
        return DriveCmd()
