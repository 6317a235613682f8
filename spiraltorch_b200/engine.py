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
