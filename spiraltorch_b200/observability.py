"""Per-op observability: observers, lazy op metadata, execution receipts and the per-epoch collector.

* Observers are global or thread-local callables ``fn(event: dict)``; ``emit_tensor_op`` costs one
  list check when nobody listens, ``emit_tensor_op_meta`` takes a closure that builds the JSON
  payload only when somebody does (crates/st-tensor/src/observability.rs:14-120).
* An execution receipt records, for every routed op, the backend that was requested, the one the
  policy selected, the one that executed and why they differ
  (crates/st-tensor/src/execution.rs ``TensorExecutionReceipt``).  Backends here are ``cpu`` and
  ``cuda`` (hand-written sm_100a kernels); a CUDA request that ran on the CPU carries the reason.
* ``TensorOpStepCollector`` folds the events of an epoch into ``EpochTensorBackendStats`` with the
  reference's counter names (crates/st-nn/src/trainer.rs:1993-2140).
"""
from __future__ import annotations

import hashlib
import json
import threading
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional

Observer = Callable[[Dict[str, Any]], None]

_global: List[Observer] = []
_local = threading.local()
_lock = threading.Lock()


def _thread_observers() -> List[Observer]:
    obs = getattr(_local, "observers", None)
    if obs is None:
        obs = _local.observers = []
    return obs


def add_observer(fn: Observer, *, thread_local: bool = False) -> Observer:
    if thread_local:
        _thread_observers().append(fn)
    else:
        with _lock:
            _global.append(fn)
    return fn


def remove_observer(fn: Observer) -> None:
    with _lock:
        if fn in _global:
            _global.remove(fn)
    if fn in _thread_observers():
        _thread_observers().remove(fn)


@contextmanager
def observe(fn: Observer, *, thread_local: bool = True):
    add_observer(fn, thread_local=thread_local)
    try:
        yield fn
    finally:
        remove_observer(fn)


def has_observers() -> bool:
    return bool(_global) or bool(getattr(_local, "observers", None))


def _dispatch(event: Dict[str, Any]) -> None:
    for fn in list(_global) + list(_thread_observers()):
        fn(event)


def emit_tensor_op(op: str, input_shape, output_shape, **fields) -> None:
    """Publishes ``{"kind": "tensor_op", "op", "input_shape", "output_shape", ...}`` to observers and, when it
    has listeners, to the plugin bus as a ``TensorOp`` event."""
    from . import plugin
    bus = plugin.has_listeners("TensorOp")
    if not bus and not has_observers():
        return
    event = {"kind": "tensor_op", "op": op, "input_shape": list(input_shape), "output_shape": list(output_shape), **fields}
    if has_observers():
        _dispatch(event)
    if bus:
        plugin.publish("TensorOp", {k: v for k, v in event.items() if k != "kind"})


def emit_tensor_op_meta(op: str, build: Callable[[], Dict[str, Any]]) -> None:
    """``build`` runs only when an observer is installed."""
    if has_observers():
        _dispatch({"kind": "tensor_op_meta", "op": op, "meta": build()})


# ---- execution receipts ---------------------------------------------------------------------------

@dataclass
class TensorExecutionReceipt:
    op: str
    requested_backend: str
    selected_backend: str
    executed_backend: str
    fallback_reason: Optional[str] = None
    workload: Dict[str, Any] = field(default_factory=dict)
    plan_commitment: Optional[str] = None

    @property
    def fell_back(self) -> bool:
        return self.executed_backend != self.selected_backend or self.selected_backend != self.requested_backend

    def as_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["fell_back"] = self.fell_back
        return d


def plan_commitment(plan: Dict[str, Any]) -> str:
    """SHA-256 of the canonical JSON of an execution plan."""
    return hashlib.sha256(json.dumps(plan, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


_last_receipt = threading.local()


def record_receipt(receipt: TensorExecutionReceipt) -> TensorExecutionReceipt:
    _last_receipt.value = receipt
    if has_observers():
        _dispatch({"kind": "execution_receipt", **receipt.as_dict()})
    return receipt


def last_receipt() -> Optional[TensorExecutionReceipt]:
    return getattr(_last_receipt, "value", None)


def resolve_backend(requested: Optional[str], on_cuda: bool, native_ok: bool, strict: bool = False):
    """``(selected, executed, reason)`` for an op whose operands live on CUDA or not.  ``requested`` is a label of
    the public API (``auto``, ``cpu``, ``cuda``, or one of the reference's CPU GEMM names)."""
    req = (requested or "auto").lower()
    cpu_names = ("cpu", "naive", "faer", "simd", "cpu-simd")
    if req in cpu_names:
        return "cpu", "cpu", None
    selected = "cuda" if on_cuda else "cpu"
    if req in ("cuda", "gpu") and not on_cuda:
        if strict:
            raise RuntimeError("backend 'cuda' was requested for host tensors and accelerator fallback is forbidden")
        return "cuda", "cpu", "operands are host tensors"
    if selected == "cuda" and not native_ok:
        if strict:
            raise RuntimeError("the native sm_100a library is not loaded and accelerator fallback is forbidden")
        return "cuda", "cpu", "native library unavailable"
    return selected, selected, None


# ---- per-epoch collector --------------------------------------------------------------------------

@dataclass
class EpochTensorBackendStats:
    ops_total: int = 0
    fallbacks: int = 0
    backend_cuda: int = 0
    backend_cpu: int = 0
    requested_cuda_hits: int = 0
    requested_cuda_misses: int = 0
    by_op: Dict[str, int] = field(default_factory=dict)

    def as_dict(self) -> Dict[str, Any]:
        return asdict(self)


class TensorOpStepCollector:
    """Install with ``with collector:`` around an epoch; ``stats`` holds the folded counters afterwards."""

    def __init__(self):
        self.stats = EpochTensorBackendStats()

    def __call__(self, event: Dict[str, Any]) -> None:
        s = self.stats
        if event["kind"] == "tensor_op":
            s.ops_total += 1
            s.by_op[event["op"]] = s.by_op.get(event["op"], 0) + 1
        elif event["kind"] == "execution_receipt":
            if event["executed_backend"] == "cuda":
                s.backend_cuda += 1
            else:
                s.backend_cpu += 1
            if event["fell_back"]:
                s.fallbacks += 1
            if event["requested_backend"] in ("cuda", "gpu"):
                if event["executed_backend"] == "cuda":
                    s.requested_cuda_hits += 1
                else:
                    s.requested_cuda_misses += 1

    def __enter__(self) -> "TensorOpStepCollector":
        add_observer(self, thread_local=True)
        return self

    def __exit__(self, *exc) -> None:
        remove_observer(self)
