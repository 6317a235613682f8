"""``SpiralSession``: backend selection, device report and a runtime execution plan.

The reference session probes WGPU/CUDA/HIP/MPS and routes every op through a per-op backend
policy (bindings/st-py/spiraltorch/__init__.py:7127-7430, crates/st-core/src/backend/
execution_plan.rs).  Here there are two backends — ``cpu`` (PyTorch fp32) and ``cuda`` (the
sm_100a kernels) — and no per-op multi-backend dispatch: ``auto`` picks ``cuda`` when a device is
present.  The plan is a small dict with a SHA-256 commitment so it can be saved and re-installed.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Optional

import torch

from .config import ExecutionConfig, determinism
from .nn.data import DataLoader, Dataset
from .nn.trainer import ModuleTrainer
from .tensor import set_default_device

BACKENDS = ("auto", "cpu", "cuda", "wgpu", "hip", "mps")


class BackendUnavailable(RuntimeError):
    pass


def describe_device(backend: str = "auto") -> dict:
    """Device report (crates/st-core/src/backend/runtime_probe.rs:1152-1275)."""
    cuda = torch.cuda.is_available()
    rep = {"requested_backend": backend, "cuda_available": cuda, "backends": {"cpu": {"ready": True}}}
    if cuda:
        p = torch.cuda.get_device_properties(0)
        rep["backends"]["cuda"] = {
            "ready": True, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
            "multiprocessors": p.multi_processor_count, "memory_bytes": p.total_memory,
            "lane_width": 32, "max_workgroup": 1024, "shared_mem": 227 * 1024,
            "native_library": _native_status(),
        }
    else:
        rep["backends"]["cuda"] = {"ready": False, "reason": "no CUDA device"}
    for b in ("wgpu", "hip", "mps"):
        rep["backends"][b] = {"ready": False, "reason": "not part of this build"}
    return rep


def _native_status() -> dict:
    from .utils import build
    return {"path": str(build.LIB_PATH), "built": build.LIB_PATH.exists(), "current": build.is_current()}


def build_info() -> dict:
    from .nn.io import VERSION
    return {"version": VERSION, "torch": torch.__version__, "cuda_arch": "sm_100a",
            "features": ["cpu", "cuda", "tcgen05", "tma", "nccl", "nvls", "golden", "kdsl", "selfsup"],
            "native": _native_status()}


def evaluate_runtime_execution_plan(report: dict, requested: str, fallback: str) -> dict:
    cuda_ready = report["backends"]["cuda"]["ready"]
    if requested == "auto":
        effective = "cuda" if cuda_ready else "cpu"
    elif requested == "cuda" and not cuda_ready:
        if fallback == "forbid":
            raise BackendUnavailable("backend 'cuda' requested but no CUDA device is present")
        effective = "cpu"
    elif requested in ("wgpu", "hip", "mps"):
        if fallback == "forbid":
            raise BackendUnavailable(f"backend '{requested}' is not part of this build")
        effective = "cuda" if cuda_ready else "cpu"
    else:
        effective = requested
    plan = {"schema": "spiraltorch.runtime_execution_plan.v1", "requested_backend": requested,
            "effective_backend": effective, "accelerator_fallback": fallback,
            "routes": {op: effective for op in ("matmul", "attention", "layer_norm", "softmax", "tensor_util", "conv")}}
    plan["sha256"] = hashlib.sha256(json.dumps(plan, sort_keys=True).encode()).hexdigest()
    return plan


class SpiralSession:
    def __init__(self, backend: str = "auto", seed: Optional[int] = None, *, runtime_execution_plan: Optional[dict] = None,
                 accelerator_fallback: Optional[str] = None, tensor_util_wgpu_min_values: Optional[int] = None):
        if backend not in BACKENDS:
            raise ValueError(f"unknown backend '{backend}' (expected one of {BACKENDS})")
        cfg = ExecutionConfig.from_env()
        self.accelerator_fallback = accelerator_fallback or cfg.accelerator_fallback
        self.requested_backend = backend
        self.device_preflight = describe_device(backend)
        if runtime_execution_plan is not None:
            body = {k: v for k, v in runtime_execution_plan.items() if k != "sha256"}
            if hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest() != runtime_execution_plan.get("sha256"):
                raise ValueError("runtime execution plan failed its commitment check")
            self._plan = runtime_execution_plan
        else:
            self._plan = evaluate_runtime_execution_plan(self.device_preflight, backend, self.accelerator_fallback)
        self.effective_backend = self._plan["effective_backend"]
        self.backend = self.effective_backend
        self.device = torch.device("cuda" if self.effective_backend == "cuda" else "cpu")
        self.seed = seed
        if seed is not None:
            torch.manual_seed(seed)
        determinism.apply()
        set_default_device(self.device)
        self._closed = False

    @classmethod
    def from_runtime_execution_plan(cls, plan: dict, seed: Optional[int] = None) -> "SpiralSession":
        return cls(plan["requested_backend"], seed, runtime_execution_plan=plan)

    def runtime_execution_plan(self) -> dict:
        return dict(self._plan)

    def dataset(self, samples=None) -> Dataset:
        return Dataset(samples)

    def dataloader(self, dataset: Dataset) -> DataLoader:
        return DataLoader(dataset, device=self.device if self.device.type == "cuda" else None)

    def trainer(self, **kw) -> ModuleTrainer:
        kw.setdefault("backend", self.effective_backend)
        return ModuleTrainer(**kw).bind_runtime_execution_plan(self._plan)

    module_trainer = trainer

    def plan_topk(self, rows: int, cols: int, k: int):
        from .ops.rank import plan_rank
        return plan_rank("topk", rows, cols, k, backend=self.effective_backend)

    def plan(self, kind: str, rows: int, cols: int, k: int):  # type: ignore[override]
        from .ops.rank import plan_rank
        return plan_rank(kind, rows, cols, k, backend=self.effective_backend)

    def close(self) -> None:
        if not self._closed:
            set_default_device("cpu")
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
