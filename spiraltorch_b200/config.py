"""Configuration surface: determinism flags, execution flags, tracing and layered config files.

Reference parity:
* ``spiral-config`` determinism (crates/spiral-config/src/determinism.rs:19-110): env
  ``SPIRAL_DETERMINISTIC``, ``SPIRAL_DETERMINISTIC_SEED`` (default 42),
  ``SPIRAL_DETERMINISTIC_SCHEDULER``, ``SPIRAL_DETERMINISTIC_REDUCTION``; seeds for unlabeled
  random streams are derived from ``(base_seed, label)``.
* execution flags (crates/spiral-config/src/execution.rs:5-95): ``SPIRALTORCH_STRICT_GPU``,
  accelerator fallback ``allow | forbid``.
* tracing (crates/spiral-config/src/tracing.rs:12-64): ``SPIRAL_TRACE_CHROME=/path.json``
  writes a Chrome-trace file; here the spans are CUDA-event timed ranges.
* layered config (crates/st-core/src/config/layered.rs:13-125): ``base.toml`` → ``site.toml`` →
  ``run.json`` merged in that order with a list of diff events; env overrides
  ``SPIRAL_CONFIG_ROOT/BASE/SITE/RUN``.
"""
from __future__ import annotations

import contextlib
import hashlib
import json
import os
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional


def _flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")


# --------------------------------------------------------------------------------------------
@dataclass
class DeterminismConfig:
    enabled: bool = False
    seed: int = 42
    scheduler: bool = False
    reduction: bool = False


class _Determinism:
    def config(self) -> DeterminismConfig:
        enabled = _flag("SPIRAL_DETERMINISTIC")
        return DeterminismConfig(
            enabled=enabled,
            seed=int(os.environ.get("SPIRAL_DETERMINISTIC_SEED", "42")),
            scheduler=_flag("SPIRAL_DETERMINISTIC_SCHEDULER", enabled),
            reduction=_flag("SPIRAL_DETERMINISTIC_REDUCTION", enabled),
        )

    def resolve_seed(self, seed: Optional[int], label: str) -> int:
        """Explicit seed wins; under ``SPIRAL_DETERMINISTIC`` derive one from (base seed, label);
        otherwise draw from the OS."""
        if seed is not None:
            return int(seed) & 0x7FFFFFFFFFFFFFFF
        cfg = self.config()
        if cfg.enabled:
            h = hashlib.sha256(f"{cfg.seed}:{label}".encode()).digest()
            return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF
        return int.from_bytes(os.urandom(8), "little") & 0x7FFFFFFFFFFFFFFF

    def apply(self) -> DeterminismConfig:
        """Push the flags into PyTorch (deterministic algorithms, single-threaded reductions)."""
        import torch
        cfg = self.config()
        if cfg.enabled:
            torch.manual_seed(cfg.seed)
            torch.use_deterministic_algorithms(True, warn_only=True)
        if cfg.reduction:
            torch.set_num_threads(1)
        return cfg


determinism = _Determinism()


# --------------------------------------------------------------------------------------------
@dataclass
class ExecutionConfig:
    strict_gpu: bool = False
    accelerator_fallback: str = "allow"      # "allow" | "forbid"
    tensor_util_min_values: int = 1024

    @staticmethod
    def from_env() -> "ExecutionConfig":
        strict = _flag("SPIRALTORCH_STRICT_GPU")
        return ExecutionConfig(
            strict_gpu=strict,
            accelerator_fallback="forbid" if strict else os.environ.get("SPIRALTORCH_ACCELERATOR_FALLBACK", "allow"),
            tensor_util_min_values=int(os.environ.get("SPIRALTORCH_TENSOR_UTIL_WGPU_MIN_VALUES", "1024")),
        )


# --------------------------------------------------------------------------------------------
class ChromeTrace:
    """Collects complete ("X") events and writes a Chrome-trace JSON file."""

    def __init__(self, path: Optional[str] = None):
        self.path = path
        self.events: list[dict] = []
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()

    @contextlib.contextmanager
    def span(self, name: str, category: str = "spiraltorch", **args):
        start = time.perf_counter()
        try:
            yield
        finally:
            end = time.perf_counter()
            with self._lock:
                self.events.append({"name": name, "cat": category, "ph": "X", "pid": os.getpid(),
                                    "tid": threading.get_ident() & 0xFFFF,
                                    "ts": (start - self._t0) * 1e6, "dur": (end - start) * 1e6, "args": args})

    def add_device_span(self, name: str, start_us: float, dur_us: float, **args) -> None:
        with self._lock:
            self.events.append({"name": name, "cat": "cuda", "ph": "X", "pid": os.getpid(), "tid": 0,
                                "ts": start_us, "dur": dur_us, "args": args})

    def flush(self) -> Optional[str]:
        if not self.path:
            return None
        tmp = f"{self.path}.tmp"
        with open(tmp, "w", encoding="utf-8") as fh:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, fh)
        os.replace(tmp, self.path)
        return self.path


_trace: Optional[ChromeTrace] = None


def init_tracing(path: Optional[str] = None) -> ChromeTrace:
    """Install the process-wide trace collector (``SPIRAL_TRACE_CHROME`` names the output file)."""
    global _trace
    if _trace is None or path is not None:
        _trace = ChromeTrace(path or os.environ.get("SPIRAL_TRACE_CHROME"))
    return _trace


def tracer() -> ChromeTrace:
    return init_tracing()


# --------------------------------------------------------------------------------------------
@dataclass
class LayeredConfig:
    values: dict = field(default_factory=dict)
    events: list = field(default_factory=list)     # [{"layer", "key", "old", "new"}]
    sources: list = field(default_factory=list)


def _load_layer(path: Path) -> dict:
    if not path.exists():
        return {}
    if path.suffix == ".json":
        return json.loads(path.read_text())
    import tomllib
    return tomllib.loads(path.read_text())


def _merge(dst: dict, src: dict, layer: str, events: list, prefix: str = "") -> None:
    for k, v in src.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v, layer, events, key + ".")
        else:
            if k not in dst or dst[k] != v:
                events.append({"layer": layer, "key": key, "old": dst.get(k), "new": v})
            dst[k] = v


def load_layered_config(root: Optional[str] = None) -> LayeredConfig:
    """base.toml → site.toml → run.json, later layers override earlier ones."""
    root_path = Path(root or os.environ.get("SPIRAL_CONFIG_ROOT") or Path.home() / ".spiraltorch" / "config")
    layers = [
        ("base", Path(os.environ.get("SPIRAL_CONFIG_BASE") or root_path / "base.toml")),
        ("site", Path(os.environ.get("SPIRAL_CONFIG_SITE") or root_path / "site.toml")),
        ("run", Path(os.environ.get("SPIRAL_CONFIG_RUN") or root_path / "run.json")),
    ]
    cfg = LayeredConfig()
    for name, path in layers:
        data = _load_layer(path)
        if data:
            cfg.sources.append(str(path))
            _merge(cfg.values, data, name, cfg.events)
    return cfg


# --------------------------------------------------------------------------------------------
def atomic_write(path, data: bytes | str) -> None:
    """tmp file → flush → fsync → rename → fsync(parent)
    (crates/st-core/src/runtime/persistence.rs:21-62)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + f".tmp.{os.getpid()}")
    mode = "wb" if isinstance(data, (bytes, bytearray)) else "w"
    with open(tmp, mode) as fh:
        fh.write(data)
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)
    try:
        dfd = os.open(str(path.parent), os.O_RDONLY)
        try:
            os.fsync(dfd)
        finally:
            os.close(dfd)
    except OSError:
        pass
