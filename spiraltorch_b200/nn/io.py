"""Weight files compatible with the reference, both ways.

* JSON (``.json``): ``{"parameters": {"<module>::<param>": {"rows": R, "cols": C, "data": [...]}}}``
  pretty-printed (crates/st-nn/src/io.rs:14-40,77-111; example models/weights/mlp_regression.json).
* Binary (``.bin`` / ``.bincode`` / ``.bc``): bincode 1.x default layout of the same struct —
  ``u64 n; n x { u64 key_len, key utf-8, u64 rows, u64 cols, u64 len, f32-LE x len }``
  (crates/st-nn/src/io.rs:113-140).
* Manifest (``<stem>.manifest.json``): ``{format_version, spiraltorch_version, module_type,
  weights: {path, format}, state_dict: [{name, shape}]}``
  (bindings/st-py/spiraltorch/__init__.py:6594-6668).

Layouts are the reference's: Linear weights ``(in, out)``, biases ``(1, out)``, convolution
weights ``(out_channels, in_channels*kh*kw)``.  Files are written atomically.
"""
from __future__ import annotations

import json
import os
import struct
from pathlib import Path
from typing import Any, Mapping

import torch

from ..config import atomic_write
from ..tensor import Tensor

FORMAT_VERSION = 1
VERSION = "0.1.0+b200"


def _entries(state) -> list[tuple[str, torch.Tensor]]:
    if hasattr(state, "state_dict") and callable(state.state_dict):
        state = state.state_dict()
    items = state.items() if isinstance(state, Mapping) else state
    out = []
    for name, t in items:
        tt = t.torch() if isinstance(t, Tensor) else torch.as_tensor(t, dtype=torch.float32)
        if tt.dim() == 1:
            tt = tt.reshape(1, -1)
        if tt.dim() != 2:
            raise ValueError(f"parameter '{name}' is not 2-D: {tuple(tt.shape)}")
        out.append((str(name), tt.detach().to("cpu", torch.float32).contiguous()))
    return out


def weights_format(path) -> str:
    p = os.fspath(path)
    if p.lower().endswith(".manifest.json"):
        return "manifest"
    suffix = Path(p).suffix.lower()
    if suffix == ".json":
        return "json"
    if suffix in (".bin", ".bincode", ".bc"):
        return "bincode"
    raise ValueError("unsupported weights extension (expected .json, .bin, .bincode, .bc, or .manifest.json)")


def save_json(state, path) -> None:
    params = {name: {"rows": t.shape[0], "cols": t.shape[1], "data": t.reshape(-1).tolist()}
              for name, t in _entries(state)}
    atomic_write(path, json.dumps({"parameters": params}, indent=2))


def load_json(path) -> list[tuple[str, Tensor]]:
    doc = json.loads(Path(path).read_text())
    if "parameters" not in doc:
        raise ValueError(f"{path}: missing 'parameters'")
    out = []
    for name, rec in doc["parameters"].items():
        rows, cols, data = int(rec["rows"]), int(rec["cols"]), rec["data"]
        if len(data) != rows * cols:
            raise ValueError(f"{path}: parameter '{name}' has {len(data)} values for shape ({rows}, {cols})")
        out.append((name, Tensor(rows, cols, data, device="cpu")))
    return sorted(out, key=lambda kv: kv[0])


def save_bincode(state, path) -> None:
    ents = _entries(state)
    buf = bytearray(struct.pack("<Q", len(ents)))
    for name, t in ents:
        key = name.encode("utf-8")
        buf += struct.pack("<Q", len(key)) + key
        buf += struct.pack("<QQQ", t.shape[0], t.shape[1], t.numel())
        buf += t.reshape(-1).numpy().astype("<f4").tobytes()
    atomic_write(path, bytes(buf))


def load_bincode(path) -> list[tuple[str, Tensor]]:
    raw = Path(path).read_bytes()
    off = 0

    def take(n: int) -> bytes:
        nonlocal off
        if off + n > len(raw):
            raise ValueError(f"{path}: truncated weights file")
        b = raw[off:off + n]
        off += n
        return b

    (n,) = struct.unpack("<Q", take(8))
    out = []
    for _ in range(n):
        (klen,) = struct.unpack("<Q", take(8))
        name = take(klen).decode("utf-8")
        rows, cols, ln = struct.unpack("<QQQ", take(24))
        if ln != rows * cols:
            raise ValueError(f"{path}: parameter '{name}' has {ln} values for shape ({rows}, {cols})")
        data = torch.frombuffer(bytearray(take(4 * ln)), dtype=torch.float32).clone()
        out.append((name, Tensor._wrap(data.reshape(rows, cols))))
    if off != len(raw):
        raise ValueError(f"{path}: {len(raw) - off} trailing bytes")
    return sorted(out, key=lambda kv: kv[0])


def manifest_path(path) -> Path:
    p = Path(os.fspath(path))
    return p if p.name.lower().endswith(".manifest.json") else p.with_suffix(".manifest.json")


def save(path, target) -> None:
    """``st.nn.save(path, model_or_state_dict)``: weights file + ``<stem>.manifest.json``."""
    p = Path(os.fspath(path))
    fmt = weights_format(p)
    if fmt == "manifest":
        raise ValueError("save() expects a weights path, not a manifest path")
    p.parent.mkdir(parents=True, exist_ok=True)
    (save_json if fmt == "json" else save_bincode)(target, p)
    ents = _entries(target)
    manifest = {
        "format_version": FORMAT_VERSION,
        "spiraltorch_version": VERSION,
        "module_type": type(target).__name__ if hasattr(target, "state_dict") else None,
        "weights": {"path": p.name, "format": fmt},
        "state_dict": [{"name": n, "shape": list(t.shape)} for n, t in ents],
    }
    atomic_write(manifest_path(p), json.dumps(manifest, indent=2))


def load(path, model=None):
    """Load a weights file or a manifest.  With ``model`` the state is loaded into it and the
    model is returned; otherwise the ``[(name, Tensor)]`` state is returned."""
    p = Path(os.fspath(path))
    fmt = weights_format(p)
    if fmt == "manifest":
        man = json.loads(p.read_text())
        if man.get("format_version") != FORMAT_VERSION:
            raise ValueError(f"unsupported manifest version {man.get('format_version')}")
        wpath = p.parent / man["weights"]["path"]
        fmt = man["weights"]["format"]
    else:
        wpath = p
    state = load_json(wpath) if fmt == "json" else load_bincode(wpath)
    if model is None:
        return state
    model.load_state_dict(state)
    return model
