"""Model-zoo run directories (models/README.md:13-22 of the reference).

A run directory holds ``command.txt``, ``run.json`` (``schema: "st.modelzoo.run.v1"``),
``metrics.jsonl`` (one JSON line per epoch with at least ``epoch``, ``batches``,
``average_loss``), ``weights.json`` and/or ``weights.bin``, and optionally ``summary.json`` and
``events.jsonl``.  Files are written atomically.
"""
from __future__ import annotations

import json
import sys
import time
from pathlib import Path
from typing import Optional

from ..config import atomic_write
from ..nn import io as nn_io

RUN_SCHEMA = "st.modelzoo.run.v1"


class RunDir:
    def __init__(self, path, arch: str, *, backend: str, hyper_params: Optional[dict] = None,
                 weight_format: str = "json", argv: Optional[list[str]] = None, extra: Optional[dict] = None):
        self.path = Path(path)
        self.path.mkdir(parents=True, exist_ok=True)
        self.weight_format = weight_format
        atomic_write(self.path / "command.txt", " ".join(argv if argv is not None else sys.argv) + "\n")
        self.meta = {"schema": RUN_SCHEMA, "arch": arch, "format": weight_format, "backend": backend,
                     "hyper_params": hyper_params or {}, "events": None, "created_unix": time.time()}
        if extra:
            self.meta.update(extra)
        atomic_write(self.path / "run.json", json.dumps(self.meta, indent=2))
        self._metrics = self.path / "metrics.jsonl"
        self._metrics.write_text("")

    def events_path(self) -> Path:
        self.meta["events"] = "events.jsonl"
        atomic_write(self.path / "run.json", json.dumps(self.meta, indent=2))
        return self.path / "events.jsonl"

    def log_epoch(self, epoch: int, batches: int, average_loss: float, **extra) -> None:
        rec = {"epoch": epoch, "batches": batches, "average_loss": average_loss, **extra}
        with open(self._metrics, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(rec) + "\n")

    def save_weights(self, model_or_state, name: str = "weights") -> Path:
        ext = ".json" if self.weight_format == "json" else ".bin"
        p = self.path / (name + ext)
        nn_io.save(p, model_or_state)
        return p

    def write_summary(self, summary: dict) -> None:
        atomic_write(self.path / "summary.json", json.dumps(summary, indent=2))


def read_metrics(run_dir) -> list[dict]:
    p = Path(run_dir) / "metrics.jsonl"
    return [json.loads(line) for line in p.read_text().splitlines() if line.strip()]


def compare_runs(run_dirs, metric: str = "average_loss") -> dict:
    """Side-by-side summary of run directories (the reference's run comparers in `tools/` and
    `examples/zspace_experiment_compare.py`): per run the architecture, backend, epochs, first / last / best
    value of `metric`, and the ranking by the last value (lower is better)."""
    rows = []
    for d in run_dirs:
        d = Path(d)
        run = json.loads((d / "run.json").read_text())
        vals = [m[metric] for m in read_metrics(d) if metric in m]
        if not vals:
            raise ValueError(f"{d}: no {metric!r} in metrics.jsonl")
        rows.append({"run_dir": str(d), "arch": run.get("arch"), "backend": run.get("backend"), "epochs": len(vals),
                     "first": vals[0], "last": vals[-1], "best": min(vals),
                     "improvement": (vals[0] - vals[-1]) / abs(vals[0]) if vals[0] else 0.0})
    order = sorted(range(len(rows)), key=lambda i: rows[i]["last"])
    for rank, i in enumerate(order, 1):
        rows[i]["rank"] = rank
    return {"schema": "st.modelzoo.compare.v1", "metric": metric, "runs": rows, "best_run": rows[order[0]]["run_dir"]}
