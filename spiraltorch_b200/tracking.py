"""Experiment-tracking connectors for search loops and training runs.

Trackers implement the ``ExperimentTracker`` interface of :mod:`spiraltorch_b200.hpo`
(``on_suggest`` / ``on_observe`` / ``on_checkpoint``) and, for plain training runs,
``log_scalar(tag, value, step)``.  The reference ships the same set as loose scripts
(tools/tracking/base.py, mlflow_connector.py, wandb_connector.py) and a TensorBoard writer in its
self-supervised example (crates/spiral-selfsup/examples/selfsup_train.rs, ``SELF_SUP_LOGDIR``).
MLflow and W&B are optional imports: without the package the tracker logs once and stays inert.  The
TensorBoard writer needs no dependency: it emits the event-file framing (length, masked CRC-32C, payload,
masked CRC-32C) and the ``Event{wall_time, step, summary{value{tag, simple_value}}}`` protobuf by hand.
"""
from __future__ import annotations

import json
import logging
import os
import socket
import struct
import time
from typing import Any, Dict, Iterable, List, Optional

from .hpo import ExperimentTracker, TrialRecord

LOGGER = logging.getLogger("spiraltorch.tracking")


class CompositeTracker(ExperimentTracker):
    """Fans every callback out to several trackers; one failing tracker does not stop the others."""

    def __init__(self, trackers: Iterable[ExperimentTracker]):
        self.trackers: List[ExperimentTracker] = list(trackers)

    def _each(self, method: str, *args) -> None:
        for t in self.trackers:
            try:
                getattr(t, method)(*args)
            except Exception:                          # a tracker must never take the search down
                LOGGER.exception("tracker %s failed in %s", type(t).__name__, method)

    def on_suggest(self, trial: TrialRecord) -> None:
        self._each("on_suggest", trial)

    def on_observe(self, trial: TrialRecord) -> None:
        self._each("on_observe", trial)

    def on_checkpoint(self, state: dict) -> None:
        self._each("on_checkpoint", state)

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        for t in self.trackers:
            if hasattr(t, "log_scalar"):
                try:
                    t.log_scalar(tag, value, step)
                except Exception:
                    LOGGER.exception("tracker %s failed in log_scalar", type(t).__name__)


class ConsoleTracker(ExperimentTracker):
    def on_suggest(self, trial: TrialRecord) -> None:
        LOGGER.info("[trial %s] started %s", trial.id, trial.suggestion)

    def on_observe(self, trial: TrialRecord) -> None:
        LOGGER.info("[trial %s] metric=%s", trial.id, trial.metric)

    def on_checkpoint(self, state: dict) -> None:
        LOGGER.debug("checkpoint: %d completed, %d pending", len(state.get("completed", [])), len(state.get("pending", [])))

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        LOGGER.info("%s[%d] = %.6g", tag, step, value)


class JsonlTracker(ExperimentTracker):
    """One JSON object per event, appended and flushed — safe to tail while a search runs."""

    def __init__(self, path: str):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def _write(self, record: Dict[str, Any]) -> None:
        with open(self.path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps({"time": time.time(), **record}, sort_keys=True) + "\n")

    def on_suggest(self, trial: TrialRecord) -> None:
        self._write({"event": "trial_start", "id": trial.id, "params": trial.suggestion})

    def on_observe(self, trial: TrialRecord) -> None:
        self._write({"event": "trial_end", "id": trial.id, "params": trial.suggestion, "metric": trial.metric})

    def on_checkpoint(self, state: dict) -> None:
        self._write({"event": "checkpoint", "completed": len(state.get("completed", [])),
                     "pending": len(state.get("pending", [])), "next_trial_id": state.get("next_trial_id")})

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        self._write({"event": "scalar", "tag": tag, "value": float(value), "step": int(step)})


# ---- TensorBoard event files ---------------------------------------------------------------------

def _crc32c_table():
    table = []
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
        table.append(c)
    return table


_CRC_TABLE = _crc32c_table()


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _len_delimited(num: int, payload: bytes) -> bytes:
    return _field(num, 2, _varint(len(payload)) + payload)


def encode_scalar_event(tag: str, value: float, step: int, wall_time: float) -> bytes:
    summary_value = _len_delimited(1, tag.encode()) + _field(2, 5, struct.pack("<f", float(value)))
    summary = _len_delimited(1, summary_value)
    return (_field(1, 1, struct.pack("<d", wall_time)) + _field(2, 0, _varint(int(step))) + _len_delimited(5, summary))


def frame_record(payload: bytes) -> bytes:
    header = struct.pack("<Q", len(payload))
    return header + struct.pack("<I", _masked_crc(header)) + payload + struct.pack("<I", _masked_crc(payload))


class TensorBoardTracker(ExperimentTracker):
    """Writes ``events.out.tfevents.<time>.<host>`` under ``logdir`` (default ``$SELF_SUP_LOGDIR``)."""

    def __init__(self, logdir: Optional[str] = None, metric_tag: str = "hpo/metric"):
        logdir = logdir or os.environ.get("SELF_SUP_LOGDIR") or "runs"
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}")
        self.metric_tag = metric_tag
        version = _field(1, 1, struct.pack("<d", time.time())) + _len_delimited(3, b"brain.Event:2")
        with open(self.path, "wb") as fh:
            fh.write(frame_record(version))

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        with open(self.path, "ab") as fh:
            fh.write(frame_record(encode_scalar_event(tag, value, step, time.time())))

    def on_observe(self, trial: TrialRecord) -> None:
        if trial.metric is not None:
            self.log_scalar(self.metric_tag, trial.metric, trial.id)


def read_scalar_events(path: str) -> List[Dict[str, Any]]:
    """Reads back the scalar events of an event file written by :class:`TensorBoardTracker`, checking both
    checksums of every record."""
    out: List[Dict[str, Any]] = []
    data = open(path, "rb").read()
    pos = 0

    def varint(buf, i):
        shift = val = 0
        while True:
            b = buf[i]
            i += 1
            val |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return val, i

    def fields(buf):
        i = 0
        while i < len(buf):
            key, i = varint(buf, i)
            num, wire = key >> 3, key & 7
            if wire == 0:
                val, i = varint(buf, i)
            elif wire == 1:
                val, i = buf[i:i + 8], i + 8
            elif wire == 5:
                val, i = buf[i:i + 4], i + 4
            else:
                n, i = varint(buf, i)
                val, i = buf[i:i + n], i + n
            yield num, wire, val

    while pos < len(data):
        header = data[pos:pos + 8]
        (n,) = struct.unpack("<Q", header)
        if struct.unpack("<I", data[pos + 8:pos + 12])[0] != _masked_crc(header):
            raise ValueError("event file: bad length checksum")
        payload = data[pos + 12:pos + 12 + n]
        if struct.unpack("<I", data[pos + 12 + n:pos + 16 + n])[0] != _masked_crc(payload):
            raise ValueError("event file: bad payload checksum")
        pos += 16 + n
        event = {num: val for num, _, val in fields(payload)}
        if 5 in event:
            for num, _, sv in fields(event[5]):
                if num == 1:
                    value = {k: v for k, _, v in fields(sv)}
                    out.append({"step": event.get(2, 0), "wall_time": struct.unpack("<d", event[1])[0],
                                "tag": value[1].decode(), "value": struct.unpack("<f", value[2])[0]})
    return out


# ---- optional services ---------------------------------------------------------------------------

class MLflowTracker(ExperimentTracker):
    """Logs trials as nested MLflow runs when ``mlflow`` is importable; otherwise inert."""

    def __init__(self, experiment: Optional[str] = None, run_name: str = "spiral-search", client=None):
        self._run_name = run_name
        if client is None:
            try:
                import mlflow as client                     # type: ignore[no-redef]
            except Exception:
                client = None
                LOGGER.warning("mlflow is not installed; MLflowTracker is disabled")
        self._mlflow = client
        if self._mlflow is not None and experiment:
            self._mlflow.set_experiment(experiment)

    @property
    def enabled(self) -> bool:
        return self._mlflow is not None

    def on_observe(self, trial: TrialRecord) -> None:
        if not self.enabled:
            return
        with self._mlflow.start_run(run_name=f"{self._run_name}-{trial.id}", nested=True):
            self._mlflow.log_params({k: v for k, v in trial.suggestion.items()})
            if trial.metric is not None:
                self._mlflow.log_metric("metric", trial.metric, step=trial.id)

    def on_checkpoint(self, state: dict) -> None:
        if self.enabled and hasattr(self._mlflow, "log_dict"):
            self._mlflow.log_dict(state, "search_checkpoint.json")

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        if self.enabled:
            self._mlflow.log_metric(tag, value, step=step)


class WandbTracker(ExperimentTracker):
    """Logs trials to Weights & Biases when ``wandb`` is importable; otherwise inert."""

    def __init__(self, project: Optional[str] = None, client=None, **init_kwargs):
        if client is None:
            try:
                import wandb as client                      # type: ignore[no-redef]
            except Exception:
                client = None
                LOGGER.warning("wandb is not installed; WandbTracker is disabled")
        self._wandb = client
        self._run = self._wandb.init(project=project, **init_kwargs) if self._wandb is not None else None

    @property
    def enabled(self) -> bool:
        return self._wandb is not None

    def on_observe(self, trial: TrialRecord) -> None:
        if self.enabled:
            self._wandb.log({"trial": trial.id, "metric": trial.metric,
                             **{f"param/{k}": v for k, v in trial.suggestion.items()}})

    def log_scalar(self, tag: str, value: float, step: int) -> None:
        if self.enabled:
            self._wandb.log({tag: value}, step=step)


def build_trackers(specs: Iterable[str]) -> CompositeTracker:
    """``console``, ``jsonl:<path>``, ``tensorboard[:<logdir>]``, ``mlflow[:<experiment>]``, ``wandb[:<project>]``."""
    trackers: List[ExperimentTracker] = []
    for spec in specs:
        kind, _, arg = spec.partition(":")
        kind = kind.strip().lower()
        if kind == "console":
            trackers.append(ConsoleTracker())
        elif kind == "jsonl":
            if not arg:
                raise ValueError("jsonl tracker needs a path: jsonl:<path>")
            trackers.append(JsonlTracker(arg))
        elif kind == "tensorboard":
            trackers.append(TensorBoardTracker(arg or None))
        elif kind == "mlflow":
            trackers.append(MLflowTracker(arg or None))
        elif kind == "wandb":
            trackers.append(WandbTracker(arg or None))
        else:
            raise ValueError(f"unknown tracker {spec!r}")
    return CompositeTracker(trackers)
