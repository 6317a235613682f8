"""In-process event bus with the reference's event vocabulary.

``subscribe(event_type, fn)`` registers a callback (``"*"`` = every event); ``publish`` fans a
dict payload out to the listeners; ``record(path, event_types=...)`` is a context manager
that streams events to a JSONL file.

Reference parity: ``PluginEventBus::{subscribe, has_listeners, publish}``
(crates/st-core/src/plugin/events.rs:126-187), ``PluginEventJsonlWriter``
(crates/st-core/src/plugin/recorder.rs:288-380), Python ``st.plugin.subscribe/unsubscribe/
record`` (bindings/st-py/spiraltorch/__init__.py:5161).
"""
from __future__ import annotations

import contextlib
import itertools
import json
import threading
import time
from typing import Callable, Iterable, Optional

EVENT_TYPES = ("SystemInit", "SystemShutdown", "TensorOp", "EpochStart", "EpochEnd", "BackendChanged",
               "Telemetry", "TrainerStep", "TrainerPhase", "RoundtablePlanned", "ZSpaceTrace",
               "TrainerAutopilotRejected", "Custom")

_lock = threading.RLock()
_listeners: dict[str, dict[int, Callable[[dict], None]]] = {}
_ids = itertools.count(1)


def subscribe(event_type: str, fn: Callable[[dict], None]) -> int:
    """Register ``fn`` for ``event_type`` (or ``"*"``); returns a subscription id."""
    with _lock:
        sid = next(_ids)
        _listeners.setdefault(event_type, {})[sid] = fn
        return sid


def unsubscribe(event_type: str, sid: int) -> bool:
    with _lock:
        return _listeners.get(event_type, {}).pop(sid, None) is not None


def has_listeners(event_type: str) -> bool:
    with _lock:
        return bool(_listeners.get(event_type)) or bool(_listeners.get("*"))


def publish(event_type: str, payload: Optional[dict] = None) -> int:
    """Deliver an event; returns the number of listeners called.  Listener exceptions propagate
    after every listener has run (first one wins)."""
    with _lock:
        targets = list(_listeners.get(event_type, {}).values()) + list(_listeners.get("*", {}).values())
    if not targets:
        return 0
    event = {"type": event_type, "ts": time.time(), **(payload or {})}
    first_error = None
    for fn in targets:
        try:
            fn(event)
        except Exception as exc:  # noqa: BLE001
            first_error = first_error or exc
    if first_error is not None:
        raise first_error
    return len(targets)


def clear() -> None:
    with _lock:
        _listeners.clear()


@contextlib.contextmanager
def record(path, event_types: Optional[Iterable[str]] = None):
    """Stream events to ``path`` as JSON lines while the block runs."""
    types = list(event_types) if event_types else ["*"]
    fh = open(path, "a", encoding="utf-8")
    wlock = threading.Lock()

    def write(event: dict) -> None:
        with wlock:
            fh.write(json.dumps(event, default=str) + "\n")

    sids = [(t, subscribe(t, write)) for t in types]
    try:
        yield path
    finally:
        for t, sid in sids:
            unsubscribe(t, sid)
        fh.flush()
        fh.close()
