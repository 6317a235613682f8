"""Plugin registry: lifecycle, dependency validation, capability lookup, loaders and event-trace writers.

A plugin is any object with ``metadata() -> PluginMetadata`` and optional ``on_load(ctx)``, ``on_unload(ctx)``,
``on_event(event, ctx)`` hooks.  The registry validates the metadata and the declared dependencies before
``on_load`` runs, publishes ``PluginLoaded`` / ``PluginUnloaded`` on the process-wide event bus
(:mod:`spiraltorch_b200.plugin`), answers capability queries, reports missing dependencies and dependency cycles,
and unloads a plugin together with its dependents in reverse topological order.

Restated from crates/st-core/src/plugin: ``PluginMetadata`` / ``PluginCapability`` / ``Plugin`` (traits.rs:15-183),
``PluginRegistry`` (registry.rs:74-520: ``register`` :98, ``unregister`` :155, ``find_by_capability`` :188,
``dependency_graph`` :209, ``validate_dependency_graph`` :237, ``unregister_safe`` :286), ``PluginLoader`` /
``StaticPluginLoader`` / ``DynamicPluginLoader`` (loader.rs), ``PluginEventRecorder`` with its JSONL, Mermaid and
HTML writers (recorder.rs:60-290).
"""
from __future__ import annotations

import html
import importlib
import json
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterable, Optional

from . import plugin as bus

CAPABILITIES = ("Backend", "Operators", "LossFunctions", "Optimizers", "DataLoaders", "Visualization", "Telemetry",
                "Language", "Vision", "ReinforcementLearning", "GraphNeuralNetworks", "Recommender", "Custom")


class PluginError(RuntimeError):
    pass


@dataclass(frozen=True)
class PluginCapability:
    kind: str
    detail: Optional[str] = None          # backend name for "Backend", free text for "Custom"

    def __post_init__(self):
        if self.kind not in CAPABILITIES:
            raise PluginError(f"unknown plugin capability '{self.kind}'")

    def __str__(self) -> str:
        return self.kind if self.detail is None else f"{self.kind}({self.detail})"


@dataclass
class PluginMetadata:
    id: str
    version: str
    name: Optional[str] = None
    description: Optional[str] = None
    author: Optional[str] = None
    dependencies: dict = field(default_factory=dict)      # plugin id → version requirement
    capabilities: list = field(default_factory=list)
    metadata: dict = field(default_factory=dict)

    def with_name(self, v): self.name = v; return self                       # noqa: E702
    def with_description(self, v): self.description = v; return self         # noqa: E702
    def with_author(self, v): self.author = v; return self                   # noqa: E702
    def with_dependency(self, pid, req="*"): self.dependencies[pid] = req; return self       # noqa: E702
    def with_capability(self, cap): self.capabilities.append(cap); return self               # noqa: E702
    def with_metadata(self, k, v): self.metadata[k] = v; return self         # noqa: E702


def _validate_metadata(m: PluginMetadata) -> None:
    if not isinstance(m, PluginMetadata):
        raise PluginError("Plugin metadata() must return PluginMetadata")
    if not m.id or m.id != m.id.strip() or any(ch.isspace() for ch in m.id):
        raise PluginError("plugin id must be non-empty and free of whitespace")
    if not m.version or not m.version.strip():
        raise PluginError(f"plugin '{m.id}' has an empty version")
    if m.id in m.dependencies:
        raise PluginError(f"plugin '{m.id}' depends on itself")


def _version_tuple(v: str) -> tuple:
    out = []
    for part in v.strip().lstrip("v").split("."):
        digits = "".join(ch for ch in part if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out + [0] * (3 - len(out)))[:3]


def version_satisfies(version: str, requirement: str) -> bool:
    """``*`` / empty, exact ``1.2.3``, comparison ``>=1.2``, caret ``^1.2`` (same major) and tilde ``~1.2``
    (same major.minor); several comma-separated clauses must all hold."""
    req = (requirement or "*").strip()
    if req in ("", "*"):
        return True
    v = _version_tuple(version)
    for clause in (c.strip() for c in req.split(",")):
        for op in (">=", "<=", "==", ">", "<", "^", "~", "="):
            if clause.startswith(op):
                want = _version_tuple(clause[len(op):])
                ok = {">=": v >= want, "<=": v <= want, "==": v == want, "=": v == want, ">": v > want, "<": v < want,
                      "^": v[0] == want[0] and v >= want, "~": v[:2] == want[:2] and v >= want}[op]
                break
        else:
            ok = v == _version_tuple(clause)
        if not ok:
            return False
    return True


@dataclass
class DependencyValidationSummary:
    ok: bool
    missing: dict
    cycles: list


class PluginContext:
    """What a plugin sees while its hooks run: a key/value store shared through the registry and the event bus."""

    def __init__(self):
        self.values: dict = {}
        self.services: dict = {}

    def set(self, key, value): self.values[key] = value          # noqa: E704
    def get(self, key, default=None): return self.values.get(key, default)      # noqa: E704
    def register_service(self, name, obj): self.services[name] = obj            # noqa: E704
    def subscribe(self, event_type: str, fn) -> int: return bus.subscribe(event_type, fn)      # noqa: E704
    def publish(self, event_type: str, payload=None) -> int: return bus.publish(event_type, payload)   # noqa: E704


class PluginHandle:
    def __init__(self, plugin):
        self._plugin, self._lock = plugin, threading.Lock()

    def metadata(self) -> PluginMetadata:
        with self._lock:
            return self._plugin.metadata()

    def with_plugin(self, fn):
        with self._lock:
            return fn(self._plugin)


class PluginRegistry:
    def __init__(self):
        self._plugins: dict = {}
        self._lock = threading.RLock()
        self._in_transition: set = set()
        self._context = PluginContext()
        self._subs: dict = {}

    # ---- lifecycle ---------------------------------------------------------------------------------------
    def _begin(self, pid: str):
        with self._lock:
            if pid in self._in_transition:
                raise PluginError(f"Plugin '{pid}' is already being loaded or unloaded")
            self._in_transition.add(pid)

    def _end(self, pid: str):
        with self._lock:
            self._in_transition.discard(pid)

    def register(self, plugin) -> None:
        try:
            meta = plugin.metadata()
        except Exception as exc:  # noqa: BLE001
            raise PluginError(f"Plugin metadata() failed: {exc}") from exc
        _validate_metadata(meta)
        self._begin(meta.id)
        try:
            with self._lock:
                if meta.id in self._plugins:
                    raise PluginError(f"Plugin '{meta.id}' is already registered")
                for dep, req in meta.dependencies.items():
                    have = self._plugins.get(dep)
                    if have is None:
                        raise PluginError(f"Plugin '{meta.id}' requires '{dep}', which is not registered")
                    ver = have.metadata().version
                    if not version_satisfies(ver, req):
                        raise PluginError(f"Plugin '{meta.id}' requires '{dep}' {req}, found {ver}")
            hook = getattr(plugin, "on_load", None)
            if hook is not None:
                try:
                    hook(self._context)
                except Exception as exc:  # noqa: BLE001
                    raise PluginError(f"Plugin '{meta.id}' failed in on_load: {exc}") from exc
            with self._lock:
                if meta.id in self._plugins:
                    raise PluginError(f"Plugin '{meta.id}' became registered during on_load")
                self._plugins[meta.id] = PluginHandle(plugin)
            on_event = getattr(plugin, "on_event", None)
            if on_event is not None:
                ctx = self._context
                self._subs[meta.id] = bus.subscribe("*", lambda ev, f=on_event: f(ev, ctx))
        finally:
            self._end(meta.id)
        bus.publish("PluginLoaded", {"plugin_id": meta.id})

    def unregister(self, plugin_id: str) -> None:
        """The plugin leaves the registry before its hook runs; a failing hook is reported but the plugin is not
        put back."""
        self._begin(plugin_id)
        try:
            with self._lock:
                handle = self._plugins.pop(plugin_id, None)
            if handle is None:
                raise PluginError(f"Plugin '{plugin_id}' not found")
            sid = self._subs.pop(plugin_id, None)
            if sid is not None:
                bus.unsubscribe("*", sid)
            err = None
            try:
                handle.with_plugin(lambda p: getattr(p, "on_unload", lambda c: None)(self._context))
            except Exception as exc:  # noqa: BLE001
                err = PluginError(f"Plugin '{plugin_id}' failed in on_unload: {exc}")
        finally:
            self._end(plugin_id)
        bus.publish("PluginUnloaded", {"plugin_id": plugin_id})
        if err is not None:
            raise err

    def get(self, plugin_id: str) -> Optional[PluginHandle]:
        with self._lock:
            return self._plugins.get(plugin_id)

    def list_plugins(self) -> list:
        with self._lock:
            return sorted(self._plugins)

    def find_by_capability(self, capability: PluginCapability) -> list:
        with self._lock:
            items = sorted(self._plugins.items())
        return [h for _, h in items if capability in h.metadata().capabilities]

    def context(self) -> PluginContext:
        return self._context

    def initialize_all(self) -> None:
        bus.publish("SystemInit", {})

    def shutdown(self) -> list:
        """Unloads every plugin, dependents before their dependencies; returns the order used."""
        order = []
        for pid in self.list_plugins():
            if self.get(pid) is not None:
                order.extend(self.unregister_safe(pid, strict=False))
        bus.publish("SystemShutdown", {})
        return order

    # ---- dependency graph --------------------------------------------------------------------------------
    def dependency_graph(self, internal_only: bool = False) -> dict:
        with self._lock:
            items = sorted(self._plugins.items())
        ids = {pid for pid, _ in items}
        graph = {}
        for pid, handle in items:
            deps = sorted(set(handle.metadata().dependencies))
            graph[pid] = [d for d in deps if d in ids] if internal_only else deps
        return graph

    def validate_dependency_graph(self, internal_only: bool = False) -> DependencyValidationSummary:
        graph = self.dependency_graph(False)
        ids = sorted(graph)
        idset = set(ids)
        missing, internal = {}, {}
        for pid in ids:
            internal[pid] = sorted(d for d in graph[pid] if d in idset)
            gone = sorted(d for d in graph[pid] if d not in idset)
            if gone and not internal_only:
                missing[pid] = gone
        cycles = _detect_cycles(ids, internal)
        cycles.sort(key=lambda c: (len(c), c))
        return DependencyValidationSummary(not missing and not cycles, missing, cycles)

    def unregister_safe(self, plugin_id: str, strict: bool = True) -> list:
        """Unloads ``plugin_id`` and everything that (transitively) depends on it; returns the unload order."""
        plugin_id = plugin_id.strip()
        if not plugin_id:
            raise PluginError("plugin_id must not be empty")
        if self.get(plugin_id) is None:
            if strict:
                raise PluginError(f"Plugin '{plugin_id}' not found")
            return []
        graph = self.dependency_graph(False)
        dependents: dict = {}
        for pid, deps in graph.items():
            for d in deps:
                dependents.setdefault(d, set()).add(pid)
        match, queue = set(), [plugin_id]
        while queue:
            cur = queue.pop(0)
            if cur in match:
                continue
            match.add(cur)
            queue.extend(sorted(dependents.get(cur, ())))
        indeg = {pid: sum(1 for d in graph.get(pid, ()) if d in match) for pid in match}
        ready = sorted(pid for pid, n in indeg.items() if n == 0)
        order = []
        while ready:
            cur = ready.pop(0)
            order.append(cur)
            for child in sorted(dependents.get(cur, ())):
                if child in indeg:
                    indeg[child] -= 1
                    if indeg[child] == 0:
                        ready.append(child)
        unload = list(reversed(order)) if len(order) == len(match) else sorted(match, reverse=True)
        done = []
        for pid in unload:
            self.unregister(pid)
            done.append(pid)
        return done


def _detect_cycles(ids: list, graph: dict) -> list:
    """Elementary cycles found by depth-first search, each reported once, rotated to start at its smallest id."""
    seen, out = set(), []
    color: dict = {}
    stack: list = []

    def visit(n):
        color[n] = 1
        stack.append(n)
        for d in graph.get(n, ()):
            if color.get(d, 0) == 0:
                visit(d)
            elif color.get(d) == 1:
                cyc = stack[stack.index(d):]
                k = cyc.index(min(cyc))
                norm = tuple(cyc[k:] + cyc[:k])
                if norm not in seen:
                    seen.add(norm)
                    out.append(list(norm))
        stack.pop()
        color[n] = 2
    for n in ids:
        if color.get(n, 0) == 0:
            visit(n)
    return out


_GLOBAL = PluginRegistry()


def global_registry() -> PluginRegistry:
    return _GLOBAL


# ---- loaders -----------------------------------------------------------------------------------------------
class PluginLoader:
    def discover(self, path) -> list:
        raise NotImplementedError

    def load_into(self, path, registry: PluginRegistry) -> int:
        plugins = self.discover(path)
        for p in plugins:
            registry.register(p)
        return len(plugins)


class StaticPluginLoader(PluginLoader):
    def __init__(self, factory: Callable[[], list]):
        self.factory = factory

    def discover(self, path=None) -> list:
        return list(self.factory())


class DynamicPluginLoader(PluginLoader):
    """Imports every ``*.py`` file of a directory (or one module path) and collects the plugins returned by its
    ``spiraltorch_plugins()`` function; files without that function are skipped.  (The reference's dynamic loader
    is a placeholder that discovers nothing; Python modules are this package's shared-library equivalent.)"""

    def discover(self, path) -> list:
        path = Path(path)
        files = sorted(path.glob("*.py")) if path.is_dir() else ([path] if path.suffix == ".py" and path.exists() else [])
        found = []
        for f in files:
            spec = importlib.util.spec_from_file_location(f"spiraltorch_plugin_{f.stem}", f)
            mod = importlib.util.module_from_spec(spec)
            try:
                spec.loader.exec_module(mod)
            except Exception as exc:  # noqa: BLE001
                raise PluginError(f"plugin module {f} failed to import: {exc}") from exc
            factory = getattr(mod, "spiraltorch_plugins", None)
            if factory is not None:
                found.extend(factory())
        return found


# ---- event recorder and trace writers ------------------------------------------------------------------------
def _label(event: dict) -> str:
    t = event.get("type", "?")
    for key in ("plugin_id", "op", "name", "step", "epoch"):
        if key in event:
            return f"{t}: {event[key]}"
    return str(t)


class PluginEventRecorder:
    """Keeps the last ``capacity`` events of the bus in memory; ``snapshot`` / ``write_jsonl`` /
    ``to_mermaid_flowchart`` / ``write_html`` render them."""

    def __init__(self, capacity: int = 4096, capture_tensor_ops: bool = False, event_types: Iterable[str] = ("*",)):
        self.capacity, self.capture_tensor_ops = max(1, capacity), capture_tensor_ops
        self._events: list = []
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()
        self._idx = 0
        self.dropped = 0
        self._subs = [(t, bus.subscribe(t, self._on_event)) for t in event_types]

    def _on_event(self, event: dict) -> None:
        if not self.capture_tensor_ops and event.get("type") == "TensorOp":
            return
        rec = {"idx": self._idx, "elapsed_ms": int((time.perf_counter() - self._t0) * 1e3), "event": dict(event)}
        with self._lock:
            self._idx += 1
            self._events.append(rec)
            if len(self._events) > self.capacity:
                self._events.pop(0)
                self.dropped += 1

    def close(self) -> None:
        for t, sid in self._subs:
            bus.unsubscribe(t, sid)
        self._subs = []

    def __enter__(self): return self                # noqa: E704
    def __exit__(self, *exc): self.close()          # noqa: E704

    def snapshot(self) -> dict:
        with self._lock:
            return {"events": list(self._events), "dropped": self.dropped}

    def clear(self) -> None:
        with self._lock:
            self._events.clear()

    def write_jsonl(self, path) -> None:
        with open(path, "w", encoding="utf-8") as f:
            for rec in self.snapshot()["events"]:
                f.write(json.dumps(rec, default=str) + "\n")

    def to_mermaid_flowchart(self, max_nodes: int = 64) -> str:
        events = self.snapshot()["events"]
        max_nodes = max(1, max_nodes)
        lines = ["flowchart TD"]
        for i, rec in enumerate(events[:max_nodes]):
            label = _label(rec["event"]).replace('"', '\\"')
            lines.append(f'  n{i}["{label}"]')
            if i > 0:
                lines.append(f"  n{i - 1} --> n{i}")
        if len(events) > max_nodes:
            lines.append(f"  n{max_nodes - 1} --> n_more")
            lines.append('  n_more["… truncated …"]')
        return "\n".join(lines)

    def write_html(self, path, title: str = "SpiralTorch plugin trace", max_nodes: int = 64) -> None:
        """Self-contained page: the Mermaid source of the flow chart and a table of the recorded events."""
        snap = self.snapshot()
        rows = "\n".join(
            f"<tr><td>{r['idx']}</td><td>{r['elapsed_ms']}</td><td>{html.escape(str(r['event'].get('type', '?')))}</td>"
            f"<td><code>{html.escape(json.dumps({k: v for k, v in r['event'].items() if k not in ('type', 'ts')}, default=str))}"
            f"</code></td></tr>" for r in snap["events"])
        page = (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title>"
                "<style>body{font-family:sans-serif}table{border-collapse:collapse}td,th{border:1px solid #ccc;"
                "padding:2px 6px;font-size:12px}</style></head><body>"
                f"<h1>{html.escape(title)}</h1><p>{len(snap['events'])} events, {snap['dropped']} dropped</p>"
                f"<pre class='mermaid'>{html.escape(self.to_mermaid_flowchart(max_nodes))}</pre>"
                "<table><tr><th>#</th><th>ms</th><th>type</th><th>payload</th></tr>"
                f"{rows}</table></body></html>")
        Path(path).write_text(page, encoding="utf-8")
