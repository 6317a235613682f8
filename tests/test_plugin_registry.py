"""Plugin registry, loaders and trace writers (reference behaviour: crates/st-core/src/plugin/registry.rs and its
tests, loader.rs, recorder.rs)."""
import pytest

from spiraltorch_b200 import plugin as bus
from spiraltorch_b200.plugin_registry import (DynamicPluginLoader, PluginCapability, PluginError, PluginEventRecorder,
                                              PluginMetadata, PluginRegistry, StaticPluginLoader, version_satisfies)


class P:
    def __init__(self, pid, version="1.0.0", deps=None, caps=(), fail_load=False):
        self.meta = PluginMetadata(pid, version, dependencies=dict(deps or {}), capabilities=list(caps))
        self.fail_load, self.log = fail_load, []

    def metadata(self): return self.meta                       # noqa: E704

    def on_load(self, ctx):
        if self.fail_load:
            raise RuntimeError("boom")
        ctx.set(f"loaded:{self.meta.id}", True)
        self.log.append("load")

    def on_unload(self, ctx): self.log.append("unload")        # noqa: E704
    def on_event(self, event, ctx): self.log.append(event["type"])      # noqa: E704


def test_version_requirements():
    assert version_satisfies("1.2.3", "*") and version_satisfies("1.2.3", ">=1.2, <2")
    assert version_satisfies("1.4.0", "^1.2") and not version_satisfies("2.0.0", "^1.2")
    assert version_satisfies("1.2.9", "~1.2") and not version_satisfies("1.3.0", "~1.2")
    assert not version_satisfies("0.9", ">=1.0") and version_satisfies("v1.0", "1.0.0")


def test_register_validates_and_publishes():
    reg = PluginRegistry()
    seen = []
    sid = bus.subscribe("PluginLoaded", seen.append)
    try:
        reg.register(P("core", caps=[PluginCapability("Telemetry")]))
        with pytest.raises(PluginError, match="already registered"):
            reg.register(P("core"))
        with pytest.raises(PluginError, match="requires 'missing'"):
            reg.register(P("x", deps={"missing": "*"}))
        with pytest.raises(PluginError, match="requires 'core' >=2"):
            reg.register(P("y", deps={"core": ">=2"}))
        with pytest.raises(PluginError, match="on_load"):
            reg.register(P("z", fail_load=True))
        with pytest.raises(PluginError):
            reg.register(P("bad id"))
        reg.register(P("viz", deps={"core": "^1.0"}, caps=[PluginCapability("Visualization"), PluginCapability("Backend", "cuda")]))
    finally:
        bus.unsubscribe("PluginLoaded", sid)
    assert reg.list_plugins() == ["core", "viz"] and [e["plugin_id"] for e in seen] == ["core", "viz"]
    assert reg.context().get("loaded:viz") is True
    assert [h.metadata().id for h in reg.find_by_capability(PluginCapability("Backend", "cuda"))] == ["viz"]
    assert reg.find_by_capability(PluginCapability("Backend", "hip")) == []
    reg.shutdown()


def test_dependency_graph_validation_and_safe_unload():
    reg = PluginRegistry()
    a, b, c, d = P("a"), P("b", deps={"a": "*"}), P("c", deps={"b": "*", "a": "*"}), P("d")
    for p in (a, b, c, d):
        reg.register(p)
    assert reg.dependency_graph() == {"a": [], "b": ["a"], "c": ["a", "b"], "d": []}
    assert reg.validate_dependency_graph().ok
    # a dependency declared after registration shows up as missing; a mutual dependency as a cycle
    d.meta.dependencies["ghost"] = "*"
    a.meta.dependencies["c"] = "*"
    summary = reg.validate_dependency_graph()
    assert not summary.ok and summary.missing == {"d": ["ghost"]} and summary.cycles == [["a", "c"], ["a", "c", "b"]]
    assert reg.validate_dependency_graph(internal_only=True).missing == {}
    del a.meta.dependencies["c"]
    assert reg.unregister_safe("a") == ["c", "b", "a"]            # dependents first
    assert reg.list_plugins() == ["d"] and c.log[-1] == "unload"
    assert reg.unregister_safe("nope", strict=False) == []
    with pytest.raises(PluginError):
        reg.unregister_safe("nope")
    reg.shutdown()


def test_plugins_receive_events_until_unloaded():
    reg = PluginRegistry()
    p = P("listener")
    reg.register(p)
    bus.publish("EpochStart", {"epoch": 1})
    assert "EpochStart" in p.log
    reg.unregister("listener")
    n = len(p.log)
    bus.publish("EpochStart", {"epoch": 2})
    assert len(p.log) == n


def test_loaders(tmp_path):
    reg = PluginRegistry()
    assert StaticPluginLoader(lambda: [P("s1"), P("s2")]).load_into(".", reg) == 2
    (tmp_path / "my_plugin.py").write_text(
        "from spiraltorch_b200.plugin_registry import PluginMetadata\n"
        "class Q:\n    def metadata(self):\n        return PluginMetadata('from_file', '0.1.0')\n"
        "def spiraltorch_plugins():\n    return [Q()]\n")
    (tmp_path / "not_a_plugin.py").write_text("x = 1\n")
    assert DynamicPluginLoader().load_into(tmp_path, reg) == 1
    assert reg.list_plugins() == ["from_file", "s1", "s2"]
    assert DynamicPluginLoader().discover(tmp_path / "absent") == []
    reg.shutdown()


def test_recorder_writers(tmp_path):
    with PluginEventRecorder(capacity=3) as rec:
        for i in range(5):
            bus.publish("TrainerStep", {"step": i})
        bus.publish("TensorOp", {"op": "matmul"})                 # filtered unless asked for
        snap = rec.snapshot()
        assert [r["event"]["step"] for r in snap["events"]] == [2, 3, 4] and snap["dropped"] == 2
        chart = rec.to_mermaid_flowchart(max_nodes=2)
        assert chart.splitlines()[0] == "flowchart TD" and 'n0["TrainerStep: 2"]' in chart and "n_more" in chart
        rec.write_jsonl(tmp_path / "trace.jsonl")
        rec.write_html(tmp_path / "trace.html")
    assert len((tmp_path / "trace.jsonl").read_text().splitlines()) == 3
    page = (tmp_path / "trace.html").read_text()
    assert "flowchart TD" in page and "<table>" in page and "TrainerStep" in page
    bus.publish("TrainerStep", {"step": 9})
    assert len(rec.snapshot()["events"]) == 3                     # closed: no longer subscribed
