"""OTLP/JSON metrics exporter (role of the reference's ``OtelExporter``,
crates/st-core/src/telemetry/monitoring.rs:526-575): payload shape, durable write, HTTP post to a collector."""
import http.server
import json
import threading

from spiraltorch_b200.nn.trainer import StepMetrics
from spiraltorch_b200.telemetry import MonitoringHub, OtelExporter


def test_payload_shape_and_accumulation(tmp_path):
    e = OtelExporter("svc")
    e.record_gauge("loss", 1.5, [("rank", "0")])
    e.record_gauge("loss", 1.25, [("rank", "0")])               # gauges keep the latest value
    e.record_gauge("loss", 2.0, [("rank", "1")])
    e.record_counter("steps", 2)
    e.record_counter("steps", 3)                                 # counters accumulate
    e.record_counter("steps", -5)                                # and never go down
    doc = e.payload()
    res = doc["resourceMetrics"][0]
    assert res["resource"]["attributes"][0] == {"key": "service.name", "value": {"stringValue": "svc"}}
    metrics = {m["name"]: m for m in res["scopeMetrics"][0]["metrics"]}
    pts = metrics["loss"]["gauge"]["dataPoints"]
    assert [(p["asDouble"], p["attributes"][0]["value"]["stringValue"]) for p in pts] == [(1.25, "0"), (2.0, "1")]
    s = metrics["steps"]["sum"]
    assert s["isMonotonic"] and s["aggregationTemporality"] == 2 and s["dataPoints"][0]["asDouble"] == 5.0
    e.write(tmp_path / "metrics.json")
    assert json.loads((tmp_path / "metrics.json").read_text()) == doc


def test_hub_exports_to_a_collector_over_http():
    got = []

    class Handler(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            got.append((self.path, json.loads(self.rfile.read(int(self.headers["Content-Length"])))))
            self.send_response(200)
            self.end_headers()

        def log_message(self, *a):
            pass
    srv = http.server.HTTPServer(("127.0.0.1", 0), Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        ex = OtelExporter()
        hub = MonitoringHub().with_exporter(ex)
        hub.observe(StepMetrics(step_time_ms=12.0, mem_peak_mb=100.0, extra={"loss": 0.7}), reward=1.0)
        assert ex.post(f"http://127.0.0.1:{srv.server_address[1]}/v1/metrics") == 200
    finally:
        srv.shutdown()
    path, doc = got[0]
    names = {m["name"] for m in doc["resourceMetrics"][0]["scopeMetrics"][0]["metrics"]}
    assert path == "/v1/metrics" and any("step_time" in n for n in names) and any("loss" in n for n in names)
