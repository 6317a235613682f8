"""Ecosystem registry (crates/st-core/src/ecosystem/mod.rs)."""
import pytest

from spiraltorch_b200 import ecosystem as E


def test_metric_digest_accumulates_stats():
    reg = E.EcosystemRegistry()
    reg.record_metric(E.MetricSample("loss", 1.0, issued_at=10.0).with_tag("stage", "train"))
    reg.record_metric(E.MetricSample("loss", 0.5, issued_at=11.0).with_tag("stage", "train").with_unit("nats"))
    reg.record_metric(E.MetricSample("loss", 2.0, issued_at=12.0).with_tag("stage", "eval"))
    reg.record_metric(E.MetricSample("acc", 0.9, issued_at=13.0))
    rep = reg.snapshot()
    assert [(d.name, d.tags) for d in rep.metric_digests] == [("acc", []), ("loss", [("stage", "eval")]), ("loss", [("stage", "train")])]
    train = rep.metric_digests[2]
    assert (train.count, train.sum, train.min, train.max, train.average, train.last_value, train.unit) == (2, 1.5, 0.5, 1.0, 0.75, 0.5, "nats")
    assert (train.first_at, train.last_at) == (10.0, 11.0) and len(rep.metrics) == 4


def test_capacities_bound_the_queues_and_configure_is_transactional():
    reg = E.EcosystemRegistry(E.EcosystemCapacity(heuristics=2, roundtables=1, connectors=0, metrics=3))
    choice = E.HeuristicChoiceSummary(True, 256, 8, 0, algo_hint="bitonic")
    for i in range(4):
        reg.record_heuristic(E.HeuristicDecision("rank", "topk", 128, 4096, i, choice, source="kv"))
        reg.record_connector(E.ConnectorEvent("push", "sent"))
        reg.record_metric(E.MetricSample("m", float(i)))
    snap = reg.snapshot()
    assert [h.k for h in snap.heuristics] == [2, 3] and snap.connectors == [] and [m.value for m in snap.metrics] == [1.0, 2.0, 3.0]

    def shrink(cap):
        cap.metrics = 1
    reg.configure(shrink)
    assert [m.value for m in reg.snapshot().metrics] == [3.0] and reg.capacity().metrics == 1

    def boom(cap):
        cap.heuristics = 0
        raise RuntimeError("no")
    with pytest.raises(RuntimeError):
        reg.configure(boom)
    assert reg.capacity().heuristics == 2 and len(reg.snapshot().heuristics) == 2
    drained = reg.drain()
    assert len(drained.heuristics) == 2 and not reg.snapshot().heuristics and not reg.snapshot().metric_digests
    with pytest.raises(ValueError):
        E.HeuristicDecision("rank", "topk", 1, 1, 1, choice, source="oracle")


def test_connectors_and_roundtable_summaries():
    hub, sqs = E.CloudConnector("azure_event_hub", "ns", "hub"), E.CloudConnector("aws_sqs", "eu-west-1", "jobs")
    assert (hub.provider(), hub.service(), hub.descriptor()) == ("azure", "event_hub", "ns/hub")
    assert (sqs.provider(), sqs.service(), sqs.descriptor()) == ("aws", "sqs", "eu-west-1/jobs")
    with pytest.raises(ValueError):
        E.CloudConnector("gcp_pubsub", "a", "b")
    reg = E.EcosystemRegistry.global_()
    assert reg is E.EcosystemRegistry.global_()
    reg.drain()
    dist = E.DistributionSummary("node-0", "push", 8, 250, ["http://meta"], [hub, sqs])
    reg.record_roundtable(E.RoundtableSummary(64, 1024, E.RoundtableConfigSummary(4, 2, 1, 0.01), [E.RankPlanSummary("topk", 64, 1024, 4)], True, dist, issued_at=5.0))
    rt = reg.drain().roundtables[0]
    assert rt.distribution.cloud_targets[1].service() == "sqs" and rt.issued_at_secs() == 5.0 and rt.plans[0].kind == "topk"
