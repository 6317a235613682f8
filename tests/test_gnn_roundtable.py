"""Roundtable signals steering graph message passing: influence derivation, per-hop scales, band-pass scales, the shared
bridge and the layer wiring (behaviour of crates/st-core/src/inference/gnn_roundtable.rs, crates/st-nn/src/gnn/mod.rs
and crates/st-nn/src/roundtable.rs `RoundtableGnnBridge`)."""
import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.nn import gnn
from spiraltorch_b200.nn.zrba import SpectralFeatureSample


def _influence(bands, sizes, drift=0.0, **spectral):
    return gnn.RoundtableBandInfluence(gnn.RoundtableBandSignal(*bands, sizes, drift, SpectralFeatureSample(**spectral) if spectral else None))


def test_directional_signal_biases_above_step():
    inf = _influence((1.4, 0.45, 0.2), (4, 2, 2), 0.35, sheet_index=1, sheet_confidence=0.9, curvature=0.6, spin=0.85, energy=0.72)
    above, here, beneath = inf.multipliers()
    assert above > beneath and above > here * 0.85 and inf.scale_for_step(1) > inf.scale_for_step(2)
    assert all(0.35 <= m <= 1.75 for m in inf.multipliers()) and 0.55 <= inf.drift_bias() <= 1.45


def test_curvature_pull_reinforces_here_band():
    inf = _influence((0.3, 1.2, 0.3), (2, 5, 2), sheet_confidence=0.88, curvature=3.4, spin=0.1, energy=0.58)
    above, here, beneath = inf.multipliers()
    assert here > above and here > beneath and inf.scale_for_step(0) >= inf.scale_for_step(1)


def test_edge_skewed_signal_can_promote_above_step():
    inf = _influence((0.19, 0.14, 0.01), (1, 2, 1), sheet_confidence=0.62, curvature=0.48, spin=0.45, energy=0.08)
    above, here, beneath = inf.multipliers()
    assert above > beneath and above >= here * 0.95 and inf.scale_for_step(1) > inf.scale_for_step(0)


def test_step_scales_decay_and_band_pass_scaling():
    inf = _influence((1.1, 0.5, 0.25), (2, 1, 1), 0.3)
    assert inf.scale_for_step(2) >= inf.scale_for_step(3) >= inf.scale_for_step(6) >= inf.scale_for_step(12) == inf.scale_for_step(40)
    assert all(0.25 <= inf.scale_for_step(k) <= 2.0 for k in range(12))
    a, h, b = inf.band_pass_scale_for_step("above", 1, 0.75), inf.band_pass_scale_for_step("here", 0, 0.75), inf.band_pass_scale_for_step("beneath", 2, 0.75)
    assert a > 1 and h > 1 and b > 1
    assert inf.band_pass_scale_for_step("above", 2, 0.75) < a and inf.band_pass_scale_for_step("beneath", 0, 0.75) < b
    assert inf.band_pass_scale_for_step("here", 1, 0.0) == 1.0
    with pytest.raises(st.TensorError):
        inf.band_pass_scale_for_step("above", 0, 1.5)
    with pytest.raises(st.TensorError):
        inf.band_pass_scale_for_step("sideways", 0, 0.5)


def test_signal_validation_and_round_trip():
    for bad in (dict(energy=(-1.0, 0.1, 0.1)), dict(energy=(float("nan"), 0.1, 0.1)), dict(sizes=(0, 1, 1)), dict(sizes=(1, 1)),
                dict(spectral=SpectralFeatureSample(spin=2.0)), dict(spectral=SpectralFeatureSample(curvature=5.0)), dict(drift=float("inf"))):
        with pytest.raises(st.TensorError):
            gnn.RoundtableBandSignal(*bad.get("energy", (0.3, 0.2, 0.1)), bad.get("sizes", (1, 1, 1)), bad.get("drift", 0.0), bad.get("spectral"))
    s = gnn.RoundtableBandSignal(0.3, 0.2, 0.1, (3, 4, 5), 0.2, SpectralFeatureSample(2, 0.5, 1.0, -0.3, 0.7), issued_at=12.5)
    again = gnn.RoundtableBandSignal.from_dict(s.as_dict())
    assert again.as_dict() == s.as_dict() and again.depth() == 12
    trainer = st.nn.ModuleTrainer()
    sched = trainer.roundtable(4, 4, st.nn.RoundtableConfig(top_k=3, mid_k=3, bottom_k=2))
    sig = gnn.RoundtableBandSignal.from_schedule(sched, {"above": 1.0, "here": 0.5, "beneath": 0.25})
    assert sig.band_sizes == (3, 11, 2)


def test_bridge_history_and_state():
    bridge = gnn.RoundtableGnnBridge(history_limit=3)
    assert bridge.latest() is None and bridge.is_empty()
    for i in range(5):
        bridge.publish(gnn.RoundtableBandSignal(0.1 * (i + 1), 0.2, 0.3, (1, 2, 3), issued_at=float(i)))
    assert len(bridge) == 3 and bridge.latest().issued_at == 4.0
    state = bridge.snapshot_state()
    other = gnn.RoundtableGnnBridge()
    other.restore_state(state)
    assert other.snapshot_state() == state and other.history_limit() == 3
    bridge.set_history_limit(1)
    assert [s.issued_at for s in bridge.drain()] == [4.0] and bridge.is_empty() and bridge.latest() is not None
    for bad in (0, 5000):
        with pytest.raises(st.TensorError):
            bridge.set_history_limit(bad)
    with pytest.raises(st.TensorError):
        other.restore_state({**state, "history_limit": 1})


def test_network_message_passing_follows_the_influence():
    torch.manual_seed(0)
    adj = torch.tensor([[0, 1, 0, 0], [1, 0, 1, 0], [0, 1, 0, 1], [0, 0, 1, 0]], dtype=torch.float32)
    net = gnn.ZSpaceGraphNetwork("g", gnn.GraphContext.from_adjacency(adj), [3, 2])
    layer = net.layers[0]
    layer.set_aggregation(gnn.NeighborhoodAggregation.multi_hop_sum(2))
    x = st.Tensor._wrap(torch.randn(4, 3))
    base = net.forward(x).torch()
    assert layer.last_step_scales == [1.0, 1.0, 1.0]
    bridge = gnn.RoundtableGnnBridge()
    net.attach_roundtable_bridge(bridge)
    assert not net.refresh_roundtable()
    bridge.publish(gnn.RoundtableBandSignal(1.4, 0.45, 0.2, (4, 2, 2), 0.35, SpectralFeatureSample(1, 0.9, 0.6, 0.85, 0.72)))
    assert net.refresh_roundtable()
    inf = layer.roundtable
    out = net.forward(x).torch()
    assert layer.last_step_scales == pytest.approx([inf.scale_for_step(k) for k in range(3)])
    # the support is the hop-weighted sum with each hop multiplied by its scale
    xt, w = x.torch(), layer.aggregation.weights()
    hops = [xt, layer.context.propagate_t(xt), layer.context.propagate_t(layer.context.propagate_t(xt))]
    want = sum(w[k] * inf.scale_for_step(k) * hops[k] for k in range(3)) @ layer.weight.value + layer.bias.value
    assert torch.allclose(out, want, atol=1e-5) and not torch.allclose(out, base)
    layer.set_active_band_pass("above", 0.75)
    net.forward(x)
    assert layer.last_step_scales[1] == pytest.approx(inf.scale_for_step(1) * inf.band_pass_scale_for_step("above", 1, 0.75))
    layer.set_active_band_pass(None)
    net.clear_roundtable_band()
    assert torch.allclose(net.forward(x).torch(), base)
