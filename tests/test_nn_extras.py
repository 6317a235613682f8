"""Graph layers, Z-RBA attention, coherence sequencer and the Z-space VAE (CPU)."""
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.nn import gnn, zspace


def test_graph_context_and_convolution():
    A = torch.tensor([[0.0, 1.0, 0.0], [1.0, 0.0, 1.0], [0.0, 1.0, 0.0]])
    ctx = gnn.GraphContext.from_adjacency(A)
    d = torch.tensor([2.0, 3.0, 2.0]).rsqrt()
    expect = d[:, None] * (A + torch.eye(3)) * d[None, :]
    assert torch.allclose(ctx.norm_adjacency, expect)
    row = gnn.GraphContext(A, 1.0, "row")
    assert torch.allclose(torch.tensor(row.row_sums()), torch.ones(3))
    conv = gnn.ZSpaceGraphConvolution("gc", ctx, 2, 2)
    assert [p.name for p in conv.parameters()] == ["gc::weight", "gc::bias"]
    assert conv.weight.value.flatten().tolist() == pytest.approx([0.01, 0.02, 0.03, 0.04])
    x = st.Tensor(3, 2, [1.0, 0.0, 0.0, 1.0, 1.0, 1.0])
    y = conv.forward(x)
    assert torch.allclose(y.torch(), (expect @ x.torch()) @ conv.weight.value, atol=1e-6)
    conv.set_aggregation(gnn.NeighborhoodAggregation.multi_hop_mean(2))
    y2 = conv.forward(x)
    sup = (x.torch() + expect @ x.torch() + expect @ expect @ x.torch()) / 3
    assert torch.allclose(y2.torch(), sup @ conv.weight.value, atol=1e-6)
    # backward accumulates into the hypergrad tapes and a step changes the weights
    before = conv.weight.value.clone()
    conv.backward(x, st.Tensor._wrap(torch.ones(3, 2)))
    conv.apply_step(0.01)
    assert not torch.equal(before, conv.weight.value)
    with pytest.raises(st.TensorError):
        conv.forward(st.Tensor.zeros(4, 2))
    with pytest.raises(st.TensorError):
        gnn.GraphContext(torch.ones(2, 3))


def test_graph_regressors_learn():
    torch.manual_seed(0)
    A = (torch.rand(6, 6) > 0.5).float()
    A = ((A + A.t()) > 0).float()
    A.fill_diagonal_(0)
    ctx = gnn.GraphContext.from_adjacency(A)
    net = gnn.ZSpaceGraphNetwork("g", ctx, [3, 4, 1], learning_rate=0.05)
    reg = gnn.ZSpaceGraphRegressor(net, gnn.GraphReadout.mean())
    x = st.Tensor._wrap(torch.randn(6, 3))
    target = st.Tensor(1, 1, [0.7])
    loss = st.nn.MeanSquaredError()
    first = float(loss.forward(reg.forward(x), target).torch())
    for _ in range(60):
        pred = reg.forward(x)
        reg.backward(x, loss.backward(pred, target))
        reg.apply_step(0.05)
        reg.zero_accumulators()
    assert float(loss.forward(reg.forward(x), target).torch()) < 0.5 * first
    batch = gnn.GraphBatch([2, 4])
    breg = gnn.ZSpaceGraphBatchRegressor(net, gnn.GraphReadout.max(), batch)
    out = breg.forward(x)
    assert out.shape() == (2, 1)
    with pytest.raises(st.TensorError):
        breg.forward_batch(x, gnn.GraphBatch([2, 3]))
    assert gnn.GraphReadout.sum().forward(st.Tensor(2, 2, [1, 2, 3, 4])).tolist() == [[4.0, 6.0]]


def test_zrba_attention_kernel_and_variance():
    att = zspace.ZRBFAttention(8, 2, ard=True)
    idx = [zspace.ZIndex(0, 0, 0), zspace.ZIndex(0, 0, 1), zspace.ZIndex(3, 2, 4), zspace.ZIndex(3, 2, 7)]
    mu = st.Tensor.randn(4, 8, seed=1)
    sigma = st.Tensor._wrap(torch.full((4, 8), 0.5))
    out = att.forward(zspace.ZTensor(mu, sigma, idx), zspace.ZFrame(echoes=8))
    assert out.mean.shape() == (4, 8) and out.variance.shape() == (4, 8)
    v = out.variance.torch()
    assert bool((v > 0).all()) and bool((v <= 0.5 + 1e-6).all())     # Σ p² σ ≤ σ
    assert len(out.telemetry.entropy) == 2 and all(0 < e <= math.log(4) + 1e-6 for e in out.telemetry.entropy)
    # the echo distance is circular: 0 and 7 are neighbours on a ring of 8
    _, _, de = zspace.ZFrame(8).distances([zspace.ZIndex(0, 0, 0), zspace.ZIndex(0, 0, 7)], "cpu")
    assert de[0, 1].item() == 1.0
    with pytest.raises(st.TensorError):
        zspace.ZRBFAttention(7, 2)
    with pytest.raises(st.TensorError):
        zspace.ZTensor(mu, sigma, idx[:2])


def test_zspace_vae_optimizers(tmp_path):
    torch.manual_seed(0)
    basis = torch.randn(2, 6)
    data = torch.randn(64, 2) @ basis
    for kind in zspace.ZSpaceVae.OPTIMIZERS:
        vae = zspace.ZSpaceVae(6, 2, seed=3)
        vae.configure_optimizer_by_name(kind)
        first = vae.evaluate_batch(data)["recon_loss"]
        lr = 0.01 if kind == "sgd" else 0.02
        for _ in range(200):
            vae.train_batch(data, learning_rate=lr, beta=0.01)
        assert vae.evaluate_batch(data)["recon_loss"] < 0.5 * first, kind
        assert vae.optimizer_step() == 200 and vae.optimizer_kind() == kind
    p = tmp_path / "vae.json"
    vae.save(p)
    again = zspace.ZSpaceVae.load(p)
    assert torch.allclose(again.forward_mean(data).reconstruction, vae.forward_mean(data).reconstruction)
    with pytest.raises(st.TensorError):
        vae.configure_optimizer_by_name("lion")


def test_field_layers_match_their_definitions():
    from spiraltorch_b200.nn import fields as F
    v = torch.tensor([[0.5, 2.0, -3.0, 1.0]])
    out = F.porous_mix(v, 1.0, 0.5)
    assert out[0, 0] == 0.5 and out[0, 3] == 1.0
    assert out[0, 1].item() == pytest.approx(1.0 * (1 - 0.125 * (1.0 / 3.0)))
    assert out[0, 2].item() == pytest.approx(-(1 - 0.125 * 0.5))
    assert torch.equal(F.porous_mix(v, 1.0, 0.0), torch.tensor([[0.5, 1.0, -1.0, 1.0]]))

    res = F.ToposResonator("tr", 3, feedback=0.5, iterations=3, saturation=10.0)
    x = st.Tensor(1, 3, [0.2, -0.4, 1.0])
    assert res.forward(x).tolist()[0] == pytest.approx([0.2 * 1.75, -0.4 * 1.75, 1.75])     # 1 + 0.5 + 0.25

    kg = F.DynamicKleinGordonField("kg", 4, dt=0.1, stiffness=1.0, self_interaction=0.2)
    s = torch.tensor([[0.1, 0.4, -0.2, 0.3, 0.0, 0.1, 0.0, -0.1]])
    field, mom = s[:, :4], s[:, 4:]
    force = lambda f: (torch.roll(f, 1, 1) - 2 * f + torch.roll(f, -1, 1)) - f - 0.2 * f ** 3   # noqa: E731
    half = mom + 0.05 * force(field)
    nf = field + 0.1 * half
    expect = torch.cat([nf, half + 0.05 * force(nf)], 1)
    assert torch.allclose(kg.forward(st.Tensor._wrap(s)).torch(), expect, atol=1e-6)
    with pytest.raises(st.TensorError):
        kg.forward(st.Tensor.zeros(1, 4))

    hj = F.DynamicHamiltonJacobiField("hj", 4, dt=0.1, kinetic=2.0, viscosity=0.05)
    a = torch.tensor([[0.0, 1.0, 0.0, -1.0]])
    grad = (torch.roll(a, -1, 1) - torch.roll(a, 1, 1)) * 0.5
    lap = torch.roll(a, 1, 1) - 2 * a + torch.roll(a, -1, 1)
    assert torch.allclose(hj.forward(st.Tensor._wrap(a)).torch(), a - 0.1 * grad ** 2 + 0.05 * lap, atol=1e-6)

    sch = F.DynamicSchrodingerField("s", 2, dt=0.5, hopping=0.0, damping=0.2)
    sch.potential.value.copy_(torch.tensor([[1.0, 2.0]]))
    y = sch.forward(st.Tensor(1, 2, [1.0, 2.0])).torch()
    d = math.exp(-0.05)
    assert torch.allclose(y, torch.tensor([[d * math.cos(0.5), 2 * d * math.cos(1.0), -d * math.sin(0.5), -2 * d * math.sin(1.0)]]), atol=1e-6)
    hop = F.DynamicSchrodingerField("h", 2, dt=1.0, hopping=0.3).forward(st.Tensor(1, 2, [1.0, 0.0])).torch()
    assert hop[0, 0].item() == pytest.approx(math.cos(0.3)) and hop[0, 3].item() == pytest.approx(-math.sin(0.3))

    cw = F.ContinuousWavelet("cw", 32, scales=3)
    sig = torch.cos(torch.arange(32.0) * 0.8).reshape(1, -1)
    w = cw.forward(st.Tensor._wrap(sig))
    assert w.shape() == (1, 3) and float(w.torch().abs().max()) > 0
    proj = F.ZSpaceProjector("zp", 4, 3, curvature=-4.0)
    out = proj.forward(st.Tensor._wrap(torch.randn(5, 4) * 50)).torch()
    assert bool((out.norm(dim=1) < 0.5).all())
    rel = F.ZRelativity("zr", 3)
    rel.rapidity.value.copy_(torch.tensor([[0.0, 1.0, -1.0]]))
    g = math.sqrt(1 - math.tanh(1.0) ** 2)
    assert rel.forward(st.Tensor(1, 3, [1.0, 1.0, 1.0])).tolist()[0] == pytest.approx([1.0, g, g])
    c1 = F.Conv1d("c1", 2, 3, 3, 8, padding=1)
    xin = torch.randn(4, 16)
    ref = torch.nn.functional.conv1d(xin.reshape(4, 2, 8), c1.weight.value.reshape(3, 2, 3), c1.bias.value.flatten(), padding=1)
    assert torch.allclose(c1.forward(st.Tensor._wrap(xin)).torch(), ref.reshape(4, 24), atol=1e-5)
    # backward through the module protocol reaches the parameters
    for layer, xx in ((kg, st.Tensor._wrap(s)), (res, x), (c1, st.Tensor._wrap(xin))):
        yy = layer.forward(xx)
        gx = layer.backward(xx, st.Tensor._wrap(torch.ones_like(yy.torch())))
        assert gx.shape() == xx.shape() and any(p.accumulators() for p in layer.parameters())


def test_curvature_scheduler_tracks_pressure():
    from spiraltorch_b200.nn import CurvatureScheduler
    s = CurvatureScheduler(-1.0, -2.0, -0.1, target_pressure=0.5)
    d = s.observe_pressure(1.5)                                  # error +1 -> step limited to +0.05
    assert d["changed"] and d["curvature"] == pytest.approx(-0.95) and d["smoothed_pressure"] == 1.5
    for _ in range(40):
        s.observe_pressure(1.5)
    assert s.current == pytest.approx(-0.1)                      # saturates at the upper bound
    s.sync(-1.0)
    assert s.ema_pressure is None
    for _ in range(7):
        assert not s.observe_pressure(0.5)["changed"]            # inside the band, stable
    d = s.observe_pressure(0.5)                                  # 8th stable step: dither +0.15 * 0.05
    assert d["changed"] and d["curvature"] == pytest.approx(-1.0 + 0.0075)
    assert s.dither_sign == -1.0
    st_ = s.state()
    s2 = CurvatureScheduler.from_state(st_)
    assert s2.state() == st_
    with pytest.raises(ValueError):
        CurvatureScheduler.from_state({**st_, "current": 0.5})
    s3 = CurvatureScheduler(-5.0, -0.5, -3.0, 0.1).apply_env_overrides({"SPIRAL_CURVATURE_STEP": "0.2", "SPIRAL_CURVATURE_DITHER_PERIOD": "3", "SPIRAL_CURVATURE_KP": "bad"})
    assert (s3.min_curvature, s3.max_curvature, s3.current) == (-3.0, -0.5, -3.0)
    assert s3.step == 0.2 and s3.dither_period == 3 and s3.kp == 1.0
    assert s3.observe(torch.full((4, 4), -2.0))["raw_pressure"] == 2.0


def test_nd_convolutions_match_torch():
    import torch.nn.functional as F
    from spiraltorch_b200 import nn
    torch.manual_seed(0)
    c2 = nn.Conv2d("c2", 3, 5, (3, 2), (2, 1), (1, 0), (1, 2), (9, 8))
    x = torch.randn(4, 3 * 9 * 8)
    params = {p.name: p for p in c2.parameters()}
    wt, bs = params["c2::weight"].value, params["c2::bias"].value
    assert wt.shape == (5, 3 * 3 * 2)
    bs.copy_(torch.randn(1, 5))
    ref = F.conv2d(x.reshape(4, 3, 9, 8), wt.reshape(5, 3, 3, 2), bs.reshape(-1), (2, 1), (1, 0), (1, 2))
    y = c2.forward(st.Tensor._wrap(x)).torch()
    assert c2.output_shape() == tuple(ref.shape[1:])
    assert torch.allclose(y, ref.reshape(4, -1), atol=1e-4)
    c3 = nn.Conv3d("c3", 2, 3, (2, 3, 2), (1, 2, 1), (0, 1, 1), (1, 1, 1), (4, 6, 5))
    x3 = torch.randn(2, 2 * 4 * 6 * 5)
    p3 = {p.name: p for p in c3.parameters()}
    ref3 = F.conv3d(x3.reshape(2, 2, 4, 6, 5), p3["c3::weight"].value.reshape(3, 2, 2, 3, 2), None, (1, 2, 1), (0, 1, 1))
    assert torch.allclose(c3.forward(st.Tensor._wrap(x3)).torch(), ref3.reshape(2, -1), atol=1e-4)
    # 4-D: a kernel of extent 1 on the first axis reduces to independent 3-D convolutions
    c4 = nn.Conv4d("c4", 2, 3, (1, 2, 2, 2), input_dims=(3, 4, 4, 4))
    x4 = torch.randn(2, 2 * 3 * 4 * 4 * 4)
    w4 = {p.name: p for p in c4.parameters()}["c4::weight"].value.reshape(3, 2, 2, 2, 2)
    y4 = c4.forward(st.Tensor._wrap(x4)).torch().reshape(2, 3, 3, 3, 3, 3)
    for a in range(3):
        ref4 = F.conv3d(x4.reshape(2, 2, 3, 4, 4, 4)[:, :, a], w4)
        assert torch.allclose(y4[:, :, a], ref4, atol=1e-4)
    # backward through the Module API: dW is averaged over the batch like Linear
    g = c2.backward(st.Tensor._wrap(x), st.Tensor._wrap(torch.ones_like(y)))
    assert g.shape() == (4, 3 * 9 * 8)
    with pytest.raises(st.TensorError):
        c2.forward(st.Tensor._wrap(torch.randn(4, 7)))
    with pytest.raises(st.TensorError):
        nn.Conv2d("bad", 1, 1, (5, 5), input_hw=(3, 3))


def test_conv6da_pools_and_wave_scan():
    from spiraltorch_b200 import nn
    from spiraltorch_b200.nn.conv import ramanujan_pi
    import math
    assert abs(ramanujan_pi(2) - math.pi) < 1e-14
    layer = nn.Conv6da("z6", 2, 3, (2, 3, 3), leech_rank=24, leech_weight=0.5)
    assert layer.neighbor_count() == 7
    x = torch.randn(2, 2 * 18)
    y = layer.forward(st.Tensor._wrap(x)).torch().reshape(2, 3, 2, 3, 3)
    params = {p.name: p for p in layer.parameters()}
    w = params["z6::weight"].value
    assert w[0, 0] == pytest.approx(0.01) and w[0, 1] == pytest.approx(0.0131)
    vol = x.reshape(2, 2, 2, 3, 3)
    # centre cell (d=0, h=1, w=1) of sample 0: neighbours in offset order, zero outside the grid
    nb = []
    for od, oh, ow in layer.offsets:
        d, h, ww = 0 + od, 1 + oh, 1 + ow
        inside = 0 <= d < 2 and 0 <= h < 3 and 0 <= ww < 3
        nb += [float(vol[0, ic, d, h, ww]) if inside else 0.0 for ic in range(2)]
    nb = torch.tensor(nb)
    density = 0.5 * (math.pi ** 12 / math.factorial(12)) * float(nb.norm()) * math.sqrt(24)
    expect = float(w[1] @ nb) + density + (ramanujan_pi(6) - math.pi)
    assert float(y[0, 1, 0, 1, 1]) == pytest.approx(expect, abs=1e-4)
    mp = nn.MaxPool2d(2, (2, 2), (2, 2), (0, 0), (4, 4))
    ap = nn.AvgPool2d(2, (2, 2), (2, 2), (0, 0), (4, 4))
    img = torch.arange(32, dtype=torch.float32).reshape(1, 32)
    assert mp.forward(st.Tensor._wrap(img)).torch()[0, :4].tolist() == [5.0, 7.0, 13.0, 15.0]
    assert ap.forward(st.Tensor._wrap(img)).torch()[0, :2].tolist() == [2.5, 4.5]
    ws = nn.WaveScan("ws", 3, 4, 2, steps=6, padding=1)
    names = sorted(p.name for p in ws.parameters())
    assert names == ["ws::conv::bias", "ws::conv::weight", "ws::gate::bias", "ws::gate::gain"]
    out = ws.forward(st.Tensor._wrap(torch.randn(5, 18)))
    assert out.shape() == (5, 4)
    assert hasattr(nn, "GoldenRetriever") and nn.ZConv6DA is nn.Conv6da


def test_text_vae_learns_and_round_trips(tmp_path):
    from spiraltorch_b200.nn import LanguageWaveEncoder, ZSpaceTextVae
    enc = LanguageWaveEncoder(-1.0, 0.5)
    z = enc.encode_z_space("spiral")
    assert z.shape == (1, 12) and float(z.norm()) < 1.0                      # inside the unit ball
    wave = enc.encode_wave("ab")
    sig = [((ord("a") % 1024) / 1024 + abs(math.sin(0.5))) * 0.5, ((ord("b") % 1024) / 1024 + abs(math.sin(1.0))) * 0.5]
    assert wave[0].real == pytest.approx(sig[0] + sig[1], rel=1e-5) and wave[1].real == pytest.approx(sig[0] - sig[1], abs=1e-5)
    vae = ZSpaceTextVae(8, 3, seed=3)
    assert vae.input_dim == 16 and vae.encode_text("hi").shape == (16,)
    assert torch.equal(vae.encode_text("hi"), vae.encode_text("hi      "))   # space padding
    texts = ["spiral torch", "z-space wave", "hello world"]
    first = vae.evaluate_text_batch(texts)["recon_loss"]
    vae.configure_optimizer_by_name("adam")
    for _ in range(150):
        vae.train_text_batch(texts, learning_rate=2e-2, beta=1e-3)
    assert vae.evaluate_text_batch(texts)["recon_loss"] < 0.5 * first
    path = tmp_path / "tv.json"
    vae.save(path)
    again = ZSpaceTextVae.load(path)
    assert again.optimizer_kind() == "adam"
    assert again.evaluate_text_batch(texts)["recon_loss"] == pytest.approx(vae.evaluate_text_batch(texts)["recon_loss"], rel=1e-5)
    basis = torch.eye(16).flip(0)
    assert torch.allclose(vae.encode_text_with_mellin("hi", basis), vae.encode_text("hi").flip(0))
    with pytest.raises(st.TensorError):
        ZSpaceTextVae(0, 3)


def test_roundtable_node_and_conductor():
    from spiraltorch_b200.nn import roundtable as RT
    assert RT.outcome_band(0.5, 0.5, 0.1) == "above" and RT.outcome_band(0.1, 0.3, 0.3) == "here"
    lo, hi = RT.wilson_bounds(0.8, 10.0, 1.0)
    assert 0.6 < lo < 0.8 < hi < 0.95
    assert RT.RoundtableNode().record_decision("p", "s", "topk", "above", 0.9) is None      # local mode
    now = [0.0]
    sent = []
    cfg = RT.DistConfig("n0", RT.PERIODIC_META, push_interval=10.0, summary_window=3).with_aws_sqs("eu", "q").with_aws_sqs("eu", "q")
    assert cfg.cloud_targets == [("aws_sqs", "eu", "q")]
    node = RT.RoundtableNode(cfg, clock=lambda: now[0], sink=sent.append)
    assert node.record_decision("plan", "wg=256", "topk", "above", 0.9, psi_total=1.0, z_signal=0.2) is None
    assert node.record_decision("plan", "wg=256", "topk", "here", 0.7) is None
    s = node.record_decision("plan", "wg=256", "topk", "above", 1.4)                        # window full; score clamped
    assert s is not None and s.events == 3 and s.winner == "above" and s.mean_score == pytest.approx((0.9 + 0.7 + 1.0) / 3)
    assert s.mean_psi == pytest.approx(1.0 / 3) and sent == [s] and len(node.pending) == 0
    node.record_decision("plan", "wg=256", "topk", "above", 0.5)
    now[0] = 11.0
    assert node.record_decision("plan", "wg=256", "topk", "above", 0.5).events == 2         # interval elapsed
    node.retune(0.0, 0)
    assert node.config.push_interval == 0.010 and node.config.summary_window == 1
    cond = RT.MetaConductor(threshold=0.5, participation=2)
    a = RT.MetaSummary("n0", "plan", "wg=256", "topk", "above", 0.9, 0.7, 0.95, 0.0, 0.0, 0.4, 3, 1.0)
    b = RT.MetaSummary("n1", "plan", "wg=256", "topk", "above", 0.8, 0.6, 0.9, 0.0, 0.5, 0.3, 3, 2.0)
    assert cond.ingest(a) is None                                                            # one node only
    prop = cond.ingest(b)
    assert prop is not None and prop.ops[0].script == "wg=256" and len(prop.evidence) == 2
    assert prop.ops[0].weight == pytest.approx((0.4 + 0.3 * 1.2) / 0.5)
    assert cond.ingest(a) is None                                                            # evidence was cleared
    log = RT.HeurOpLog()
    ok, metrics = RT.simulate_proposal_locally(prop, log)
    assert ok and metrics == {"wg=256": prop.ops[0].weight} and log.high_watermark() == 1
    log.append(prop.ops[0]); log.append(prop.ops[0])
    other = RT.HeurOpLog(); other.merge(log); other.merge(log)
    assert other.high_watermark() == 2 and other.top_winners(5)[0].script == "wg=256" and RT.HeurOpLog().missing_ranges() == [(0, 0)]
    assert RT.exchange_summaries(a) == [a] and RT.exchange_summaries(None) == []


def test_zrba_block_gate_covariance_and_metrics():
    """Parity: crates/st-nn/src/z_rba/{mod,beta_residual,cov_head,telemetry}.rs unit tests."""
    import math
    from spiraltorch_b200.nn import (BetaGate, CovHead, SpectralFeatureSample, ZRBA, ZRBAConfig, ZRBAMetrics,
                                     ZFrame, ZIndex)
    from spiraltorch_b200.nn.zspace import ZTensor
    from spiraltorch_b200.nn.zrba import spearman_rank_correlation
    from spiraltorch_b200.tensor import Tensor, TensorError

    stats = SpectralFeatureSample(1, 0.8, 0.1, 0.05, 0.2)
    gate = BetaGate()
    s = gate.forward(stats, [ZIndex(1, 2, 3)])
    assert 0.0 <= s.sample <= 1.0 and s.alpha > 0 and s.beta > 0 and s.applied == s.sample
    assert abs(s.expected - s.alpha / (s.alpha + s.beta)) < 1e-12
    before = gate.ema()
    with pytest.raises(TensorError):
        gate.try_forward(SpectralFeatureSample(1, 0.8, math.inf, 0.05, 0.2), [ZIndex(1, 2, 3)])
    assert gate.ema() == before                                   # a rejected draw leaves the averages alone
    assert gate.forward(SpectralFeatureSample(1, 0.8, math.inf, 0.05, 0.2), []).expected == 0.5
    # same seed, same stream
    assert BetaGate().forward(stats, [ZIndex(1, 2, 3)]).sample == s.sample

    g = torch.Generator().manual_seed(0)
    mu, sig = torch.randn(12, 6, generator=g), torch.rand(12, 6, generator=g)
    out = CovHead(2).forward(mu, sig)
    cov = out.covariance.torch()
    assert torch.allclose(cov, cov.T, atol=1e-6)
    assert float(torch.linalg.eigvalsh(cov.double()).min()) >= 1e-4 - 1e-7
    assert out.telemetry.condition_number >= 1.0
    # full rank: covariance is exactly the sample covariance plus the mean diagonal
    full = CovHead(6).forward(mu, sig).covariance.torch()
    c = mu - mu.mean(0)
    assert torch.allclose(full, c.T @ c / 12 + torch.diag(sig.mean(0)), atol=1e-5)

    idx = [ZIndex(i % 3, i % 2, i % 4) for i in range(12)]
    blk = ZRBA(ZRBAConfig(d_model=6, n_heads=2, cov_rank=3))
    z, zc, tel = blk.forward(ZTensor(Tensor._wrap(mu), Tensor._wrap(sig), idx), ZFrame(4), stats)
    assert z.mu.shape() == (12, 6) and zc.covariance.shape() == (6, 6) and zc.gate.applied == zc.gate.expected
    # targets at the predicted mean: full coverage, and the NLL is the entropy term alone
    pred, var = z.mu.torch(), z.sigma.torch()
    m = tel.metrics(z.mu, z.sigma, pred.mean(1).tolist(), 0.9, idx)
    assert m.picp == 1.0 and [b.band for b in m.reliability_by_band] == [0, 1, 2]
    want = 0.5 * torch.log(2 * math.pi * var.clamp(min=1e-6).mean(1)).mean()
    assert abs(m.nll - float(want)) < 1e-5
    assert abs(m.pinaw - float(2 * 1.6448536 * var.mean(1).sqrt().mean())) < 1e-4
    bundle = tel.bundle_metrics(m).to_json()
    assert set(bundle) == {"metrics", "gate", "covariance"}
    assert abs(spearman_rank_correlation([1, 2, 3, 4], [10, 20, 30, 40]) - 1.0) < 1e-12
    assert abs(spearman_rank_correlation([1, 2, 3, 4], [4, 3, 2, 1]) + 1.0) < 1e-12
    with pytest.raises(TensorError):
        ZRBAMetrics.compute(z.mu, z.sigma, [0.0], 0.9, idx)


def test_zspace_vae_closed_form_gradients_match_autograd_and_stats():
    torch.manual_seed(4)
    vae = zspace.ZSpaceVae(6, 3, seed=1)
    x = torch.randn(5, 6)
    leaves = {k: v.clone().requires_grad_(True) for k, v in vae.p.items()}
    mu = x @ leaves["enc_mu"] + leaves["b_mu"]
    lv = x @ leaves["enc_logvar"] + leaves["b_logvar"]
    rec = mu @ leaves["dec"] + leaves["b_dec"]
    loss = (((rec - x) ** 2).mean(-1) + 0.3 * (-0.5 * (1 + lv - mu ** 2 - lv.exp()).sum(-1))).mean()
    want = torch.autograd.grad(loss, list(leaves.values()))
    _, got = vae._gradients(x, 0.3)
    for (k, _), w in zip(leaves.items(), want):
        assert torch.allclose(got[k], w, atol=1e-6), k
    vae.configure_optimizer_by_name("adam", grad_clip=1e-3)
    before = {k: v.clone() for k, v in vae.p.items()}
    st_ = vae.train_batch(x, learning_rate=1e-2, beta=0.3)
    assert st_.batch_size == 5 and st_["samples"] == 5 and st_.optimizer == "adam" and st_.optimizer_step == 1
    assert st_.gradient_l2 > 1e-3 and st_.clipped_gradient_l2 == pytest.approx(1e-3) and st_.update_l2 > 0
    assert st_.weighted_loss == pytest.approx(st_.recon_loss + 0.3 * st_.kl_loss)
    assert st_.evidence_lower_bound == pytest.approx(-(st_.recon_loss + st_.kl_loss))
    assert any(not torch.equal(before[k], vae.p[k]) for k in before)
    ev = vae.evaluate_batch(x, beta=0.0)
    assert ev.learning_rate == 0.0 and ev.gradient_l2 == 0.0 and ev.kl_weight == 0.0
    state = vae.forward_mean(x)
    assert torch.equal(state.latent, state.mu) and state.recon_loss == state.stats.recon_loss
    r0 = state.recon_loss
    for _ in range(20):
        vae.refine_decoder(vae.forward_mean(x), 0.05)
    assert vae.forward_mean(x).recon_loss < r0
    for bad in (dict(learning_rate=0.0), dict(learning_rate=float("nan")), dict(beta=-1.0)):
        with pytest.raises(st.TensorError):
            vae.train_batch(x, **{"learning_rate": 1e-2, "beta": 1.0, **bad})
    with pytest.raises(st.TensorError):
        vae.configure_optimizer_by_name("adam", grad_clip=-1.0)
    with pytest.raises(st.TensorError):
        vae.train_batch(torch.full((2, 6), float("inf")))


def test_mellin_basis_projection():
    b = zspace.MellinBasis([1.0, 2.0, 0.5])
    p = b.project(torch.tensor([1.0, -2.0, 3.0]))
    assert float(p.norm()) == pytest.approx(1.0, abs=1e-6) and p[1] < 0
    raw = torch.tensor([1.0, -4.0, 3.0 ** 0.5])
    assert torch.allclose(p, raw / raw.norm(), atol=1e-6)
    ramp = zspace.MellinBasis.ramp(4, 0.5, 2.0)
    assert ramp.exponents.tolist() == pytest.approx([0.5, 1.0, 1.5, 2.0]) and ramp.dimension() == 4
    assert zspace.MellinBasis.ramp(1, 0.7, 9.0).exponents.tolist() == [0.7]
    assert zspace.MellinBasis.constant(3, 2.0).exponents.tolist() == [2.0] * 3
    short = zspace.MellinBasis([2.0]).project(torch.tensor([[2.0, 3.0]]))          # missing exponents default to 1
    assert torch.allclose(short, torch.tensor([[4.0, 3.0]]) / 5.0, atol=1e-6)
    vae = zspace.ZSpaceVae(3, 2, seed=0)
    mu, _ = vae.encode_with_mellin(torch.tensor([[1.0, -2.0, 3.0]]), b)
    assert torch.allclose(mu, vae.encode(p.reshape(1, 3))[0], atol=1e-6)
    assert float(vae.decode_with_mellin(mu, b).norm()) == pytest.approx(1.0, abs=1e-5)
    tv = zspace.ZSpaceTextVae(4, 2)
    assert float(tv.encode_text_with_mellin("abcd", zspace.MellinBasis.constant(8, 1.5)).norm()) == pytest.approx(1.0, abs=1e-5)


def test_reorder_feature_tensor_layouts():
    x = torch.arange(2 * 2 * 3 * 4, dtype=torch.float32).reshape(2, -1)          # C=4, H=2, W=3 stored NHWC
    t = st.nn.reorder_feature_tensor(st.Tensor._wrap(x), 4, 2, 3, "nhwc", "to")
    assert torch.equal(st.nn.reorder_feature_tensor(t, 4, 2, 3, "NHWC", "from_canonical").torch(), x)
    row, can = x[0], t.torch()[0]
    assert all(can[c * 6 + h * 3 + w] == row[(h * 3 + w) * 4 + c] for c in range(4) for h in range(2) for w in range(3))
    assert torch.equal(st.nn.reorder_feature_tensor(st.Tensor._wrap(x), 4, 2, 3, "NCHW").torch(), x)
    v = torch.arange(2 * 3 * 2 * 2 * 2, dtype=torch.float32).reshape(2, -1)       # C=3, D=H=W=2 stored NDHWC
    t3 = st.nn.reorder_feature_tensor_3d(st.Tensor._wrap(v), 3, 2, 2, 2)
    assert torch.equal(st.nn.reorder_feature_tensor_3d(t3, 3, 2, 2, 2, direction="from").torch(), v)
    assert t3.torch()[0][1 * 8 + 1 * 4 + 0 * 2 + 1] == v[0][((1 * 2 + 0) * 2 + 1) * 3 + 1]
    with pytest.raises(ValueError):
        st.nn.reorder_feature_tensor(t, 4, 2, 3, "CHWN")
    with pytest.raises(ValueError):
        st.nn.reorder_feature_tensor(t, 4, 2, 3, "NHWC", "sideways")
    with pytest.raises(st.TensorError):
        st.nn.reorder_feature_tensor(t, 5, 2, 3)
    with pytest.raises(ValueError):
        st.nn.FeatureReorder2d(4, 2, 3, layout="HWCN")
