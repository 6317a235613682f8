"""Public API semantics (Tensor, nn modules, losses, trainer, weight files) on the CPU backend."""
import json
import math

import pytest
import torch

import spiraltorch as st


def test_tensor_constructors_and_basics():
    a = st.Tensor(2, 3, [1, 2, 3, 4, 5, 6])
    b = st.Tensor((2, 3), data=[1, 2, 3, 4, 5, 6])
    c = st.Tensor(data=[[1, 2, 3], [4, 5, 6]])
    assert a.shape() == b.shape() == c.shape() == (2, 3)
    assert a.tolist() == b.tolist() == c.tolist() == [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]
    assert st.Tensor(2, 2).tolist() == [[0.0, 0.0], [0.0, 0.0]]
    with pytest.raises(st.TensorError):
        st.Tensor(2, 2, [1, 2, 3])
    with pytest.raises(TypeError):
        st.Tensor(1, 2, 3, 4)
    r1, r2 = st.Tensor.rand(3, 4, seed=7), st.Tensor.rand(3, 4, seed=7)
    assert r1.tolist() == r2.tolist() and st.Tensor.randn(3, 4, seed=1).shape() == (3, 4)
    assert a.transpose().shape() == (3, 2) and a.reshape(3, 2).shape() == (3, 2)
    assert a.sum_axis0() == [5.0, 7.0, 9.0] and a.sum_axis1() == [6.0, 15.0]
    assert a.squared_l2_norm() == 91.0
    assert a.add(b).scale(0.5).tolist() == a.tolist()
    assert a.hadamard(b).tolist()[1] == [16.0, 25.0, 36.0]
    assert a.cat_rows(b).shape() == (4, 3)
    back = st.Tensor.from_dlpack(a.to_dlpack())
    assert back.tolist() == a.tolist()


def test_matmul_family_and_softmax_attention():
    torch.manual_seed(0)
    x, w = st.Tensor.randn(5, 4, seed=1), st.Tensor.randn(4, 3, seed=2)
    bias, res = st.Tensor.randn(1, 3, seed=3), st.Tensor.randn(5, 3, seed=4)
    ref = x.torch() @ w.torch()
    assert torch.allclose(x.matmul(w).torch(), ref, atol=1e-6)
    assert torch.allclose(x.matmul(w, backend="naive").torch(), ref, atol=1e-6)
    with pytest.raises(st.TensorError):
        x.matmul(w, backend="quantum")
    with pytest.raises(st.TensorError):
        w.matmul(x)
    assert torch.allclose(x.matmul_bias_relu(w, bias).torch(), torch.relu(ref + bias.torch()), atol=1e-6)
    g = torch.nn.functional.gelu(ref + bias.torch() + res.torch(), approximate="tanh")
    assert torch.allclose(x.matmul_bias_add_gelu(w, bias, res).torch(), g, atol=1e-6)
    sm, hard = x.row_softmax_hardmax()
    assert torch.allclose(sm.torch().sum(1), torch.ones(5), atol=1e-6)
    assert hard.torch().sum().item() == 5 and torch.equal(hard.torch().argmax(1), x.torch().argmax(1))
    q = st.Tensor.randn(6, 4, seed=5)
    zb = st.Tensor.randn(2, 3, seed=6)
    ab = st.Tensor(6, 3, [0.0 if c <= r % 3 else -1e9 for r in range(6) for c in range(3)])
    out = q.scaled_dot_attention(q, q, contexts=2, sequence=3, scale=0.5, z_bias=zb, attn_bias=ab)
    qq = q.torch().view(2, 3, 4)
    s = qq @ qq.transpose(1, 2) * 0.5 + zb.torch().view(2, 1, 3) + ab.torch().view(2, 3, 3)
    assert torch.allclose(out.torch(), (torch.softmax(s, -1) @ qq).reshape(6, 4), atol=1e-5)
    p = st.Tensor(2, 2, [3.0, 4.0, 0.0, 0.0]).project_to_poincare(-1.0).tolist()
    assert abs(math.hypot(*p[0]) - math.tanh(5.0)) < 1e-6 and p[1] == [0.0, 0.0]
    with pytest.raises(st.TensorError):
        q.project_to_poincare(0.5)
    ln = x.layer_norm_affine(st.Tensor(1, 4, [1, 1, 1, 1]), st.Tensor(1, 4, [0, 0, 0, 0]), epsilon=1e-5)
    assert torch.allclose(ln.torch().mean(1), torch.zeros(5), atol=1e-5)


def test_linear_matches_reference_conventions():
    layer = st.nn.Linear("fc", 2, 3)
    assert [n for n, _ in layer.state_dict()] == ["fc::bias", "fc::weight"]
    w = dict(layer.state_dict())["fc::weight"]
    assert w.shape() == (2, 3)
    assert [round(v, 6) for v in w.data()] == [0.01, 0.02, 0.03, 0.04, 0.05, 0.06]
    assert st.nn.Linear(2, 3, name="alt").state_dict()[0][0] == "alt::bias"
    x = st.Tensor(2, 2, [0.5, -0.1, 0.2, 0.3])
    target = st.Tensor(2, 3, [0.2] * 6)
    loss = st.nn.MeanSquaredError()
    pred = layer.forward(x)
    value, grad = loss.forward(pred, target), loss.backward(pred, target)
    assert value.shape() == (1, 1)
    manual = 2.0 / 6.0 * (pred.torch() - target.torch())
    assert torch.allclose(grad.torch(), manual, atol=1e-7)
    gx = layer.backward(x, grad)
    assert torch.allclose(gx.torch(), manual @ w.torch().t(), atol=1e-7)
    dw = layer.weight.gradient
    assert torch.allclose(dw, x.torch().t() @ manual / 2.0, atol=1e-7)        # the extra 1/batch
    assert torch.allclose(layer.bias.gradient, manual.sum(0, keepdim=True) / 2.0, atol=1e-7)
    before = layer.forward(x).tolist()
    layer.apply_step(0.05)
    layer.zero_accumulators()
    assert layer.forward(x).tolist() != before


def test_sequential_moves_layers_and_trains():
    model = st.nn.Sequential()
    linear = st.nn.Linear("l1", 2, 4)
    model.add(linear)
    model.add(st.nn.Relu())
    model.add(st.nn.Linear("l2", 4, 1))
    assert model.len() == 3 and len(model) == 3
    with pytest.raises(ValueError):
        linear.forward(st.Tensor(1, 2, [0.1, 0.2]))
    x = st.Tensor(4, 2, [0.1, 0.2, -0.3, 0.4, 0.5, -0.6, 0.7, 0.8])
    y = st.Tensor(4, 1, [0.3, -0.1, 0.2, 0.5])
    loss = st.nn.MeanSquaredError()
    l0 = loss.forward(model.forward(x), y).data()[0]
    for _ in range(50):
        pred = model.forward(x)
        model.backward(x, loss.backward(pred, y))
        model.apply_step(0.5)
        model.zero_accumulators()
    assert loss.forward(model.forward(x), y).data()[0] < l0
    assert [n for n, _ in model.state_dict()] == ["l1::bias", "l1::weight", "l2::bias", "l2::weight"]
    other = st.nn.Sequential([st.nn.Linear("l1", 2, 4), st.nn.Relu(), st.nn.Linear("l2", 4, 1)])
    other.load_state_dict(model.state_dict())
    assert other.forward(x).tolist() == model.forward(x).tolist()
    with pytest.raises(KeyError):
        other.load_state_dict([("l1::weight", st.Tensor(2, 4))])
    rep = other.state_dict_compatibility([("l1::weight", st.Tensor(3, 4)), ("zz", st.Tensor(1, 1))])
    assert not rep["compatible"] and "zz" in rep["unexpected"] and "l1::weight" in rep["shape_mismatch"]


def test_lora_linear_contract():
    with pytest.raises(ValueError, match="lora_alpha"):
        st.nn.LoraLinear(2, 1, 1, alpha=0.0, name="adapter")
    with pytest.raises(ValueError, match="lora_rank"):
        st.nn.LoraLinear(2, 1, 2, alpha=2.0, name="adapter")
    layer = st.nn.LoraLinear(2, 1, 1, alpha=2.0, name="adapter")
    assert layer.rank == 1 and layer.scale == pytest.approx(2.0)
    assert [n for n, _ in layer.state_dict()] == ["adapter::lora_a", "adapter::lora_b"]
    assert [n for n, _ in layer.base_state_dict()] == ["adapter::bias", "adapter::weight"]
    x, g = st.Tensor((1, 2), data=[0.5, -0.1]), st.Tensor((1, 1), data=[0.3])
    before = layer.forward(x).tolist()
    layer.backward(x, g)
    layer.apply_step(0.05)
    assert layer.forward(x).tolist() != before


@pytest.mark.parametrize("make", [
    lambda: st.nn.LayerNorm("ln", 6, -1.0, 1e-5), lambda: st.nn.ZSpaceLayerNorm("zln", 6, -1.0, 1e-5),
    lambda: st.nn.BatchNorm1d("bn", 6, 0.1, 1e-5), lambda: st.nn.Gelu(), lambda: st.nn.Scaler("sc", 6),
    lambda: st.nn.WaveGate("wg", 6, -1.0, 1.0), lambda: st.nn.SpiralRnn("rnn", 2, 5, 3),
    lambda: st.nn.Lstm("lstm", 2, 4, 3), lambda: st.nn.WaveRnn("wr", 2, 4, 3),
    lambda: st.nn.ZSpaceCoherenceScan(2, 3, 2, -1.0, 1.0), lambda: st.nn.ZSpaceCoherenceWaveBlock(2, 3, 2, -1.0, 1.0),
    lambda: st.nn.ZConv("conv", 1, 2, (2, 3), (2, 2), padding=(1, 1)), lambda: st.nn.Pool2d("max", 1, 2, 3, (1, 2)),
    lambda: st.nn.NonLiner("nl", 6), lambda: st.nn.Dropout(0.25, seed=3, training=False), lambda: st.nn.ZSpaceSoftmax(-1.0, 0.5),
])
def test_layer_backward_matches_finite_differences(make):
    layer = make()
    x = st.Tensor.randn(3, 6, seed=11)
    y = layer.forward(x)
    g = st.Tensor.randn(*y.shape(), seed=12)
    gx = layer.backward(x, g).torch()
    eps = 1e-3
    for (r, c) in [(0, 0), (1, 3), (2, 5)]:
        xp, xm = x.torch().clone(), x.torch().clone()
        xp[r, c] += eps
        xm[r, c] -= eps
        fd = ((layer.forward(st.Tensor(xp)).torch() - layer.forward(st.Tensor(xm)).torch()) * g.torch()).sum() / (2 * eps)
        assert abs(fd.item() - gx[r, c].item()) < 5e-3 * max(1.0, abs(fd.item())), (r, c, fd.item(), gx[r, c].item())


def test_losses():
    p, t = st.Tensor(2, 2, [0.7, 0.3, 0.2, 0.8]), st.Tensor(2, 2, [1, 0, 0, 1])
    cce = st.nn.CategoricalCrossEntropy()
    assert cce.forward(p, t).data()[0] == pytest.approx(-(math.log(0.7) + math.log(0.8)) / 2, rel=1e-5)
    hce = st.nn.HyperbolicCrossEntropy(-1.0)
    z = torch.tensor([[0.7, 0.3], [0.2, 0.8]])
    tt = torch.tensor([[1, 0], [0, 1.0]]).clamp(1e-5, 1 - 1e-5)
    ref = (tt * torch.nn.functional.softplus(-z) + (1 - tt) * torch.nn.functional.softplus(z)).mean()
    assert hce.forward(p, t).data()[0] == pytest.approx(ref.item(), rel=1e-5)
    assert st.nn.CrossEntropy is st.nn.HyperbolicCrossEntropy
    with pytest.raises(ValueError):
        st.nn.HyperbolicCrossEntropy(0.5)
    for loss in (st.nn.FocalLoss(), st.nn.ContrastiveLoss(1.0), st.nn.TripletLoss(0.5), st.nn.SoftmaxCrossEntropy()):
        v, g = loss.forward(p, t), loss.backward(p, t)
        assert v.shape() == (1, 1) and g.shape() == (2, 2) and math.isfinite(v.data()[0])
    ids = st.Tensor(2, 1, [0, 1])
    sce = st.nn.SoftmaxCrossEntropy()
    assert sce.forward(p, ids).data()[0] == pytest.approx(sce.forward(p, t).data()[0], rel=1e-6)


def test_trainer_events_roundtable_and_checkpoints(tmp_path):
    events = []
    sid = st.plugin.subscribe("EpochEnd", events.append)
    model = st.nn.Sequential([st.nn.Linear("l1", 2, 8), st.nn.Relu(), st.nn.Linear("l2", 8, 1)])
    model.attach_hypergrad(curvature=-1.0, learning_rate=1e-2)
    trainer = st.nn.ModuleTrainer(backend="cpu", curvature=-1.0, hyper_learning_rate=1e-2, fallback_learning_rate=1e-2)
    trainer.set_grad_clip_max_norm(1.0)
    sched = trainer.roundtable(8, 1, st.nn.RoundtableConfig(top_k=1, mid_k=1, bottom_k=1, here_tolerance=1e-5))
    x = st.Tensor.rand(8, 2, seed=1)
    y = st.Tensor(8, 1, [0.7 * r[0] - 0.2 * r[1] for r in x.tolist()])
    with st.plugin.record(tmp_path / "events.jsonl", event_types=["TrainerStep"]):
        stats = trainer.train_epoch(model, st.nn.MeanSquaredError(), [(x, y)], sched)
    st.plugin.unsubscribe("EpochEnd", sid)
    assert stats.batches == 1 and stats.average_loss == stats.total_loss
    assert events and events[0]["epoch"] == 1 and "loss" in events[0]
    assert json.loads((tmp_path / "events.jsonl").read_text().splitlines()[0])["type"] == "TrainerStep"
    g = st.Tensor(8, 1, [0.5, -0.01, 0.02, 0.0, -0.9, 0.03, 0.2, 0.000001])
    above, here, beneath = sched.split(g)
    assert torch.allclose(above.torch() + here.torch() + beneath.torch(), g.torch())
    assert above.data()[4] == pytest.approx(-0.9) and beneath.data()[1] == pytest.approx(-0.01)
    energy = sched.band_energy(g)
    assert energy["above"] == pytest.approx(0.81, rel=1e-5)
    # band-wise backward accumulates the same result as one backward
    a = st.nn.Linear("a", 2, 1)
    b = st.nn.Linear("a", 2, 1)
    t1, t2 = st.nn.ModuleTrainer(band_backward=True), st.nn.ModuleTrainer()
    t1.train_epoch(a, st.nn.MeanSquaredError(), [(x, y)], sched)
    t2.train_epoch(b, st.nn.MeanSquaredError(), [(x, y)], sched)
    assert torch.allclose(a.weight.value, b.weight.value, atol=1e-7)
    # optimizer / runtime checkpoints
    model.backward(x, st.Tensor(8, 1, [0.1] * 8))
    bundle = trainer.runtime_checkpoint_bundle(model)
    assert bundle["contract_version"].endswith(".v2")
    kept = [p.hypergrad.gradient.clone() for p in model.parameters()]
    model.zero_accumulators()
    trainer.restore_runtime_checkpoint_bundle(model, json.loads(json.dumps(bundle)))
    for p, k in zip(model.parameters(), kept):
        assert torch.allclose(p.hypergrad.gradient, k)
    model.apply_step(0.01)
    with pytest.raises(ValueError, match="fingerprint"):
        trainer.restore_optimizer_checkpoint(model, bundle["optimizer"])
    report = st.nn.ModuleTrainer().train_epochs(st.nn.Linear("z", 2, 1), st.nn.MeanSquaredError(), [(x, y)],
                                                epochs=3, validation_batches=[(x, y)], patience=1, restore_best=True)
    assert report["epochs_run"] >= 1 and "validation" in report["epochs"][0]


def test_weight_files_roundtrip_and_reference_layout(tmp_path):
    model = st.nn.Sequential([st.nn.Linear("fc1", 8, 32), st.nn.Relu(), st.nn.Linear("head", 32, 1)])
    for ext in (".json", ".bin", ".bincode"):
        path = tmp_path / f"weights{ext}"
        st.nn.save(path, model)
        manifest = json.loads((tmp_path / "weights.manifest.json").read_text())
        assert manifest["format_version"] == 1 and manifest["weights"]["format"] in ("json", "bincode")
        assert {e["name"] for e in manifest["state_dict"]} == {"fc1::weight", "fc1::bias", "head::weight", "head::bias"}
        for source in (path, tmp_path / "weights.manifest.json"):
            state = st.nn.load(source)
            assert [n for n, _ in state] == ["fc1::bias", "fc1::weight", "head::bias", "head::weight"]
            assert dict(state)["fc1::weight"].shape() == (8, 32)
            fresh = st.nn.Sequential([st.nn.Linear("fc1", 8, 32), st.nn.Relu(), st.nn.Linear("head", 32, 1)])
            st.nn.load(source, fresh)
            assert fresh.state_dict()[1][1].tolist() == model.state_dict()[1][1].tolist()
    doc = json.loads((tmp_path / "weights.json").read_text())
    assert set(doc) == {"parameters"} and doc["parameters"]["head::bias"] == {"rows": 1, "cols": 1, "data": [0.0]}
    # binary layout: u64 count, then (u64 key_len, key, u64 rows, u64 cols, u64 n, f32 x n)
    raw = (tmp_path / "weights.bin").read_bytes()
    import struct
    assert struct.unpack_from("<Q", raw, 0)[0] == 4
    klen = struct.unpack_from("<Q", raw, 8)[0]
    name = raw[16:16 + klen].decode()
    rows, cols, n = struct.unpack_from("<QQQ", raw, 16 + klen)
    assert name in doc["parameters"] and n == rows * cols
    with pytest.raises(ValueError):
        st.nn.save(tmp_path / "weights.manifest.json", model)
    with pytest.raises(ValueError):
        st.nn.save(tmp_path / "weights.txt", model)


def test_mlp_regression_config(tmp_path):
    from spiraltorch_b200.models import mlp_regression
    from spiraltorch_b200.models.zoo import read_metrics
    out = mlp_regression.run(tmp_path / "run", steps=200, quiet=True)
    assert out["final_loss"] < out["initial_loss"] and out["steps"] == 200
    run = json.loads((tmp_path / "run" / "run.json").read_text())
    assert run["schema"] == "st.modelzoo.run.v1"
    metrics = read_metrics(tmp_path / "run")
    assert metrics and {"epoch", "batches", "average_loss"} <= set(metrics[0])
    w = json.loads((tmp_path / "run" / "weights.json").read_text())["parameters"]
    assert (w["fc1::weight"]["rows"], w["fc1::weight"]["cols"]) == (8, 32) and "head::bias" in w


def test_session_and_dataloader():
    s = st.SpiralSession(backend="cpu", seed=3)
    assert s.backend == s.effective_backend == "cpu" and s.requested_backend == "cpu"
    plan = s.runtime_execution_plan()
    assert st.SpiralSession.from_runtime_execution_plan(plan).effective_backend == "cpu"
    plan["effective_backend"] = "cuda"
    with pytest.raises(ValueError):
        st.SpiralSession.from_runtime_execution_plan(plan)
    with pytest.raises(ValueError):
        st.SpiralSession(backend="tpu")
    ds = s.dataset([(st.Tensor(1, 2, [i, i]), st.Tensor(1, 1, [i])) for i in range(7)])
    loader = s.dataloader(ds).shuffle(5).batched(3).prefetch(2)
    batches = list(loader)
    assert [b[0].rows for b in batches] == [3, 3, 1]
    again = list(s.dataloader(ds).shuffle(5).batched(3))
    assert [b[1].tolist() for b in again] == [b[1].tolist() for b in batches]
    dyn = list(s.dataloader(ds).dynamic_batch_by_rows(2))
    assert [b[0].rows for b in dyn] == [2, 2, 2, 1]
    assert isinstance(s.trainer(), st.nn.ModuleTrainer)
    info = st.build_info()
    assert "cuda" in info["features"] and st.describe_device()["backends"]["cpu"]["ready"]
    s.close()


def test_spiral_lightning_plans():
    from spiraltorch_b200.nn import lightning as L
    sess = st.SpiralSession("cpu", seed=3)
    model = st.nn.Sequential()
    model.add(st.nn.Linear("fc", 4, 2))
    g = torch.Generator().manual_seed(0)
    w = torch.randn(4, 2, generator=g)
    def batches(n):
        out = []
        for _ in range(n):
            x = torch.randn(8, 4, generator=g)
            out.append((st.Tensor._wrap(x), st.Tensor._wrap(x @ w)))
        return out
    lt = L.SpiralLightning(sess, 8, 2)
    stats = lt.fit_epochs(model, st.nn.MeanSquaredError(), [batches(3), batches(3)])
    assert len(stats) == 2 and stats[0].batches == 3
    cfg2 = L.LightningConfig.builder(8, 2).roundtable(st.nn.RoundtableConfig(top_k=2, mid_k=1, bottom_k=1)).build()
    rep = lt.fit_plan(model, st.nn.MeanSquaredError(), [
        L.LightningStage(L.LightningConfig(8, 2), [batches(4) for _ in range(3)], "warm"),
        L.LightningStage(cfg2, [batches(4) for _ in range(3)], "refine")])
    assert rep.total_epochs() == 6 and rep.total_batches() == 24 and [s.label for s in rep.stages] == ["warm", "refine"]
    best = min(rep.epochs(), key=lambda e: e.average_loss)
    assert rep.best_epoch() is best and rep.stages[rep.best_stage_index()].best_epoch() is best
    assert lt.schedule().describe()["top_k"] == 2 if "top_k" in lt.schedule().describe() else True

    # self-supervised plan: an encoder learns to align two noisy views
    enc = st.nn.Sequential()
    enc.add(st.nn.Linear("enc", 6, 4))
    def views(n):
        out = []
        for _ in range(n):
            base = torch.randn(16, 6, generator=g)
            out.append((st.Tensor._wrap(base + 0.05 * torch.randn(16, 6, generator=g)),
                        st.Tensor._wrap(base + 0.05 * torch.randn(16, 6, generator=g))))
        return out
    lt2 = L.SpiralLightning(sess, 32, 4)
    got = []
    sid = st.plugin.subscribe("Telemetry", got.append)
    plan = lt2.fit_selfsup_plan(enc, [L.SelfSupStage(L.LightningConfig(32, 4), [views(4) for _ in range(6)], 0.2, True, "ssl")])
    st.plugin.unsubscribe("Telemetry", sid)
    eps = plan.stages[0].epochs
    assert plan.total_epochs() == 6 and eps[0].telemetry.batches == 4
    assert eps[-1].telemetry.mean_loss < eps[0].telemetry.mean_loss
    assert 0.0 <= eps[-1].telemetry.mean_accuracy <= 1.0 and any(e.get("selfsup") == "info_nce" for e in got)
    loss = L.InfoNCELoss(0.1)
    with pytest.raises(st.TensorError):
        loss.forward(st.Tensor.zeros(3, 4), None)


def test_mapped_state_dict_loading():
    lin = st.nn.Linear(3, 2, name="fc")
    ckpt = {"dense.kernel": torch.arange(6, dtype=torch.float32).reshape(2, 3),        # (out, in): needs a transpose
            "dense.bias": torch.ones(1, 4), "junk": torch.zeros(1, 1)}
    key_map = {"dense.kernel": {"target": "fc::weight", "transform": "transpose"},
               "dense.bias": {"target": "fc::bias", "transform": "copy_overlap_zeros"},
               "dense.gone": "fc::nothing"}
    rep = lin.state_dict_compatibility_with_key_map(ckpt, key_map)
    assert rep["matched"] == 2 and rep["missing"] == 0 and rep["extra"] == 2 and rep["compatible"]
    assert {e["status"] for e in rep["entries"]} == {"matched", "unexpected_target"}
    rep2 = lin.load_state_dict_subset_mapped_checked(ckpt, key_map)
    assert rep2["matched_subset_hash"] == rep["matched_subset_hash"]
    w = dict(lin.state_dict())["fc::weight"].torch()
    assert torch.equal(w, ckpt["dense.kernel"].t()) and dict(lin.state_dict())["fc::bias"].torch().tolist() == [[1.0, 1.0]]
    bad = lin.state_dict_compatibility_with_key_map(ckpt, {"dense.kernel": "fc::weight"})
    assert not bad["compatible"] and bad["shape_mismatched"] == 1 and bad["missing"] == 1
    with pytest.raises(ValueError):
        lin.state_dict_compatibility_with_key_map(ckpt, {"dense.kernel": {"target": "fc::weight", "transform": "rot"}})
    seq = st.nn.Sequential()
    seq.eval()
    assert seq.training is False


def test_observers_receipts_and_collector():
    from spiraltorch_b200 import observability as O
    events = []
    a = st.Tensor(2, 3, [1, 2, 3, 4, 5, 6])
    b = st.Tensor(3, 2, [1, 0, 0, 1, 1, 1])
    a.matmul(b)                                   # nobody listens: nothing is built
    built = []
    O.emit_tensor_op_meta("x", lambda: built.append(1) or {})
    assert built == []
    with O.observe(events.append):
        a.matmul(b, backend="cpu")
        a.add(a).row_softmax()
        O.emit_tensor_op_meta("matmul", lambda: {"tile": 128})
    kinds = [e["kind"] for e in events]
    assert kinds == ["execution_receipt", "tensor_op", "tensor_op", "tensor_op", "tensor_op_meta"]
    assert events[1]["op"] == "matmul" and events[1]["output_shape"] == [2, 2] and events[2]["op"] == "add"
    assert events[0]["requested_backend"] == "cpu" and not events[0]["fell_back"] and events[-1]["meta"] == {"tile": 128}
    assert O.last_receipt().workload == {"kind": "dense_matmul", "rows": 2, "inner": 3, "cols": 2}
    a.matmul(b)
    assert len(events) == 5                       # observer removed
    with O.TensorOpStepCollector() as col:
        a.matmul(b)
        a.hadamard(a)
    assert col.stats.ops_total == 2 and col.stats.by_op == {"matmul": 1, "hadamard": 1} and col.stats.backend_cpu == 1
    assert O.resolve_backend("cuda", False, True) == ("cuda", "cpu", "operands are host tensors")
    assert O.resolve_backend(None, True, False) == ("cuda", "cpu", "native library unavailable")
    assert O.resolve_backend("faer", True, True) == ("cpu", "cpu", None)
    with pytest.raises(RuntimeError):
        O.resolve_backend("cuda", False, True, strict=True)
    assert len(O.plan_commitment({"b": 1, "a": 2})) == 64 and O.plan_commitment({"a": 2, "b": 1}) == O.plan_commitment({"b": 1, "a": 2})
    # thread-local observers do not see other threads' ops
    import threading
    seen = []
    O.add_observer(seen.append, thread_local=True)
    t = threading.Thread(target=lambda: a.matmul(b))
    t.start(); t.join()
    O.remove_observer(seen.append)
    assert seen == []


def test_hf_bridge_round_trip_and_lora():
    from spiraltorch_b200 import hf_bridge as HB
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.ReLU(), torch.nn.Linear(4, 3))
    model = st.nn.Sequential()
    model.add(st.nn.Linear(6, 4, name="fc1")); model.add(st.nn.Relu()); model.add(st.nn.Linear(4, 3, name="head"))
    rep = HB.load_torch_module(model, ref, [("0", "fc1"), ("2", "head")])
    assert rep["compatible"] and rep["matched"] == 4
    x = torch.randn(5, 6)
    assert torch.allclose(model.forward(st.Tensor._wrap(x)).torch(), ref(x), atol=1e-5)
    back = HB.export_torch_state(model, [("fc1", "0"), ("head", "2")])
    assert all(torch.equal(back[k], v) for k, v in ref.state_dict().items())
    # GPT-2 Conv1D layout is (in, out): inferred from the shapes
    conv1d_state = {"c_fc.weight": torch.randn(6, 4), "c_fc.bias": torch.randn(4)}
    lin = st.nn.Linear(6, 4, name="fc")
    rules = HB.key_map_for_linears([("c_fc", "fc")], HB._rows(conv1d_state), lin)
    assert rules["c_fc.weight"]["transform"] == "identity"
    assert HB.load_torch_module(lin, conv1d_state, [("c_fc", "fc")])["matched"] == 2
    with pytest.raises(KeyError):
        HB.key_map_for_linears([("c_fc", "nope")], conv1d_state, lin)
    lora = st.nn.LoraLinear(6, 4, 2, alpha=4.0, name="ad")
    delta = torch.randn(6, 2) @ torch.randn(2, 4)
    a, b = HB.lora_from_delta(delta, 2, alpha=4.0)
    HB.attach_lora_factors(lora, a, b, peft_layout=False)
    base = {p.name: p.value for p in lora.parameters()}["ad::weight"]
    assert torch.allclose(HB.merge_lora(lora), base + delta, atol=1e-4)
    HB.attach_lora_factors(lora, a.t().contiguous(), b.t().contiguous())       # PEFT layout: (rank, in) and (out, rank)
    assert torch.allclose(HB.merge_lora(lora), base + delta, atol=1e-4)
    with pytest.raises(ValueError):
        HB.attach_lora_factors(lora, torch.zeros(3, 6), torch.zeros(4, 3))


def test_loader_iteration_object_and_binding_alias():
    import spiraltorch_b200 as st
    samples = [(st.Tensor(1, 1, [float(i)]), st.Tensor(1, 1, [float(2 * i)])) for i in range(5)]
    loader = st.nn.from_samples(samples).loader().batched(2)
    it = iter(loader)
    assert isinstance(it, st.nn.DataLoaderIter) and iter(it) is it and isinstance(loader.iter(), st.nn.DataLoaderIter)
    x, y = next(it)
    assert x.shape() == (2, 1) and y.tolist() == [[0.0], [2.0]]
    assert len(list(it)) == 2 and len(list(loader)) == 3                # a new pass per iter(); the old one is exhausted
    with __import__("pytest").raises(StopIteration):
        next(it)
    assert st.nn.py_is_swap_invariant is st.nn.is_swap_invariant
