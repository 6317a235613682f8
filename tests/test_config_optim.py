"""Configuration flags, layered config, tracing, plugin bus and the Amegagrad tapes."""
import json
import math

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200 import config
from spiraltorch_b200.ops import optim as K
from spiraltorch_b200.optim import Amegagrad, AmegaHypergrad, AmegaRealgrad, DesireGradientControl, Topos


def test_determinism_flags(monkeypatch):
    monkeypatch.delenv("SPIRAL_DETERMINISTIC", raising=False)
    assert not config.determinism.config().enabled and config.determinism.config().seed == 42
    monkeypatch.setenv("SPIRAL_DETERMINISTIC", "1")
    monkeypatch.setenv("SPIRAL_DETERMINISTIC_SEED", "7")
    cfg = config.determinism.config()
    assert cfg.enabled and cfg.seed == 7 and cfg.reduction and cfg.scheduler
    a = config.determinism.resolve_seed(None, "rand/2x2")
    assert a == config.determinism.resolve_seed(None, "rand/2x2") != config.determinism.resolve_seed(None, "other")
    assert config.determinism.resolve_seed(5, "x") == 5
    assert st.Tensor.rand(2, 2).tolist() == st.Tensor.rand(2, 2).tolist()     # label-derived seed
    monkeypatch.setenv("SPIRALTORCH_STRICT_GPU", "1")
    assert config.ExecutionConfig.from_env().accelerator_fallback == "forbid"


def test_layered_config_and_atomic_write(tmp_path, monkeypatch):
    (tmp_path / "base.toml").write_text('lr = 0.1\n[trainer]\nepochs = 3\nbackend = "cpu"\n')
    (tmp_path / "site.toml").write_text('[trainer]\nbackend = "cuda"\n')
    (tmp_path / "run.json").write_text(json.dumps({"lr": 0.01, "trainer": {"epochs": 5}}))
    monkeypatch.setenv("SPIRAL_CONFIG_ROOT", str(tmp_path))
    cfg = config.load_layered_config()
    assert cfg.values == {"lr": 0.01, "trainer": {"epochs": 5, "backend": "cuda"}}
    assert {"layer": "run", "key": "lr", "old": 0.1, "new": 0.01} in cfg.events and len(cfg.sources) == 3
    config.atomic_write(tmp_path / "deep" / "x.txt", "hello")
    assert (tmp_path / "deep" / "x.txt").read_text() == "hello"
    tr = config.init_tracing(str(tmp_path / "trace.json"))
    with tr.span("step", phase="fwd"):
        pass
    doc = json.loads(open(tr.flush()).read())
    assert doc["traceEvents"][0]["name"] == "step" and doc["traceEvents"][0]["ph"] == "X"


def test_plugin_bus():
    seen = []
    a = st.plugin.subscribe("Custom", seen.append)
    b = st.plugin.subscribe("*", seen.append)
    assert st.plugin.has_listeners("Custom") and st.plugin.publish("Custom", {"x": 1}) == 2
    assert st.plugin.unsubscribe("Custom", a) and not st.plugin.unsubscribe("Custom", a)
    st.plugin.unsubscribe("*", b)
    assert seen[0]["type"] == "Custom" and seen[0]["x"] == 1
    ops = []
    sid = st.plugin.subscribe("TensorOp", ops.append)
    st.Tensor.randn(2, 3, seed=1).matmul(st.Tensor.randn(3, 2, seed=2))
    st.plugin.unsubscribe("TensorOp", sid)
    assert ops and ops[0]["op"] == "matmul" and ops[0]["output_shape"] == [2, 2]


def test_porous_mix_matches_reference_cases():
    x = torch.tensor([0.5, -2.0, 4.0, float("nan"), float("inf")])
    out = K.porous_mix(x, 1.0, 0.2)
    assert out[0] == 0.5 and out[3] == 0 and out[4] == 0
    bleed = (4.0 - 1.0) / (4.0 + 1.0)
    assert out[2].item() == pytest.approx(1.0 * (1 - 0.05 * bleed))
    assert out[1].item() == pytest.approx(-(1 - 0.05 * (1.0 / 3.0)))
    assert K.porous_mix(x[:3], 1.0, 0.0).tolist() == [0.5, -1.0, 1.0]


def test_hypergrad_and_realgrad_tapes():
    tape = AmegaHypergrad(-1.0, 0.05, 2, 3)
    with pytest.raises(ValueError):
        AmegaHypergrad(0.5, 0.05, 2, 3)
    wave = torch.tensor([[0.5, -1.0, 2.0], [0.0, 0.25, -0.75]])
    tape.accumulate_wave(wave)
    expect = wave / (1 + wave * wave).abs().clamp(min=1e-6)
    assert torch.allclose(tape.gradient, expect, atol=1e-6)
    tape.accumulate_pair(torch.ones(2, 3), torch.zeros(2, 3))
    assert torch.allclose(tape.gradient, expect + 1, atol=1e-6)
    w = torch.tensor([[0.3, -0.2, 0.1], [0.0, 0.0, 0.0]])
    w0, g0 = w.clone(), tape.gradient.clone()
    tape.apply(w)
    stepped = w0 - 0.05 / (1 + w0 * w0) * g0
    norm = stepped.norm(dim=1, keepdim=True)
    assert torch.allclose(w, stepped * torch.tanh(norm) / norm, atol=1e-6)
    assert tape.gradient.abs().max() == 0
    ck = json.loads(json.dumps(tape.checkpoint()))
    assert AmegaHypergrad.from_checkpoint(ck).shape() == (2, 3)
    real = AmegaRealgrad(0.1, 2, 3)
    real.accumulate(torch.ones(2, 3))
    w = torch.zeros(2, 3)
    real.apply(w)
    assert torch.allclose(w, torch.full((2, 3), -0.1)) and real.gradient.abs().max() == 0


def test_amegagrad_combined_step_and_tuning():
    opt = Amegagrad(2, 2, curvature=-1.0, hyper_learning_rate=0.1, real_learning_rate=0.05, gain=1.0)
    assert opt.shape() == (2, 2)
    opt.accumulate_wave(torch.tensor([[0.2, -0.4], [0.1, 0.3]]))
    w = st.Tensor(2, 2, [0.5, -0.5, 0.25, 0.75])
    w0 = w.torch().clone()
    hg, rg = opt.hyper.gradient.clone(), opt.real.gradient.clone()
    opt.desire_control(DesireGradientControl(hyper_rate_scale=0.5, real_rate_scale=2.0))
    opt.step(w)
    assert opt.hyper.learning_rate == pytest.approx(0.05) and opt.real.learning_rate == pytest.approx(0.1)
    stepped = w0 - 0.05 / (1 + w0 * w0) * hg
    n = stepped.norm(dim=1, keepdim=True)
    expect = stepped * torch.tanh(n) / n - 0.1 * rg
    assert torch.allclose(w.torch(), expect, atol=1e-6)
    assert opt.hyper.gradient.abs().max() == 0 and opt.real.gradient.abs().max() == 0
    assert "gradient_norm" in opt.topos_diagnostics()
    assert st.hypergrad(2, 2, curvature=-0.5, learning_rate=0.1).curvature == -0.5
    assert st.realgrad(2, 2, learning_rate=0.2).learning_rate == 0.2
    assert Topos().saturate(torch.tensor([2e6]))[0] < 2e6


def test_selfsup_objectives():
    torch.manual_seed(0)
    base = torch.randn(16, 8)
    res = st.selfsup.info_nce(base + 0.01 * torch.randn(16, 8), base + 0.01 * torch.randn(16, 8), temperature=0.1)
    assert res.top1_accuracy == 1.0 and res.mean_margin > 1.0 and 0 < res.loss < 1.0
    a = torch.nn.functional.normalize(base, dim=-1)
    logits = a @ a.t() / 0.1
    manual = (torch.logsumexp(logits, -1) - logits.diag()).mean()
    assert st.selfsup.info_nce(base, base, 0.1).loss == pytest.approx(manual.item(), rel=1e-5)
    with pytest.raises(ValueError):
        st.selfsup.info_nce(base, base[:4], 0.1)
    p, t = st.Tensor(2, 3, [1, 2, 3, 4, 5, 6]), st.Tensor(2, 3, [1, 0, 3, 4, 5, 0])
    assert st.selfsup.masked_mse(p, t, [[1], [2]]) == pytest.approx((4 + 36) / 2)
    with pytest.raises(IndexError):
        st.selfsup.masked_mse(p, t, [[9], []])


def test_grad_scaler_and_warmup_cosine_schedule():
    import math
    import spiraltorch_b200 as st
    from spiraltorch_b200.nn import amp

    assert not amp.autocast_enabled()
    with amp.AutocastGuard.enable():
        assert amp.autocast_enabled()
        with amp.AutocastGuard.disable():
            assert not amp.autocast_enabled()
        assert amp.autocast_enabled()
    assert not amp.autocast_enabled()

    layer = st.nn.Linear("amp", 2, 2)
    opt = amp.ZSpaceParameterOptimizer(0.05)
    opt.set_mode(amp.OptimizerMode.realgrad(0.05))
    opt.prepare_module(layer)
    scaler = amp.GradScaler(2.0, 2.0, 0.5, 2).with_limits(1.0, 16.0)
    x = st.Tensor(1, 2, [0.3, -0.7])
    before = layer.weight.value.clone()
    loss_grad = layer.forward(x)
    layer.backward(x, scaler.scale_tensor(loss_grad))
    assert scaler.step(opt, layer) is True and not torch.equal(layer.weight.value, before)
    # the unscaled step equals a step taken without a scaler
    ref = st.nn.Linear("amp", 2, 2)
    ref.attach_realgrad(0.05)
    ref.backward(x, ref.forward(x))
    ref.apply_step(0.05)
    assert torch.allclose(ref.weight.value, layer.weight.value, atol=1e-6)
    layer.zero_accumulators()
    layer.backward(x, scaler.scale_tensor(layer.forward(x)))
    assert scaler.step(opt, layer) and scaler.scale() == 4.0          # grown after 2 clean steps
    # overflow: step skipped, scale backed off, accumulators cleared
    held = layer.weight.value.clone()
    layer.zero_accumulators()
    layer.backward(x, st.Tensor(1, 2, [3e38, 3e38]).scale(1.0))
    for p in layer.parameters():
        for a in p.accumulators():
            a.mul_(1e30)
    assert scaler.step(opt, layer) is False and scaler.scale() == 2.0 and torch.equal(layer.weight.value, held)
    with pytest.raises(st.TensorError):
        amp.GradScaler(1.0, 1.0, 0.5, 2)
    with pytest.raises(st.TensorError):
        scaler.try_scale_loss(float("inf"))

    sch = amp.WarmupCosineScheduler(1e-2, 1e-4, 4, 12)
    lrs = [sch.step() for _ in range(14)]
    assert abs(lrs[0] - (1e-4 + (1e-2 - 1e-4) / 4)) < 1e-9 and abs(lrs[3] - 1e-2) < 1e-9
    assert abs(lrs[7] - (1e-4 + (1e-2 - 1e-4) * 0.5 * (1 + math.cos(math.pi * 0.5)))) < 1e-9
    assert abs(lrs[11] - 1e-4) < 1e-9 and lrs[13] == lrs[11] and all(a >= b for a, b in zip(lrs[3:], lrs[4:]))
    opt2 = amp.ZSpaceParameterOptimizer(1e-2)
    sch2 = amp.WarmupCosineScheduler(1e-2, 0.0, 0, 10)
    lr = sch2.step_optimizer(opt2, layer)
    assert abs(opt2.fallback_learning_rate() - lr) < 1e-9
    with pytest.raises(st.TensorError):
        amp.WarmupCosineScheduler(1e-2, 0.0, 5, 4)
    ad = amp.SpectralLrAdapter()
    opt2.set_adapter(ad)
    layer.zero_accumulators()
    layer.backward(x, layer.forward(x))
    opt2.step(layer)
    assert ad.min_scale <= ad.scale_for("w", torch.randn(4, 4)) <= ad.max_scale
    assert amp.SpectralLrAdapter.from_state(ad.state()).avg_energy == ad.avg_energy


def test_native_pointer_guard_refuses_host_tensors():
    import torch
    from spiraltorch_b200.ops import native
    assert native.ptr(None).value in (None, 0)
    with pytest.raises(ValueError):
        native.ptr(torch.zeros(4))
    with pytest.raises(ValueError):
        native.same_device("op", torch.zeros(1), torch.zeros(1, device="meta"))
