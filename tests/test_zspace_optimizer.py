"""Z-space meta-optimizer: fractional regulariser and its analytic gradient, topos control scales, the Adam transition,
checkpoint / restore rules and the parameter control derived from a report (behaviour of
crates/st-core/src/runtime/zspace_optimizer.rs)."""
import copy
import math

import pytest
import torch

from spiraltorch_b200.runtime import zspace_optimizer as Z


def _energy(z, order):
    n = z.numel()
    bins = n // 2 + 1
    spec = torch.fft.fft(z.to(torch.complex128))[:bins]
    w = (torch.arange(bins, dtype=torch.float64) / (bins - 1)) ** (2 * order)
    return (w * (spec.real ** 2 + spec.imag ** 2)).sum() / bins


def test_fractional_regularizer_energy_and_gradient_match_autograd():
    torch.manual_seed(0)
    for n in (2, 5, 8, 33):
        z = torch.randn(n, dtype=torch.float64, requires_grad=True)
        e = _energy(z, 0.35)
        (g,) = torch.autograd.grad(e, z)
        rep = Z.fractional_regularizer(z.detach().tolist(), 0.35)
        assert rep["energy"] == pytest.approx(float(e.detach()), rel=1e-10)
        assert rep["raw_gradient"] == pytest.approx(g.tolist(), rel=1e-9, abs=1e-12)
        scale = max(1.0, float(g.abs().max()))
        assert rep["gradient_normalization_scale"] == pytest.approx(scale)
        assert rep["normalized_gradient"] == pytest.approx((g / scale).tolist(), rel=1e-9, abs=1e-12)
    one = Z.fractional_regularizer([3.0], 0.5)
    assert one["energy"] == 0.0 and one["normalized_gradient"] == [0.0]
    assert Z.fractional_regularizer([2.0, 2.0, 2.0, 2.0], 0.5)["energy"] == pytest.approx(0.0)        # a constant has only the DC bin
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.fractional_regularizer([], 0.5)
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.fractional_regularizer([1.0, float("nan")], 0.5)


def test_topos_control_is_neutral_without_telemetry_or_gain():
    cfg = Z.Config(topos_control_gain=0.5)
    quiet = Z.resolve_topos_control(cfg, {}, 0.1)
    assert not quiet["present"] and not quiet["active"] and quiet["learning_rate_scale"] == 1.0 and quiet["clip_scale"] == 1.0
    assert quiet["effective_fractional_weight"] == 0.1 and quiet["gradient_bias_scale"] == 0.0 and quiet["pressure"] == 0.0
    tel = {"topos.closure_pressure": 0.8, "topos.learning_rate_scale": 0.5, "topos.clip_scale": 0.5, "topos.regularization_scale": 3.0,
           "topos.gradient_bias_scale": 0.2}
    off = Z.resolve_topos_control(Z.Config(), tel, 0.1)
    assert off["present"] and not off["active"] and off["learning_rate_scale"] == 1.0 and off["pressure"] == pytest.approx(0.8)
    on = Z.resolve_topos_control(cfg, tel, 0.1)
    assert on["active"] and on["learning_rate_scale"] == pytest.approx(0.75) and on["clip_scale"] == pytest.approx(0.75)
    assert on["regularization_scale"] == pytest.approx(2.0) and on["effective_fractional_weight"] == pytest.approx(0.2)
    assert on["gradient_bias_scale"] == pytest.approx(0.1) and on["effective_learning_rate"] == pytest.approx(0.0075)
    assert on["guard_strength"] == 0.8 and on["step_damping"] == pytest.approx(0.64) and on["openness"] == pytest.approx(0.2)
    assert on["gradient_bias_basis"][:3] == pytest.approx([0.3, -0.5, -0.5]) and on["gradient_bias_basis"][6] == pytest.approx(0.5)
    assert Z.gradient_clip_threshold(2.0, 0.75) == pytest.approx(8.0) and Z.gradient_clip_threshold(2.0, 1.0) is None


def test_transition_is_adam_on_the_regularised_projected_gradient():
    cfg = Z.Config(dimension=4, learning_rate=0.1)
    opt = Z.ZSpaceMetaOptimizer(cfg)
    obs = Z.Observation(speed=0.5, memory=-0.2, stability=1.0, gradient=[0.3, -2.0])
    rep = opt.try_step(obs)
    proj = [math.tanh(0.3), math.tanh(-2.0)] * 2
    assert rep["gradient"]["projected_normalized"] == pytest.approx(proj) and rep["gradient"]["applied"] == pytest.approx(proj)   # z = 0: no regulariser pull
    # first Adam step moves every coordinate by lr * sign(g) (bias-corrected m / sqrt(v) = sign)
    assert opt.state.z == pytest.approx([-0.1 * math.copysign(1, g) for g in proj], rel=1e-6)
    assert rep["adam"]["step"] == 1 and rep["adam"]["first_moment_bias_correction"] == pytest.approx(0.1)
    obj = rep["objective"]
    assert obj["observed_resource_penalty"] == pytest.approx(0.5 * math.tanh(0.5) + 0.3 * math.tanh(-0.2) + 0.2 * math.tanh(1.0))
    assert obj["fractional_term"] == 0.0 and rep["state_before"]["step"] == 0 and rep["state_after"]["z"] == opt.state.z
    rep2 = opt.try_step(obs)
    frac = Z.fractional_regularizer(rep["state_after"]["z"], cfg.fractional_order)
    want = [p + 0.1 * g for p, g in zip(proj, frac["normalized_gradient"])]
    assert rep2["gradient"]["before_clip"] == pytest.approx(want) and rep2["objective"]["fractional_term"] == pytest.approx(0.1 * frac["energy"])
    m = [0.9 * 0.1 * p + 0.1 * w for p, w in zip(proj, want)]
    v = [0.999 * 0.001 * p * p + 0.001 * w * w for p, w in zip(proj, want)]
    delta = [-(0.1 * mi / (1 - 0.9 ** 2)) / (math.sqrt(vi / (1 - 0.999 ** 2)) + 1e-8) for mi, vi in zip(m, v)]
    assert rep2["adam"]["parameter_delta"] == pytest.approx(delta, rel=1e-9)
    # clipping: an outlier coordinate is clamped to rms / (1 - clip_scale)
    clip = Z.ZSpaceMetaOptimizer(Z.Config(dimension=4, topos_control_gain=1.0))
    r = clip.try_step(Z.Observation(gradient=[5.0, 0.01, 0.01, 0.01], telemetry={"topos.clip_scale": 0.25, "topos.gradient_bias_scale": 0.0}))
    th = r["topos_control"]["gradient_clip_threshold"]
    assert th == pytest.approx(r["topos_control"]["biased_gradient_rms"] / 0.75) and r["gradient"]["clipped_values"] == 1
    assert r["gradient"]["applied"][0] == pytest.approx(th)
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.ZSpaceMetaOptimizer(Z.Config(dimension=4, gradient_projection="exact")).try_step(Z.Observation(gradient=[1.0]))
    bad = Z.ZSpaceMetaOptimizer(cfg)
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        bad.try_step(Z.Observation(speed=float("inf")))
    assert bad.state.step == 0 and bad.last_report is None                                  # nothing committed


def test_checkpoint_restore_rules():
    opt = Z.ZSpaceMetaOptimizer(Z.Config(dimension=3))
    opt.try_step(Z.Observation(gradient=[1.0, -1.0, 0.5]))
    ck = opt.checkpoint()
    again = Z.ZSpaceMetaOptimizer.from_checkpoint(copy.deepcopy(ck))
    assert again.state == opt.state and again.checkpoint() == ck
    wide = copy.deepcopy(ck)
    wide["config"]["dimension"] = 5
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.ZSpaceMetaOptimizer.from_checkpoint(copy.deepcopy(wide))                          # strict: lengths must match
    relaxed = Z.ZSpaceMetaOptimizer.from_checkpoint(wide, strict=False)
    assert relaxed.state.z[:3] == opt.state.z and relaxed.state.z[3:] == [0.0, 0.0]
    narrow = copy.deepcopy(ck)
    narrow["config"]["dimension"] = 2
    narrow["state"]["z"][2] = float("nan")
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.ZSpaceMetaOptimizer.from_checkpoint(narrow, strict=False)                         # a discarded tail may not hide a NaN
    neg = copy.deepcopy(ck)
    neg["state"]["second_moment"][0] = -1.0
    with pytest.raises(Z.ZSpaceMetaOptimizerError):
        Z.ZSpaceMetaOptimizer.from_checkpoint(neg)
    assert Z.Config.from_dict({"alpha": 0.5, "lr": 0.2, "weights": {"drs": 0.4}}).weights.drift_response == 0.4
    for bad in ({"dimension": 0}, {"dimension": 5000}, {"learning_rate": 0.0}, {"first_moment_decay": 1.0}, {"bogus": 1}):
        with pytest.raises(Z.ZSpaceMetaOptimizerError):
            Z.Config.from_dict(bad).validate()
    assert Z.initialize(Z.Config(dimension=2))["state"]["z"] == [0.0, 0.0]


def test_parameter_control_rederives_the_report():
    opt = Z.ZSpaceMetaOptimizer(Z.Config(dimension=2, learning_rate=0.02, topos_control_gain=0.5))
    assert opt.parameter_control() is None
    rep = opt.try_step(Z.Observation(gradient=[0.1, 0.2], telemetry={"topos.learning_rate_scale": 0.4}))
    ctl = opt.parameter_control()
    assert ctl.absolute_learning_rate_scale == pytest.approx(0.7) and ctl.source_effective_learning_rate == pytest.approx(0.014)
    assert ctl.source_step == 1 and ctl.kind == Z.PARAMETER_CONTROL_KIND
    for path, value, code in ((("topos_control", "learning_rate_scale"), 0.9, "invariant_violation"), (("adam", "effective_learning_rate"), 0.5, "invariant_violation"),
                              (("state_after", "step"), 7, "inconsistent_step"), (("semantic_backend",), "python", "contract_field"),
                              (("transition_validated",), False, "unvalidated_transition")):
        forged = copy.deepcopy(rep)
        node = forged
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(Z.ZSpaceMetaOptimizerError) as e:
            Z.parameter_control_from_report(forged)
        assert e.value.code == code
    del rep["adam"]
    with pytest.raises(Z.ZSpaceMetaOptimizerError) as e:
        Z.parameter_control_from_report(rep)
    assert e.value.code == "malformed_report"
