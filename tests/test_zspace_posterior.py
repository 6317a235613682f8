"""Latent Z-space posterior against the values of crates/st-core/src/inference/zspace_posterior.rs's unit tests."""
import math

import pytest
import torch

from spiraltorch_b200 import zspace_posterior as ZP

STATE = [0.12, -0.03, 0.48, -0.2]


def test_decode_is_parseval_normalised_and_matches_the_reference_values():
    d = ZP.decode_zspace_posterior(STATE, 0.35)
    assert d.spectral_bins == 3 and float(d.energy) == pytest.approx(0.2857, abs=1e-14)
    assert float(d.spectral_energy) == pytest.approx(float(d.energy), abs=1e-14) and float(d.parseval_relative_error) <= 1e-14
    assert float(d.frac_energy) == pytest.approx(0.2210090973787923, abs=1e-12)
    assert float(d.fractional_energy_ratio) == pytest.approx(0.7735705193517406, abs=1e-12)
    assert float(d.spectral_centroid) == pytest.approx(0.7415120756037802, abs=1e-12)
    m = d.metric_floats()
    assert m["speed"] == pytest.approx(0.4463024613684294, abs=1e-12) and m["memory"] == pytest.approx(0.10991043037290935, abs=1e-12)
    assert m["stability"] == pytest.approx(0.672934550609384, abs=1e-12) and m["drs"] == pytest.approx(0.6413201743341207, abs=1e-12)
    assert m["frac"] == pytest.approx(0.6490008507207798, abs=1e-12)
    assert float(d.barycentric.sum()) == pytest.approx(1.0, abs=1e-14) and d.gradient.shape == (4,)
    assert torch.allclose(d.gradient, torch.tensor([0.5 * (0.12 + (-0.15)), 0.5 * (-0.15 + 0.51), 0.5 * (0.51 - 0.68), 0.5 * (-0.68 + 0.2)], dtype=torch.float64))


def test_batched_decode_matches_single_states_and_edge_cases():
    torch.manual_seed(0)
    batch = torch.randn(6, 9, dtype=torch.float64)
    all_ = ZP.decode_zspace_posterior(batch, 0.5)
    for i in range(6):
        one = ZP.decode_zspace_posterior(batch[i], 0.5)
        for k in ZP.BASE_METRICS:
            assert float(all_.metrics[k][i]) == pytest.approx(float(one.metrics[k]), abs=1e-12)
        assert torch.allclose(all_.barycentric[i], one.barycentric) and torch.allclose(all_.gradient[i], one.gradient)
    zero = ZP.decode_zspace_posterior([0.0, 0.0, 0.0])
    assert zero.metric_floats()["frac"] == 0.0 and zero.metric_floats()["drs"] == 0.0 and float(zero.spectral_centroid) == 0.0
    single = ZP.decode_zspace_posterior([0.7])
    assert single.spectral_bins == 1 and float(single.frac_energy) == 0.0 and single.metric_floats()["speed"] == pytest.approx(math.tanh(0.25 * 0.7))
    big = ZP.decode_zspace_posterior([0.0, 5.0, -5.0])
    assert float(big.gradient.abs().max()) == pytest.approx(1.0)                     # scaled to unit sup norm
    for bad in ([], [float("nan")], torch.zeros(5000)):
        with pytest.raises(ZP.ZSpacePosteriorError):
            ZP.decode_zspace_posterior(bad)


def test_projection_blends_barycentres_and_scales_confidence_by_telemetry():
    prior = ZP.decode_zspace_posterior(STATE, 0.35)
    proj = ZP.project_zspace_posterior(STATE, {"speed": 0.3, "mem": -0.2, "gradient": [2.0, -1.0]}, 0.35, 0.35,
                                       gradient_basis="test.posterior.control.v1", telemetry=[{"psi": {"energy": 2.0, "focus": 0.4}}])
    pm = prior.metric_floats()
    assert proj.metrics["speed"] == 0.3 and proj.metrics["memory"] == -0.2 and proj.metrics["stability"] == pm["stability"]
    assert proj.applied == {"memory": -0.2, "speed": 0.3} and proj.residual_metric_count == 2
    assert proj.residual == pytest.approx(math.sqrt(((0.3 - pm["speed"]) ** 2 + (-0.2 - pm["memory"]) ** 2) / 2))
    assert torch.equal(proj.gradient, prior.gradient) and proj.gradient_source == "latent_state"
    cg = proj.control_gradient
    assert cg.basis == "test.posterior.control.v1" and cg.dimension == 2 and cg.l2 == pytest.approx(math.sqrt(5.0)) and cg.linf == 2.0
    sp = lambda x: math.log1p(math.exp(x))                                            # noqa: E731
    ov = [sp(0.3), sp(-0.2), sp(pm["stability"])]
    ov = [v / sum(ov) for v in ov]
    expect = [0.35 * float(prior.barycentric[i]) + 0.65 * ov[i] for i in range(3)]
    assert proj.barycentric == pytest.approx([v / sum(expect) for v in expect], abs=1e-12) and sum(proj.barycentric) == pytest.approx(1.0)
    adj = proj.telemetry_adjustment                                                  # leaves (2.0, 0.4): variance 0.64, all positive
    assert adj.variance_reliability == pytest.approx(1.0 / 1.64) and adj.focus_reliability == 1.0
    assert proj.confidence == pytest.approx(math.exp(-proj.residual) / 1.64) and proj.telemetry_reliability == pytest.approx(1.0 / 1.64)
    plain = ZP.project_zspace_posterior(STATE)
    assert plain.residual == 0.0 and plain.confidence == 1.0 and plain.telemetry is None and plain.metrics == pm
    for kwargs in ({"smoothing": 1.5}, {"partial": {"nonsense": 1.0}}, {"partial": {"gradient": [1.0]}}, {"gradient_basis": "b"},
                   {"partial": {"speed": float("inf")}}):
        with pytest.raises(ZP.ZSpacePosteriorError):
            ZP.project_zspace_posterior(STATE, **kwargs)
