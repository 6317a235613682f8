"""Closed forms of the psi-spiral stability helpers."""
import math

import pytest

import spiraltorch_b200 as st
from spiraltorch_b200 import spiral_dynamics as sd


def test_barriers_and_force():
    assert sd.hard_barrier_max_c(-0.2, 0.5) == pytest.approx(0.4)
    assert sd.hard_barrier_satisfied(-0.2, 0.5, 0.3) and not sd.hard_barrier_satisfied(-0.2, 0.5, 0.5)
    assert sd.hard_barrier_max_c(-0.1, 0.0) == math.inf and sd.hard_barrier_max_c(0.1, 0.0) is None and sd.hard_barrier_max_c(0.2, 0.5) is None
    f = sd.LogisticForce.evaluate(0.4, 0.3, 0.3, 0.7)
    sig = 1 / (1 + math.exp(-(0.4 - 0.21)))
    assert f.value == pytest.approx(0.3 * sig) and f.du == pytest.approx(0.3 * sig * (1 - sig)) and f.ds == pytest.approx(-0.7 * f.du)
    assert sd.LogisticForce.evaluate(0.4, 0.3, 0.0, 0.7) == sd.LogisticForce()
    assert sd.soft_barrier_ceiling(0.6, 0.5, 2.0) == pytest.approx(0.3) and sd.soft_barrier_ceiling(-1, 0.5, 2.0) == 0.0
    assert sd.soft_barrier_force(0.4, 2.0, 0.6, 0.5, 0.1) == pytest.approx(0.3 / (1 + math.exp(-0.2)))
    assert sd.soft_barrier_mu_eff(-0.2, 0.5, 0.6, 0.5, 2.0) == pytest.approx(-0.05)
    assert sd.soft_barrier_margin_satisfied(-0.5, 0.5, 0.6, 0.5, 0.1) and not sd.soft_barrier_margin_satisfied(-0.5, 0.5, 0.6, 0.5, 0.3)
    assert sd.cbf_dot_h(0.5, f, 2.0) == pytest.approx(-0.5 * f.du * 2.0)
    assert sd.cbf_boundary_projection(1, 2, 3, 0.5, 0.1, 0.2, 0.7, 0.3, 0.4, 0.9, 0.6, 0.8) == pytest.approx(
        (0.2 - 0.6 - 0.5) - 0.21 + 0.4 * 0.9 * 0.6 - 0.4 * 0.8 * 0.2)


def test_steady_radius_solves_its_equation():
    args = dict(mu0=0.3, eta=0.05, gamma=-0.4, c1=0.5, q=2.0, nu=0.8, sigma_s=0.3, s=0.2)
    y = sd.steady_radius_squared(**args)
    # the stationarity condition: mu0 - eta + gamma (c1 / (1 + q y) - sigma_s s) - nu y = 0
    assert args["mu0"] - args["eta"] + args["gamma"] * (args["c1"] / (1 + args["q"] * y) - args["sigma_s"] * args["s"]) - args["nu"] * y == pytest.approx(0.0, abs=1e-12)
    assert sd.steady_radius(**args) == pytest.approx(math.sqrt(y))
    eps = 1e-6
    fd = (sd.steady_radius_squared(**{**args, "s": args["s"] + eps}) - sd.steady_radius_squared(**{**args, "s": args["s"] - eps})) / (2 * eps)
    assert sd.steady_radius_sensitivity(**args) == pytest.approx(fd, rel=1e-6)
    assert sd.steady_radius_squared(**{**args, "q": 0.0}) is None and sd.steady_radius_squared(**{**args, "mu0": -5.0}) is None


def test_hopf_metrics_and_bounds():
    bal = sd.audit_container_balance(0.8, 0.5, 2.0, 0.4, 0.3, 1.5)
    assert bal.audit_gain == pytest.approx(0.2) and bal.container_gain == pytest.approx(0.08) and bal.difference == pytest.approx(0.12)
    assert sd.audit_container_balance(0.8, 0.5, 0.0, 0.4, 0.3, 1.5) is None
    events = []
    with st.observability.observe(events.append):
        m = sd.psi_spiral_metrics(-0.1, 0.5, 1.2, 0.7, 0.8, 0.5, 2.0, 0.1, 0.4, 0.3, 1.5, 0.3)
    sig = 1 / (1 + math.exp(0.8 * 0.1 / 2.0))
    assert m.hopf.forcing.value == pytest.approx(0.3 * sig) and m.hopf.mu_eff0 == pytest.approx(-0.1 + 0.5 * 0.3 * sig)
    ratio = 1 - sig
    assert m.hopf.center_manifold_c == pytest.approx(ratio * (1 - ratio) * 0.12) and m.hopf.alpha3 == pytest.approx(0.7 - 0.5 * m.hopf.center_manifold_c)
    assert m.hopf.regime == "supercritical" and m.dimensionless.omega_bar == pytest.approx(1.2 / 0.7) and m.balance == bal
    meta = [e["meta"] for e in events if e["kind"] == "tensor_op_meta"][0]
    assert meta["hopf_regime"] == "supercritical" and meta["hard_barrier_max_c"] == pytest.approx(0.2) and meta["hard_barrier_satisfied"] is False
    assert sd.hopf_normal_form(-0.1, 50.0, 0.7, 1.2, 8.0, 5.0, 2.0, 0.1, 0.4, 0.3, 1.5, 0.3).regime == "subcritical"
    assert sd.psi_spiral_metrics(-0.1, 0.5, 1.2, 0.0, 0.8, 0.5, 2.0, 0.1, 0.4, 0.3, 1.5, 0.3) is None
    y = sd.ito_mean_square_bound(0.2, 0.5, 0.3)
    assert 0.5 * y * y - 0.2 * y - 0.15 == pytest.approx(0.0, abs=1e-12) and sd.ito_mean_square_bound(-0.2, 0.5, 0.0) == 0.0
    assert sd.ito_mean_square_bound(0.2, 0.0, 0.3) is None
    assert sd.gershgorin_contraction_bound(1.0, 0.5, 0.8, 0.5, 0.2, 0.4, 0.3, 2.0, 1.5) == pytest.approx(min(1 - 0.05, 1 - 0.5 * (0.16 + 0.1), 2 - 0.5 * (0.1 + 0.16 + 0.4), 1.5 - 0.25))
    assert sd.contraction_with_cubic(-0.1, 0.5, 2.0) == pytest.approx(1.9)
