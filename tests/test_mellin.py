"""Mellin log-lattice transforms: Gamma-function oracle, plan forms, derivative, stable evaluation, training step."""
import cmath
import math

import pytest
import torch

from spiraltorch_b200 import mellin as M
from scipy.special import gamma, digamma


def exp_grid(n=1200, t0=-14.0, t1=5.0):
    h = (t1 - t0) / (n - 1)
    return M.MellinLogGrid.from_function(t0, h, n, lambda x: torch.exp(-x))


def test_mellin_of_exp_decay_is_gamma():
    g = exp_grid()
    for s in (1.5 + 0j, 2.0 + 1.0j, 1.6 - 2.5j):
        assert abs(g.evaluate(s) - gamma(s)) < 1e-7
        assert abs(g.evaluate_stable(s) - gamma(s)) < 1e-7
    vals = g.evaluate_many([1.5, 2.0 + 1j])
    assert vals.shape == (2,) and abs(complex(vals[1]) - gamma(2 + 1j)) < 1e-7
    # d/ds Gamma(s) = Gamma(s) psi(s)
    v, d = g.evaluate_with_derivative(2.0 + 0j)
    assert abs(d - gamma(2.0) * digamma(2.0)) < 1e-6
    v2, d2 = g.evaluate_with_derivative(2.0 + 0.5j, stable=True)
    fd = (g.evaluate(2.0 + 0.5j + 1e-6) - g.evaluate(2.0 + 0.5j - 1e-6)) / 2e-6
    assert abs(d2 - fd) < 1e-6
    assert M.mellin_transform(lambda x: torch.exp(-x), 3.0, (1e-6, 60.0), 4000) == pytest.approx(2.0, abs=1e-6)
    samples = M.sample_log_uniform_exp_decay(-14.0, 0.02, 1000, rate=2.0)
    assert abs(M.mellin_transform_log_samples(-14.0, 0.02, samples, 2.0) - gamma(2.0) / 4.0) < 1e-6      # rate^-s Gamma(s)


def test_plans_line_mesh_and_magnitudes():
    g = exp_grid(400)
    line = g.evaluate_vertical_line(1.2, [-1.0, 0.0, 1.0])
    assert abs(complex(line[1]) - gamma(1.2)) < 1e-5 and complex(line[0]) == pytest.approx(complex(line[2]).conjugate())
    mesh = g.evaluate_mesh([1.0, 2.0], [0.0, 0.5, 1.0])
    assert mesh.shape == (2, 3) and abs(complex(mesh[1, 0]) - 1.0) < 1e-5
    plan = g.plan_mesh([1.0, 2.0], [0.0, 0.5, 1.0])
    assert plan.shape == (2, 3) and len(plan) == 6
    assert torch.allclose(g.evaluate_plan_magnitude(plan), mesh.abs().reshape(-1))
    assert torch.allclose(g.evaluate_plan_log_magnitude(plan), torch.log1p(mesh.abs().reshape(-1)))
    assert torch.allclose(g.evaluate_plan_log_magnitude(plan, 1e-3), torch.log(mesh.abs().reshape(-1) + 1e-3))
    empty = M.MellinEvalPlan.many(g.log_start, g.log_step, [])
    assert empty.shape == (0, 0) and g.evaluate_plan(empty).numel() == 0
    other = M.MellinEvalPlan.many(g.log_start, g.log_step * 2, [1.0])
    with pytest.raises(M.MellinError) as e:
        g.evaluate_plan(other)
    assert e.value.kind == "lattice_mismatch"


def test_z_transform_matches_horner_and_handles_zero():
    c = [1 + 1j, 2.0, -0.5j, 0.25]
    w = [0.5, 1.0, 1.0, 0.5]
    z = 0.7 - 0.3j
    want = sum(ci * wi * z ** k for k, (ci, wi) in enumerate(zip(c, w)))
    dwant = sum(k * ci * wi * z ** (k - 1) for k, (ci, wi) in enumerate(zip(c, w)) if k)
    v, d = M.weighted_z_transform(c, w, z, derivative=True)
    assert abs(v - want) < 1e-12 and abs(d - dwant) < 1e-12
    v0, d0 = M.weighted_z_transform(c, w, 0.0, derivative=True)
    assert v0 == pytest.approx(0.5 + 0.5j) and d0 == pytest.approx(2.0)
    many = M.weighted_z_transform(c, w, torch.tensor([z, 0.0, 1.0], dtype=torch.complex128))
    assert abs(complex(many[0]) - want) < 1e-12 and abs(complex(many[2]) - sum(ci * wi for ci, wi in zip(c, w))) < 1e-12
    with pytest.raises(M.MellinError):
        M.weighted_z_transform(c, w[:3], z)
    with pytest.raises(M.MellinError):
        M.weighted_z_transform([float("nan")], [1.0], z)


def test_windows_and_weights():
    assert M.trapezoidal_weights(1).tolist() == [1.0] and M.trapezoidal_weights(4).tolist() == [0.5, 1, 1, 0.5]
    hann = M.trapezoidal_weights(5, "hann")
    assert hann[0] == 0 and hann[2] == pytest.approx(1.0) and hann[1] == pytest.approx(0.5)
    kept = M.trapezoidal_weights(9, "blackman", preserve_sum=True)
    assert float(kept.sum()) == pytest.approx(8.0)
    tukey = M.trapezoidal_weights(9, "tukey")
    assert tukey[4] == 1.0 and tukey[0] == pytest.approx(0.0) and 0 < tukey[1] < 1
    with pytest.raises(M.MellinError):
        M.trapezoidal_weights(0)
    with pytest.raises(M.MellinError):
        M.trapezoidal_weights(4, "kaiser")
    p, z = M.mellin_log_lattice_prefactor(-1.0, 0.25, 2 + 1j)
    assert p == pytest.approx(0.25 * cmath.exp(-(2 + 1j))) and z == pytest.approx(cmath.exp(0.25 * (2 + 1j)))
    with pytest.raises(M.MellinError) as e:
        M.mellin_log_lattice_prefactor(0.0, 0.0, 1.0)
    assert e.value.kind == "invalid_log_step"


def test_stable_evaluation_survives_large_powers():
    n = 4000
    g = M.MellinLogGrid(0.0, 0.5, torch.exp(-0.6 * torch.arange(n, dtype=torch.float64)))    # f(x) = x^-1.2 on the lattice
    s = 0.9 + 0j                                                         # z^n = e^{0.45 n} overflows past n ~ 1577 on its own
    with pytest.raises(M.MellinError):
        g.evaluate(s)
    v = g.evaluate_stable(s)
    assert math.isfinite(abs(v))
    want = 0.5 * (sum(math.exp(-0.15 * k) for k in range(n)) - 0.5 - 0.5 * math.exp(-0.15 * (n - 1)))
    assert v.real == pytest.approx(want, rel=1e-9)


def test_hilbert_structure_and_training_step():
    a = M.MellinLogGrid.from_function(-3.0, 0.1, 61, lambda x: torch.exp(-x))
    b = M.MellinLogGrid.from_function(-3.0, 0.1, 61, lambda x: torch.exp(-2 * x) * (1 + 0.5j))
    ip = a.hilbert_inner_product(b)
    assert b.hilbert_inner_product(a) == pytest.approx(ip.conjugate())
    assert a.hilbert_norm() == pytest.approx(math.sqrt(a.hilbert_inner_product(a).real))
    l2 = M.mellin_l2_inner_product(lambda x: torch.exp(-x), lambda x: torch.exp(-2 * x) * (1 + 0.5j), (math.exp(-3.0), math.exp(3.0)), 60)
    assert l2 == pytest.approx(ip, rel=1e-9)
    with pytest.raises(M.MellinError):
        a.hilbert_inner_product(M.MellinLogGrid(-3.0, 0.2, torch.ones(61)))
    # gradient against finite differences, then descent reduces the loss
    plan = a.plan_mesh([0.5, 1.0], [-1.0, 0.0, 1.0])
    loss, grad = a.l2_loss_grad_plan_match_grid(plan, b)
    k, eps = 7, 1e-6
    bumped = M.MellinLogGrid(-3.0, 0.1, a.samples + eps * torch.nn.functional.one_hot(torch.tensor(k), 61))
    fd_re = (bumped.l2_loss_grad_plan_match_grid(plan, b)[0] - loss) / eps
    bumped = M.MellinLogGrid(-3.0, 0.1, a.samples + 1j * eps * torch.nn.functional.one_hot(torch.tensor(k), 61))
    fd_im = (bumped.l2_loss_grad_plan_match_grid(plan, b)[0] - loss) / eps
    assert complex(grad[k]).real == pytest.approx(fd_re, rel=1e-3) and complex(grad[k]).imag == pytest.approx(fd_im, rel=1e-3, abs=1e-9)
    losses = [a.train_step_l2_plan_match_grid(plan, b, 0.02) for _ in range(20)]
    assert losses[-1] < losses[0] * 0.8 and all(b2 <= a2 for a2, b2 in zip(losses, losses[1:]))
    with pytest.raises(M.MellinError):
        a.train_step_l2_plan_match_grid(plan, b, 0.0)
