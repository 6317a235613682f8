"""Stochastic and imaginary-time Schrödinger evolutions (crates/st-core/src/dynamics/stochastic_schrodinger.rs,
crates/st-core/src/inference/imaginary_time_schrodinger.rs)."""
import math

import pytest
import torch

from spiraltorch_b200 import schrodinger as S


def test_stochastic_step_is_a_damped_unitary_and_matches_the_pair_formula():
    torch.manual_seed(0)
    cfg = S.StochasticSchrodingerConfig(loss_rate=0.3, noise_scale=0.2).with_time_step(0.05).with_hopping_rate(1.7)
    x, pot, xi = torch.randn(6, 5, dtype=torch.float64), torch.randn(5, dtype=torch.float64), torch.randn(6, 5, dtype=torch.float64)
    st = S.apply_stochastic_schrodinger_step(x, pot, xi, cfg)
    assert torch.allclose(st.phase, pot * 0.05 + xi * 0.2 * math.sqrt(0.05))
    c, s, d = math.cos(1.7 * 0.05), math.sin(1.7 * 0.05), math.exp(-0.5 * 0.3 * 0.05)
    r, col, partner = 2, 2, 3
    mean = 0.5 * st.phase[r, col] + 0.5 * st.phase[r, partner]
    assert float(st.output_real[r, col]) == pytest.approx(d * (c * x[r, col] * math.cos(st.phase[r, col]) - s * x[r, partner] * math.sin(mean)))
    assert float(st.output_imaginary[r, 4]) == pytest.approx(-d * x[r, 4] * math.sin(st.phase[r, 4]))           # the unpaired last feature
    # with a common phase inside each pair the split is exactly unitary up to the attenuation
    st0 = S.apply_stochastic_schrodinger_step(x, torch.zeros(5, dtype=torch.float64), torch.zeros_like(x), cfg)
    assert torch.allclose(st0.norm_ratio(x), torch.full((6,), math.exp(-0.3 * 0.05), dtype=torch.float64))
    assert cfg.ensemble_dephasing_rate == pytest.approx(0.04) and cfg.decoherence_rate == 0.3
    with pytest.raises(S.SchrodingerError):
        S.StochasticSchrodingerConfig(loss_rate=-1.0)
    with pytest.raises(S.SchrodingerError):
        S.apply_stochastic_schrodinger_step(x, pot[:3], xi, cfg)


def test_stochastic_backward_matches_autograd():
    torch.manual_seed(1)
    cfg = S.StochasticSchrodingerConfig(loss_rate=0.1, noise_scale=0.3)
    x = torch.randn(4, 7, dtype=torch.float64, requires_grad=True)
    pot = torch.randn(7, dtype=torch.float64, requires_grad=True)
    xi, g = torch.randn(4, 7, dtype=torch.float64), torch.randn(4, 7, dtype=torch.float64)
    S.apply_stochastic_schrodinger_step(x, pot, xi, cfg).output_real.backward(g)            # plain autograd through the tensor program
    ref_x, ref_p = x.grad.clone(), pot.grad.clone()
    x.grad = pot.grad = None
    S.StochasticSchrodingerFunction.apply(x, pot, xi, cfg).backward(g)                        # the analytic backward
    assert torch.allclose(x.grad, ref_x, atol=1e-12) and torch.allclose(pot.grad, ref_p, atol=1e-12)
    assert torch.autograd.gradcheck(lambda a, b: S.StochasticSchrodingerFunction.apply(a, b, xi, cfg), (x, pot), atol=1e-6)


def test_imaginary_time_prefers_the_lower_potential():
    out = S.apply_imaginary_time_schrodinger([0.0, 2.0], [(0, 1, 1.0)], S.ImaginaryTimeSchrodingerConfig(1.0), tags=["left", "right"])
    assert out.probability[0] > out.probability[1] and float(out.log_amplitude_boost[0]) == 0.0 and float(out.log_amplitude_boost[1]) < 0.0
    eff = out.effects
    assert eff.final_rayleigh_energy < eff.initial_rayleigh_energy and eff.rayleigh_energy_drop > 0.0 and abs(out.probability_sum - 1.0) < 1e-12
    assert eff.substeps == math.ceil(1.0 * 4.0 / 0.9) and eff.spectral_upper_bound == 4.0 and eff.edge_count == 1
    assert abs(eff.initial_l2_norm - 1.0) < 1e-12 and abs(eff.final_l2_norm - 1.0) < 1e-12 and eff.final_residual_l2 < eff.initial_residual_l2
    # long evolution converges to the ground state of [[1, -1], [-1, 3]]
    long = S.apply_imaginary_time_schrodinger([0.0, 2.0], [(0, 1, 1.0)], S.ImaginaryTimeSchrodingerConfig(40.0))
    vals, vecs = torch.linalg.eigh(torch.tensor([[1.0, -1.0], [-1.0, 3.0]], dtype=torch.float64))
    assert torch.allclose(long.final_amplitude, vecs[:, 0].abs(), atol=1e-8) and long.effects.final_rayleigh_energy == pytest.approx(float(vals[0]), abs=1e-8)


def test_imaginary_time_on_a_larger_graph_matches_the_dense_euler_iteration():
    torch.manual_seed(2)
    n = 9
    edges = [(i, j, float(torch.rand(()) + 0.1)) for i in range(n) for j in range(i + 1, n) if (i + 2 * j) % 3 == 0]
    pot = torch.rand(n, dtype=torch.float64) * 3.0
    cfg = S.ImaginaryTimeSchrodingerConfig(0.7, cfl_limit=0.5)
    out = S.apply_imaginary_time_schrodinger(pot, edges, cfg, initial_amplitude=torch.rand(n, dtype=torch.float64) + 0.2)
    lap = torch.zeros(n, n, dtype=torch.float64)
    for a, b, w in edges:
        lap[a, a] += w; lap[b, b] += w; lap[a, b] -= w; lap[b, a] -= w
    h = lap + torch.diag(pot - pot.min())
    a = out.initial_amplitude.clone()
    for _ in range(out.effects.substeps):
        a = a - out.effects.substep_imaginary_time * (h @ a)
        a = a / a.norm()
    assert torch.allclose(out.final_amplitude, a, atol=1e-10) and bool((out.final_amplitude > 0).all())
    assert out.effects.probability_entropy == pytest.approx(float(-(out.probability * out.probability.log()).sum()))
    nothing = S.apply_imaginary_time_schrodinger(pot, edges, S.ImaginaryTimeSchrodingerConfig(0.0))
    assert not nothing.effects.evolution_applied and nothing.effects.substeps == 0


def test_imaginary_time_validation():
    for bad in ([(1, 0, 1.0)], [(0, 0, 1.0)], [(0, 5, 1.0)], [(0, 1, -1.0)], [(0, 1, 1.0), (0, 1, 2.0)]):
        with pytest.raises(S.SchrodingerError):
            S.apply_imaginary_time_schrodinger([0.0, 1.0], bad)
    with pytest.raises(S.SchrodingerError):
        S.apply_imaginary_time_schrodinger([0.0, 1.0], [(0, 1, 1.0)], S.ImaginaryTimeSchrodingerConfig(100.0, max_substeps=3))
    with pytest.raises(S.SchrodingerError):
        S.apply_imaginary_time_schrodinger([0.0, 1.0], [], initial_amplitude=[1.0, -1.0])
    with pytest.raises(S.SchrodingerError):
        S.ImaginaryTimeSchrodingerConfig(1.0, cfl_limit=1.0)
