"""Psi synchronisation: circle-map identification, rotation numbers, Arnold-tongue scan."""
import math

import pytest
import torch

from spiraltorch_b200 import psi_sync as ps


def scalar_rotation(omega, kappa, burn, sample):
    phi, scale = 0.0, kappa / (2 * math.pi)
    for _ in range(burn):
        phi = (phi + omega - scale * math.sin(2 * math.pi * phi)) % 1.0
    total = 0.0
    for _ in range(sample):
        prev = phi
        phi = (phi + omega - scale * math.sin(2 * math.pi * phi)) % 1.0
        total += (phi - prev) % 1.0
    return total / sample


def test_rotation_number_grid_matches_scalar_loop_and_locks():
    om = torch.tensor([[0.21, 0.5], [0.33, -0.3]], dtype=torch.float64)
    ka = torch.tensor([[0.0, 0.9], [0.5, 0.2]], dtype=torch.float64)
    got = ps.rotation_number(om, ka, 50, 80)
    for i in range(2):
        for j in range(2):
            assert float(got[i, j]) == pytest.approx(scalar_rotation(float(om[i, j]), float(ka[i, j]), 50, 80), abs=1e-12)
    assert float(ps.rotation_number(0.21, 0.0, 10, 100)) == pytest.approx(0.21)          # no coupling: the bare frequency
    assert float(ps.rotation_number(0.49, 0.9, 300, 400)) == pytest.approx(0.5, abs=1e-9)  # inside the 1/2 tongue


def test_nearest_rational_and_wrap():
    p, q, e = ps.nearest_rational(torch.tensor([0.3334, 0.5, 0.71, 0.0]), 8)
    assert (p.tolist(), q.tolist()) == ([1, 1, 5, 0], [3, 2, 7, 1]) and float(e[0]) == pytest.approx(0.3334 - 1 / 3, abs=1e-7)
    assert ps.wrap_unit(torch.tensor([0.7, -0.7, 0.2])).tolist() == pytest.approx([-0.3, 0.3, 0.2])
    assert ps.linspace(0.0, 1.0, 1) == [0.0] and ps.linspace(0.0, 1.0, 3) == [0.0, 0.5, 1.0]
    assert ps.gradient_color(0.0) == (0, 0, 255) and ps.gradient_color(1.0) == (255, 0, 0) and ps.gradient_color(0.5) == (127, 255, 127)


def test_identify_kappa_recovers_a_circle_map():
    omega, k = 0.13, 0.8
    phi = [0.2]
    for _ in range(400):
        phi.append((phi[-1] + omega - k / (2 * math.pi) * math.sin(2 * math.pi * phi[-1])) % 1.0)
    o, kap, rmse = ps.identify_kappa(phi, lam=2.0)
    assert o == pytest.approx(omega, abs=1e-9) and kap == pytest.approx(k / 2.0, abs=1e-8) and rmse < 1e-9
    assert ps.identify_kappa([0.1], 1.0) == (0.0, 0.0, 0.0)


def test_branch_run_and_heatmap(tmp_path):
    state = ps.SyncState()
    cfg = ps.PsiSynchroConfig(lam_range=(0.0, 2.0, 6), wd_range=(0.3, 1.2, 9), burn=40, sample=60, qmax=6, out_dir=str(tmp_path))
    mono = ps.PsiSynchroMonolith(state, cfg)
    branch = ps.PsiBranchConfig.with_state("main:alpha", state, 48)
    (rep,) = mono.synchronise_branches([branch])
    assert len(rep.phi_samples) == 48 and all(0.0 <= v < 1.0 for v in rep.phi_samples)
    # stroboscopic sampling: the k-th sample sits at the first step at or after k drive periods
    td = 2 * math.pi / branch.wd
    t3 = math.ceil((3 * td - 1e-12) / branch.step) * branch.step
    assert rep.phi_samples[3] == pytest.approx(mono.model.phi_sample(t3, branch))
    assert rep.heatmap.shape == (6, 9) and len(rep.lam_grid) == 6 and len(rep.wd_grid) == 9
    # every cell agrees with the scalar loop
    i, j = 4, 2
    rho = scalar_rotation(branch.omega0 / rep.wd_grid[j] - 1.0, rep.kappa_hat * rep.lam_grid[i], 40, 60)
    _, _, err = ps.nearest_rational(torch.tensor(rho), 6)
    assert float(rep.heatmap[i, j]) == pytest.approx(1.0 / (float(err) + 1e-6), rel=1e-6)
    assert rep.best_lock.error == pytest.approx(1.0 / float(rep.heatmap.max()) - 1e-6, abs=1e-9) and rep.best_lock.q <= 6
    assert "@ λ=" in str(rep.best_lock)
    assert rep.heatmap_path.name == "heatmap_main-alpha_gamma_1.30.png" and rep.heatmap_path.read_bytes()[:8] == b"\x89PNG\r\n\x1a\n"
    with pytest.raises(ps.PsiSyncError) as e:
        mono.run_branch(ps.PsiBranchConfig.with_state("tiny", state, 1))
    assert e.value.kind == "insufficient_samples"
