"""Qubit-lattice model: the tensor expressions against element-by-element restatements of the formulas of
crates/st-logic/src/quantum_reality.rs, and the engine's summaries."""
import math

import pytest
import torch

from spiraltorch_b200 import quantum_reality as Q
from spiraltorch_b200.meta_narrative import ZSpace

PI = math.pi


def _engine():
    lattice = Q.QubitLattice([5.0, 5.2, 4.8], torch.tensor([PI / 4, PI / 3, PI / 6], dtype=torch.float64),
                             torch.tensor([0.0, PI / 8, PI / 7], dtype=torch.float64), torch.tensor([0.0, 0.01, 0.0]), torch.tensor([0.0, 0.02, 0.0]))
    return Q.QuantumRealityEngine(Q.ClusterStructure([2, 1]), lattice, Q.BloomSignature(0.7, 0.05, 1.2), Q.DriftField(0.3, 0.15, torch.ones(3)), 0.2, 0.3)


def _amp(e, n, t):
    return e.bloom.varphi0 ** 4 * math.sin(float(e.lattice.theta(t)[n])) * math.log(1 + n + e.bloom.epsilon_t * t) ** 1.2


def _dphi(e, n, t):
    return 0.3 * math.cos(0.15 * t + float(e.lattice.phi(t)[n])) / math.sin(float(e.lattice.theta(t)[n]))


def test_cluster_structure_and_layout():
    c = Q.ClusterStructure([2, 3, 1])
    assert (c.cluster_count(), c.total_qubits(), c.cluster_bounds(1), c.cluster_bounds(5)) == (3, 6, (2, 5), None)
    assert list(c.cluster_indices(2)) == [5] and c.cluster_of(4) == 1 and c.cluster_of(6) is None
    assert c.labels(7).tolist() == [0, 0, 1, 1, 1, 2, -1]
    lay = Q.TaxicabLayout.from_cluster(c)
    assert lay.coordinate_of(3) == (1, 1) and lay.coordinate_of(9) == (9, 0)
    assert lay.manhattan(6)[0, 4].item() == 3.0
    with pytest.raises(ValueError):
        Q.ClusterStructure([])


def test_state_geometry():
    e, t = _engine(), 0.1
    b = e.lattice.bloch_vectors(t)
    assert torch.allclose(b.norm(dim=-1), torch.ones(3, dtype=torch.float64))
    f = e.lattice.fidelity_matrix(t)
    th, ph = e.lattice.theta(t), e.lattice.phi(t)
    for m in range(3):
        for n in range(3):
            ref = 0.5 * (1 + math.cos(th[m]) * math.cos(th[n]) + math.sin(th[m]) * math.sin(th[n]) * math.cos(ph[m] - ph[n]))
            assert abs(float(f[m, n]) - ref) < 1e-12
    # the velocity is the time derivative of the Bloch vector for linear-in-time angles
    lat = Q.QubitLattice([1.0], lambda t: torch.tensor([0.4 + 0.3 * t], dtype=torch.float64), lambda t: torch.tensor([0.1 - 0.2 * t], dtype=torch.float64), 0.3, -0.2)
    h = 1e-6
    num = (lat.bloch_vectors(0.5 + h) - lat.bloch_vectors(0.5 - h)) / (2 * h)
    assert torch.allclose(lat.bloch_velocities(0.5), num, atol=1e-8)


def test_kernels_match_the_elementwise_formulas():
    e, t = _engine(), 0.1
    amp = e.bloom.amplitude(e.lattice, t)
    assert all(abs(float(amp[n]) - _amp(e, n, t)) < 1e-12 for n in range(3))
    dphi = e.drift.phi_component(e.lattice, t)
    assert all(abs(float(dphi[n]) - _dphi(e, n, t)) < 1e-12 for n in range(3))
    k = Q.interference_kernel(e.lattice, t, e.bloom, e.drift, 0.2, 0.3)
    for m in range(3):
        for n in range(3):
            ref = math.exp(-(_dphi(e, m, t) - _dphi(e, n, t)) ** 2 / (2 * 0.04)) * math.exp(-(_amp(e, m, t) - _amp(e, n, t)) ** 2 / (2 * 0.09)) / (math.sqrt(2 * PI) * 0.3)
            assert abs(float(k[m, n]) - ref) < 1e-12
    lam = e.lambda_(t)
    assert torch.allclose(lam.sum(-1), torch.ones(3, dtype=torch.float64)) and torch.allclose(lam, k / k.sum(-1, keepdim=True))
    aff = Q.spiral_phase_affinity(e.lattice, t, e.bloom)
    assert abs(aff[0, 1] - math.sqrt(abs(_amp(e, 0, t) * _amp(e, 1, t))) * float(e.lattice.fidelity_matrix(t)[0, 1]) * complex(math.cos(-0.02), math.sin(-0.02))) < 1e-12
    w = Q.wavelet_modulation(e.clusters, 0, 0.7, t, e.bloom, e.lattice)
    assert abs(w - (_amp(e, 0, t) + _amp(e, 1, t) * complex(math.cos(-0.7), math.sin(-0.7)))) < 1e-12
    p = Q.collapse_redistribution(lam, [0.2, 0.5, 0.3], 0.4)
    assert torch.allclose(p, 0.6 * torch.tensor([0.2, 0.5, 0.3], dtype=torch.float64) + 0.4 * (lam @ torch.tensor([0.2, 0.5, 0.3], dtype=torch.float64)))
    assert abs(float(p.sum()) - (0.6 + 0.4 * float((lam @ torch.tensor([0.2, 0.5, 0.3], dtype=torch.float64)).sum()))) < 1e-12
    sd = Q.superposed_drift(lam, e.lattice, t, e.drift)
    assert sd.shape == (3, 2) and torch.allclose(sd[:, 1], lam @ dphi) and float(sd[:, 0].abs().max()) == 0.0


def test_collapse_manifold_and_bridge():
    e, t = _engine(), 0.1
    man = e.collapse_manifold(t, 0.05, 0.4)
    assert man.degeneracy.shape == (3,) and man.pressure_map.shape == (3,) and man.cluster_entropies.shape == (2,)
    assert abs(man.average_entropy - float(man.cluster_entropies.mean())) < 1e-12 and bool(torch.isfinite(man.pressure_map).all())
    # a wide tolerance makes every qubit degenerate with the two others
    wide = e.collapse_manifold(t, 10.0, 0.4)
    assert wide.degeneracy.tolist() == [2, 2, 2]
    dl = [math.log1p(abs(_amp(e, n, t) - e.bloom.varphi0 ** 4 * math.cos(float(e.lattice.theta(t)[n])) * math.log(1 + n + 0.05 * t) ** 1.2)) for n in range(3)]
    assert torch.allclose(wide.cluster_entropies, torch.tensor([2 * (dl[0] + dl[1]), 2 * dl[2]], dtype=torch.float64))
    ent = sum(((1 + math.cos(float(e.lattice.theta(t)[n]))) / 2) * dl[n] for n in range(3)) / 3
    assert abs(Q.shadow_entropy(e.lattice, t, e.bloom) - ent) < 1e-12
    bridge = e.connect_zspace_monad(ZSpace([2.0, 1.0, 1.0]), Q.MonadBiome([1.0, 0.0]), t, 0.25)
    p0 = torch.tensor([0.5, 0.25, 0.25], dtype=torch.float64)
    assert torch.allclose(bridge.probability, 0.75 * p0 + 0.25 * (e.lambda_(t) @ p0), atol=1e-12)
    assert abs(bridge.coherence - float(bridge.probability[0])) < 1e-12 and abs(bridge.shadow_entropy - ent) < 1e-12


def test_atlas_and_auto_tune():
    n = 12
    g = torch.Generator().manual_seed(1)
    clusters = Q.ClusterStructure([4, 4, 4])
    omega = torch.tensor([5.0] * 4 + [5.6] * 4 + [6.2] * 4, dtype=torch.float64) + 0.01 * torch.randn(n, generator=g, dtype=torch.float64)
    lattice = Q.QubitLattice(omega, 0.4 + torch.rand(n, generator=g, dtype=torch.float64), torch.rand(n, generator=g, dtype=torch.float64))
    bloom, drift = Q.BloomSignature(0.9, 0.02, 1.0), Q.DriftField(0.1, 0.2)
    layout = Q.TaxicabLayout.from_cluster(clusters)
    atlas = Q.interference_atlas(lattice, 0.3, bloom, drift, layout, 1.5, clusters, Q.NoiseModel(20.0, 0.05, 0.001))
    k = atlas.base.kernel
    assert torch.allclose(k, k.T, atol=1e-12) and float(torch.linalg.eigvalsh(k).min()) > -1e-9
    assert atlas.base.diffusion_coordinates.shape == (n, 3) and atlas.noisy is not None and 0.0 <= atlas.stability <= 1.0
    assert Q.interference_atlas(lattice, 0.3, bloom, drift, layout, 1.5, clusters, Q.NoiseModel()).noisy is None
    eng = Q.QuantumRealityEngine(clusters, lattice, bloom, drift, 0.2, 0.3)
    tuned = eng.tuned_collapse_drive(0.3, layout, [0, 2, 3, 5], [0.1, 1.0], [1.0, 2.0, 4.0])
    assert tuned is not None
    params, lam = tuned
    assert params.k_nn in (2, 3, 5) and params.connectivity >= 1 and 0.0 <= params.objective <= 1.0
    rows = lam.sum(-1)
    assert torch.allclose(rows[rows > 0], torch.ones_like(rows[rows > 0])) and lam.shape == (n, n)
    # graph helpers on a graph with two obvious components
    adj = torch.zeros(5, 5, dtype=torch.float64)
    adj[0, 1] = adj[1, 0] = adj[1, 2] = adj[2, 1] = 1.0
    adj[3, 4] = adj[4, 3] = 2.0
    assert Q.connected_components(adj) == 2 and Q.laplacian_lambda2(adj) == pytest.approx(0.0, abs=1e-9)
    kk = torch.tensor([[0.0, 0.9, 0.1, 0.2], [0.9, 0.0, 0.3, 0.1], [0.1, 0.3, 0.0, 0.8], [0.2, 0.1, 0.8, 0.0]], dtype=torch.float64)
    a1 = Q.knn_adjacency(kk, 1)
    assert a1[0, 1] == 0.9 and a1[2, 3] == 0.8 and a1[0, 2] == 0.0 and torch.equal(a1, a1.T)
