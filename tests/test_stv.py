"""Spino-tensor-vector kernels against the values of crates/st-core/src/theory/stv.rs's unit tests, and batched
evaluation against the one-at-a-time results."""
import math

import pytest
import torch

from spiraltorch_b200 import observability as obs
from spiraltorch_b200 import stv as S

DIAG = torch.diag(torch.tensor([2.0, 1.0, 3.0], dtype=torch.float64))


def _mink(v):
    return float(v[0] ** 2 - (v[1:] ** 2).sum())


def test_determinants_and_invariants():
    k = S.SpinoTensorKernel(1.5, DIAG, [0.0, 1.5, 0.0], [0.0, 0.0, 1.0])
    assert abs(float(k.det_d()) - 9.0) < 1e-9 and abs(float(k.det_t())) < 1e-9
    assert abs(float(k.alpha()) - 1.5) < 1e-9 and abs(float(k.beta()) - 1.25) < 1e-9
    assert abs(float(torch.linalg.det(k.block_tensor())) - float(k.det_t())) < 1e-9
    v = torch.tensor([0.3, -1.0, 2.0, 0.5], dtype=torch.float64)
    assert torch.allclose(k.apply_tensor(v), k.block_tensor() @ v, atol=1e-12)
    assert k.z_scale_hint().physical_radius == pytest.approx(math.sqrt(2.25))
    with pytest.raises(S.NonSymmetric):
        S.SpinoTensorKernel(1.0, [[1.0, 0.2, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]], [0.0] * 3, [0.0] * 3)
    with pytest.raises(S.SingularD):
        S.SpinoTensorKernel(1.0, torch.zeros(3, 3), [1.0, 0.0, 0.0], [0.0] * 3).alpha()


def test_spinor_bloch_round_trip():
    theta, phi = 1.1, -0.7
    sp = S.PauliSpinor.from_bloch_angles(theta, phi)
    j = sp.bloch_current()
    expect = [1.0, math.sin(theta) * math.cos(phi), math.sin(theta) * math.sin(phi), math.cos(theta)]
    assert torch.allclose(j, torch.tensor(expect, dtype=torch.float64), atol=1e-9)
    th2, ph2 = sp.bloch_angles()
    assert abs(float(th2) - theta) < 1e-9 and abs(float(ph2) - phi) < 1e-9
    again = S.PauliSpinor.from_bloch_vector(sp.bloch_vector() * 3.0)
    assert torch.allclose(again.bloch_current(), j, atol=1e-9)
    assert torch.allclose(sp.phase_shift(0.9).bloch_current(), j, atol=1e-12)            # a global phase is invisible
    with pytest.raises(S.InvalidBlochVector):
        S.PauliSpinor.from_bloch_vector([0.0, 0.0, 0.0])
    with pytest.raises(S.ZeroSpinor):
        S.PauliSpinor([0.0, 0.0])
    batch = S.PauliSpinor.from_bloch_angles(torch.tensor([0.0, math.pi / 2, math.pi], dtype=torch.float64), torch.zeros(3))
    assert torch.allclose(batch.bloch_vector()[:, 2], torch.tensor([1.0, 0.0, -1.0], dtype=torch.float64), atol=1e-12)


def test_causal_classes_and_normalisation():
    k = S.SpinoTensorKernel(2.0 / 3.0, DIAG, [0.0, 1.0, 0.0], [0.0, 0.0, 1.0])
    assert k.classify(1e-9) == "timelike"
    cls, vec, beta = k.normalise_kernel(1e-9)
    assert cls == "timelike" and abs(float(beta) - 5.0 / 9.0) < 1e-9 and abs(_mink(vec) - 1.0) < 1e-9
    # beta = 1 exactly when |D^-1 E| = 1: scale E of the kernel above by 1 / sqrt(beta)
    kl = S.SpinoTensorKernel(1.0, DIAG, [0.0, 1.0 / math.sqrt(5.0 / 9.0), 0.0], [0.0, 0.0, 1.0])
    assert kl.classify(1e-8) == "lightlike" and abs(float(kl.beta()) - 1.0) < 1e-8
    ks = S.SpinoTensorKernel(1.0, DIAG, [0.0, 3.0, 0.0], [0.0, 0.0, 1.0])
    assert ks.classify() == "spacelike"
    # the kernel vector is annihilated by the spatial rows of T, and by T itself when det T = 0
    k0 = S.SpinoTensorKernel(1.5, DIAG, [0.0, 1.5, 0.0], [0.0, 0.0, 1.0])
    assert torch.allclose(k0.apply_tensor(k0.kernel_direction()), torch.zeros(4, dtype=torch.float64), atol=1e-9)


def test_intersection_curve_lies_on_both_surfaces():
    k = S.SpinoTensorKernel(2.1, DIAG, [0.0] * 3, [0.0, 0.0, 1.0])
    ell = k.intersection_curve(1e-9)
    assert ell is not None
    for branch in (1, -1):
        e = ell.electric_field(torch.tensor([0.3, 1.7, 4.0]), branch)
        adj, inv = k.adj_d(), torch.linalg.inv(k.dd_t())
        lhs = (e * (adj @ e.T).T).sum(-1)
        assert torch.allclose(lhs, torch.full((3,), float(k.s0 * k.det_d()), dtype=torch.float64), atol=1e-6)
        assert torch.allclose((e * (inv @ e.T).T).sum(-1), torch.ones(3, dtype=torch.float64), atol=1e-6)
    assert S.SpinoTensorKernel(50.0, DIAG, [0.0] * 3, [0.0, 0.0, 1.0]).intersection_curve() is None


def test_minimal_field_and_vorticity():
    sol = S.SpinoTensorKernel(1.5, DIAG, [0.0] * 3, [0.0, 0.0, 1.0]).minimal_electric_field()
    assert abs(float(sol.magnitude_squared) - 2.25) < 1e-9 and abs(abs(float(sol.vector[1])) - 1.5) < 1e-9
    assert abs(float(sol.vector[0])) < 1e-9 and abs(float(sol.vector[2])) < 1e-9
    # that field makes the tensor singular
    assert abs(float(S.SpinoTensorKernel(1.5, DIAG, sol.vector, [0.0, 0.0, 1.0]).det_t())) < 1e-9
    vor = S.SpinoTensorKernel(1.5, DIAG, [0.0, math.sqrt(2.0), 0.0], [0.0] * 3).minimal_vorticity()
    assert abs(float(vor.magnitude_squared) - 2.0 / 3.0) < 1e-9 and abs(abs(float(vor.vector[2])) - math.sqrt(2.0 / 3.0)) < 1e-9
    assert abs(float(S.SpinoTensorKernel(1.5, DIAG, [0.0, math.sqrt(2.0), 0.0], vor.vector).det_t())) < 1e-9
    assert not bool(S.SpinoTensorKernel(-1.0, DIAG, [0.0] * 3, [0.0, 0.0, 1.0]).minimal_electric_field().exists())


def test_batched_kernels_match_single_ones():
    g = torch.Generator().manual_seed(3)
    n = 17
    m = torch.randn(n, 3, 3, generator=g, dtype=torch.float64)
    a = m + m.transpose(-1, -2) + 4.0 * torch.eye(3, dtype=torch.float64)
    s0, e, w = torch.rand(n, generator=g, dtype=torch.float64) + 0.5, torch.randn(n, 3, generator=g, dtype=torch.float64), torch.randn(n, 3, generator=g, dtype=torch.float64)
    kb = S.SpinoTensorKernel(s0, a, e, w)
    det_t, alpha, beta, cls = kb.det_t(), kb.alpha(), kb.beta(), kb.classify()
    vort, field = kb.minimal_vorticity(), S.SpinoTensorKernel(s0, a, torch.zeros(n, 3), w).minimal_electric_field()
    names = {-1: "timelike", 0: "lightlike", 1: "spacelike"}
    for i in range(n):
        k = S.SpinoTensorKernel(s0[i], a[i], e[i], w[i])
        assert abs(float(k.det_t()) - float(det_t[i])) < 1e-9 and abs(float(k.alpha()) - float(alpha[i])) < 1e-9
        assert abs(float(k.beta()) - float(beta[i])) < 1e-9 and k.classify() == names[int(cls[i])]
        assert abs(float(torch.linalg.det(k.block_tensor())) - float(det_t[i])) < 1e-8
        one = k.minimal_vorticity().magnitude_squared
        assert (math.isnan(float(one)) and math.isnan(float(vort.magnitude_squared[i]))) or abs(float(one) - float(vort.magnitude_squared[i])) < 1e-9
        if bool(field.exists()[i]):
            assert abs(float(S.SpinoTensorKernel(s0[i], a[i], field.vector[i], w[i]).det_t())) < 1e-8


def test_projection_onto_a_z_pulse():
    k = S.SpinoTensorKernel(2.0 / 3.0, DIAG, [0.0, 1.0, 0.0], [0.0, 0.0, 1.0])
    stv = S.SpinoTensorVector(S.PauliSpinor.from_bloch_angles(0.9, 0.4), k)
    proj = stv.z_projection()
    spatial = stv.induced_vector()[1:]
    assert abs(proj.tempo - float(spatial.norm())) < 1e-9 and abs(sum(proj.band_energy) - proj.tempo) < 1e-9
    assert abs(proj.z_bias - (1.0 - 5.0 / 9.0)) < 1e-9 and proj.quality == 1.0 and abs(proj.support.total() - 1.0) < 1e-9
    assert abs(proj.drift - math.cos(0.9)) < 1e-9 and abs(proj.stderr - math.sqrt(abs(float(k.det_t())))) < 1e-12
    seen = []
    obs.add_observer(seen.append)
    try:
        pulse = stv.project_to_zpulse(128, "graph")
    finally:
        obs.remove_observer(seen.append)
    assert pulse.source == "graph" and pulse.ts == 128 and pulse.tempo > 0.0 and pulse.scale is not None
    assert pulse == proj.into_pulse(128, "graph")
    meta = [ev["meta"] for ev in seen if ev.get("kind") == "tensor_op_meta" and ev.get("op") == "spino_tensor_zpulse_project"]
    assert meta and meta[0]["causal_class"] == "timelike" and meta[0]["has_beta"] and meta[0]["band_total"] > 0.0
    flipped = stv.with_bloch_vector([0.0, 0.0, -2.0])
    assert torch.allclose(flipped.bloch_current(), torch.tensor([1.0, 0.0, 0.0, -1.0], dtype=torch.float64), atol=1e-9)
    assert torch.allclose(stv.with_phase_shift(1.3).induced_vector(), stv.induced_vector(), atol=1e-12)
