"""Inflaton Z-space helpers against the values of crates/st-core/src/theory/inflaton_zspace.rs's unit tests."""
import math

import pytest
import torch

from spiraltorch_b200 import inflaton as I
from spiraltorch_b200 import observability as obs


def test_weights_and_hann_window():
    lat = I.LogLattice.from_samples(0.0, 0.25, [1.0, 2.0, 3.0, 4.0])
    assert abs(float(lat.weights.sum()) - 1.0) < 1e-12 and lat.weights[0] == lat.weights[-1] == lat.weights[1] / 2
    flat = I.LogLattice(0.0, 0.25, [1.0, 1.0, 1.0, 1.0])
    before = flat.weights.clone()
    flat.apply_hann_window()
    assert flat.weights[0] < before[0] and flat.weights[1] > 0.0 and abs(float(flat.weights.sum()) - 1.0) < 1e-12
    with pytest.raises(ValueError):
        I.LogLattice(0.0, 0.0, [1.0, 2.0])
    with pytest.raises(ValueError):
        I.LogLattice(0.0, 0.1, [1.0])


def test_horner_matches_the_direct_sum_for_many_points():
    samples = [1.0, 2.0, 4.0, 8.0]
    lat = I.LogLattice(0.0, 0.5, samples)
    z = torch.tensor([0.8 + 0.2j, 0.3 - 0.9j, 1.0 + 0.0j], dtype=torch.complex128)
    k = torch.arange(4, dtype=torch.float64)
    direct = ((lat.weights * lat.samples).to(torch.complex128)[None, :] * z[:, None] ** k[None, :]).sum(dim=1)
    assert torch.allclose(lat.z_transform(z), direct, atol=1e-12, rtol=0)
    assert I.z_transform(lat.weights, lat.samples, 0.8 + 0.2j).shape == ()


def test_spectrum_is_scale_invariant_for_constant_channels():
    spec = I.assemble_primordial_spectrum([0.5, 0.25], [10.0, 10.0], [0.01, 0.01], 2.435e18)
    expected = 100.0 / (8.0 * math.pi ** 2 * 0.01 * 2.435e18 ** 2)
    assert spec.shape == (2,) and abs(float(spec[0]) - expected) < 1e-24 and float(spec[0]) == float(spec[1])
    assert float(I.assemble_primordial_spectrum([1.0], [1.0], [-5.0], 1.0)[0]) == pytest.approx(1.0 / (8 * math.pi ** 2 * 1e-20))
    with pytest.raises(ValueError):
        I.assemble_primordial_spectrum([1.0], [1.0, 2.0], [1.0], 1.0)


def test_projection_bundles_channels_and_reports():
    s = torch.tensor([1.0 + 0.0j, 1.0 + 0.5j, 1.0 - 0.5j], dtype=torch.complex128)
    z = torch.exp(s * 0.25)
    seen = []
    obs.add_observer(seen.append)
    try:
        proj = I.PrimordialProjection.new(0.0, 0.25, 4, s, z, [2.0, 2.0 + 0.1j, 2.0 - 0.1j], [0.01, 0.02, 0.015], 2.435e18)
    finally:
        obs.remove_observer(seen.append)
    assert len(proj) == 3 and not proj.is_empty() and proj.spectrum.shape == (3,) and proj.lattice_len == 4
    assert torch.equal(proj.z_points, z) and float(proj.spectrum[0]) > float(proj.spectrum[1])
    meta = [e["meta"] for e in seen if e.get("kind") == "tensor_op_meta" and e.get("op") == "inflaton_primordial_projection"]
    assert meta and meta[0]["kind"] == "st_core_inflaton_primordial_projection" and meta[0]["evaluation_count"] == 3
    assert meta[0]["spectrum_count"] == 3 and meta[0]["epsilon_clamp_count"] == 0


def test_from_background_reproduces_a_de_sitter_like_plateau():
    # constant H and epsilon on the lattice: both transforms share the geometric factor, so the spectrum is flat in Im s
    n, dt = 64, 0.125
    hub = I.LogLattice(0.0, dt, torch.full((n,), 1.0e-5, dtype=torch.float64))
    eps = I.LogLattice(0.0, dt, torch.full((n,), 0.01, dtype=torch.float64))
    s = torch.complex(torch.zeros(5, dtype=torch.float64), torch.zeros(5, dtype=torch.float64))
    proj = I.PrimordialProjection.from_background(hub, eps, s, 1.0)
    expected = (1.0e-5) ** 2 / (8 * math.pi ** 2 * 0.01)
    assert torch.allclose(proj.spectrum, torch.full((5,), expected, dtype=torch.float64), rtol=1e-12)
    with pytest.raises(ValueError):
        I.PrimordialProjection.from_background(hub, I.LogLattice(0.0, dt, [1.0, 2.0]), s, 1.0)
