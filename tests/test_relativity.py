"""General relativity helpers and the product-geometry module.  Analytic oracles: Minkowski is flat; Schwarzschild is
Ricci-flat with Kretschmann 48 M^2 / r^6; exponentially expanding FLRW has R = 12 H^2, K = 24 H^4 and no Weyl part."""
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import relativity as gr

ETA = torch.diag(torch.tensor([-1.0, 1.0, 1.0, 1.0], dtype=torch.float64))


def schwarzschild(c, mass=1.0):
    r, th = c[:, 1], c[:, 2]
    f = 1 - 2 * mass / r
    g = torch.zeros(c.shape[0], 4, 4, dtype=torch.float64)
    g[:, 0, 0], g[:, 1, 1], g[:, 2, 2], g[:, 3, 3] = -f, 1 / f, r * r, r * r * torch.sin(th) ** 2
    return g


def test_metric_validation():
    m = gr.LorentzianMetric.try_scaled(ETA, 3.0)
    assert m.components[0, 0] == -3.0 and m.signature.count(-1) == 1
    assert gr.LorentzianMetric(ETA).scaled(2.0).components[1, 1] == 2.0
    assert gr.LorentzianMetric(ETA).volume_element() == pytest.approx(1.0)
    with pytest.raises(gr.MetricError) as e:
        gr.LorentzianMetric(torch.eye(4))
    assert e.value.kind == "non_lorentzian"
    bad = ETA.clone()
    bad[0, 1] = 0.5
    with pytest.raises(gr.MetricError) as e:
        gr.LorentzianMetric(bad)
    assert e.value.kind == "non_symmetric"
    with pytest.raises(gr.MetricError) as e:
        gr.LorentzianMetric(torch.zeros(4, 4))
    assert e.value.kind == "degenerate"
    assert gr.InternalMetric(torch.diag(torch.tensor([1.0, 4.0, 9.0]))).volume_density() == pytest.approx(6.0)
    with pytest.raises(gr.MetricError) as e:
        gr.InternalMetric(torch.diag(torch.tensor([1.0, -1.0])))
    assert e.value.kind == "non_positive_definite"
    with pytest.raises(gr.MetricError):
        gr.WarpFactor.from_multiplier(0.0)
    assert gr.WarpFactor.from_exponent(0.5).scale == pytest.approx(math.e)


def test_minkowski_is_flat_and_solves_the_vacuum_equation():
    metric, first, second = gr.finite_difference_metric_data(lambda c: ETA, [0.0] * 4, 1e-3)
    model = gr.GeneralRelativityModel(gr.ZManifold.canonical(), metric, first, second)
    assert model.connection.coefficients.abs().max() == 0 and model.riemann.is_near_zero(1e-12)
    d = model.diagnostics
    assert d.kretschmann == d.ricci_square == d.weyl_square == d.weyl_self_dual_squared == 0.0
    eq = gr.FieldEquation.vacuum(model.einstein, 0.0, metric)
    assert eq.residual(gr.EnergyMomentumTensor.zero(), gr.PhysicalConstants()).abs().max() == 0


def test_schwarzschild_batch_matches_closed_forms():
    pts = torch.tensor([[0, 10.0, math.pi / 2, 0], [0, 6.0, 1.0, 0.3], [1.0, 25.0, 2.0, 1.0]], dtype=torch.float64)
    cf = gr.curvature_at_points(schwarzschild, pts, 1e-3)
    assert cf.ricci.abs().max() < 1e-5 and cf.einstein.abs().max() < 1e-4
    want = 48.0 / pts[:, 1] ** 6
    assert torch.allclose(cf.kretschmann, want, rtol=1e-4)
    assert torch.allclose(cf.weyl_square, want, rtol=1e-4)            # vacuum: Riemann is all Weyl
    # the single-point classes agree with the batched path
    one = gr.GeneralRelativityModel.from_metric_fn(lambda c: schwarzschild(torch.tensor([c], dtype=torch.float64))[0], pts[0].tolist())
    assert torch.allclose(one.riemann.components, cf.riemann[0], atol=1e-12)
    assert one.diagnostics.kretschmann == pytest.approx(float(cf.kretschmann[0]), rel=1e-9)
    # Gamma^r_{tt} = f M / r^2
    assert one.connection.coefficient(1, 0, 0) == pytest.approx((1 - 0.2) * 1.0 / 100.0, rel=1e-6)


def test_de_sitter_curvature():
    h = 0.3

    def flrw(c):
        a2 = torch.exp(2 * h * c[:, 0])
        g = torch.zeros(c.shape[0], 4, 4, dtype=torch.float64)
        g[:, 0, 0] = -1
        g[:, 1, 1] = g[:, 2, 2] = g[:, 3, 3] = a2
        return g
    cf = gr.curvature_at_points(flrw, torch.tensor([[0.0, 0, 0, 0], [0.7, 1, 2, 3]], dtype=torch.float64), 1e-3)
    assert torch.allclose(cf.scalar, torch.full((2,), 12 * h * h, dtype=torch.float64), rtol=1e-5)
    assert torch.allclose(cf.kretschmann, torch.full((2,), 24 * h ** 4, dtype=torch.float64), rtol=1e-4)
    assert cf.weyl_square.abs().max() < 1e-9
    # maximally symmetric: G = -3 H^2 g
    assert torch.allclose(cf.einstein, -3 * h * h * cf.metric, atol=1e-5)


def test_self_dual_decomposition_of_an_electric_weyl_mode():
    """A tensor that acts diagonally on the six bivectors with entries (2, -1, -1, 2, -1, -1): the self-dual projector
    pairs rows (0,5), (1,4), (2,3), so the 3x3 matrix is diag(0.5, -1, 0.5), I = 0.75, J = 0.125, discriminant 0 (the
    values the reference's own test pins, general_relativity.rs:2684-2703)."""
    metric = gr.LorentzianMetric(ETA)
    expected = [2.0, -1.0, -1.0]
    weyl = torch.zeros(4, 4, 4, 4, dtype=torch.float64)
    for a, (m, n) in enumerate(gr.BIVECTOR_BASIS):
        v = 2.0 * expected[a % 3]
        weyl[m, n, m, n] = weyl[n, m, n, m] = v
        weyl[n, m, m, n] = weyl[m, n, n, m] = -v
    ricci = gr.RicciTensor(torch.zeros(4, 4))
    d = gr.CurvatureDiagnostics._from_lower(weyl, weyl, metric, ricci, 0.0)
    assert torch.allclose(d.weyl_self_dual_matrix, torch.diag(torch.tensor([0.5, -1.0, 0.5], dtype=torch.complex128)))
    assert d.weyl_self_dual_invariant_i == pytest.approx(0.75) and d.weyl_self_dual_invariant_j == pytest.approx(0.125)
    assert abs(d.weyl_self_dual_discriminant) < 1e-12
    assert [z.real for z in d.weyl_self_dual_eigenvalues] == pytest.approx([-1.0, 0.5, 0.5])
    assert d.weyl_self_dual_squared + d.weyl_anti_self_dual_squared == pytest.approx(d.weyl_square)


def test_cubic_solver_branches():
    roots = gr.solve_self_dual_eigenvalues(3.0, -1.0)                          # double root
    assert sorted(r.real for r in roots) == pytest.approx([-1.0, -1.0, 2.0])
    for i, j in ((7.0, 3.0), (1.0, 2.0), (2 + 1j, 0.5 - 0.3j)):             # three real / one real / complex
        for x in gr.solve_self_dual_eigenvalues(i, j):
            assert abs(x ** 3 - i * x + 2 * j) < 1e-9


def _product(learnable=True):
    base = gr.LorentzianMetric(ETA)
    internal = gr.InternalMetric(torch.eye(2, dtype=torch.float64)).with_learnable(learnable)
    mixed = gr.MixedBlock([[0.0, 0.1], [-0.1, 0.0], [0.05, -0.05], [0.02, -0.02]], 4, 2).with_learnable(learnable)
    warp = gr.WarpFactor.from_multiplier(1.5).with_learnable(learnable)
    space = gr.InternalSpace("compact Z", gr.InternalPatch("torus", ["psi", "chi"]))
    return base, gr.ProductGeometry(gr.ZManifold.canonical(), space, gr.ProductMetric(base, internal, mixed, warp))


def test_product_metric_reduction_and_field_equation():
    base = gr.LorentzianMetric(ETA)
    internal = gr.InternalMetric([[1.0, 0.0], [0.0, 4.0]])
    mixed = gr.MixedBlock([[0, 0], [0.5, 0], [0, -0.5], [0, 0]], 4, 2)
    pm = gr.ProductMetric(base, internal, mixed, gr.WarpFactor.from_multiplier(4.0))
    b = pm.block_matrix()
    assert pm.total_dimension() == 6 and b[0, 0] == -4.0 and b[4, 4] == 1.0 and b[5, 5] == 4.0
    assert b[1, 4] == b[4, 1] == 0.5 and b[2, 5] == b[5, 2] == -0.5
    consts = gr.PhysicalConstants()
    vol = 2 * math.pi * 2.0
    assert pm.effective_newton_constant(consts, vol) == pytest.approx(consts.gravitational_constant / vol)
    with pytest.raises(gr.MetricError):
        gr.MixedBlock(torch.zeros(3, 2), 4, 2)
    space = gr.InternalSpace("Z", gr.InternalPatch("torus", ["a", "b"]))
    geo = gr.ProductGeometry(gr.ZManifold.canonical(), space, pm)
    red = gr.DimensionalReduction.project(geo, consts, vol)
    assert red.effective_metric.components[0, 0] == -4.0 and red.gauge_component(1, 0) == 0.5 and red.modulus_component(1, 1) == 4.0
    flat = gr.GeneralRelativityModel(gr.ZManifold.canonical(), base, gr.MetricDerivatives.zero(), gr.MetricSecondDerivatives.zero())
    lam = 0.25
    model = gr.ZRelativityModel.assemble(geo, flat, consts, vol, lam)
    assert torch.allclose(model.field_equations.lhs, lam * b)                   # flat base: only the Lambda terms remain
    assert model.field_equations.prefactor == pytest.approx(8 * math.pi * consts.gravitational_constant / vol / consts.speed_of_light ** 4)
    t = gr.ExtendedStressEnergy(torch.eye(6, dtype=torch.float64))
    assert torch.allclose(model.field_equations.residual(t), lam * b - model.field_equations.prefactor * torch.eye(6, dtype=torch.float64))
    with pytest.raises(gr.MetricError):
        gr.ExtendedStressEnergy(torch.tensor([[0.0, 1.0], [0.0, 0.0]]))


def test_zrelativity_module_exposes_and_trains_the_geometry():
    base, geo = _product(True)
    flat = gr.GeneralRelativityModel(gr.ZManifold.canonical(), base, gr.MetricDerivatives.zero(), gr.MetricSecondDerivatives.zero(),
                                     symmetry=gr.SymmetryAnsatz.HOMOGENEOUS_ISOTROPIC)
    model = gr.ZRelativityModel.assemble(geo, flat)
    events = []
    with st.observability.observe(events.append):
        mod = st.nn.ZRelativityModule.from_model(model)
        dummy = st.Tensor.zeros(1, 1)
        out = mod.forward(dummy)
        assert out.shape() == (1, mod.parameter_dimension()) and mod.parameter_dimension() == 36 + 8 + 4 + 1
        assert out.tolist()[0][0] == pytest.approx(-1.5) and out.tolist()[0][-1] == pytest.approx(1.5)
        back = mod.backward(dummy, st.Tensor._wrap(torch.ones(1, mod.parameter_dimension())))
    assert back.shape() == (1, 1) and back.tolist() == [[0.0]]
    assert all(p.gradient is not None for p in mod.parameters()) and mod.learnable_segments() == 4
    ops = {e["op"] for e in events if e["kind"] == "tensor_op_meta"}
    assert {"zrelativity_module_forward", "zrelativity_module_backward"} <= ops
    before = mod.warp.value.clone()
    mod.apply_step(0.1)
    assert torch.allclose(mod.warp.value, before - 0.1)
    with pytest.raises(st.TensorError):
        mod.backward(dummy, st.Tensor.zeros(1, 3))
    # constants stay constants
    _, geo2 = _product(False)
    frozen = st.nn.ZRelativityModule(gr.ZRelativityModel.assemble(geo2, flat))
    frozen.backward(dummy, st.Tensor._wrap(torch.ones(1, frozen.parameter_dimension())))
    assert frozen.learnable_segments() == 1 and frozen.gauge.gradient is None and frozen.block.gradient is not None
