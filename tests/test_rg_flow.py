"""RG flows on a log lattice (user beta functions, operator flows with Mellin resonances) and the gravity potential."""
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.mellin import MellinLogGrid
from spiraltorch_b200.rg_flow import (GravityField, GravityWell, RGFlowModel, RGOperator, RgFlowError, RgFlowLattice)


def beta_profile(log_scale, couplings):
    target = math.tanh(log_scale)
    return [-0.35 * (g - target) for g in couplings]


def test_lattice_from_mellin_grid_and_fixed_points():
    grid = MellinLogGrid.from_function(-1.5, 0.3, 10, lambda x: torch.complex(torch.sin(1.3 * x), torch.cos(torch.sin(1.3 * x))))
    flow = RgFlowLattice.from_mellin_grid(grid, [0.1, 0.05], beta_profile)
    assert len(flow) == 10 and flow.mellin_series() is not None and len(flow.nodes[0].couplings) == 2
    # Euler step
    n0, n1 = flow.nodes[0], flow.nodes[1]
    assert n1.couplings[0] == pytest.approx(n0.couplings[0] + 0.3 * n0.beta[0]) and n1.log_scale == pytest.approx(-1.2)
    assert n0.scale == pytest.approx(math.exp(-1.5)) and n0.narrative_depth() == n0.scale
    assert min(n.beta_norm() for n in flow.nodes) < 0.1
    tol = sorted(n.beta_norm() for n in flow.nodes)[2]
    events = []
    with st.observability.observe(events.append):
        fixed = flow.fixed_points(tol)
    assert len(fixed) == 3 and all(math.isfinite(c) for p in fixed for c in p.couplings)
    meta = [e["meta"] for e in events if e["kind"] == "tensor_op_meta"][0]
    assert meta["fixed_points"] == 3 and meta["has_mellin_series"] and meta["beta_norm_min"] <= tol
    s = 1.1 + 0.4j
    assert flow.evaluate_mellin(s) == pytest.approx(grid.evaluate(s))
    many = flow.evaluate_mellin_many([s, 0.8 - 0.2j])
    assert many.shape == (2,) and complex(many[0]) == pytest.approx(grid.evaluate(s))
    plain = RgFlowLattice.new_with_beta(0.0, 0.1, 4, [1.0], lambda t, g: [-g[0]])
    assert [n.couplings[0] for n in plain.nodes] == pytest.approx([1.0, 0.9, 0.81, 0.729])
    with pytest.raises(RgFlowError) as e:
        plain.evaluate_mellin(1.0)
    assert e.value.kind == "missing_mellin_series"
    for args, kind in (((float("nan"), 0.1, 4, [1.0]), "invalid_log_start"), ((0.0, 0.0, 4, [1.0]), "invalid_log_step"),
                       ((0.0, 0.1, 0, [1.0]), "empty_lattice"), ((0.0, 0.1, 4, []), "empty_couplings")):
        with pytest.raises(RgFlowError) as e:
            RgFlowLattice.new_with_beta(*args, lambda t, g: list(g))
        assert e.value.kind == kind
    with pytest.raises(RgFlowError) as e:
        RgFlowLattice.new_with_beta(0.0, 0.1, 4, [1.0], lambda t, g: [0.0, 0.0])
    assert e.value.kind == "beta_dimension"


def test_operator_flow_matches_the_scalar_recurrence():
    model = RGFlowModel(-1.0, 0.1, 12)
    res = RGFlowModel.gaussian_resonance(-2.0, 0.1, 41, 1.0, 0.5, 0.3)
    model.register_operator(RGOperator("relevant", 3.0, 0.2))
    model.register_operator(RGOperator("marginal", 4.0, 0.1).with_nonlinear_feedback(-0.5))
    model.register_operator(RGOperator("driven", 4.5, 0.05).with_resonance(res))
    model.damping = 0.05
    sol = model.propagate()
    assert sol.tensor.shape == (3, 12) and [t.name for t in sol] == ["relevant", "marginal", "driven"]
    for idx, op in enumerate(model.operators):                          # one operator at a time, through sample_beta
        g, want = op.initial_coupling, [op.initial_coupling]
        for log_scale in model.lattice[1:]:
            g += model.log_step * model.sample_beta(g, idx, log_scale)
            want.append(g)
        assert sol.trajectory(op.name).values == pytest.approx(want, rel=1e-9)
    rel = sol.trajectory("relevant")
    assert rel.at(11) < rel.at(0) and rel.at(99) is None                 # Delta < 4 and damping: the coupling decays along the flow
    assert res.evaluate(0.3) == pytest.approx(complex(res.evaluate_lattice([0.3])[0]))
    assert sol.trajectory("missing") is None
    with pytest.raises(RgFlowError):
        model.sample_beta(0.1, 7, 0.0)
    empty = RGFlowModel.from_lattice([0.0, 0.5, 1.0]).propagate()
    assert empty.trajectories == [] and empty.lattice == [0.0, 0.5, 1.0]
    nd = RGFlowModel.narrative_depth(8, 0.0)
    assert nd.lattice[-1] + nd.log_step == pytest.approx((math.sqrt(5) - 1) / 2)
    breath = RGFlowModel.breathing_resonance(res.grid, 1.5 + 0.2j, math.pi / 2, 2.0)
    assert breath.residue == pytest.approx(2j)
    with pytest.raises(RgFlowError):
        RGFlowModel(0.0, -1.0, 3)


def test_gravity_potential():
    field = GravityField()
    field.add_well("pose", GravityWell.newtonian(10.0))
    assert field.potential("pose", 2.0) == pytest.approx(-6.67430e-11 * 5.0) and field.potential("nope", 2.0) is None
    assert field.potential("pose", 0.0) == 0.0
    field.add_well("rel", GravityWell.relativistic(10.0, 10.0))
    assert field.potential("rel", 2.0) == pytest.approx(field.potential("pose", 2.0) / 1.2)
    assert field("nope", 1.0) == 0.0 and field("pose", 2.0) < 0
