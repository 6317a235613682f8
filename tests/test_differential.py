"""Spiral differentials (parity: crates/st-tensor/src/pure/differential.rs unit tests; barycenter path of measure.rs)."""
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.differential import (FunctorDifferential, HomotopyDifferential, InfinityDifferential,
                                           RecursiveDifferential, SpiralDifferential)
from spiraltorch_b200.measure import z_space_barycenter
from spiraltorch_b200.tensor import TensorError
from spiraltorch_b200.topos import OpenCartesianTopos


def T(rows):
    return st.Tensor(torch.tensor(rows, dtype=torch.float32))


def _bary():
    return z_space_barycenter([1.0, 2.0], [T([[0.7, 0.2, 0.1]]), T([[0.1, 0.3, 0.6]])], 0.1, 0.0)


def test_barycenter_path_descends_and_feeds_a_tape():
    b = _bary()
    alphas = [s.interpolation for s in b.intermediates]
    objs = [s.objective for s in b.intermediates]
    assert alphas == [0.0, 0.25, 0.5, 0.75, 1.0] and all(x >= y - 1e-6 for x, y in zip(objs, objs[1:]))
    assert abs(objs[-1] - b.objective) < 1e-5
    assert torch.allclose(b.intermediates[-1].density.torch(), b.density.torch(), atol=1e-6)
    want0 = (torch.tensor([0.7, 0.2, 0.1]) + 2 * torch.tensor([0.1, 0.3, 0.6])) / 3
    assert torch.allclose(b.intermediates[0].density.torch().flatten(), want0, atol=1e-6)
    tape, ref = st.hypergrad(1, 3), st.hypergrad(1, 3)
    RecursiveDifferential(b).accumulate(tape)
    ref.accumulate_wave(b.intermediates[0].density)
    for prev, cur in zip(b.intermediates, b.intermediates[1:]):
        ref.accumulate_pair(cur.density, prev.density)
    assert torch.allclose(tape.gradient, ref.gradient)
    with pytest.raises(ValueError):
        tape.accumulate_barycenter_path([])


def test_homotopy_functor_infinity():
    h1 = HomotopyDifferential(T([[1.0, 2.0]]), T([[0.5, -1.0]]), T([[2.0, 3.0]]))
    assert h1.flow().data() == [2.0, -1.0] and h1.directional_energy() == 1.0 + 9.0
    h2 = HomotopyDifferential(T([[1.0, 2.0]]), T([[1.0, 1.0]]), T([[1.0, -1.0]]))
    assert h1.commutator(h2).data() == [0.0, 0.0]                       # translations commute
    topos = OpenCartesianTopos(-1.0, 1e-6, 1.5, 4, 64, porosity=0.0)
    assert h1.flow_guarded(topos).data() == [1.5, -1.0]
    with pytest.raises(TensorError):
        HomotopyDifferential(T([[1.0, 2.0]]), T([[1.0]]), T([[1.0, 2.0]]))
    f = FunctorDifferential(T([[1.0, 2.0]]), T([[1.0, 0.0], [0.0, 2.0]]), 1e-3)
    assert f.apply().data() == [1.0, 4.0] and f.linearise(T([[3.0, 1.0]])).data() == [3.0, 2.0]
    with pytest.raises(TensorError):
        FunctorDifferential(T([[1.0, 2.0]]), T([[1.0, 0.0]]), 1e-3)
    with pytest.raises(TensorError):
        FunctorDifferential(T([[1.0, 2.0]]), T([[1.0, 0.0], [0.0, 2.0]]), 0.0)
    inf = InfinityDifferential([T([[1.0, 3.0]]), T([[3.0, 5.0]])], [-2.0, 0.5])
    assert inf.collapse().data() == [2.0, 4.0] and inf.hierarchical_energy_tensor().data() == [20.0, 17.0]
    with pytest.raises(TensorError):
        InfinityDifferential([])
    with pytest.raises(TensorError):
        InfinityDifferential([T([[1.0]])], [1.0, 2.0])


def test_spiral_differential_resonates_under_a_topos():
    b = _bary()
    h = HomotopyDifferential(T([[0.2, 0.3, 0.5]]), T([[1.0, 1.0, 1.0]]), T([[0.1, 0.0, -0.1]]))
    f = FunctorDifferential(T([[0.2, 0.3, 0.5]]), st.Tensor(torch.eye(3) * 2), 1e-3)
    inf = InfinityDifferential([T([[0.0, 0.0, 3.0]]), T([[0.0, 4.0, 0.0]])])
    topos = OpenCartesianTopos(-1.0, 1e-6, 10.0, 4, 64, porosity=0.0)
    sd = SpiralDifferential(topos, h, f, RecursiveDifferential.from_barycenter(b), inf)
    tape = st.hypergrad(1, 3)
    r = sd.resonate(tape)
    assert torch.allclose(r.homotopy_flow.torch(), torch.tensor([[0.3, 0.3, 0.4]]), atol=1e-6)
    assert torch.allclose(r.functor_linearisation.torch(), torch.tensor([[0.2, 0.0, -0.2]]), atol=1e-6)
    assert r.recursive_objective.shape() == (1, 5) and r.infinity_projection.data() == [0.0, 2.0, 1.5]
    assert r.infinity_energy.data() == [9.0, 10.0]                      # 16 saturates at 10
    assert float(tape.gradient.abs().sum()) > 0
    with pytest.raises(TensorError, match="shape"):
        SpiralDifferential(None, h, f, RecursiveDifferential(b), InfinityDifferential([T([[1.0, 2.0]])]))
    broken = _bary()
    broken.intermediates[2].objective = broken.intermediates[1].objective + 1.0
    with pytest.raises(TensorError, match="objective"):
        RecursiveDifferential(broken)
