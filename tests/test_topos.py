"""Topos guards (parity: crates/st-tensor/src/pure/topos.rs unit tests for the guard, the
probability projection, the control signal and the biome)."""
import math

import pytest
import torch

from spiraltorch_b200.tensor import Tensor, TensorError
from spiraltorch_b200.topos import LawvereTierneyGuard, OpenCartesianTopos, RewriteMonad, TensorBiome


def test_constructor_validates_every_parameter():
    OpenCartesianTopos(-1.0, 1e-6, 10.0, 8, 1024)
    for args in ((0.5, 1e-6, 10.0, 8, 1024), (-1.0, 0.0, 10.0, 8, 1024), (-1.0, 1e-6, -1.0, 8, 1024),
                 (-1.0, 1e-6, 10.0, 0, 1024), (-1.0, 1e-6, 10.0, 8, 0), (math.nan, 1e-6, 10.0, 8, 1024)):
        with pytest.raises(TensorError):
            OpenCartesianTopos(*args)
    with pytest.raises(TensorError):
        OpenCartesianTopos(-1.0, 1e-6, 10.0, 8, 1024).with_porosity(1.5)
    with pytest.raises(TensorError):
        LawvereTierneyGuard(1e-3, 1e-4, 1e-5)


def test_guards_reject_non_finite_oversized_and_deep():
    t = OpenCartesianTopos(-1.0, 1e-6, 10.0, 4, 6)
    t.guard_tensor("ok", torch.zeros(2, 3))
    with pytest.raises(TensorError, match="volume"):
        t.guard_tensor("big", torch.zeros(2, 4))
    with pytest.raises(TensorError, match="non-finite"):
        t.guard_tensor("nan", torch.tensor([[1.0, math.nan]]))
    t.ensure_loop_free(3)
    with pytest.raises(TensorError, match="loop"):
        t.ensure_loop_free(4)


def test_probability_projection_repairs_and_normalises():
    t = OpenCartesianTopos(-1.0, 1e-6, 2.0, 4, 64)
    p = t.guard_probability_slice("p", [0.2, 0.0, 5.0, math.nan, -1.0, 0.3])
    assert abs(sum(p) - 1.0) < 1e-5 and p[1] == p[3] == p[4] == 0.0
    assert abs(p[2] / p[0] - 10.0) < 1e-4                       # 5.0 was clipped to the saturation 2.0 first
    with pytest.raises(TensorError, match="infeasible"):
        t.guard_probability_slice("p", [0.0, -3.0])
    # a tight density window: the upper bound forces a flat answer
    g = LawvereTierneyGuard(0.2, 0.3, 1e-4)
    q = g.project("q", [1.0, 1.0, 100.0, 1.0], 10.0)
    assert abs(float(q.sum()) - 1.0) < 1e-4 and float(q.max()) <= 0.3 + 1e-6 and float(q.min()) >= 0.2 - 1e-6
    m = t.guard_probability_tensor("m", torch.tensor([[1.0, 1.0], [2.0, 0.0]]))
    assert m.shape() == (2, 2) and abs(sum(m.data()) - 1.0) < 1e-5


def test_saturation_and_slope_match_the_closed_form():
    t = OpenCartesianTopos(-1.0, 1e-6, 2.0, 4, 64, porosity=0.25)
    for x in (-5.0, -0.5, 0.0, 1.0, 3.0):
        mag, sign = abs(x), (1.0 if x >= 0 else -1.0)
        absorb = 0.25 * 0.25
        want = x if mag <= 2.0 else sign * 2.0 * (1.0 - absorb * (mag - 2.0) / (mag + 2.0))
        slope = 1.0 if mag <= 2.0 else -2.0 * 4.0 * absorb / (mag + 2.0) ** 2
        y, dy = t.saturate_with_slope(x)
        assert abs(y - want) < 1e-6 and abs(t.saturate_scalar(x) - want) < 1e-6
        assert abs(dy - slope) < 1e-5
    out = RewriteMonad(t).rewrite_tensor("r", torch.tensor([[100.0, -100.0, 0.1]]))
    assert max(abs(v) for v in out.data()) <= 2.0 + 1e-6


def test_control_signal_tightens_with_pressure():
    t = OpenCartesianTopos(-1.0, 1e-6, 2.0, 8, 100)
    free, tight = t.control_signal(0, 0), t.control_signal(7, 95)
    assert free.openness == 1.0 and free.remaining_volume == 100 and tight.remaining_volume == 5
    assert tight.closure_pressure == 0.95 and tight.learning_rate_scale < free.learning_rate_scale
    assert tight.regularization_scale > free.regularization_scale
    assert 0.1 <= tight.learning_rate_scale <= 1.25 and set(free.as_dict()) >= {"sampling_focus", "step_damping"}
    ck = t.checkpoint()
    assert OpenCartesianTopos.from_checkpoint(ck).checkpoint() == ck


def test_biome_canopy_is_the_weighted_mean_under_the_guard():
    t = OpenCartesianTopos(-1.0, 1e-6, 50.0, 4, 18, porosity=0.0)
    b = TensorBiome(t)
    with pytest.raises(TensorError):
        b.canopy()
    b.absorb("a", torch.ones(2, 3))
    b.absorb_weighted("b", Tensor._wrap(torch.full((2, 3), 3.0)), 3.0)
    assert len(b) == 2 and b.total_weight() == 4.0 and b.stored_volume() == 12 and b.remaining_volume() == 6
    assert torch.allclose(b.canopy().torch(), torch.full((2, 3), 2.5))
    with pytest.raises(TensorError, match="shape"):
        b.absorb("c", torch.ones(3, 2))
    with pytest.raises(TensorError, match="weight"):
        b.absorb_weighted("c", torch.ones(2, 3), 0.0)
    b.absorb("c", torch.ones(2, 3))
    with pytest.raises(TensorError, match="volume"):
        b.absorb("d", torch.ones(2, 3))                              # 4 x 6 values > 18
    doubled = b.map_shoots("x2", lambda m, s: Tensor._wrap(s.torch() * 2))
    assert torch.allclose(doubled.canopy().torch(), b.canopy().torch() * 2)
    b.renormalise_weights()
    assert abs(b.total_weight() - 1.0) < 1e-5 and abs(b.weights()[1] - 0.6) < 1e-5
    # a failing rewrite (shoots of different shapes) leaves the biome as it was
    before = b.canopy().data()
    with pytest.raises(TensorError):
        b.bind_shoots("bad", lambda m, s: Tensor._wrap(torch.ones(1, 1 + int(s.torch()[0, 0] > 1))))
    assert b.canopy().data() == before
    b.clear()
    assert b.is_empty() and b.shape() is None


def test_fractal_scheduler_ring_and_fold():
    import asyncio
    from spiraltorch_b200.topos import FractalPatch, UringFractalScheduler
    for bad in ((0.0, 1.0), (1.0, 0.0), (math.nan, 1.0)):
        with pytest.raises(TensorError):
            FractalPatch(torch.ones(1, 2), *bad)
    with pytest.raises(TensorError):
        UringFractalScheduler(0)
    s = UringFractalScheduler(2)
    with pytest.raises(TensorError):
        s.fold_coherence()
    s.push(FractalPatch(torch.tensor([[3.0, 4.0]]), 1.0, 1.0, depth=0))        # weight 0.5, unit (0.6, 0.8)
    s.push(FractalPatch(torch.tensor([[0.0, 2.0]]), 3.0, 1.0, depth=1))        # weight 1.5, unit (0, 1)
    assert abs(s.total_weight() - 2.0) < 1e-9 and s.relation_shape() == (1, 2)
    assert torch.allclose(s.fold_coherence().torch(), torch.tensor([[0.25 * 0.6, 0.25 * 0.8 + 0.75]]), atol=1e-6)
    with pytest.raises(TensorError, match="shape"):
        s.push(FractalPatch(torch.ones(2, 2), 1.0, 1.0))
    assert len(s) == 2                                                           # the rejected push changed nothing
    s.push(FractalPatch(torch.tensor([[1.0, 0.0]]), 1.0, 1.0, depth=2))        # evicts depth 0
    snap = s.snapshot()
    assert (snap.queued, snap.oldest_depth, snap.newest_depth, snap.capacity) == (2, 1, 2, 2)
    # a full ring of capacity 1 accepts a new shape, because the only old patch is evicted
    one = UringFractalScheduler(1)
    one.push(FractalPatch(torch.ones(1, 2), 1.0, 1.0))
    one.push(FractalPatch(torch.ones(2, 2), 1.0, 1.0))
    assert one.relation_shape() == (2, 2)
    out = Tensor._wrap(torch.zeros(1, 2))
    s.fold_coherence_into(out)
    assert torch.allclose(out.torch(), s.fold_coherence().torch())
    assert asyncio.run(s.pop_async()).depth == 1 and s.pop().depth == 2 and s.pop() is None
    zero = FractalPatch(torch.zeros(1, 2), 1.0, 1.0)
    assert zero.normalized_relation().data() == [0.0, 0.0]
    # biome absorbs a patch under its weight and refuses one that is too deep
    b = TensorBiome(OpenCartesianTopos(-1.0, 1e-6, 50.0, 2, 64))
    b.absorb_fractal_patch(FractalPatch(torch.ones(1, 2), 3.0, 1.0, depth=1))
    assert b.weights() == [1.5]
    with pytest.raises(TensorError, match="loop"):
        b.absorb_fractal_patch(FractalPatch(torch.ones(1, 2), 3.0, 1.0, depth=2))
