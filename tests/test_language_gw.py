"""Entropic Gromov-Wasserstein solver and the semantic bridge (parity:
crates/st-nn/src/language/gw.rs tests; geometry.rs `SemanticBridge`)."""
import math

import pytest
import torch

from spiraltorch_b200.language import EntropicGwSolver, SemanticBridge
from spiraltorch_b200.tensor import TensorError


def _line(n):
    x = torch.arange(n, dtype=torch.float32)
    return (x[:, None] - x[None, :]).abs()


def _loop_cost(ds, dz, pi):
    n, m = ds.shape[0], dz.shape[0]
    out = torch.zeros(n, m)
    for i in range(n):
        for j in range(m):
            out[i, j] = (((ds[i][:, None] - dz[j][None, :]) ** 2) * pi).sum()
    return out


def test_gemm_form_of_the_cost_equals_the_four_loop_form():
    g = torch.Generator().manual_seed(0)
    ds, dz = _line(5) * 0.7, _line(4) * 1.3
    pi = torch.rand(5, 4, generator=g)
    pi /= pi.sum()
    fast = ((ds * ds) @ pi.sum(1))[:, None] + ((dz * dz) @ pi.sum(0))[None, :] - 2 * ds @ pi @ dz.T
    assert torch.allclose(fast, _loop_cost(ds, dz, pi), atol=1e-5)


def test_solver_recovers_an_isometry_with_one_anchor():
    n = 5
    d = _line(n)
    bridge = EntropicGwSolver(epsilon=0.1, anchor_strength=1.0, max_iter=30, sinkhorn_iter=60).solve(
        d, d, [1.0] * n, [1.0] * n, anchors=[(0, 0)])          # the anchor breaks the reflection symmetry
    pi = torch.exp(bridge.log_pi_matrix)
    assert pi.argmax(1).tolist() == list(range(n))
    assert torch.allclose(bridge.row_marginal(), torch.full((n,), 1 / n), atol=1e-3)
    assert torch.allclose(bridge.col_marginal(), torch.full((n,), 1 / n), atol=1e-3)
    assert bridge.anchors() == {(0, 0)} and bridge.vocab_size() == n and bridge.concept_count() == n


def test_solver_validates_marginals():
    s = EntropicGwSolver()
    with pytest.raises(TensorError, match="match"):
        s.solve(_line(3), _line(2), [1, 1], [1, 1])
    with pytest.raises(TensorError, match="non-negative"):
        s.solve(_line(2), _line(2), [1, -1], [1, 1])
    with pytest.raises(TensorError, match="positive"):
        s.solve(_line(2), _line(2), [0, 0], [1, 1])
    with pytest.raises(TensorError, match="empty"):
        s.solve(_line(2), _line(2), [], [1, 1])


def test_cooperative_tuning_moves_parameters_the_documented_way():
    s = EntropicGwSolver()
    z, w = s.propose()
    assert w > 0 and -1 < z < 1
    a0, e0 = s.anchor_strength, s.epsilon
    s.observe(-0.4, 0.6)
    assert s.anchor_strength >= a0 and s.epsilon <= e0 * (1 + 0.03)
    e1 = s.epsilon
    s.observe(0.2, -0.7)
    assert s.epsilon >= e1 * 0.99 and 0.5 <= s.anchor_strength <= 24.0


def test_bridge_queries():
    pi = torch.tensor([[0.4, 0.0], [0.1, 0.5]])
    b = SemanticBridge.from_dense(pi, anchors=[(0, 0)], epsilon=1e-6)
    assert abs(b.log_pi(0, 0) - math.log(0.4)) < 1e-6 and abs(b.log_pi(0, 1) - math.log(1e-6)) < 1e-5
    assert b.log_pi(9, 0) == b.log_epsilon
    assert abs(b.expectation(1, [1.0, 1.0]) - 0.5 * (math.log(0.1) + math.log(0.5))) < 1e-6
    assert b.expectation(1, [0.0, 0.0]) == b.log_epsilon
    assert torch.allclose(b.expectations([1.0, 1.0])[1], torch.tensor(b.expectation(1, [1.0, 1.0])))
    d = b.infer_from_window([(1, 2.0), (7, 1.0), (0, -1.0)])
    assert torch.allclose(d, torch.tensor([0.1, 0.5]) / 0.6, atol=1e-6)
    assert torch.allclose(b.infer_from_window([]), torch.tensor([0.5, 0.5]))
    assert torch.allclose(b.infer_from_window([], smoothing=1.0), torch.tensor([0.5, 0.5]))
    with pytest.raises(TensorError):
        SemanticBridge.from_dense(torch.tensor([[1.0, -1.0]]))
