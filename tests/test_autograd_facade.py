"""AutogradTensor contract and hypergradient solvers (CPU)."""
import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import autograd as ag
from spiraltorch_b200.autograd import AutogradTensor as AT


def test_contract_example_and_accumulation():
    x = AT.variable(st.Tensor(1, 3, [1.0, 2.0, -1.0]))
    loss = x.hadamard(x).add(x.scale(3.0)).sum()
    rep = loss.backward()
    assert x.grad().tolist() == [[5.0, 7.0, 1.0]]
    p = rep.contract_payload()
    assert p["contract_version"] == "spiraltorch.autograd.v1" and p["semantic_owner"] == "st-tensor"
    assert p["leaf_count"] == 1 and p["trainable_leaf_count"] == 1 and p["leaf_gradient_count"] == 1 and p["seed_l2"] == 1.0
    loss.backward()                                   # repeated passes accumulate
    assert x.grad().tolist() == [[10.0, 14.0, 2.0]]
    loss.zero_grad_graph()
    assert x.grad() is None
    assert loss.operation_name() == "sum" and loss.item_f32() == 1 + 4 + 1 + 3 * 2


def test_backward_rules_and_vjp():
    a = AT.variable(torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    b = AT.constant(torch.tensor([[0.5, -1.0], [2.0, 1.0]]))
    y = a.matmul(b).transpose()
    with pytest.raises(st.TensorError, match="1 x 1"):
        y.backward()
    seed = torch.tensor([[1.0, 0.0], [0.0, 2.0]])
    y.backward_with_grad(seed)
    expect = seed.t() @ b.value().torch().t()
    assert torch.allclose(a.grad().torch(), expect) and b.grad() is None
    # vjp is side-effect free and returns zeros for a disconnected input
    before = a.grad().tolist()
    other = AT.variable(torch.ones(2, 2))
    assert y.vector_jacobian_product(other, seed).tolist() == [[0.0, 0.0], [0.0, 0.0]]
    assert torch.allclose(y.vector_jacobian_product(a, seed).torch(), expect) and a.grad().tolist() == before
    mse = a.mean_squared_error(b)
    mse.backward()
    s = mse.graph_summary()
    assert s.leaf_count == 2 and s.trainable_leaf_count == 1 and s.operation_count == 3 and s.max_depth == 3
    with pytest.raises(st.TensorError):
        a.add(AT.constant(torch.ones(3, 2)))
    with pytest.raises(st.TensorError):
        AT.variable(torch.tensor([[float("nan")]]))
    assert a.detach().requires_grad() is False and a.dot(a).item_f32() == 30.0


def test_non_finite_gradient_commits_nothing():
    with pytest.raises(st.TensorError, match="non-finite value"):
        AT.variable(torch.tensor([[1e30, 1.0]])).hadamard(AT.variable(torch.tensor([[1e30, 1.0]])))
    x = AT.variable(torch.tensor([[1e-30]]))
    z = AT.variable(torch.tensor([[2.0]]))
    out = x.hadamard(AT.constant(torch.tensor([[1e30]]))).add(z)          # forward value 3.0
    with pytest.raises(st.TensorError, match="nothing was committed"):
        out.backward_with_grad(torch.tensor([[1e30]]))                    # d/dx overflows, d/dz is finite
    assert x.grad() is None and z.grad() is None
    out.backward_with_grad(torch.tensor([[1.0]]))
    assert z.grad().tolist() == [[1.0]] and abs(x.grad().tolist()[0][0] / 1e30 - 1) < 1e-6


def _quadratic_problem():
    # inner problem: w <- w - lr * (A w - b) with hyper = lr vector per coordinate; fixed point w* = A^{-1} b
    A = torch.tensor([[2.0, 0.3], [0.3, 1.0]])
    b = torch.tensor([[1.0], [-0.5]])
    target = torch.tensor([[0.2], [0.1]])
    Ac, bc, tc = AT.constant(A), AT.constant(b), AT.constant(target)

    def step(w, hyper, batch):
        grad = Ac.matmul(w).sub(bc)
        return w.sub(hyper.hadamard(grad))

    def val(w):
        return w.mean_squared_error(tc)

    return A, b, target, step, val


def test_unrolled_hypergradient_matches_torch():
    A, b, target, step, val = _quadratic_problem()
    hyper = AT.variable(torch.tensor([[0.1], [0.2]]))
    out = ag.unrolled(step, AT.variable(torch.zeros(2, 1)), hyper, iter([None] * 5), 5, val)
    h = torch.tensor([[0.1], [0.2]], requires_grad=True)
    w = torch.zeros(2, 1)
    for _ in range(5):
        w = w - h * (A @ w - b)
    ((w - target) ** 2).mean().backward()
    assert torch.allclose(out.dval_dhyper.torch(), h.grad, atol=1e-6)
    with pytest.raises(ag.HypergradError):
        ag.unrolled(step, AT.variable(torch.zeros(2, 1)), hyper, iter([None]), 3, val)
    with pytest.raises(ag.HypergradError):
        ag.unrolled(step, AT.variable(torch.zeros(2, 1)), AT.constant(torch.ones(2, 1)), iter([None]), 1, val)


@pytest.mark.parametrize("solver", ["neumann", "cg"])
def test_implicit_hypergradient_solves_the_sensitivity_equation(solver):
    A, b, target, step, val = _quadratic_problem()
    lr = torch.tensor([[0.3], [0.4]])
    w_star = torch.linalg.solve(A, b)
    out = ag.implicit(step, AT.variable(w_star), AT.variable(lr), iter([None]), val, solver, 200,
                      options=ag.ImplicitOptions(solver=solver, max_iters=200, tolerance=1e-6))
    # closed form: J = I - diag(lr) A, dstep/dlr = -diag(A w - b) = 0 at the fixed point -> hypergradient 0;
    # evaluate instead at a point off the fixed point, against a dense solve
    w0 = torch.tensor([[0.5], [0.5]])
    out = ag.implicit(step, AT.variable(w0), AT.variable(lr), iter([None]), val, solver, 300,
                      options=ag.ImplicitOptions(solver=solver, max_iters=300, tolerance=1e-6))
    J = torch.eye(2) - torch.diag(lr.flatten()) @ A
    g = 2 * (w0 - target) / 2
    v = torch.linalg.solve((torch.eye(2) - J).t(), g)
    dstep_dlr = -torch.diag((A @ w0 - b).flatten())
    expect = dstep_dlr.t() @ v
    assert torch.allclose(out.dval_dhyper.torch(), expect, atol=2e-3), (out.dval_dhyper.tolist(), expect.tolist())
    d = out.diagnostics
    assert d.solver == solver and d.converged and d.residual < 1e-2 and len(d.residual_history) >= 2
    with pytest.raises(ag.HypergradError):
        ag.implicit(step, AT.variable(w0), AT.variable(lr), iter([None]), val, "newton")
