"""``AutogradTensor``: the reverse-mode graph API of the reference on top of ``torch.autograd``,
plus unrolled and implicit hypergradients.

Contract ``spiraltorch.autograd.v1`` (crates/st-tensor/src/autograd.rs:87-640,
docs/autograd_contract.md): immutable graph nodes with atomically assigned ids; leaves declare
``requires_grad``; ``backward()`` only for ``1 x 1`` outputs, ``backward_with_grad(seed)`` otherwise;
every gradient of a pass is validated (finite) before any is committed; repeated passes accumulate;
``vector_jacobian_product`` has no side effects and returns zeros for a disconnected input;
operations: add, sub, hadamard, matmul, scale, transpose, sum, mean, dot, mean_squared_error.
Matrix products of CUDA tensors run the tcgen05 GEMM (forward and both gradient products).

Hypergradients follow crates/st-core/src/autograd/hypergrad.rs:238-520: ``unrolled`` differentiates
the validation loss through ``steps`` applications of ``step_fn``; ``implicit`` solves the
fixed-point sensitivity ``(I - Jᵀ) v = ∂L/∂w`` by a Neumann series or conjugate gradients on the
normal equations and returns ``(∂step/∂hyper)ᵀ v`` with solver diagnostics.
"""
from __future__ import annotations

import itertools
import threading
from dataclasses import dataclass, field
from typing import Callable, Iterator, Optional

import torch

from .ops import gemm as gemm_ops
from .ops import native
from .tensor import Tensor, TensorError

CONTRACT_VERSION = "spiraltorch.autograd.v1"
SEMANTIC_OWNER = "st-tensor"
_ids = itertools.count(1)
_backward_lock = threading.Lock()


class _MatMul(torch.autograd.Function):
    """``a @ b`` whose three products run on the sm_100a GEMM for CUDA operands."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        if native.use_native(a):
            return gemm_ops.gemm(a.to(torch.bfloat16), b.to(torch.bfloat16), b_mn=True, out_dtype=torch.float32)
        return a @ b

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        if native.use_native(a):
            gb, ab, bb = g.to(torch.bfloat16), a.to(torch.bfloat16), b.to(torch.bfloat16)
            da = gemm_ops.gemm(gb, bb, out_dtype=torch.float32)                         # g @ bᵀ
            db = gemm_ops.gemm(ab, gb, a_mn=True, b_mn=True, out_dtype=torch.float32)   # aᵀ @ g
            return da, db
        return g @ b.t(), a.t() @ g


@dataclass
class AutogradGraphSummary:
    node_count: int = 0
    operation_count: int = 0
    leaf_count: int = 0
    trainable_leaf_count: int = 0
    max_depth: int = 0

    def contract_payload(self) -> dict:
        return {"contract_version": CONTRACT_VERSION, "semantic_owner": SEMANTIC_OWNER, "node_count": self.node_count,
                "operation_count": self.operation_count, "leaf_count": self.leaf_count,
                "trainable_leaf_count": self.trainable_leaf_count, "max_depth": self.max_depth}


@dataclass
class AutogradBackwardReport:
    graph: AutogradGraphSummary = field(default_factory=AutogradGraphSummary)
    gradient_node_count: int = 0
    leaf_gradient_count: int = 0
    seed_l2: float = 0.0

    def contract_payload(self) -> dict:
        p = self.graph.contract_payload()
        p.update(gradient_node_count=self.gradient_node_count, leaf_gradient_count=self.leaf_gradient_count,
                 seed_l2=self.seed_l2)
        return p


class AutogradTensor:
    def __init__(self, t: torch.Tensor, op: str, parents: tuple = (), requires_grad: bool = False):
        self._t = t
        self._op = op
        self._parents = parents
        self._leaf_requires = requires_grad
        self._id = next(_ids)
        self._grad: Optional[torch.Tensor] = None

    # ---- construction -------------------------------------------------------------------------
    @staticmethod
    def _raw(value) -> torch.Tensor:
        t = value.torch() if isinstance(value, Tensor) else torch.as_tensor(value, dtype=torch.float32)
        if t.dim() != 2:
            raise TensorError(f"autograd values are 2-D, got shape {tuple(t.shape)}")
        if not bool(torch.isfinite(t).all()):
            raise TensorError("non-finite value in autograd leaf")
        return t.detach().float().clone()

    @classmethod
    def from_tensor(cls, value, requires_grad: bool) -> "AutogradTensor":
        t = cls._raw(value)
        t.requires_grad_(requires_grad)
        return cls(t, "leaf", (), requires_grad)

    @classmethod
    def variable(cls, value) -> "AutogradTensor":
        return cls.from_tensor(value, True)

    @classmethod
    def constant(cls, value) -> "AutogradTensor":
        return cls.from_tensor(value, False)

    @classmethod
    def zeros_like(cls, other: "AutogradTensor") -> "AutogradTensor":
        return cls.constant(torch.zeros_like(other._t))

    # ---- accessors ----------------------------------------------------------------------------
    def id(self) -> int:
        return self._id

    def value(self) -> Tensor:
        return Tensor._wrap(self._t.detach())

    def shape(self) -> tuple:
        return tuple(self._t.shape)

    def requires_grad(self) -> bool:
        return bool(self._t.requires_grad)

    def operation_name(self) -> str:
        return self._op

    def detach(self) -> "AutogradTensor":
        return AutogradTensor.constant(self._t.detach())

    def grad(self) -> Optional[Tensor]:
        return None if self._grad is None else Tensor._wrap(self._grad.clone())

    def zero_grad(self) -> None:
        self._grad = None

    def zero_grad_graph(self) -> None:
        for n in self._topological():
            n._grad = None

    def item_f32(self) -> float:
        if self.shape() != (1, 1):
            raise TensorError(f"item_f32 needs a 1 x 1 tensor, got {self.shape()}")
        return float(self._t.detach())

    # ---- operations ---------------------------------------------------------------------------
    def _new(self, t: torch.Tensor, op: str, *parents: "AutogradTensor") -> "AutogradTensor":
        if not bool(torch.isfinite(t.detach()).all()):
            raise TensorError(f"non-finite value produced by autograd {op}")
        return AutogradTensor(t, op, parents)

    def _same(self, rhs: "AutogradTensor", op: str) -> None:
        if self.shape() != rhs.shape():
            raise TensorError(f"{op}: shape mismatch {self.shape()} vs {rhs.shape()}")

    def add(self, rhs):
        self._same(rhs, "add")
        return self._new(self._t + rhs._t, "add", self, rhs)

    def sub(self, rhs):
        self._same(rhs, "sub")
        return self._new(self._t - rhs._t, "sub", self, rhs)

    def hadamard(self, rhs):
        self._same(rhs, "hadamard")
        return self._new(self._t * rhs._t, "hadamard", self, rhs)

    def matmul(self, rhs):
        if self.shape()[1] != rhs.shape()[0]:
            raise TensorError(f"matmul: inner dimensions differ, {self.shape()} x {rhs.shape()}")
        return self._new(_MatMul.apply(self._t, rhs._t), "matmul", self, rhs)

    def scale(self, factor: float):
        return self._new(self._t * float(factor), "scale", self)

    def transpose(self):
        return self._new(self._t.t(), "transpose", self)

    def sum(self):
        return self._new(self._t.sum().reshape(1, 1), "sum", self)

    def mean(self):
        return self._new(self._t.mean().reshape(1, 1), "mean", self)

    def dot(self, rhs):
        return self.hadamard(rhs).sum()

    def mean_squared_error(self, target):
        d = self.sub(target)
        return d.hadamard(d).mean()

    # ---- graph --------------------------------------------------------------------------------
    def _topological(self) -> list:
        order, seen, stack = [], set(), [(self, False)]
        while stack:
            node, expanded = stack.pop()
            if expanded:
                order.append(node)
                continue
            if node._id in seen:
                continue
            seen.add(node._id)
            stack.append((node, True))
            for p in reversed(node._parents):
                stack.append((p, False))
        return order

    def graph_summary(self) -> AutogradGraphSummary:
        s = AutogradGraphSummary()
        depth: dict[int, int] = {}
        stack = [(self, 0)]
        while stack:
            node, d = stack.pop()
            if node._id in depth and depth[node._id] >= d:
                continue
            if node._id not in depth:
                s.node_count += 1
                if node._op == "leaf":
                    s.leaf_count += 1
                    s.trainable_leaf_count += int(node._leaf_requires)
                else:
                    s.operation_count += 1
            depth[node._id] = d
            s.max_depth = max(s.max_depth, d)
            for p in node._parents:
                stack.append((p, d + 1))
        return s

    # ---- differentiation ----------------------------------------------------------------------
    def vector_jacobian_product(self, input: "AutogradTensor", seed) -> Tensor:
        seed_t = AutogradTensor._raw(seed).to(self._t.device)
        if tuple(seed_t.shape) != self.shape():
            raise TensorError(f"seed shape {tuple(seed_t.shape)} does not match output {self.shape()}")
        if not input._t.requires_grad or not self._t.requires_grad:
            return Tensor._wrap(torch.zeros_like(input._t))
        (g,) = torch.autograd.grad(self._t, input._t, seed_t, retain_graph=True, allow_unused=True)
        return Tensor._wrap(torch.zeros_like(input._t) if g is None else g)

    def backward(self) -> AutogradBackwardReport:
        if self.shape() != (1, 1):
            raise TensorError(f"backward() needs a 1 x 1 output, got {self.shape()}; use backward_with_grad(seed)")
        return self.backward_with_grad(torch.ones(1, 1))

    def backward_with_grad(self, seed) -> AutogradBackwardReport:
        seed_t = AutogradTensor._raw(seed).to(self._t.device)
        if tuple(seed_t.shape) != self.shape():
            raise TensorError(f"seed shape {tuple(seed_t.shape)} does not match output {self.shape()}")
        nodes = [n for n in self._topological() if n._t.requires_grad]
        report = AutogradBackwardReport(self.graph_summary(), seed_l2=float(seed_t.norm()))
        if not nodes or not self._t.requires_grad:
            return report
        with _backward_lock:
            grads = torch.autograd.grad(self._t, [n._t for n in nodes], seed_t, retain_graph=True, allow_unused=True)
            # validate everything before committing anything
            for n, g in zip(nodes, grads):
                if g is not None and not bool(torch.isfinite(g).all()):
                    raise TensorError(f"non-finite gradient at autograd node {n._id} ({n._op}); nothing was committed")
            for n, g in zip(nodes, grads):
                if g is None:
                    continue
                report.gradient_node_count += 1
                if n._op == "leaf":
                    report.leaf_gradient_count += 1
                    n._grad = g.clone() if n._grad is None else n._grad + g
        return report


# ---- hypergradients --------------------------------------------------------------------------------
class HypergradError(ValueError):
    pass


@dataclass
class UnrolledOut:
    w_final: AutogradTensor
    dval_dhyper: Tensor


@dataclass
class ImplicitDiagnostics:
    requested_solver: str
    solver: str
    iterations: int
    residual: float
    residual_history: list
    finite_diff_eps: float
    converged: bool
    fallback_reason: Optional[str] = None


@dataclass
class ImplicitOut:
    dval_dhyper: Tensor
    diagnostics: ImplicitDiagnostics


@dataclass
class ImplicitOptions:
    solver: str = "neumann"
    max_iters: int = 32
    tolerance: float = 1e-5
    finite_diff_eps: float = 1e-3
    cg_fallback: bool = True

    def validate(self) -> None:
        if self.solver.lower() not in ("neumann", "cg"):
            raise HypergradError(f"unknown solver '{self.solver}'")
        if self.max_iters <= 0:
            raise HypergradError("max_iters must be positive")
        if not self.tolerance > 0 or not self.finite_diff_eps > 0:
            raise HypergradError("tolerance and finite-difference step must be positive")


def _scalar_vjp(loss: AutogradTensor, wrt: AutogradTensor) -> torch.Tensor:
    if loss.shape() != (1, 1):
        raise HypergradError(f"validation loss must be 1 x 1, got {loss.shape()}")
    return loss.vector_jacobian_product(wrt, torch.ones(1, 1)).torch()


def unrolled(step_fn: Callable, w0: AutogradTensor, hyper: AutogradTensor, data_loader: Iterator, steps: int,
             val_loss_fn: Callable) -> UnrolledOut:
    if steps <= 0:
        raise HypergradError("unrolled_steps must be positive")
    if not hyper.requires_grad():
        raise HypergradError("hyper must require gradients")
    it = iter(data_loader)
    w = w0
    for step in range(steps):
        try:
            batch = next(it)
        except StopIteration:
            raise HypergradError(f"data loader ran out at step {step}") from None
        nxt = step_fn(w, hyper, batch)
        if nxt.shape() != w.shape():
            raise HypergradError(f"step changed the weight shape from {w.shape()} to {nxt.shape()}")
        w = nxt
    return UnrolledOut(w, Tensor._wrap(_scalar_vjp(val_loss_fn(w), hyper)))


def implicit(step_fn: Callable, w0: AutogradTensor, hyper: AutogradTensor, data_loader: Iterator, val_loss_fn: Callable,
             solver: str = "neumann", iterations: int = 32, options: Optional[ImplicitOptions] = None) -> ImplicitOut:
    opt = options or ImplicitOptions(solver=solver, max_iters=iterations)
    opt.validate()
    if not w0.requires_grad() or not hyper.requires_grad():
        raise HypergradError("w0 and hyper must require gradients")
    try:
        batch = next(iter(data_loader))
    except StopIteration:
        raise HypergradError("data loader ran out at step 0") from None
    base = step_fn(w0, hyper, batch)
    if base.shape() != w0.shape():
        raise HypergradError(f"step changed the weight shape from {w0.shape()} to {base.shape()}")
    g = _scalar_vjp(val_loss_fn(w0), w0)

    def vjp_w(v: torch.Tensor) -> torch.Tensor:          # Jᵀ v
        return base.vector_jacobian_product(w0, v).torch()

    def jvp_w(v: torch.Tensor) -> torch.Tensor:          # J v by central differences of the step
        eps = opt.finite_diff_eps
        with torch.no_grad():
            wp = AutogradTensor.constant(w0._t.detach() + eps * v)
            wm = AutogradTensor.constant(w0._t.detach() - eps * v)
            return (step_fn(wp, hyper.detach(), batch)._t - step_fn(wm, hyper.detach(), batch)._t) / (2 * eps)

    requested = opt.solver.lower()
    history: list = []
    fallback = None
    if requested == "neumann":
        v, term = g.clone(), g.clone()
        res = float(term.norm())
        history.append(res)
        it_count = 0
        while it_count < opt.max_iters and res > opt.tolerance:
            term = vjp_w(term)
            v = v + term
            res = float(term.norm())
            if not torch.isfinite(torch.tensor(res)):
                raise HypergradError("implicit Neumann series diverged (the step is not a contraction)")
            history.append(res)
            it_count += 1
        res = float((v - vjp_w(v) - g).norm())
        history.append(res)
        used = "neumann"
    else:
        # normal equations  B Bᵀ v = B g  with  B = I - J  (Bᵀ v = g is the sensitivity equation)
        def B(x):
            return x - jvp_w(x)

        def Bt(x):
            return x - vjp_w(x)

        rhs = B(g)
        v = torch.zeros_like(g)
        r = rhs.clone()
        d = r.clone()
        rs = float((r * r).sum())
        history.append(rs ** 0.5)
        it_count = 0
        while it_count < opt.max_iters and rs ** 0.5 > opt.tolerance:
            Ad = B(Bt(d))
            denom = float((d * Ad).sum())
            if abs(denom) < 1e-30:
                fallback = "cg_breakdown"
                break
            alpha = rs / denom
            v = v + alpha * d
            r = r - alpha * Ad
            rs_new = float((r * r).sum())
            history.append(rs_new ** 0.5)
            d = r + (rs_new / rs) * d
            rs = rs_new
            it_count += 1
        res = float((Bt(v) - g).norm())
        history.append(res)
        used = "cg"
    dval = base.vector_jacobian_product(hyper, v)
    return ImplicitOut(dval, ImplicitDiagnostics(requested, used, it_count, res, history, opt.finite_diff_eps,
                                                 res <= max(opt.tolerance, 1e-3 * float(g.norm())), fallback))
