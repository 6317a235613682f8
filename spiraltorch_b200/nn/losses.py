"""Losses with the reference protocol: ``forward(pred, target) -> (1,1) Tensor`` and
``backward(pred, target) -> gradient Tensor`` (crates/st-nn/src/loss/mod.rs:26-32).

* ``MeanSquaredError``: mean over all elements, gradient ``2/(rows*cols)*(pred-target)``
  (loss/mean_squared_error.rs:60-93).
* ``CategoricalCrossEntropy``: expects probabilities, clamps with ``epsilon`` (1e-9), mean over rows
  (loss/categorical_cross_entropy.rs:13-36).
* ``HyperbolicCrossEntropy`` (= ``CrossEntropy``): element-wise sigmoid BCE on ``logits*sqrt(-c)`` with
  targets clamped to ``[eps, 1-eps]``, mean over all elements (loss/hyperbolic_cross_entropy.rs:160-178).
* ``FocalLoss``, ``ContrastiveLoss`` (on distances), ``TripletLoss``.
* ``SoftmaxCrossEntropy``: logits + integer/one-hot targets on the fused CUDA kernel (new).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from ..tensor import Tensor, TensorError
from .modules import assert_finite


class Loss:
    def _value(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def _check(self, pred: Tensor, target: Tensor):
        if pred.shape() != target.shape():
            raise TensorError(f"loss: shape mismatch {pred.shape()} vs {target.shape()}")
        p, t = pred.torch(), target.torch()
        assert_finite([p, t], lambda i: "loss: non-finite input")
        return p, t

    def forward(self, pred: Tensor, target: Tensor) -> Tensor:
        p, t = self._check(pred, target)
        if p.numel() == 0:
            return Tensor(1, 1, [0.0])
        with torch.no_grad():
            return Tensor._wrap(self._value(p, t).reshape(1, 1))

    __call__ = forward

    def backward(self, pred: Tensor, target: Tensor) -> Tensor:
        p, t = self._check(pred, target)
        if p.numel() == 0:
            return Tensor._wrap(torch.zeros_like(p))
        x = p.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            (g,) = torch.autograd.grad(self._value(x, t), x)
        return Tensor._wrap(g)


class MeanSquaredError(Loss):
    def _value(self, p, t):
        return (p - t).pow(2).mean()


class CategoricalCrossEntropy(Loss):
    def __init__(self, *, epsilon: Optional[float] = None):
        self.epsilon = 1e-9 if epsilon is None else float(epsilon)

    def _value(self, p, t):
        return -(t * torch.log(p.clamp(min=self.epsilon))).sum() / p.shape[0]


class HyperbolicCrossEntropy(Loss):
    def __init__(self, curvature: float = -1.0, *, epsilon: Optional[float] = None):
        if not (curvature < 0 and math.isfinite(curvature)):
            raise ValueError(f"non-hyperbolic curvature {curvature}")
        self.curvature = float(curvature)
        self.epsilon = 1e-5 if epsilon is None else float(epsilon)

    def _value(self, p, t):
        z = p * math.sqrt(-self.curvature)
        tt = t.clamp(self.epsilon, 1 - self.epsilon)
        return (tt * F.softplus(-z) + (1 - tt) * F.softplus(z)).mean()


CrossEntropy = HyperbolicCrossEntropy


class FocalLoss(Loss):
    def __init__(self, alpha: float = 0.25, gamma: float = 2.0, *, epsilon: Optional[float] = None):
        self.alpha, self.gamma = float(alpha), float(gamma)
        self.epsilon = 1e-6 if epsilon is None else float(epsilon)

    def _value(self, p, t):
        tt = t.clamp(0, 1)
        prob = p.clamp(self.epsilon, 1 - self.epsilon)
        pos = tt > 0.5
        pt = torch.where(pos, prob, 1 - prob)
        a = torch.where(pos, torch.full_like(p, self.alpha), torch.full_like(p, 1 - self.alpha))
        return (-a * (1 - pt).pow(self.gamma) * torch.log(pt)).mean()


class ContrastiveLoss(Loss):
    """``pred`` holds pair distances, ``target`` the similarity labels in [0, 1]."""

    def __init__(self, margin: float = 1.0):
        self.margin = max(0.0, margin) if math.isfinite(margin) else 0.0

    def _value(self, p, t):
        lab = t.clamp(0, 1)
        return (lab * p.pow(2) + (1 - lab) * torch.relu(self.margin - p).pow(2)).mean()


class TripletLoss(Loss):
    """``pred`` columns = (d(anchor, positive), d(anchor, negative)); target is ignored."""

    def __init__(self, margin: float = 1.0):
        self.margin = max(0.0, margin) if math.isfinite(margin) else 0.0

    def _value(self, p, t):
        if p.shape[1] < 2:
            raise TensorError("TripletLoss expects at least two distance columns")
        return torch.relu(p[:, 0] - p[:, 1] + self.margin).mean()


class SoftmaxCrossEntropy(Loss):
    """Mean softmax cross-entropy on logits; ``target`` is one-hot / soft ``(rows, classes)`` or a
    column of class ids ``(rows, 1)``.  CUDA inputs with hard labels use the fused kernels."""

    def _check(self, pred, target):
        p, t = pred.torch(), target.torch()
        if t.shape[0] != p.shape[0] or t.shape[1] not in (1, p.shape[1]):
            raise TensorError("SoftmaxCrossEntropy: target must be (rows, 1) ids or (rows, classes)")
        return p, t

    def _value(self, p, t):
        if t.shape[1] == 1 and p.shape[1] != 1:
            return F.cross_entropy(p, t.reshape(-1).long())
        return -(t * torch.log_softmax(p, -1)).sum(-1).mean()
