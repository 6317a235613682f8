"""Optimizers over a model's flat parameter buffer (one fused kernel launch per range).

``FlatAdamW`` keeps fp32 master weights and Adam moments next to the model's flat bf16
weights and fp32 gradient buffer.  A step is: (tensor-parallel) sum of the replicated
gradients → global gradient norm on the device → clip coefficient on the device → fused
AdamW that also writes the bf16 working weights and zeroes the gradient buffer.  Nothing in
the step synchronises with the host.

``FlatSGD`` is the SGD-momentum twin used by the convolutional classifier.

Reference parity: the reference has no AdamW (Adam exists only inside ``ZSpaceVae``,
crates/st-nn/src/zspace_coherence/vae.rs:303-334); the step order (synchronise → clip →
apply) follows ``ModuleTrainer::step`` (crates/st-nn/src/trainer.rs:7259-7268).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import optim as K


class _FlatBase:
    def __init__(self, model, max_grad_norm: float = 0.0):
        self.model = model
        self.w = model.flat_w
        self.grad = model.flat_grad
        self.decay_elems = getattr(model, "decay_elems", self.w.numel())
        self.max_grad_norm = max_grad_norm
        dev = self.w.device
        self.master = self.w.float().clone()
        self._sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.step_count = 0

    def _ranges(self):
        n, d = self.w.numel(), self.decay_elems
        out = []
        if d > 0:
            out.append((0, d, True))
        if n > d:
            out.append((d, n, False))
        return out

    def _prepare(self, grad_scale: float) -> Optional[torch.Tensor]:
        """Sync replicated grads, compute the clip coefficient (device scalar)."""
        model = self.model
        if hasattr(model, "sync_replicated_grads"):
            model.sync_replicated_grads()
        if self.max_grad_norm <= 0:
            return None
        tp = getattr(model, "tp", None)
        self._sumsq.zero_()
        d = self.decay_elems
        K.sumsq(self.grad[:d], self._sumsq[0:1])
        if tp is not None and tp.world > 1:
            tp.all_reduce_(self._sumsq[0:1])
        if self.grad.numel() > d:
            K.sumsq(self.grad[d:], self._sumsq[1:2])
        total = self._sumsq.sum().reshape(1)
        K.clip_coef(total, grad_scale, self.max_grad_norm, self._coef, self.grad_norm)
        return self._coef


class FlatAdamW(_FlatBase):
    def __init__(self, model, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0):
        super().__init__(model, max_grad_norm)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)

    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        """Apply one update; ``grad_scale`` multiplies the accumulated gradient first."""
        self.step_count += 1
        coef = self._prepare(grad_scale)
        for lo, hi, decay in self._ranges():
            K.adamw_step(self.grad[lo:hi], self.master[lo:hi], self.m[lo:hi], self.v[lo:hi], self.w[lo:hi],
                         lr=self.lr if lr is None else lr, beta1=self.betas[0], beta2=self.betas[1],
                         eps=self.eps, weight_decay=self.weight_decay if decay else 0.0,
                         step=self.step_count, grad_scale=grad_scale, scale_tensor=coef, zero_grad=True)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.w.copy_(self.master.to(self.w.dtype))


class FlatSGD(_FlatBase):
    def __init__(self, model, lr: float = 0.1, momentum: float = 0.9, weight_decay: float = 0.0,
                 nesterov: bool = False, max_grad_norm: float = 0.0):
        super().__init__(model, max_grad_norm)
        self.lr, self.momentum, self.weight_decay, self.nesterov = lr, momentum, weight_decay, nesterov
        self.buf = torch.zeros_like(self.master) if momentum > 0 else None

    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        self.step_count += 1
        coef = self._prepare(grad_scale)
        for lo, hi, decay in self._ranges():
            K.sgd_step(self.grad[lo:hi], self.master[lo:hi], None if self.buf is None else self.buf[lo:hi],
                       self.w[lo:hi], lr=self.lr if lr is None else lr, momentum=self.momentum,
                       weight_decay=self.weight_decay if decay else 0.0, nesterov=self.nesterov,
                       grad_scale=grad_scale, scale_tensor=coef, zero_grad=True)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "momentum": self.buf}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        if self.buf is not None and sd.get("momentum") is not None:
            self.buf.copy_(sd["momentum"])
        self.w.copy_(self.master.to(self.w.dtype))
