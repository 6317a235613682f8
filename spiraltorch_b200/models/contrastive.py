"""Self-supervised contrastive encoder: MLP 512 → 2048 → 2048 → 256 with LayerNorm + GELU, output
L2-normalised, trained with InfoNCE (temperature 0.1) on two noisy views of the same base vectors.

Layers run on the sm_100a kernels through the autograd wrappers (``ops.gemm.linear``,
``ops.norm.layer_norm``, ``ops.elementwise.gelu``).  On several GPUs the loss is
:class:`spiraltorch_b200.parallel.contrastive.FusedInfoNCE` (embeddings of all ranks gathered
inside the similarity kernel).

Reference: crates/spiral-selfsup (objectives and the self-sup trainer, crates/st-nn/src/trainer/
selfsup.rs:591-706) and docs/benchmarks/selfsup.md for the expected metric ranges.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import elementwise as ew
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from ..selfsup import info_nce_torch


class ContrastiveEncoder(nn.Module):
    def __init__(self, in_dim: int = 512, hidden: int = 2048, out_dim: int = 256, device="cuda",
                 dtype=torch.bfloat16, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        dims = [in_dim, hidden, hidden, out_dim]
        self.weights = nn.ParameterList()
        self.biases = nn.ParameterList()
        self.gammas = nn.ParameterList()
        self.betas = nn.ParameterList()
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            self.weights.append(nn.Parameter((torch.randn(b, a, generator=g) * math.sqrt(1.0 / a)).to(device, dtype)))
            self.biases.append(nn.Parameter(torch.zeros(b, device=device, dtype=dtype)))
            if i < 2:
                self.gammas.append(nn.Parameter(torch.ones(b, device=device, dtype=dtype)))
                self.betas.append(nn.Parameter(torch.zeros(b, device=device, dtype=dtype)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = x.to(self.weights[0].dtype)
        for i in range(3):
            h = gemm_ops.linear(h, self.weights[i], self.biases[i])
            if i < 2:
                h = ew.gelu(norm_ops.layer_norm(h, self.gammas[i], self.betas[i], 1e-5))
        hf = h.float()
        return hf / hf.norm(dim=-1, keepdim=True).clamp(min=1e-12)


def make_views(base: torch.Tensor, noise: float = 0.1, seed: Optional[int] = None):
    g = None
    if seed is not None:
        g = torch.Generator(device=base.device).manual_seed(seed)
    n1 = torch.randn(base.shape, generator=g, device=base.device, dtype=base.dtype)
    n2 = torch.randn(base.shape, generator=g, device=base.device, dtype=base.dtype)
    return base + noise * n1, base + noise * n2


def contrastive_step(encoder: ContrastiveEncoder, base: torch.Tensor, temperature: float = 0.1,
                     fused_loss=None, noise: float = 0.1, seed: Optional[int] = None) -> torch.Tensor:
    """Forward + backward of one batch; returns the loss (gradients are in ``.grad``)."""
    v1, v2 = make_views(base, noise, seed)
    za, zp = encoder(v1), encoder(v2)
    if fused_loss is not None:
        loss = fused_loss.apply(za, zp)
    else:
        loss, _ = info_nce_torch(za, zp, temperature, normalize=False)
    loss.backward()
    return loss.detach()
