"""Self-supervised objectives: InfoNCE and masked MSE.

``info_nce`` restates crates/spiral-selfsup/src/contrastive.rs:96-153: rows of ``anchors`` and
``positives`` are L2-normalised (optional), logits are ``anchor · positiveᵀ / temperature``, the
loss is the mean over rows of ``logsumexp(row) − row[i]``; the report also carries top-1
accuracy and the mean margin between the positive logit and the best negative.
``masked_mse`` restates crates/spiral-selfsup/src/masked.rs:48.

On several GPUs :func:`spiraltorch_b200.parallel.contrastive.fused_info_nce` computes the same
loss against the embeddings of all ranks inside one kernel (all-gather + similarity GEMM +
row softmax).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .tensor import Tensor


@dataclass
class InfoNCEResult:
    loss: float
    top1_accuracy: float
    mean_margin: float
    logits: Optional[torch.Tensor] = None


def info_nce_torch(anchors: torch.Tensor, positives: torch.Tensor, temperature: float = 0.1,
                   normalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Differentiable loss and the logits matrix."""
    if anchors.shape[0] != positives.shape[0] or anchors.shape[1] != positives.shape[1]:
        raise ValueError(f"info_nce: shape mismatch {tuple(anchors.shape)} vs {tuple(positives.shape)}")
    if not temperature > 0:
        raise ValueError("info_nce: temperature must be positive")
    a, p = anchors.float(), positives.float()
    if normalize:
        a = torch.nn.functional.normalize(a, dim=-1, eps=1e-12)
        p = torch.nn.functional.normalize(p, dim=-1, eps=1e-12)
    logits = a @ p.t() / temperature
    idx = torch.arange(a.shape[0], device=a.device)
    loss = (torch.logsumexp(logits, dim=-1) - logits[idx, idx]).mean()
    return loss, logits


def info_nce(anchors, positives, temperature: float = 0.1, normalize: bool = True) -> InfoNCEResult:
    a = anchors.torch() if isinstance(anchors, Tensor) else torch.as_tensor(anchors, dtype=torch.float32)
    p = positives.torch() if isinstance(positives, Tensor) else torch.as_tensor(positives, dtype=torch.float32)
    with torch.no_grad():
        loss, logits = info_nce_torch(a, p, temperature, normalize)
        n = logits.shape[0]
        idx = torch.arange(n, device=logits.device)
        pos = logits[idx, idx]
        neg = logits.clone()
        neg[idx, idx] = float("-inf")
        best_neg = neg.max(dim=-1).values if n > 1 else torch.zeros_like(pos)
        top1 = (logits.argmax(dim=-1) == idx).float().mean()
        margin = (pos - best_neg).mean() if n > 1 else pos.mean()
    return InfoNCEResult(float(loss), float(top1), float(margin), logits)


def masked_mse(predictions, targets, mask_indices: Sequence[Sequence[int]]) -> float:
    """Mean squared error over the masked positions of each row."""
    p = predictions.torch() if isinstance(predictions, Tensor) else torch.as_tensor(predictions, dtype=torch.float32)
    t = targets.torch() if isinstance(targets, Tensor) else torch.as_tensor(targets, dtype=torch.float32)
    if p.shape != t.shape or len(mask_indices) != p.shape[0]:
        raise ValueError("masked_mse: shape mismatch")
    total, count = 0.0, 0
    for r, idxs in enumerate(mask_indices):
        for c in idxs:
            if not 0 <= c < p.shape[1]:
                raise IndexError(f"mask index {c} out of range for row {r}")
            total += float((p[r, c] - t[r, c]) ** 2)
            count += 1
    return total / count if count else 0.0
