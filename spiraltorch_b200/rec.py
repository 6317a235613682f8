"""Recommenders: matrix factorisation with saturating updates, a user-neighbourhood model and a
damped knowledge-graph walker.

Restated from crates/st-rec/src/lib.rs: ``NeighborhoodModel`` (:86-198, cosine similarity with
additive smoothing), ``KnowledgeGraphRecommender`` (:201-327) and ``SpiralRecommender`` (:329-560:
deterministic sin/cos factor initialisation, per-rating SGD with L2 regularisation, every updated
factor clamped to the topos saturation, RMSE report).  ``recommend_top_k`` ranks with the row
top-k kernel on CUDA tensors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .ops import rank as rank_ops


class SpiralRecError(ValueError):
    pass


@dataclass
class RatingTriple:
    user: int
    item: int
    rating: float


@dataclass
class RecEpochReport:
    rmse: float
    samples: int
    regularization_penalty: float


@dataclass
class Recommendation:
    item: int
    score: float


def _top(scores: torch.Tensor, k: int) -> list:
    k = min(k, scores.numel())
    if k == 0:
        return []
    v, i = rank_ops.rank_select(scores.reshape(1, -1), k, "topk")
    return [Recommendation(int(ii), float(vv)) for vv, ii in zip(v[0].tolist(), i[0].tolist()) if ii >= 0]


class NeighborhoodModel:
    def __init__(self, matrix: torch.Tensor, smoothing: float):
        self.matrix, self.smoothing = matrix, smoothing
        self.users, self.items = matrix.shape

    @classmethod
    def fit(cls, users: int, items: int, ratings: Sequence[RatingTriple], smoothing: float, device="cpu"):
        if users <= 0 or items <= 0:
            raise SpiralRecError(f"invalid dimensions ({users}, {items})")
        if smoothing < 0:
            raise SpiralRecError("smoothing must not be negative")
        total = torch.zeros(users * items, device=device)
        count = torch.zeros(users * items, device=device)
        if ratings:
            u = torch.tensor([r.user for r in ratings])
            i = torch.tensor([r.item for r in ratings])
            if int(u.max()) >= users or int(i.max()) >= items or int(u.min()) < 0 or int(i.min()) < 0:
                bad = next(r for r in ratings if not (0 <= r.user < users and 0 <= r.item < items))
                raise SpiralRecError(f"rating ({bad.user}, {bad.item}) is out of bounds")
            idx = (u * items + i).to(device)
            total.index_add_(0, idx, torch.tensor([r.rating for r in ratings], device=device))
            count.index_add_(0, idx, torch.ones(len(ratings), device=device))
        mat = torch.where(count > 0, total / count.clamp(min=1), total).view(users, items)
        return cls(mat, max(smoothing, 1e-5))

    def recommend(self, user: int, k: int) -> list:
        if not 0 <= user < self.users:
            raise SpiralRecError(f"user {user} is out of bounds")
        if k == 0:
            return []
        target = self.matrix[user]
        norms = self.matrix.norm(dim=1) + self.smoothing
        sim = (self.matrix @ target) / (norms * norms[user]).clamp(min=self.smoothing)
        sim[user] = 0.0
        return _top(sim @ self.matrix, k)


class KnowledgeGraphRecommender:
    """Users and items as graph nodes; a recommendation is the mass that reaches an item after
    ``hops`` damped propagation steps from the user."""

    def __init__(self, users: int, items: int, damping: float):
        if users <= 0 or items <= 0:
            raise SpiralRecError(f"invalid dimensions ({users}, {items})")
        if not 0.0 < damping <= 1.0:
            raise SpiralRecError(f"damping {damping} is outside (0, 1]")
        self.users, self.items, self.damping = users, items, damping
        self.user_item = torch.zeros(users, items)
        self.item_item = torch.zeros(items, items)

    def add_edge(self, kind: str, a: int, b: int, weight: float = 1.0) -> None:
        if not math.isfinite(weight) or weight < 0:
            raise SpiralRecError("edge weight must be finite and non-negative")
        if kind == "user_item":
            if not (0 <= a < self.users and 0 <= b < self.items):
                raise SpiralRecError(f"edge ({a}, {b}) is out of bounds")
            self.user_item[a, b] += weight
        elif kind == "item_item":
            if not (0 <= a < self.items and 0 <= b < self.items):
                raise SpiralRecError(f"edge ({a}, {b}) is out of bounds")
            self.item_item[a, b] += weight
            self.item_item[b, a] += weight
        else:
            raise SpiralRecError(f"unknown edge kind '{kind}'")

    def item_degree(self, item: int) -> int:
        if not 0 <= item < self.items:
            raise SpiralRecError(f"item {item} is out of bounds")
        return int((self.item_item[item] > 0).sum() + (self.user_item[:, item] > 0).sum())

    def recommend(self, user: int, k: int, hops: int) -> list:
        if not 0 <= user < self.users:
            raise SpiralRecError(f"user {user} is out of bounds")
        mass = self.user_item[user].clone()
        total = mass.clone()
        for _ in range(max(0, hops)):
            mass = self.damping * (mass @ self.item_item)
            total += mass
        total[self.user_item[user] > 0] = -math.inf           # already known to the user
        return [r for r in _top(total, k) if math.isfinite(r.score) and r.score > 0.0]   # unreachable items are not offered


class SpiralRecommender:
    SATURATION = 64.0

    def __init__(self, users: int, items: int, factors: int, learning_rate: float, regularization: float,
                 curvature: float = -1.0, device="cpu"):
        if users <= 0 or items <= 0 or factors <= 0:
            raise SpiralRecError(f"invalid dimensions ({users}, {items}, {factors})")
        if learning_rate <= 0:
            raise SpiralRecError(f"learning rate must be positive, got {learning_rate}")
        if regularization < 0:
            raise SpiralRecError("regularization must not be negative")
        if not curvature < 0:
            raise SpiralRecError("curvature must be negative")
        f = torch.arange(1, factors + 1, dtype=torch.float32)[None, :]
        self.user_factors = (torch.sin(torch.arange(1, users + 1, dtype=torch.float32)[:, None] * f) * 0.05).to(device)
        self.item_factors = (torch.cos(torch.arange(1, items + 1, dtype=torch.float32)[:, None] * f) * 0.05).to(device)
        self._users, self._items, self._factors = users, items, factors
        self.learning_rate, self.regularization, self.curvature = learning_rate, regularization, curvature

    def users(self) -> int:
        return self._users

    def items(self) -> int:
        return self._items

    def factors(self) -> int:
        return self._factors

    def _guard(self, user: int, item: int) -> None:
        if not (0 <= user < self._users and 0 <= item < self._items):
            raise SpiralRecError(f"rating ({user}, {item}) is out of bounds")

    def predict(self, user: int, item: int) -> float:
        self._guard(user, item)
        return float(self.user_factors[user] @ self.item_factors[item])

    def user_embedding(self, user: int) -> torch.Tensor:
        self._guard(user, 0)
        return self.user_factors[user:user + 1].clone()

    def item_embedding(self, item: int) -> torch.Tensor:
        self._guard(0, item)
        return self.item_factors[item:item + 1].clone()

    def train_epoch(self, ratings: Sequence[RatingTriple]) -> RecEpochReport:
        """One pass of per-rating SGD in the given order (later ratings see earlier updates)."""
        if not ratings:
            raise SpiralRecError("empty rating batch")
        for r in ratings:
            self._guard(r.user, r.item)
        U, I = self.user_factors.cpu().clone(), self.item_factors.cpu().clone()
        lr, reg, sat = self.learning_rate, self.regularization, self.SATURATION
        sq, pen = 0.0, 0.0
        for r in ratings:
            u, i = U[r.user].clone(), I[r.item].clone()
            diff = float(u @ i) - r.rating
            sq += diff * diff
            U[r.user] = (u - lr * (diff * i + reg * u)).clamp(-sat, sat)
            I[r.item] = (i - lr * (diff * u + reg * i)).clamp(-sat, sat)
            pen += reg * float((u * u + i * i).sum())
        if not (torch.isfinite(U).all() and torch.isfinite(I).all()):
            raise SpiralRecError("non-finite factors after the epoch")
        self.user_factors.copy_(U)
        self.item_factors.copy_(I)
        return RecEpochReport(math.sqrt(sq / len(ratings)), len(ratings), pen / len(ratings))

    def recommend_top_k(self, user: int, k: int, exclude: Optional[Sequence[int]] = None) -> list:
        if k == 0:
            return []
        self._guard(user, 0)
        scores = self.item_factors @ self.user_factors[user]
        if exclude:
            scores = scores.clone()
            scores[torch.tensor(list(exclude), device=scores.device)] = float("nan")   # non-finite entries are skipped
        return _top(scores, k)
