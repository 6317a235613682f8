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


# ------------------------------------------------------------------------------------------------------
# Data side: augmented view pairs from a multi-view dataset, batching, TOML configuration.
# Reference: ViewPair / ViewPairSampler / InfoNCEBatchConfig / InfoNCEBatcher
# (crates/spiral-selfsup/src/dataset/mod.rs:12-269).
# ------------------------------------------------------------------------------------------------------
@dataclass
class ViewPair:
    anchor: torch.Tensor        # [3, H, W]
    positive: torch.Tensor


def colors_to_image(colors: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """Per-ray RGB rows ``[H*W, 3]`` (row-major pixels) → image ``[3, H, W]``."""
    if height <= 0 or width <= 0:
        raise ValueError("image dimensions must be > 0")
    if colors.dim() != 2 or colors.shape[1] != 3:
        raise ValueError(f"expected RGB colors with 3 columns, found {tuple(colors.shape)}")
    if colors.shape[0] != height * width:
        raise ValueError(f"color rows ({colors.shape[0]}) do not match target image size {height}x{width}")
    return colors.t().reshape(3, height, width).contiguous()


class ViewPairSampler:
    """Draws a frame, turns its colours into an image and augments it twice with independently reseeded copies
    of the pipeline's operations."""

    def __init__(self, dataset, image_height: int, image_width: int, seed: Optional[int] = None, pipeline=None):
        from .config import determinism
        if dataset.num_frames() == 0:
            raise ValueError("dataset must contain at least one frame")
        if image_height <= 0 or image_width <= 0:
            raise ValueError("image dimensions must be > 0")
        self.dataset, self.image_height, self.image_width = dataset, image_height, image_width
        label = f"spiral-selfsup/view_pair_sampler:{dataset.num_frames()}:{image_height}:{image_width}"
        self._gen = torch.Generator()
        self._gen.manual_seed(determinism.resolve_seed(seed, label))
        self.operations = [] if pipeline is None else pipeline.operations()

    def _augment(self, img: torch.Tensor) -> torch.Tensor:
        if not self.operations:
            return img
        from .vision import TransformPipeline
        pipe = TransformPipeline(int(torch.randint(0, 2 ** 62, (), generator=self._gen)))
        for op in self.operations:
            pipe.add(op)
        return pipe.apply(img)

    def sample_pair(self) -> ViewPair:
        n = self.dataset.num_frames()
        idx = 0 if n <= 1 else int(torch.randint(0, n, (), generator=self._gen))
        base = colors_to_image(self.dataset.frames()[idx].colors, self.image_height, self.image_width)
        return ViewPair(self._augment(base.clone()), self._augment(base))


@dataclass
class InfoNCEBatchConfig:
    batch_size: int
    image_height: int
    image_width: int
    temperature: float
    normalize: bool = True
    seed: Optional[int] = None

    def validate(self) -> None:
        if self.batch_size <= 0:
            raise ValueError("batch_size must be > 0")
        if self.image_height <= 0 or self.image_width <= 0:
            raise ValueError("image dimensions must be > 0")
        if not (self.temperature > 0 and self.temperature == self.temperature and self.temperature != float("inf")):
            raise ValueError(f"temperature must be > 0, got {self.temperature}")

    @classmethod
    def from_toml_str(cls, text: str) -> "InfoNCEBatchConfig":
        import tomllib
        try:
            data = tomllib.loads(text)
            cfg = cls(int(data["batch_size"]), int(data["image_height"]), int(data["image_width"]),
                      float(data["temperature"]), bool(data.get("normalize", True)),
                      None if data.get("seed") is None else int(data["seed"]))
        except (tomllib.TOMLDecodeError, KeyError, TypeError, ValueError) as exc:
            raise ValueError(f"failed to parse InfoNCE batch config: {exc}") from exc
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, path) -> "InfoNCEBatchConfig":
        try:
            with open(path, "r", encoding="utf-8") as f:
                text = f.read()
        except OSError as exc:
            raise ValueError(f"failed to read InfoNCE batch config {path}: {exc}") from exc
        return cls.from_toml_str(text)


@dataclass
class InfoNCEBatch:
    anchors: Tensor
    positives: Tensor


class InfoNCEBatcher:
    """Dataset sampling → augmentation → ``[batch, 3*H*W]`` anchor / positive matrices → InfoNCE loss."""

    def __init__(self, dataset, pipeline, config: InfoNCEBatchConfig):
        config.validate()
        self.config = config
        self.sampler = ViewPairSampler(dataset, config.image_height, config.image_width, config.seed, pipeline)

    def sample_batch(self) -> InfoNCEBatch:
        anchors, positives = [], []
        dim = None
        for _ in range(self.config.batch_size):
            pair = self.sampler.sample_pair()
            a, p = pair.anchor.reshape(-1), pair.positive.reshape(-1)
            if a.numel() != p.numel():
                raise ValueError(f"anchor/positive feature mismatch (anchor={a.numel()}, positive={p.numel()})")
            if dim is not None and dim != a.numel():
                raise ValueError(f"inconsistent feature dims across batch: expected {dim}, got {a.numel()}")
            dim = a.numel()
            anchors.append(a)
            positives.append(p)
        return InfoNCEBatch(Tensor(torch.stack(anchors)), Tensor(torch.stack(positives)))

    def next_loss(self) -> InfoNCEResult:
        batch = self.sample_batch()
        return info_nce(batch.anchors, batch.positives, self.config.temperature, self.config.normalize)
