"""Data side of the self-supervised crate: view-pair sampling, TOML batch configuration, batching into
InfoNCE losses, and the transform pipeline they use (reference behaviour:
crates/spiral-selfsup/src/dataset/mod.rs:74-269, crates/st-vision/src/lib.rs:3404-3540)."""
import math

import pytest
import torch

from spiraltorch_b200 import selfsup as S
from spiraltorch_b200 import vision as V


def _dataset(frames=3, h=4, w=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(frames):
        n = h * w
        out.append(V.MultiViewFrame(torch.zeros(n, 3), torch.randn(n, 3, generator=g), torch.rand(n, 3, generator=g),
                                    torch.tensor([[0.1, 4.0]]).repeat(n, 1)))
    return V.MultiViewDatasetAdapter(out)


def test_colors_to_image_is_channel_major():
    colors = torch.arange(12, dtype=torch.float32).reshape(4, 3)        # 2x2 image, pixel-major RGB rows
    img = S.colors_to_image(colors, 2, 2)
    assert img.shape == (3, 2, 2)
    assert img[0].reshape(-1).tolist() == [0, 3, 6, 9] and img[2, 1, 1].item() == 11
    with pytest.raises(ValueError):
        S.colors_to_image(colors, 3, 2)
    with pytest.raises(ValueError):
        S.colors_to_image(torch.zeros(4, 2), 2, 2)


def test_view_pair_sampler_without_pipeline_returns_identical_views():
    ds = _dataset()
    s = S.ViewPairSampler(ds, 4, 4, seed=5)
    pair = s.sample_pair()
    assert torch.equal(pair.anchor, pair.positive) and pair.anchor.shape == (3, 4, 4)
    # the same seed reproduces the same frame choices
    a = [S.ViewPairSampler(ds, 4, 4, seed=5).sample_pair().anchor for _ in range(2)]
    assert torch.equal(a[0], a[1])
    with pytest.raises(ValueError):
        S.ViewPairSampler(ds, 0, 4)


def test_view_pair_sampler_augments_the_two_views_independently():
    ds = _dataset(frames=1)
    pipe = V.TransformPipeline(1).add(V.RandomColorJitter(0.4, 0.4, 0.4, 0.1)).add(V.RandomHorizontalFlip(0.5))
    s = S.ViewPairSampler(ds, 4, 4, seed=3, pipeline=pipe)
    pairs = [s.sample_pair() for _ in range(6)]
    assert any(not torch.allclose(p.anchor, p.positive) for p in pairs)
    assert all(torch.isfinite(p.anchor).all() and p.anchor.shape == (3, 4, 4) for p in pairs)


def test_batch_config_from_toml():
    cfg = S.InfoNCEBatchConfig.from_toml_str("batch_size = 4\nimage_height = 4\nimage_width = 4\ntemperature = 0.2\nseed = 9\n")
    assert (cfg.batch_size, cfg.normalize, cfg.seed, cfg.temperature) == (4, True, 9, 0.2)
    for bad in ("batch_size = 0\nimage_height = 4\nimage_width = 4\ntemperature = 0.2",
                "batch_size = 2\nimage_height = 4\nimage_width = 4\ntemperature = -1.0",
                "batch_size = 2\nimage_height = 4\ntemperature = 0.5",
                "this is not toml ["):
        with pytest.raises(ValueError):
            S.InfoNCEBatchConfig.from_toml_str(bad)


def test_batcher_shapes_and_loss(tmp_path):
    ds = _dataset(frames=5)
    path = tmp_path / "cfg.toml"
    path.write_text("batch_size = 6\nimage_height = 4\nimage_width = 4\ntemperature = 0.1\nnormalize = true\nseed = 2\n")
    cfg = S.InfoNCEBatchConfig.load(path)
    b = S.InfoNCEBatcher(ds, None, cfg)
    batch = b.sample_batch()
    assert batch.anchors.shape() == (6, 48) and batch.positives.shape() == (6, 48)
    res = b.next_loss()
    # identical views: every positive logit is the row maximum (ties only between copies of one frame)
    assert math.isfinite(res.loss) and 0.0 <= res.top1_accuracy <= 1.0 and res.mean_margin >= -1e-5
    with pytest.raises(ValueError):
        S.InfoNCEBatchConfig.load(tmp_path / "missing.toml")


def test_transform_pipeline_operations():
    img = torch.rand(3, 40, 48)
    pipe = V.standard_classification_pipeline(8, seed=4)
    assert [op.name for op in pipe.operations()] == ["Resize", "CenterCrop", "RandomHorizontalFlip", "Normalize"]
    out = pipe.apply(img)
    assert out.shape == (3, 8, 8)
    again = V.standard_classification_pipeline(8, seed=4).apply(img)
    assert torch.equal(out, again)
    with pytest.raises(ValueError):
        V.Normalize([0.5], [0.0])
    with pytest.raises(ValueError):
        V.RandomColorJitter(hue=0.7)
    with pytest.raises(TypeError):
        V.TransformPipeline().add(object())


def test_multiview_adapter_weights_and_batches():
    ds = _dataset(frames=3)
    ds.set_frame_weights([0.0, 1.0, 0.0])
    g = torch.Generator().manual_seed(0)
    batch = ds.sample_batch(g, 16)
    assert batch["colors"].shape == (16, 3) and batch["bounds"].shape == (16, 2)
    frame1 = ds.frames()[1].colors
    assert all(any(torch.equal(c, row) for row in frame1) for c in batch["colors"])
    with pytest.raises(ValueError):
        ds.set_frame_weights([0.0, 0.0, 0.0])
    with pytest.raises(ValueError):
        V.MultiViewFrame(torch.zeros(4, 3), torch.zeros(4, 3), torch.zeros(4, 2), torch.zeros(4, 2))
