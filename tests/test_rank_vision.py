"""Rank selection, compaction, image transforms, NeRF compositing, canvas and fractional stencil:
CPU statements against hand-computed cases, CUDA kernels against the CPU statements."""
import math

import pytest
import torch

from spiraltorch_b200 import frac, vision
from spiraltorch_b200.ops import rank as R

NAN = float("nan")


def _dev_params():
    return ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("dev", _dev_params())
def test_rank_selection_reference_cases(dev):
    x = torch.tensor([[NAN, 4.0, float("inf"), 3.0, -2.0, 5.0]], device=dev)
    v, i = R.topk(x, 3)
    assert v.tolist() == [[5.0, 4.0, 3.0]] and i.tolist() == [[5, 1, 3]]          # non-finite ignored
    v, i = R.bottomk(x, 2)
    assert v.tolist() == [[-2.0, 3.0]] and i.tolist() == [[4, 3]]
    t = torch.tensor([[2.0, 7.0, 7.0, 1.0, 7.0]], device=dev)
    assert R.topk(t, 2)[1].tolist() == [[1, 2]]                                   # ties: lower index first
    assert R.bottomk(torch.tensor([[1.0, 0.0, 0.0]], device=dev), 2)[1].tolist() == [[1, 2]]
    m = torch.tensor([[9.0, 1.0, 5.0, 3.0, 7.0, NAN]], device=dev)
    v, i = R.midk(m, 3)
    assert v.tolist() == [[3.0, 5.0, 7.0]] and i.tolist() == [[3, 2, 4]]          # centred in ascending order
    few = torch.tensor([[NAN, 2.0, NAN, 1.0]], device=dev)
    v, i = R.topk(few, 3)
    assert v[0, :2].tolist() == [2.0, 1.0] and math.isnan(v[0, 2].item()) and i.tolist() == [[1, 3, -1]]
    v, i = R.topk(torch.tensor([[3.0, 9.0, 9.0]], device=dev), 1)
    assert v.tolist() == [[9.0]] and i.tolist() == [[1]]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,k", [(7, 50, 5), (33, 1000, 64), (4, 8192, 1024), (16, 4096, 1), (3, 129, 129)])
def test_rank_kernels_match_cpu(rows, cols, k):
    torch.manual_seed(0)
    x = torch.randn(rows, cols)
    x[0, :3] = float("nan")
    x[:, 5] = x[:, 6]                       # ties
    for kind in ("topk", "bottomk", "midk"):
        cv, ci = R.rank_select(x, k, kind)
        gv, gi = R.rank_select(x.cuda(), k, kind)
        assert torch.equal(ci, gi.cpu()), kind
        assert torch.equal(torch.nan_to_num(cv, nan=-7.0), torch.nan_to_num(gv.cpu(), nan=-7.0))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,k", [(5, 50304, 40), (3, 20000, 1), (2, 9000, 2500), (2, 70000, 5000)])
def test_rank_two_stage_for_wide_rows_matches_cpu(rows, cols, k):
    """Rows wider than one CTA's shared-memory sort (a 50,304-wide vocabulary row) stay on the kernel: select per
    column chunk, then among the candidates; values, indices and the lower-column tie rule must match the CPU path."""
    torch.manual_seed(1)
    x = torch.randn(rows, cols)
    x[0, 100:110] = float("nan")
    x[:, 8191] = x[:, 8193] = x[:, 17] = 9.0          # ties across chunk boundaries, all in the top
    before = R.launch_count
    for kind in ("topk", "bottomk"):
        cv, ci = R.rank_select(x, k, kind)
        gv, gi = R.rank_select(x.cuda(), k, kind)
        assert torch.equal(ci, gi.cpu()), kind
        assert torch.equal(torch.nan_to_num(cv, nan=-7.0), torch.nan_to_num(gv.cpu(), nan=-7.0))
    assert R.launch_count - before >= 4               # two stages per call, on the kernel
    assert R.plan_rank("topk", rows, cols, k, backend="cuda").kernel.startswith("two_stage")


@pytest.mark.parametrize("dev", _dev_params())
def test_compaction(dev):
    x = torch.tensor([[0.1, 5.0, 0.3, NAN, 0.2, -1.0], [9.0, 9.0, 9.0, 9.0, 9.0, 9.0]], device=dev)
    v, i, n = R.compact_rows(x, 0.0, 1.0)
    assert n.tolist() == [3, 0]
    assert torch.allclose(v[0, :3].cpu(), torch.tensor([0.1, 0.3, 0.2])) and i[0, :3].tolist() == [0, 2, 4]
    assert v[0, 3:].abs().sum().item() == 0 and v[1].abs().sum().item() == 0 and i[1].sum().item() == 0
    with pytest.raises(ValueError):
        R.compact_rows(x, 1.0, 0.0)
    if dev == "cuda":
        big = torch.randn(37, 1000)
        cv, ci, cn = R.compact_rows(big, -0.5, 0.25)
        gv, gi, gn = R.compact_rows(big.cuda(), -0.5, 0.25)
        assert torch.equal(cn, gn.cpu()) and torch.equal(ci, gi.cpu()) and torch.equal(cv, gv.cpu())


def test_merge_topk_shards_and_plan():
    torch.manual_seed(1)
    x = torch.randn(5, 64)
    x[:, 40] = x[:, 3]                      # a tie across shards
    shards = x.chunk(4, dim=1)
    vs, ids = [], []
    for s, sh in enumerate(shards):
        v, i = R.topk(sh, 6)
        vs.append(v)
        ids.append(i + s * 16)
    mv, mi = R.merge_topk_shards(torch.cat(vs, 1), torch.cat(ids, 1), 6)
    rv, ri = R.topk(x, 6)
    assert torch.equal(mi, ri) and torch.equal(mv, rv)
    assert torch.equal(R.distributed_topk(x, 6, group=False)[1], ri)
    plan = R.plan_rank("topk", 128, 4096, 32, backend="cuda")
    assert plan.kernel == "smem_bitonic" and plan.shared_bytes == 4096 * 8
    assert R.plan_rank("topk", 4, 512, 1, backend="cuda").kernel == "block_argmax"
    assert R.plan_rank("midk", 4, 100000, 8, backend="cuda").backend == "cpu"
    with pytest.raises(ValueError):
        R.plan_rank("topk", 1, 4, 8)


@pytest.mark.parametrize("dev", _dev_params())
def test_transforms(dev):
    torch.manual_seed(2)
    img = torch.rand(2, 3, 32, 48, device=dev)
    same = vision.resize(img, 32, 48)
    assert torch.allclose(same, img)
    down = vision.resize(img, 16, 24)
    ref = torch.nn.functional.interpolate(img.cpu(), size=(16, 24), mode="bilinear", align_corners=False)
    assert torch.allclose(down.cpu(), ref, atol=1e-5)                              # interior == half-pixel bilinear
    crop = vision.center_crop(img, 16, 20)
    assert torch.equal(crop, img[:, :, 8:24, 14:34])
    assert torch.equal(vision.horizontal_flip(img), img.flip(-1))
    j = vision.ColorJitter(brightness=1.2, contrast=0.8, saturation=1.5, hue=0.3, means=[0.4, 0.5, 0.6])
    out = vision.color_jitter(img, j)
    assert torch.allclose(out.cpu(), vision._jitter_ref(img.cpu(), j, [0.4, 0.5, 0.6, 0.0]), atol=1e-5)
    ident = vision.color_jitter(img, vision.ColorJitter())
    assert torch.allclose(ident, img, atol=1e-6)
    fused = vision.classification_pipeline(img, size=20, resize_to=24, jitter=j, flip=True)
    step = vision.horizontal_flip(vision.color_jitter(vision.center_crop(vision.resize(img, 24, 24), 20, 20), j))
    assert fused.shape == (2, 3, 20, 20) and torch.allclose(fused, step, atol=1e-5)
    assert vision.resize(img[0], 8, 8).shape == (3, 8, 8)
    with pytest.raises(ValueError):
        vision.center_crop(img, 64, 64)


@pytest.mark.parametrize("dev", _dev_params())
def test_nerf_sampling_compositing_and_canvas(dev):
    torch.manual_seed(3)
    Rn, S = 33, 17
    rays = torch.cat([torch.randn(Rn, 3), torch.nn.functional.normalize(torch.randn(Rn, 3), dim=-1),
                      torch.full((Rn, 1), 0.5), torch.full((Rn, 1), 4.0)], 1).to(dev)
    pts, t, d = vision.nerf_sample(rays, S)
    cp, ct, cd = vision.nerf_sample(rays.cpu(), S)
    assert torch.allclose(pts.cpu(), cp, atol=1e-5) and torch.allclose(d.cpu(), cd, atol=1e-5)
    assert torch.allclose(t[:, 0].cpu(), torch.full((Rn,), 0.5 + 0.5 * 3.5 / S), atol=1e-5)
    st_pts, _, st_d = vision.nerf_sample(rays, S, stratified=True, seed=4)
    assert (st_d > 0).all() and not torch.allclose(st_pts, pts)
    sigma = torch.randn(Rn, S, device=dev).requires_grad_(True)
    rad = torch.rand(Rn, S, 3, device=dev).requires_grad_(True)
    acc = vision.nerf_composite(sigma, rad, d)
    g = torch.randn(Rn, 4, device=dev)
    acc.backward(g)
    s2, r2 = sigma.detach().cpu().clone().requires_grad_(True), rad.detach().cpu().clone().requires_grad_(True)
    ref = vision._composite_ref(s2, r2, d.cpu(), 1.0)
    ref.backward(g.cpu())
    assert torch.allclose(acc.detach().cpu(), ref.detach(), atol=1e-5)
    assert torch.allclose(sigma.grad.cpu(), s2.grad, atol=1e-4) and torch.allclose(rad.grad.cpu(), r2.grad, atol=1e-5)
    assert (acc[:, 3] <= 1.0 + 1e-5).all()
    x = torch.linspace(-1, 1, 64, device=dev).reshape(8, 8)
    for pal in vision.PALETTES:
        img = vision.canvas_paint(x, pal)
        assert img.shape == (8, 8, 4) and img.dtype == torch.uint8 and (img[..., 3] == 255).all()
        assert torch.equal(img.cpu(), vision.canvas_paint(x.cpu(), pal))
    gray = vision.canvas_paint(x, "grayscale")
    assert gray[0, 0, 0].item() == 0 and gray[7, 7, 0].item() == 255
    vol = torch.rand(5, 6, 7, device=dev)
    assert vision.temporal_volume_render(vol).shape == (6, 7, 4)
    f = vision.canvas_fft(torch.rand(4, 8, device=dev), "row")
    assert f.shape == (4, 8) and torch.is_complex(f)
    field = vision.NerfField(hidden=16, frequencies=2, layers=2).to(dev)
    assert vision.nerf_render(field, rays, samples=8).shape == (Rn, 4)


@pytest.mark.parametrize("dev", _dev_params())
def test_fractional_gl(dev):
    w = frac.gl_coeffs(0.5, 4)
    assert torch.allclose(w, torch.tensor([1.0, -0.5, -0.125, -0.0625, -0.0390625]))
    assert torch.allclose(frac.gl_coeffs(1.0, 3), torch.tensor([1.0, -1.0, 0.0, 0.0]))
    x = torch.arange(10, dtype=torch.float32, device=dev) ** 2
    d1 = frac.fracdiff_gl(x, 1.0, h=1.0)
    assert torch.allclose(d1[1:].cpu(), (x[1:] - x[:-1]).cpu())                     # alpha=1 is the backward difference
    torch.manual_seed(5)
    xr = torch.randn(3, 300, device=dev)
    y = frac.fracdiff_gl(xr, 0.7, h=0.5, m=64)
    ref = frac.fracdiff_gl(xr.cpu(), 0.7, h=0.5, m=64)
    assert torch.allclose(y.cpu(), ref, atol=1e-4)
    assert abs(frac.mellin_log_grid(torch.exp(-torch.exp(torch.linspace(math.log(1e-4), math.log(40), 4000))), 1e-4, 40, 2 + 0j) - 1.0) < 1e-3
