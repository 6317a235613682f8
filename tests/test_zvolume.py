"""Z-space volume and vision projector semantics (crates/st-vision/src/lib.rs): slice statistics, collapse, depth
interpolation, bilinear upscale, diffusion stencil, EMA streaming, sequence blending, spectral windows, the temporal
resonance buffer and the projector's depth / time weights."""
import math
from types import SimpleNamespace

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import zvolume as Z
from spiraltorch_b200.telemetry import AtlasFrame


def _vol():
    return Z.ZSpaceVolume(torch.arange(24, dtype=torch.float32).reshape(3, 2, 4))


def _resonance(depth=3):
    t = lambda v: st.Tensor._wrap(torch.tensor([v], dtype=torch.float32))           # noqa: E731
    return SimpleNamespace(infinity_energy=t([1.0, 2.0, 3.0][:depth]), recursive_objective=t([0.0] * depth),
                           homotopy_flow=t([0.0] * depth))


def test_profile_and_report():
    v = _vol()
    p = v.profile()
    assert p.depth() == 3 and p.means == pytest.approx([3.5, 11.5, 19.5])
    assert p.std(0) == pytest.approx(math.sqrt(5.25)) and p.energy(0) == pytest.approx(sum(i * i for i in range(8)) / 8)
    r = v.telemetry_report()
    assert r.depth == 3 and r.mean_intensity == pytest.approx(11.5) and r.max_energy == pytest.approx(p.energy(2))
    shares = [e / p.total_energy() for e in p.energies]
    assert r.energy_entropy == pytest.approx(-sum(s * math.log2(s) for s in shares))
    assert Z.ZSpaceVolume.zeros(2, 2, 2).profile().energy_entropy() == 0.0
    assert p.mean(9) == 0.0
    with pytest.raises(st.TensorError):
        Z.ZSliceProfile([1.0], [1.0, 2.0], [1.0])


def test_constructors_and_collapse():
    v = Z.ZSpaceVolume.from_voxels(2, 1, 2, [1.0, 2.0, 3.0, 4.0])
    assert v.collapse_with_weights([0.25, 0.75]).torch().tolist() == [[2.5, 3.5]]
    s = Z.ZSpaceVolume.from_slices([st.Tensor._wrap(torch.ones(2, 2)), st.Tensor._wrap(torch.zeros(2, 2))])
    assert (s.depth, s.height, s.width) == (2, 2, 2) and s.slice(0).torch().sum() == 4 and float(s.resonance_decay.min()) == 1.0
    h = Z.ZSpaceVolume.zeros_with_temporal(2, 2, 2, 3)
    assert h.harmonic_channels == 3
    h.ensure_harmonic_channels(5)
    assert h.temporal_harmonics.shape == (2, 2, 2, 5)
    for bad in (lambda: Z.ZSpaceVolume.zeros(0, 2, 2), lambda: Z.ZSpaceVolume.from_voxels(2, 2, 2, [1.0]), lambda: Z.ZSpaceVolume.from_slices([]),
                lambda: Z.ZSpaceVolume.from_slices([torch.ones(2, 2), torch.ones(2, 3)]), lambda: v.collapse_with_weights([1.0]),
                lambda: v.collapse_with_weights([float("nan"), 1.0]), lambda: v.slice(2)):
        with pytest.raises(st.TensorError):
            bad()
    w = _vol().resonance_weights(_resonance())
    assert w == pytest.approx([1 / 6, 2 / 6, 3 / 6], rel=1e-5)                      # |energy| shares; tanh(0) factors are 1
    assert torch.allclose(_vol().project_resonance(_resonance()).torch(), (_vol().voxels * torch.tensor(w)[:, None, None]).sum(0))


def test_interpolate_and_upscale():
    v = Z.ZSpaceVolume(torch.tensor([0.0, 1.0, 4.0, 9.0]).reshape(4, 1, 1))
    assert v.interpolate("nearest").voxels.flatten().tolist() == [0, 0, 1, 1, 4, 4, 9]
    assert v.interpolate("linear").voxels.flatten().tolist() == [0, 0.5, 1, 2.5, 4, 6.5, 9]
    cub = v.interpolate("cubic").voxels.flatten().tolist()
    assert cub[1] == pytest.approx((-0 + 9 * 0 + 9 * 1 - 4) / 16) and cub[3] == pytest.approx((-0 + 9 * 1 + 9 * 4 - 9) / 16)
    assert cub[5] == pytest.approx((-1 + 9 * 4 + 9 * 9 - 9) / 16)
    assert Z.ZSpaceVolume.zeros(1, 2, 2).interpolate().depth == 1
    with pytest.raises(ValueError):
        v.interpolate("spline")
    img = Z.ZSpaceVolume(torch.tensor([[[0.0, 1.0], [2.0, 3.0]]]))
    up = img.upscale(2)
    assert (up.height, up.width) == (4, 4)
    assert up.voxels[0, 0].tolist() == pytest.approx([0, 1 / 3, 2 / 3, 1]) and up.voxels[0, 3, 3] == 3.0      # corners aligned
    assert img.upscale(1).voxels.equal(img.voxels)
    with pytest.raises(st.TensorError):
        img.upscale(0)


def test_diffuser_stencil():
    v = Z.ZSpaceVolume(torch.zeros(1, 1, 3))
    v.voxels[0, 0, 1] = 3.0
    out = Z.ZDiffuser(1, 0.5).diffuse(v).voxels.flatten().tolist()
    assert out == pytest.approx([1.5, 1.5, 1.5])                   # ends see one neighbour (3.0); the centre two zeros
    torch.manual_seed(0)
    big = Z.ZSpaceVolume(torch.rand(3, 4, 5))
    ref = big.voxels.clone()
    nxt = ref.clone()
    for z in range(3):
        for y in range(4):
            for x in range(5):
                nb = [ref[a, b, c] for a, b, c in ((z - 1, y, x), (z + 1, y, x), (z, y - 1, x), (z, y + 1, x), (z, y, x - 1), (z, y, x + 1))
                      if 0 <= a < 3 and 0 <= b < 4 and 0 <= c < 5]
                nxt[z, y, x] = ref[z, y, x] * 0.75 + 0.25 * sum(nb) / len(nb)
    assert torch.allclose(Z.ZDiffuser(1, 0.25).diffuse(big).voxels, nxt, atol=1e-6)
    assert torch.equal(Z.ZDiffuser(3, 0.5).diffuse(Z.ZSpaceVolume(torch.full((1, 1, 1), 2.0))).voxels, torch.full((1, 1, 1), 2.0))
    assert Z.ZDiffuser(1, float("nan")).rate == 0.25 and Z.ZDiffuser(1, 7.0).rate == 1.0


def test_accumulate_and_blend_sequence():
    a = Z.ZSpaceVolume(torch.zeros(1, 1, 2), torch.ones(1, 1, 2, 1))
    b = Z.ZSpaceVolume(torch.ones(1, 1, 2) * 4, torch.ones(1, 1, 2, 3) * 2, torch.full((1, 1, 2), 3.0))
    a.accumulate(b, 0.25)
    assert a.voxels.flatten().tolist() == [1.0, 1.0] and a.harmonic_channels == 3
    assert a.temporal_harmonics[0, 0, 0].tolist() == pytest.approx([1.25, 0.5, 0.5]) and a.resonance_decay[0, 0, 0] == 1.5
    with pytest.raises(st.TensorError):
        a.accumulate(b, 1.5)
    with pytest.raises(st.TensorError):
        a.accumulate(Z.ZSpaceVolume.zeros(2, 1, 2), 0.5)
    seq = [Z.ZSpaceVolume(torch.full((1, 1, 1), float(i))) for i in (1, 2, 3)]
    blend = Z.ZSpaceVolume.blend_sequence(seq, [1.0, 1.0, 2.0])
    assert float(blend.voxels) == pytest.approx((1 + 2 + 6) / 4) and float(blend.resonance_decay) == pytest.approx(1.0)
    with pytest.raises(st.TensorError):
        Z.ZSpaceVolume.blend_sequence(seq, [1.0])
    with pytest.raises(st.TensorError):
        Z.ZSpaceVolume.blend_sequence([], [])


def test_windows_and_resonance_buffer():
    assert Z.SpectralWindow.rectangular().weights(4) == [0.25] * 4
    hann = Z.SpectralWindow.hann().weights(5)
    assert hann[0] == 0.0 and hann[2] == max(hann) and sum(hann) == pytest.approx(1.0)
    assert Z.SpectralWindow.hamming().weights(1) == [1.0] and Z.SpectralWindow.blackman().weights(0) == []
    g = Z.SpectralWindow.gaussian(0.2).weights(7)
    assert g[3] == max(g) and g[0] == pytest.approx(g[6]) and Z.SpectralWindow.gaussian(-1.0).sigma == 0.4
    buf = Z.TemporalResonanceBuffer(0.25)
    assert buf.apply([2.0, 2.0]) == [0.5, 0.5] and buf.frames_accumulated() == 1
    assert buf.apply([1.0, 0.0]) == pytest.approx([0.625, 0.375]) and buf.frames_accumulated() == 2
    assert buf.apply([1.0, 1.0, 1.0]) == pytest.approx([1 / 3] * 3) and buf.frames_accumulated() == 1       # depth changed: restart
    assert buf.apply([]) == [] and buf.history is None
    with pytest.raises(st.TensorError):
        buf.apply([float("inf")])
    assert Z.TemporalResonanceBuffer(float("nan")).decay == 0.5


def test_vision_projector_weights():
    proj = Z.VisionProjector(1.0, 0.2, 0.0, Z.SpectralWindow.rectangular())
    w = proj.depth_weights(_vol(), _resonance())
    assert sum(w) == pytest.approx(1.0) and w[2] > w[1] > w[0]
    raw = [e * math.exp(-0.5 * ((i / 2 - 1.0) / 0.2) ** 2) for i, e in enumerate([1 / 6, 2 / 6, 3 / 6])]
    assert w == pytest.approx([max(r, 0) / sum(raw) for r in raw], rel=1e-4)
    assert torch.allclose(proj.project(_vol(), _resonance()).torch(), (_vol().voxels * torch.tensor(w)[:, None, None]).sum(0), atol=1e-5)
    buf = Z.TemporalResonanceBuffer(0.5)
    first = proj.depth_weights_with_temporal(_vol(), _resonance(), buf)
    assert first == pytest.approx(w) and proj.project_with_temporal(_vol(), _resonance(), buf).shape() == (2, 4)
    tw = proj.temporal_weights(4)
    assert sum(tw) == pytest.approx(1.0) and tw[3] == max(tw) and proj.temporal_weights(1) == [1.0] and proj.temporal_weights(0) == []
    assert proj.streaming_alpha() == pytest.approx(0.65)
    fused = proj.fuse_sequence([Z.ZSpaceVolume(torch.full((1, 1, 1), float(i))) for i in range(4)])
    assert float(fused.voxels) == pytest.approx(sum(i * t for i, t in enumerate(tw)))
    state = Z.ZSpaceVolume.zeros(1, 1, 1)
    proj.accumulate_temporal(state, Z.ZSpaceVolume(torch.ones(1, 1, 1)))
    assert float(state.voxels) == pytest.approx(0.65)
    summary = SimpleNamespace(max_energy=3.0, min_energy=1.0, mean_energy=2.5, energy_std=0.5, mean_abs_drift=1.0, mean_decay=0.2)
    p2 = Z.VisionProjector.from_summary(summary)
    assert p2.focus == pytest.approx(0.75) and p2.spread == pytest.approx(0.125) and p2.energy_bias == 0.2 and p2.temporal_decay == 0.5
    atlas = AtlasFrame(timestamp=1.0, z_signal=0.3, collapse_total=0.5)
    atlas.push_metric("temporal_focus", 0.2)
    atlas.push_metric("pace", -0.7, district="Temporal")
    p2.calibrate_from_atlas(atlas)
    assert p2.focus == pytest.approx(0.3) and p2.energy_bias == pytest.approx(math.tanh(0.5)) and p2.temporal_focus == 0.2 and p2.temporal_decay == pytest.approx(0.7)
    assert Z.VisionProjector(0.5, float("nan"), float("inf")).spread == 0.35


def test_stream_frames_and_aggregator():
    f1 = Z.ZSpaceStreamFrame([torch.ones(2, 2), torch.ones(2, 2) * 2], atlas_frame=AtlasFrame(timestamp=1.0))
    assert f1.depth() == 2 and f1.slice_shape() == (2, 2) and f1.telemetry_report().depth == 2
    agg = Z.ZSpaceStreamFrameAggregator(max_depth=3)
    assert agg.is_empty() and agg.as_frame() is None and agg.telemetry_report() is None
    agg.extend(f1)
    agg.extend(Z.ZSpaceStreamFrame([torch.ones(2, 2) * 3, torch.ones(2, 2) * 4]))
    assert len(agg) == 3 and agg.as_frame().volume.voxels[:, 0, 0].tolist() == [2.0, 3.0, 4.0] and agg.atlas_frame.timestamp == 1.0
    with pytest.raises(st.TensorError):
        agg.extend(Z.ZSpaceStreamFrame([torch.ones(3, 3)]))
    agg.set_max_depth(1)
    assert len(agg) == 1 and agg.slice_shape() == (2, 2)
    with pytest.raises(st.TensorError):
        agg.set_max_depth(0)
    agg.clear()
    assert agg.is_empty()
    played = Z.ZSpaceVolume(torch.ones(2, 2, 2), torch.zeros(2, 2, 2, 1)).render_temporal(frames=3, sample_rate_hz=2.0)
    assert played.data.shape == (3, 2, 2, 2) and float(played.data[2, 0, 0, 0]) == pytest.approx(math.exp(-1.0))


@pytest.mark.gpu
def test_volume_ops_on_gpu_match_cpu():
    torch.manual_seed(1)
    v = Z.ZSpaceVolume(torch.rand(5, 16, 16), torch.rand(5, 16, 16, 2), torch.rand(5, 16, 16))
    g = v.to("cuda")
    assert g.profile().means == pytest.approx(v.profile().means, rel=1e-5)
    assert torch.allclose(Z.ZDiffuser(2, 0.3).diffuse(g).voxels.cpu(), Z.ZDiffuser(2, 0.3).diffuse(v).voxels, atol=1e-6)
    assert torch.allclose(g.interpolate("cubic").voxels.cpu(), v.interpolate("cubic").voxels, atol=1e-6)
    assert torch.allclose(g.upscale(2).voxels.cpu(), v.upscale(2).voxels, atol=1e-5)
    res = SimpleNamespace(infinity_energy=st.Tensor._wrap(torch.rand(1, 5).cuda()), recursive_objective=st.Tensor._wrap(torch.rand(1, 5).cuda()),
                          homotopy_flow=st.Tensor._wrap(torch.rand(1, 5).cuda()))
    out = Z.VisionProjector(0.4, 0.3, 0.1).project(g, res)
    assert out.torch().is_cuda and out.shape() == (16, 16)
    assert torch.allclose(g.render_temporal(4, 12.0).data.cpu(), v.render_temporal(4, 12.0).data, atol=2e-5)
