"""Spectral ops: FFT conventions, windows, canvas vector-field spectra, spectral multipliers, temporal renderer.
CPU cases pin the semantics; GPU cases compare the shared-memory FFT / multiplier / renderer kernels with ``torch.fft``
and the fp32 statement of each formula."""
import math

import pytest
import torch

from spiraltorch_b200 import frac, vision
from spiraltorch_b200.ops import spectral


def test_fft_conventions_and_windows():
    x = torch.randn(3, 8)
    z = spectral.fft(x)
    assert torch.allclose(z, torch.fft.fft(x.to(torch.complex64)), atol=1e-5)
    assert torch.allclose(spectral.fft(z, inverse=True).real, x, atol=1e-5)          # inverse carries the 1/N
    assert torch.allclose(spectral.fft(x, dim=0), torch.fft.fft(x.to(torch.complex64), dim=0), atol=1e-5)
    hann = spectral.window_coefficients("hann", 5)
    assert hann.tolist() == pytest.approx([0.0, 0.5, 1.0, 0.5, 0.0], abs=1e-6)
    assert spectral.window_coefficients("hamming", 3).tolist() == pytest.approx([0.08, 1.0, 0.08], abs=1e-6)
    assert spectral.window_coefficients("blackman", 3).tolist() == pytest.approx([0.0, 1.0, 0.0], abs=1e-6)
    assert spectral.window_coefficients("hann", 1).tolist() == [1.0]
    assert torch.allclose(spectral.fft(x, window=spectral.window_coefficients("hann", 8)),
                          torch.fft.fft((x * spectral.window_coefficients("hann", 8)).to(torch.complex64)), atol=1e-5)
    with pytest.raises(ValueError):
        spectral.window_coefficients("kaiser", 4)
    with pytest.raises(ValueError):
        spectral.fft(x, window=torch.ones(3))


def test_color_vector_field_spectra_layout():
    torch.manual_seed(0)
    f = vision.ColorVectorField(torch.rand(4, 6, 4))
    rows = f.fft_rows_tensor().reshape(4, 6, 4, 2)
    want = torch.fft.fft(f.vectors.to(torch.complex64), dim=1)
    assert torch.allclose(torch.view_as_complex(rows.contiguous()), want, atol=1e-5)          # (re, im) pairs per channel
    cols = f.fft_cols_tensor(window="hann").reshape(4, 6, 4, 2)
    w = spectral.window_coefficients("hann", 4).reshape(4, 1, 1)
    assert torch.allclose(torch.view_as_complex(cols.contiguous()), torch.fft.fft((f.vectors * w).to(torch.complex64), dim=0), atol=1e-5)
    both = torch.view_as_complex(f.fft_2d_tensor().reshape(4, 6, 4, 2).contiguous())
    assert torch.allclose(both, torch.fft.fft2(f.vectors.to(torch.complex64), dim=(0, 1)), atol=1e-4)
    mag, power, db, phase = (f.fft_magnitude_tensor(), f.fft_power_tensor(), f.fft_power_db_tensor(), f.fft_phase_tensor())
    assert mag.shape == (4, 24) and torch.allclose(mag ** 2, power, atol=1e-4)
    assert torch.allclose(db, (10 * torch.log10(power.clamp(min=1e-12))).clamp(min=-160.0), atol=1e-4)
    assert torch.allclose(phase.reshape(4, 6, 4), torch.angle(want), atol=1e-4)
    back = vision.ColorVectorField(f.vectors).fft_rows_tensor(inverse=True).reshape(4, 6, 4, 2)
    assert torch.allclose(torch.view_as_complex(back.contiguous()), torch.fft.ifft(f.vectors.to(torch.complex64), dim=1), atol=1e-5)
    assert f.as_tensor().shape == (4, 24) and f.energy_tensor().shape == (4, 6)
    e = vision.ColorVectorField.from_energy(torch.rand(5, 7))
    assert e.vectors.shape == (5, 7, 4) and float(e.energy_tensor().min()) == 0.0 and float(e.energy_tensor().max()) == pytest.approx(1.0)
    with pytest.raises(ValueError):
        vision.ColorVectorField(torch.rand(4, 6, 3))
    g = torch.rand(4, 8)
    assert torch.allclose(vision.canvas_fft(g, "2d"), torch.fft.fft2(g.to(torch.complex64)), atol=1e-4)
    assert torch.allclose(vision.canvas_fft(g, "col", inverse=True), torch.fft.ifft(g.to(torch.complex64), dim=0), atol=1e-5)


def test_spectral_multipliers():
    z = torch.randn(2, 8, dtype=torch.complex64)
    lap = spectral.specmul_frac_laplace(z, 1.5)
    env = torch.tensor([0, 1, 2, 3, 3, 2, 1, 0], dtype=torch.float32) ** 1.5
    assert torch.allclose(lap, z * env, atol=1e-5) and torch.allclose(frac.specmul_frac_laplace(z, 1.5), lap)
    # the derivative multiplier differentiates a sine exactly: d/dt sin(2 pi t) sampled on [0, 1)
    n = 64
    t = torch.arange(n, dtype=torch.float32) / n
    d1 = frac.fracdiff_spectral(torch.sin(2 * math.pi * t), 1.0, h=1.0 / n)
    assert torch.allclose(d1, 2 * math.pi * torch.cos(2 * math.pi * t), atol=1e-3)
    half = frac.fracdiff_spectral(frac.fracdiff_spectral(torch.sin(2 * math.pi * t), 0.5, h=1.0 / n), 0.5, h=1.0 / n)
    assert torch.allclose(half, d1, atol=1e-3)                                    # semigroup: D^0.5 D^0.5 = D^1
    with pytest.raises(ValueError):
        spectral.specmul_frac_derivative(z, 1.0, h=0.0)
    with pytest.raises(ValueError):
        spectral.specmul_frac_laplace(z, float("nan"))


def _temporal_case(device):
    torch.manual_seed(1)
    vox = torch.rand(2, 3, 4, device=device)
    harm = torch.randn(2, 3, 4, 3, device=device) * 0.2
    harm[0, 0, 0] = 0.0
    decay = torch.rand(2, 3, 4, device=device)
    decay[0, 0, 1], decay[0, 0, 2], decay[0, 0, 3] = float("nan"), -2.0, 0.0
    return vox, harm, decay


def _temporal_oracle(vox, harm, decay, frames, rate):
    out = torch.zeros(frames, *vox.shape)
    for f in range(frames):
        t = f / rate
        base = vox.clone()
        for c in range(harm.shape[-1]):
            base += harm[..., c] * math.sin((c + 1) * 2 * math.pi * t)
        d = torch.where(torch.isfinite(decay), decay.clamp(min=0), torch.ones_like(decay))
        out[f] = torch.where(d <= 1.1920929e-07, torch.zeros_like(base), base * torch.exp(-d * t))
    return out


def test_temporal_renderer_matches_formula():
    vox, harm, decay = _temporal_case("cpu")
    out = vision.TemporalRenderer(frames=5, sample_rate_hz=10.0).render(vox, decay, harm)
    assert (out.frames, out.depth, out.height, out.width) == (5, 2, 3, 4) and out.times[2] == pytest.approx(0.2)
    assert torch.allclose(out.data, _temporal_oracle(vox, harm, decay, 5, 10.0), atol=1e-5)
    assert torch.equal(out.frame(0)[0, 0, :2], vox[0, 0, :2])                        # t = 0: undamped (NaN decay counts as 1)
    assert float(out.data[:, 0, 0, 2:].abs().max()) == 0.0 and out.frame(9) is None     # negative -> 0, and zero decay silences
    no_harm = vision.TemporalRenderer(3, 24.0).render(vox, decay)
    assert torch.allclose(no_harm.data[1], _temporal_oracle(vox, harm * 0, decay, 3, 24.0)[1], atol=1e-6)
    for bad in (lambda: vision.TemporalRenderer(0).render(vox, decay), lambda: vision.TemporalRenderer(4, 0.0).render(vox, decay),
                lambda: vision.TemporalRenderer().render(vox, decay[:1]), lambda: vision.TemporalRenderer().render(vox, decay, harm[..., :2, :])):
        with pytest.raises(ValueError):
            bad()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [2, 8, 64, 1024, 8192, 6, 100, 1000])
def test_fft_kernel_matches_torch(n):
    torch.manual_seed(n)
    before = spectral.launch_count
    x = torch.randn(5, n, device="cuda")
    z = spectral.fft(x)
    assert spectral.launch_count == before + 1
    ref = torch.fft.fft(x.double().cpu()).to(torch.complex64)
    scale = float(ref.abs().max())
    assert float((z.cpu() - ref).abs().max()) <= 2e-5 * scale * max(math.log2(n), 1)
    c = torch.randn(3, n, device="cuda", dtype=torch.complex64)
    back = spectral.fft(spectral.fft(c), inverse=True)
    assert float((back - c).abs().max()) <= 5e-5 * max(math.log2(n), 1) * float(c.abs().max())
    col = spectral.fft(x.t().contiguous(), dim=0)                                 # transform along the outer dimension
    assert float((col.cpu().t() - ref).abs().max()) <= 2e-5 * scale * max(math.log2(n), 1)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,n", [(2048, 4096), (1500, 512), (4001, 64), (700, 2048)])
def test_streamed_fft_of_long_batches_matches_torch(rows, n):
    """Batches longer than four rows per SM take the persistent kernel that prefetches the next row with a bulk
    asynchronous copy; forward and inverse against torch, including a row count that leaves some CTAs one row short."""
    torch.manual_seed(rows + n)
    x = torch.randn(rows, n, device="cuda", dtype=torch.complex64)
    ref = torch.fft.fft(x)
    z = spectral.fft(x)
    assert float((z - ref).abs().max()) <= 2e-5 * float(ref.abs().max()) * math.log2(n)
    back = spectral.fft(z, inverse=True)
    assert float((back - x).abs().max()) <= 5e-5 * math.log2(n) * float(x.abs().max())
    from spiraltorch_b200.ops import native
    native.raise_on_device_error()


@pytest.mark.gpu
def test_field_spectra_multipliers_and_renderer_on_gpu():
    torch.manual_seed(3)
    v = torch.rand(16, 32, 4)
    cpu, gpu = vision.ColorVectorField(v), vision.ColorVectorField(v.cuda())
    before = spectral.launch_count
    for fn in ("fft_rows_tensor", "fft_cols_tensor", "fft_2d_tensor"):
        a, b = getattr(cpu, fn)(window="hamming"), getattr(gpu, fn)(window="hamming")
        assert b.is_cuda and float((a - b.cpu()).abs().max()) <= 1e-4 * float(a.abs().max()), fn
    assert spectral.launch_count - before == 4                                    # rows, cols, rows + cols of the 2-D pass
    assert torch.allclose(gpu.fft_power_db_tensor("col").cpu(), cpu.fft_power_db_tensor("col"), atol=1e-2)
    z = torch.randn(7, 48, dtype=torch.complex64)
    assert torch.allclose(spectral.specmul_frac_laplace(z.cuda(), 0.75).cpu(), spectral.specmul_frac_laplace(z, 0.75), atol=1e-4)
    for alpha in (0.5, 1.0, 1.7):
        a, b = spectral.specmul_frac_derivative(z, alpha, 0.1), spectral.specmul_frac_derivative(z.cuda(), alpha, 0.1).cpu()
        assert float((a - b).abs().max()) <= 2e-4 * float(a.abs().max())
    x = torch.randn(4, 256)
    assert torch.allclose(frac.fracdiff_spectral(x.cuda(), 0.6, 0.05).cpu(), frac.fracdiff_spectral(x, 0.6, 0.05), atol=2e-3)
    vox, harm, decay = _temporal_case("cuda")
    out = vision.TemporalRenderer(frames=7, sample_rate_hz=12.0).render(vox, decay, harm)
    assert out.data.is_cuda and torch.allclose(out.data.cpu(), _temporal_oracle(vox.cpu(), harm.cpu(), decay.cpu(), 7, 12.0), atol=2e-5)
