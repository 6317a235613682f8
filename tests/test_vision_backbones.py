"""Vision backbones and explainability on the CPU reference path (the GPU numerics of the kernels they
use are covered by the op-level tests); a GPU smoke test checks that they train on the native kernels."""
import pytest
import torch

from spiraltorch_b200.models import vision_backbones as V


def _finite_grads(model):
    gs = [p.grad for p in model.parameters() if p.requires_grad]
    assert all(g is not None and torch.isfinite(g.float()).all() for g in gs)


@pytest.mark.parametrize("make", [
    lambda dev: V.ResNet(num_classes=5, widths=(64, 128), blocks=1, device=dev, dtype=torch.float32),
    lambda dev: V.ConvNeXt(num_classes=5, widths=(64, 128), depth=1, device=dev, dtype=torch.float32),
    lambda dev: V.ViT(image=16, patch=4, dim=128, depth=2, heads=2, num_classes=5, device=dev, dtype=torch.float32),
])
def test_backbones_forward_backward_cpu(make):
    torch.manual_seed(0)
    m = make("cpu")
    x = torch.randn(2, 3, 16, 16)
    y = torch.tensor([1, 3])
    logits = m(x)
    assert logits.shape == (2, 5)
    loss = torch.nn.functional.cross_entropy(logits.float(), y)
    loss.backward()
    _finite_grads(m)


def test_conv3x3_function_matches_torch_conv_cpu():
    torch.manual_seed(1)
    conv = V.Conv3x3(64, 64, relu=True, dtype=torch.float32)
    x = torch.randn(2, 6, 6, 64, requires_grad=True)
    y = conv(x)
    y.sum().backward()
    from spiraltorch_b200.ops import conv as C
    w_ref = C.from_tap_major(conv.weight.detach(), 64).reshape(64, 64, 3, 3)
    x2 = x.detach().permute(0, 3, 1, 2).clone().requires_grad_(True)
    y2 = torch.relu(torch.nn.functional.conv2d(x2, w_ref, conv.bias.detach(), padding=1))
    y2.sum().backward()
    assert torch.allclose(y, y2.permute(0, 2, 3, 1), atol=1e-4)
    assert torch.allclose(x.grad, x2.grad.permute(0, 2, 3, 1), atol=1e-4)


def test_grad_cam_and_integrated_gradients_cpu():
    torch.manual_seed(2)
    m = V.ResNet(num_classes=4, widths=(64,), blocks=1, device="cpu", dtype=torch.float32)
    x = torch.randn(2, 3, 8, 8)
    cam = V.grad_cam(m, x)
    assert cam.shape == (2, 8, 8) and float(cam.min()) >= 0.0 and float(cam.max()) <= 1.0 + 1e-6
    t = torch.tensor([0, 2])
    ig = V.integrated_gradients(m, x, t, steps=32)
    with torch.no_grad():
        delta = m(x).float().gather(1, t[:, None]).flatten() - m(torch.zeros_like(x)).float().gather(1, t[:, None]).flatten()
    assert torch.allclose(ig.sum(dim=(1, 2, 3)), delta, rtol=0.1, atol=0.05)


@pytest.mark.gpu
def test_backbones_train_on_native_kernels():
    from spiraltorch_b200.ops import conv as C, gemm as G, attention as A, native
    torch.manual_seed(0)
    for make in (lambda: V.ResNet(num_classes=10, widths=(64, 128), device="cuda"),
                 lambda: V.ConvNeXt(num_classes=10, widths=(64, 128), device="cuda"),
                 lambda: V.ViT(image=32, patch=4, dim=128, depth=2, heads=2, device="cuda")):
        m = make()
        opt = torch.optim.SGD(m.parameters(), lr=2e-3)
        x = torch.randn(16, 3, 32, 32, device="cuda")
        y = torch.randint(0, 10, (16,), device="cuda")
        before = (C.launch_count, G.launch_count, A.launch_count)
        losses = []
        for _ in range(12):
            opt.zero_grad(set_to_none=True)
            loss = torch.nn.functional.cross_entropy(m(x).float(), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        native.raise_on_device_error()
        assert min(losses[-3:]) < losses[0], losses
        assert G.launch_count > before[1]
        assert (C.launch_count > before[0]) or (A.launch_count > before[2])
