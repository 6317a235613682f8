"""Implicit-GEMM 3x3 convolution, pooling and the conv classifier."""
import pytest
import torch
import torch.nn.functional as F

from spiraltorch_b200.models.conv_classifier import ConvClassifier
from spiraltorch_b200.ops import conv as C


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def test_weight_layout_conversions():
    w = torch.arange(2 * 3 * 9, dtype=torch.float32).reshape(2, 27)
    tap = C.to_tap_major(w, 3)
    assert torch.equal(C.from_tap_major(tap, 3), w)
    assert tap[0, 0 * 3 + 1] == w[0, 1 * 9 + 0]            # [tap][ic] <- [ic][tap]
    x = torch.randn(2, 5, 5, 3)
    y = C.conv3x3(x, tap, None)
    ref = F.conv2d(x.permute(0, 3, 1, 2), w.reshape(2, 3, 3, 3), padding=1).permute(0, 2, 3, 1)
    assert torch.allclose(y, ref, atol=1e-5)
    dy = torch.randn(2, 5, 5, 2)
    xg = x.clone().requires_grad_(True)
    F.conv2d(xg.permute(0, 3, 1, 2), w.reshape(2, 3, 3, 3), padding=1).permute(0, 2, 3, 1).backward(dy)
    dx = C.conv3x3(dy, C.dgrad_weights(tap, 3), None)
    assert torch.allclose(dx, xg.grad, atol=1e-5)


def test_classifier_backward_matches_autograd_cpu():
    torch.manual_seed(0)
    model = ConvClassifier(num_classes=10, image=16, device="cpu", dtype=torch.float32)
    imgs, labels = torch.randn(4, 3, 16, 16), torch.randint(0, 10, (4,))
    loss = model.forward_backward(imgs, labels)
    P = {k: v.detach().clone().requires_grad_(True) for k, v in model.p.items()}
    x = imgs
    for s in range(4):
        for i in range(2):
            w = P[f"conv{s}_{i}.weight"]
            ic = w.shape[1] // 9
            w4 = w.reshape(w.shape[0], 3, 3, ic).permute(0, 3, 1, 2)
            x = torch.relu(F.conv2d(x, w4, P[f"conv{s}_{i}.bias"], padding=1))
        x = F.max_pool2d(x, 2)
    logits = x.mean((2, 3)) @ P["head.weight"].t() + P["head.bias"]
    ref = F.cross_entropy(logits[:, :10], labels)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    for name, p in model.p.items():
        g, r = p.main_grad, P[name].grad
        assert torch.allclose(g, r, atol=1e-4, rtol=1e-3), (name, (g - r).abs().max().item())
    assert model(imgs).shape == (4, 10)
    names = [n for n, _ in model.reference_state_dict()]
    assert "conv0_0::weight" in names and dict(model.reference_state_dict())["head::weight"].shape() == (512, 10)


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,Cin,OC", [(4, 64, 64, 64), (8, 32, 64, 128), (8, 16, 128, 256), (16, 8, 256, 512), (2, 32, 3, 64)])
def test_conv_kernels_match_reference(N, H, Cin, OC):
    torch.manual_seed(1)
    x = torch.randn(N, H, H, Cin, device="cuda").bfloat16()
    w = (torch.randn(OC, 9 * Cin, device="cuda") * (2.0 / (9 * Cin)) ** 0.5).bfloat16()
    b = torch.randn(OC, device="cuda").bfloat16()
    y = C.conv3x3(x, w, b, relu=True)
    ref = C._conv_ref(x.cpu().float(), w.cpu().float(), b.cpu().float(), 1, None)
    assert _rel(y.cpu(), ref) < 2e-2
    dy = torch.randn(N, H, H, OC, device="cuda").bfloat16()
    dw = torch.full((OC, 9 * Cin), 0.25, device="cuda")
    C.conv3x3_wgrad(dy, x, dw)
    rdw = torch.full((OC, 9 * Cin), 0.25)
    C.conv3x3_wgrad(dy.cpu().float(), x.cpu().float(), rdw)
    assert _rel(dw.cpu(), rdw) < 2e-2
    if Cin % 64 == 0:
        dx = C.conv3x3(dy, C.dgrad_weights(w, Cin), relu_mask_of=x)
        rdx = C._conv_ref(dy.cpu().float(), C.dgrad_weights(w.cpu().float(), Cin), None, 4, x.cpu().float())
        assert _rel(dx.cpu(), rdx) < 2e-2
    p, idx = C.maxpool2(y)
    rp, ridx = C.maxpool2(y.cpu().float())
    assert torch.equal(p.cpu().float(), rp)
    g = torch.randn_like(p)
    assert torch.equal(C.maxpool2_backward(g, idx, H, H).cpu().float(), C.maxpool2_backward(g.cpu().float(), idx.cpu(), H, H))
    assert _rel(C.global_avgpool(p).cpu(), C.global_avgpool(p.cpu().float())) < 1e-2
    from spiraltorch_b200.ops import native
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


@pytest.mark.gpu
def test_classifier_cuda_tracks_cpu():
    torch.manual_seed(2)
    gpu = ConvClassifier(num_classes=100, image=64, device="cuda")
    cpu = ConvClassifier(num_classes=100, image=64, device="cpu", dtype=torch.float32)
    cpu.flat_w.copy_(gpu.flat_w.float().cpu())
    imgs, labels = torch.randn(8, 3, 64, 64), torch.randint(0, 100, (8,))
    lg = gpu.forward_backward(imgs.cuda(), labels.cuda())
    lc = cpu.forward_backward(imgs, labels)
    assert abs(lg.item() - lc.item()) < 5e-2
    cos = torch.nn.functional.cosine_similarity(gpu.flat_grad.cpu(), cpu.flat_grad, dim=0).item()
    assert cos > 0.98, cos
