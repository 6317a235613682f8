"""Vision backbones (ResNet-style, ConvNeXt-style, ViT) and explainability (Grad-CAM, integrated
gradients) on the framework's kernels.

The reference ships ResNet / ConvNeXt / ViT backbones (crates/st-vision/src/models/{resnet,
convnext,vit}.rs; the ViT is forward-only there) and Grad-CAM / integrated gradients
(crates/st-vision/src/xai/*).  Here the 3x3 convolutions run as implicit GEMMs
(``ops.conv``: forward, data gradient with fused ReLU mask, split-K weight gradient), linears on the
tcgen05 GEMM, attention on the flash-style kernel with its backward — so the ViT trains — and norms
on the fused norm kernels.  Activations are NHWC bf16 inside the conv nets.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import conv as C
from ..ops import elementwise as ew
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops


class _Conv3x3Fn(torch.autograd.Function):
    """conv3x3 (+bias, optional ReLU) over NHWC activations with tap-major weights ``[OC, 9*IC]``."""

    @staticmethod
    def forward(ctx, x, w, b, relu):
        y = C.conv3x3(x, w, b, relu=relu)
        ctx.save_for_backward(x, w, y if relu else None)
        ctx.relu, ctx.has_bias = relu, b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.relu:
            dy = torch.where(y > 0, dy, torch.zeros_like(dy))
        ic = x.shape[-1]
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        C.conv3x3_wgrad(dy, x, dw)
        db = dy.reshape(-1, dy.shape[-1]).float().sum(0).to(w.dtype) if ctx.has_bias else None
        dx = C.conv3x3(dy, C.dgrad_weights(w, ic)) if ctx.needs_input_grad[0] else None
        return dx, dw.to(w.dtype), db, None


class Conv3x3(nn.Module):
    def __init__(self, ic: int, oc: int, relu: bool = False, bias: bool = True, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.ic, self.oc, self.relu = ic, oc, relu
        self.weight = nn.Parameter((torch.randn(oc, 9 * ic, device=device) * math.sqrt(2.0 / (9 * ic))).to(dtype))
        self.bias = nn.Parameter(torch.zeros(oc, device=device, dtype=dtype)) if bias else None

    def forward(self, x):                       # x: [N, H, W, IC]
        return _Conv3x3Fn.apply(x, self.weight, self.bias, self.relu)


class _Pool2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y, idx = C.maxpool2(x)
        ctx.save_for_backward(idx)
        ctx.hw = (x.shape[1], x.shape[2])
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        return C.maxpool2_backward(dy.contiguous(), idx, *ctx.hw)


def maxpool2(x):
    return _Pool2Fn.apply(x)


class Linear(nn.Module):
    def __init__(self, i: int, o: int, device=None, dtype=torch.bfloat16, std: Optional[float] = None):
        super().__init__()
        self.weight = nn.Parameter((torch.randn(o, i, device=device) * (std or math.sqrt(1.0 / i))).to(dtype))
        self.bias = nn.Parameter(torch.zeros(o, device=device, dtype=dtype))

    def forward(self, x):
        shp = x.shape
        return gemm_ops.linear(x.reshape(-1, shp[-1]), self.weight, self.bias).reshape(*shp[:-1], -1)


class LayerNorm(nn.Module):
    def __init__(self, d: int, device=None, dtype=torch.bfloat16, eps: float = 1e-5):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(d, device=device, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(d, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x):
        return norm_ops.layer_norm(x, self.gamma, self.beta, self.eps)


# ---- ResNet-style ------------------------------------------------------------------------------------
class BasicBlock(nn.Module):
    """conv-ReLU-conv + identity, ReLU (channel-preserving; the stem / transitions change width)."""

    def __init__(self, ch: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.c1 = Conv3x3(ch, ch, relu=True, device=device, dtype=dtype)
        self.c2 = Conv3x3(ch, ch, relu=False, device=device, dtype=dtype)

    def forward(self, x):
        return ew.relu(self.c2(self.c1(x)) + x)


class ResNet(nn.Module):
    """Stem conv (IC padded to 64 lanes is handled by the small-channel im2col path), ``blocks`` residual
    blocks per stage, 2x2 max-pool + widening conv between stages, global average pool, linear head."""

    def __init__(self, num_classes: int = 10, widths=(64, 128, 256), blocks: int = 1, in_channels: int = 3, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.stem = Conv3x3(in_channels, widths[0], relu=True, device=device, dtype=dtype)
        layers, ch = [], widths[0]
        for i, w in enumerate(widths):
            if i > 0:
                layers.append(("pool", None))
                layers.append(("widen", Conv3x3(ch, w, relu=True, device=device, dtype=dtype)))
                ch = w
            for _ in range(blocks):
                layers.append(("block", BasicBlock(ch, device=device, dtype=dtype)))
        self.kinds = [k for k, _ in layers]
        self.layers = nn.ModuleList([m if m is not None else nn.Identity() for _, m in layers])
        self.head = Linear(ch, num_classes, device=device, dtype=dtype)
        self.feature_channels = ch

    def features(self, images):                 # NCHW -> NHWC feature map
        x = images.to(self.dtype).permute(0, 2, 3, 1).contiguous()
        x = self.stem(x)
        for kind, m in zip(self.kinds, self.layers):
            x = maxpool2(x) if kind == "pool" else m(x)
        return x

    def forward(self, images, return_features: bool = False):
        f = self.features(images)
        logits = self.head(f.float().mean(dim=(1, 2)).to(self.dtype))
        return (logits, f) if return_features else logits


# ---- ConvNeXt-style ------------------------------------------------------------------------------------
class ConvNeXtBlock(nn.Module):
    """Spatial mixing by a 3x3 convolution, LayerNorm over channels, inverted-bottleneck MLP
    (expansion 4, GELU), layer scale, residual."""

    def __init__(self, ch: int, device=None, dtype=torch.bfloat16, layer_scale: float = 1e-2):
        super().__init__()
        self.mix = Conv3x3(ch, ch, device=device, dtype=dtype)
        self.norm = LayerNorm(ch, device=device, dtype=dtype)
        self.fc1 = Linear(ch, 4 * ch, device=device, dtype=dtype)
        self.fc2 = Linear(4 * ch, ch, device=device, dtype=dtype)
        self.scale = nn.Parameter(torch.full((ch,), layer_scale, device=device, dtype=dtype))

    def forward(self, x):
        h = self.norm(self.mix(x))
        h = self.fc2(ew.gelu(self.fc1(h)))
        return x + h * self.scale


class ConvNeXt(nn.Module):
    def __init__(self, num_classes: int = 10, widths=(64, 128), depth: int = 1, in_channels: int = 3, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.stem = Conv3x3(in_channels, widths[0], device=device, dtype=dtype)
        mods, kinds, ch = [], [], widths[0]
        for i, w in enumerate(widths):
            if i > 0:
                kinds.append("down")
                mods.append(Conv3x3(ch, w, device=device, dtype=dtype))
                ch = w
            for _ in range(depth):
                kinds.append("block")
                mods.append(ConvNeXtBlock(ch, device=device, dtype=dtype))
        self.kinds, self.mods = kinds, nn.ModuleList(mods)
        self.norm = LayerNorm(ch, device=device, dtype=dtype)
        self.head = Linear(ch, num_classes, device=device, dtype=dtype)

    def forward(self, images):
        x = self.stem(images.to(self.dtype).permute(0, 2, 3, 1).contiguous())
        for kind, m in zip(self.kinds, self.mods):
            x = m(maxpool2(x)) if kind == "down" else m(x)
        return self.head(self.norm(x.float().mean(dim=(1, 2)).to(self.dtype)))


# ---- ViT -------------------------------------------------------------------------------------------------
class ViTBlock(nn.Module):
    def __init__(self, dim: int, heads: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.heads = heads
        self.n1, self.n2 = LayerNorm(dim, device=device, dtype=dtype), LayerNorm(dim, device=device, dtype=dtype)
        self.qkv = Linear(dim, 3 * dim, device=device, dtype=dtype)
        self.proj = Linear(dim, dim, device=device, dtype=dtype)
        self.fc1 = Linear(dim, 4 * dim, device=device, dtype=dtype)
        self.fc2 = Linear(4 * dim, dim, device=device, dtype=dtype)

    def forward(self, x):                      # [B, S, D]
        B, S, D = x.shape
        qkv = self.qkv(self.n1(x)).reshape(B, S, 3, self.heads, D // self.heads)
        o = attn_ops.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=False)
        x = x + self.proj(o.reshape(B, S, D))
        return x + self.fc2(ew.gelu(self.fc1(self.n2(x))))


class ViT(nn.Module):
    """Patch embedding (a GEMM over flattened patches), class token, learned positions, pre-norm blocks
    with bidirectional attention (head dim 64 or 128), LayerNorm, linear head on the class token."""

    def __init__(self, image: int = 32, patch: int = 4, dim: int = 128, depth: int = 2, heads: int = 2,
                 num_classes: int = 10, in_channels: int = 3, device=None, dtype=torch.bfloat16):
        super().__init__()
        assert image % patch == 0 and dim % heads == 0 and dim // heads in (64, 128)
        self.patch, self.dtype = patch, dtype
        n = (image // patch) ** 2
        self.embed = Linear(in_channels * patch * patch, dim, device=device, dtype=dtype)
        self.cls = nn.Parameter(torch.zeros(1, 1, dim, device=device, dtype=dtype))
        self.pos = nn.Parameter((torch.randn(1, n + 1, dim, device=device) * 0.02).to(dtype))
        self.blocks = nn.ModuleList([ViTBlock(dim, heads, device=device, dtype=dtype) for _ in range(depth)])
        self.norm = LayerNorm(dim, device=device, dtype=dtype)
        self.head = Linear(dim, num_classes, device=device, dtype=dtype)

    def forward(self, images):
        B, Cc, H, W = images.shape
        p = self.patch
        x = images.to(self.dtype).reshape(B, Cc, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
        x = self.embed(x.reshape(B, (H // p) * (W // p), Cc * p * p))
        x = torch.cat([self.cls.expand(B, -1, -1), x], 1) + self.pos
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x)[:, 0])


# ---- explainability -----------------------------------------------------------------------------------------
def grad_cam(model: ResNet, images: torch.Tensor, target: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grad-CAM over the last feature map of a conv backbone: channel weights = spatial mean of the
    class-score gradient; map = ReLU(Σ_c w_c · A_c), normalised to [0, 1] per image.  ``[N, H, W]``."""
    logits, feat = model(images, return_features=True)
    feat.retain_grad()
    if target is None:
        target = logits.argmax(-1)
    score = logits.float().gather(1, target.reshape(-1, 1).to(logits.device)).sum()
    model.zero_grad(set_to_none=True)
    score.backward()
    w = feat.grad.float().mean(dim=(1, 2), keepdim=True)
    cam = torch.relu((w * feat.detach().float()).sum(-1))
    lo = cam.amin(dim=(1, 2), keepdim=True)
    hi = cam.amax(dim=(1, 2), keepdim=True)
    return (cam - lo) / (hi - lo).clamp(min=1e-12)


def integrated_gradients(model: nn.Module, images: torch.Tensor, target: torch.Tensor, steps: int = 16,
                         baseline: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Riemann (midpoint) approximation of integrated gradients; attributions have the image's shape and
    sum, per image, to about ``score(image) - score(baseline)``."""
    baseline = torch.zeros_like(images) if baseline is None else baseline
    total = torch.zeros_like(images, dtype=torch.float32)
    for k in range(steps):
        alpha = (k + 0.5) / steps
        x = (baseline + alpha * (images - baseline)).detach().float().requires_grad_(True)
        score = model(x).float().gather(1, target.reshape(-1, 1).to(images.device)).sum()
        (g,) = torch.autograd.grad(score, x)
        total += g
    return (images - baseline).float() * total / steps
