"""Differentiable layer math of the public ``nn`` API on the sm_100a kernels.

The modules in :mod:`spiraltorch_b200.nn.modules` state their forward once as ``_fwd(x, params)`` over
fp32 tensors and obtain gradients by differentiating it.  For CUDA tensors the heavy pieces of those
forwards are the functions below: each is a ``torch.autograd.Function`` whose forward AND backward run on
the hand-written kernels of :mod:`spiraltorch_b200.ops` (tcgen05 GEMM for forward / data gradient /
weight gradient, the LayerNorm kernels, embedding gather / scatter-add, implicit-GEMM 3x3 convolution,
2x2 max-pool), so that ``Module.backward`` never reaches a library GEMM or convolution.  The public
tensors stay fp32; operands are rounded to bf16 at the kernel boundary and results / gradients come back
in fp32 (the GEMM accumulates in fp32 in TMEM).

Every function falls back to the plain PyTorch statement on CPU tensors, which is also the oracle the GPU
tests compare against.

Reference parity (what each mirrors):
  linear      crates/st-nn/src/layers/linear.rs:87-170      (x·W + b, dW = xᵀ·dy, db = Σ dy, dx = dy·Wᵀ)
  layer_norm  crates/st-tensor/src/pure.rs:3712             (layer_norm_affine_with_backend)
  embedding   crates/st-nn/src/layers/embedding.rs:449
  conv2d      crates/st-nn/src/layers/conv.rs:951-969,2602  (im2col GEMM; weights (OC, IC*kh*kw))
  max_pool2x2 crates/st-nn/src/layers/conv.rs (Pool2d)
  attention   crates/st-tensor/src/pure.rs:4083-4157        (scaled_dot_attention_with_backend)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import attention as _attn
from ..ops import conv as _conv
from ..ops import elementwise as _ew
from ..ops import gemm as _gemm
from ..ops import norm as _norm

#: kernel-path calls per op since import (tests assert that the public API reached the kernels)
launch_counts = {"linear": 0, "layer_norm": 0, "embedding": 0, "conv2d": 0, "max_pool2x2": 0, "attention": 0,
                 "gelu": 0}

bf16_of = _gemm.cached_bf16


def _on_kernels(*ts: Optional[torch.Tensor]) -> bool:
    return all(t is None or t.is_cuda for t in ts) and any(t is not None for t in ts)


# ------------------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act):
        xb = x.detach().to(torch.bfloat16).contiguous()
        wb = bf16_of(weight)                      # (in, out): the B operand in MN-major form
        bb = None if bias is None else bf16_of(bias).reshape(-1)
        pre = None
        if act == "gelu":
            pre = torch.empty((xb.shape[0], wb.shape[1]), dtype=torch.bfloat16, device=x.device)
        y = _gemm.gemm(xb, wb, b_mn=True, bias=bb, out_dtype=torch.float32, act=act, aux_out=pre)
        if act == "relu":
            pre = y
        ctx.save_for_backward(xb, wb, pre)
        ctx.act, ctx.has_bias = act, bias is not None
        launch_counts["linear"] += 1
        return y

    @staticmethod
    def backward(ctx, dy):
        xb, wb, pre = ctx.saved_tensors
        dyf = dy
        if ctx.act == "gelu":
            dyf = dy * _gemm.gelu_tanh_grad(pre.float())
        elif ctx.act == "relu":
            dyf = dy * (pre > 0)
        dyb = dyf.to(torch.bfloat16).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _gemm.gemm(dyb, wb, out_dtype=torch.float32)                    # dy · Wᵀ  (W is [N=in, K=out])
        if ctx.needs_input_grad[1]:
            dw = _gemm.gemm(xb, dyb, a_mn=True, b_mn=True, out_dtype=torch.float32)   # xᵀ · dy → (in, out)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _ew.colsum(dyb).reshape(1, -1)
        return dx, dw, db, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ weight + bias)`` with ``weight`` stored ``(in, out)`` and ``bias`` ``(1, out)``;
    ``act`` is ``None``, ``"relu"`` or ``"gelu"`` (tanh form), fused into the GEMM epilogue on CUDA."""
    if _on_kernels(x, weight, bias):
        return _LinearFn.apply(x, weight, bias, act)
    y = x @ weight
    if bias is not None:
        y = y + bias
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = F.gelu(y, approximate="tanh")
    return y


# ------------------------------------------------------------------------------------------------------
# layer norm (optionally with a residual added first)
# ------------------------------------------------------------------------------------------------------
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, residual):
        xb = x.detach().to(torch.bfloat16).contiguous()
        rb = None if residual is None else residual.detach().to(torch.bfloat16).contiguous()
        gb, bb = bf16_of(gamma).reshape(-1), bf16_of(beta).reshape(-1)
        y, summed, mean, rstd = _norm.norm_forward(xb, gb, bb, float(eps), False, rb)
        ctx.save_for_backward(xb if summed is None else summed, gb, mean, rstd)
        ctx.has_residual = residual is not None
        ctx.pshape = gamma.shape
        launch_counts["layer_norm"] += 1
        return y.float()

    @staticmethod
    def backward(ctx, dy):
        xin, gb, mean, rstd = ctx.saved_tensors
        dyb = dy.to(torch.bfloat16).contiguous()
        dg = torch.empty(xin.shape[1], dtype=torch.float32, device=xin.device)
        db = torch.empty_like(dg)
        dx = _norm.norm_backward(dyb, xin, gb, mean, rstd, False, dg, db, False).float()
        return dx, dg.reshape(ctx.pshape), db.reshape(ctx.pshape), None, (dx if ctx.has_residual else None)


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
               residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise ``gamma * (v - mean) / sqrt(var + eps) + beta`` with ``v = x (+ residual)``."""
    if _on_kernels(x, gamma, beta, residual) and x.shape[-1] % 8 == 0:
        return _LayerNormFn.apply(x, gamma, beta, eps, residual)
    v = x if residual is None else x + residual
    return F.layer_norm(v, (v.shape[-1],), gamma.reshape(-1), beta.reshape(-1), eps)


# ------------------------------------------------------------------------------------------------------
# embedding
# ------------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        wb = bf16_of(weight)
        out = _ew.embedding_forward(ids, wb)
        ctx.save_for_backward(ids)
        ctx.wshape = weight.shape
        launch_counts["embedding"] += 1
        return out.float()

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        dw = torch.zeros(ctx.wshape, dtype=torch.float32, device=dy.device)
        _ew.embedding_backward(ids, dy.to(torch.bfloat16).contiguous(), dw)
        return None, dw


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``weight[ids]`` for integer ``ids`` of any shape → ``[ids.numel(), dim]``."""
    ids = ids.reshape(-1)
    if _on_kernels(weight) and ids.is_cuda and weight.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids.to(torch.int64), weight)
    return weight[ids]


# ------------------------------------------------------------------------------------------------------
# convolution
# ------------------------------------------------------------------------------------------------------
class _Conv3x3Fn(torch.autograd.Function):
    """3x3, stride 1, padding 1: implicit GEMM (4-D TMA boxes) on the tcgen05 kernel; bias and ReLU fused."""

    @staticmethod
    def forward(ctx, x_nchw, weight, bias, relu):
        N, C, H, W = x_nchw.shape
        OC = weight.shape[0]
        xn = x_nchw.detach().permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()          # NHWC
        w_tap = _conv.to_tap_major(bf16_of(weight), C)
        bb = None if bias is None else bf16_of(bias).reshape(-1)
        y = _conv.conv3x3(xn, w_tap, bb, relu=relu)                                       # [N, H, W, OC]
        ctx.save_for_backward(xn, w_tap, y if relu else None)
        ctx.relu, ctx.has_bias, ctx.C = relu, bias is not None, C
        launch_counts["conv2d"] += 1
        return y.permute(0, 3, 1, 2).float()

    @staticmethod
    def backward(ctx, dy_nchw):
        xn, w_tap, y = ctx.saved_tensors
        N, H, W, C = xn.shape
        OC = w_tap.shape[0]
        d = dy_nchw.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        if ctx.relu:
            d = torch.where(y > 0, d, torch.zeros_like(d))
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw_tap = torch.zeros((OC, 9 * C), dtype=torch.float32, device=xn.device)
            _conv.conv3x3_wgrad(d, xn, dw_tap)
            dw = _conv.from_tap_major(dw_tap, C)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _ew.colsum(d.reshape(-1, OC)).reshape(1, OC)
        if ctx.needs_input_grad[0]:
            dxn = _conv.conv3x3(d, _conv.dgrad_weights(w_tap, C))                        # [N, H, W, C]
            dx = dxn.permute(0, 3, 1, 2).float()
        return dx, dw, db, None


class _ConvGemmFn(torch.autograd.Function):
    """Any kernel / stride / padding / dilation: explicit im2col (``unfold``), then the tcgen05 GEMM for the
    forward, the data gradient (followed by ``fold``) and the weight gradient."""

    @staticmethod
    def forward(ctx, x_nchw, weight, bias, kernel, stride, padding, dilation):
        N, C, H, W = x_nchw.shape
        OC = weight.shape[0]
        cols = F.unfold(x_nchw.detach().to(torch.bfloat16), kernel, dilation, padding, stride)   # [N, C*kh*kw, L]
        L = cols.shape[-1]
        cols2 = cols.transpose(1, 2).reshape(N * L, -1).contiguous()                    # [N*L, C*kh*kw]
        wb = bf16_of(weight)                                                            # [OC, C*kh*kw]
        bb = None if bias is None else bf16_of(bias).reshape(-1)
        y = _gemm.gemm(cols2, wb, bias=bb, out_dtype=torch.float32)                     # [N*L, OC]
        ctx.save_for_backward(cols2, wb)
        ctx.geom = (N, C, H, W, OC, L, kernel, stride, padding, dilation)
        ctx.has_bias = bias is not None
        launch_counts["conv2d"] += 1
        oh = (H + 2 * padding[0] - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1
        return y.reshape(N, L, OC).permute(0, 2, 1).reshape(N, OC, oh, L // oh)

    @staticmethod
    def backward(ctx, dy):
        cols2, wb = ctx.saved_tensors
        N, C, H, W, OC, L, kernel, stride, padding, dilation = ctx.geom
        d2 = dy.reshape(N, OC, L).permute(0, 2, 1).reshape(N * L, OC).to(torch.bfloat16).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw = _gemm.gemm(d2, cols2, a_mn=True, b_mn=True, out_dtype=torch.float32)   # [OC, C*kh*kw]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _ew.colsum(d2).reshape(1, OC)
        if ctx.needs_input_grad[0]:
            dcols = _gemm.gemm(d2, wb, b_mn=True, out_dtype=torch.float32)              # [N*L, C*kh*kw]
            dcols = dcols.reshape(N, L, -1).transpose(1, 2)
            dx = F.fold(dcols, (H, W), kernel, dilation, padding, stride)
        return dx, dw, db, None, None, None, None


def conv2d(x_nchw: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], kernel, stride=(1, 1),
           padding=(0, 0), dilation=(1, 1), relu: bool = False) -> torch.Tensor:
    """2-D convolution of ``[N, C, H, W]`` with ``weight`` ``(OC, C*kh*kw)`` (K ordered ``[ic][kh][kw]``)
    and ``bias`` ``(1, OC)``."""
    kernel, stride, padding, dilation = tuple(kernel), tuple(stride), tuple(padding), tuple(dilation)
    N, C, H, W = x_nchw.shape
    OC = weight.shape[0]
    if _on_kernels(x_nchw, weight, bias):
        if kernel == (3, 3) and stride == (1, 1) and padding == (1, 1) and dilation == (1, 1) and OC % 8 == 0 \
                and C % 8 == 0:
            return _Conv3x3Fn.apply(x_nchw, weight, bias, relu)
        y = _ConvGemmFn.apply(x_nchw, weight, bias, kernel, stride, padding, dilation)
        return torch.relu(y) if relu else y
    y = F.conv2d(x_nchw, weight.reshape(OC, C, *kernel), None if bias is None else bias.reshape(-1), stride, padding,
                 dilation)
    return torch.relu(y) if relu else y


# ------------------------------------------------------------------------------------------------------
# pooling
# ------------------------------------------------------------------------------------------------------
class _MaxPool2x2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_nchw):
        N, C, H, W = x_nchw.shape
        xn = x_nchw.detach().permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        y, idx = _conv.maxpool2(xn)
        ctx.save_for_backward(idx)
        ctx.hw = (H, W)
        launch_counts["max_pool2x2"] += 1
        return y.permute(0, 3, 1, 2).float()

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        d = dy.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        dx = _conv.maxpool2_backward(d, idx, *ctx.hw)
        return dx.permute(0, 3, 1, 2).float()


def max_pool2x2(x_nchw: torch.Tensor) -> torch.Tensor:
    """2x2 max-pool with stride 2 of ``[N, C, H, W]`` (H, W, C even on the kernel path)."""
    N, C, H, W = x_nchw.shape
    if _on_kernels(x_nchw) and H % 2 == 0 and W % 2 == 0 and C % 2 == 0:
        return _MaxPool2x2Fn.apply(x_nchw)
    return F.max_pool2d(x_nchw, 2, 2)


# ------------------------------------------------------------------------------------------------------
# attention (per-context, additive biases)
# ------------------------------------------------------------------------------------------------------
def scaled_dot_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                         z_bias: Optional[torch.Tensor] = None, attn_bias: Optional[torch.Tensor] = None,
                         causal: bool = False, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(scale * q·kᵀ + z_bias[ctx, key] + attn_bias[ctx, query, key]) · v`` per context.

    ``q``, ``k``, ``v``: ``[contexts, sequence, head_dim]``; ``z_bias``: ``[contexts, sequence]``; ``attn_bias``:
    ``[contexts, sequence, sequence]``; ``lengths``: valid keys per context (int).  Differentiable in q, k, v."""
    ctxs, S, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if _on_kernels(q, k, v) and D in (64, 128) and v.shape[-1] == D:
        launch_counts["attention"] += 1
        o = _attn.attention(q.to(torch.bfloat16).unsqueeze(2), k.to(torch.bfloat16).unsqueeze(2),
                            v.to(torch.bfloat16).unsqueeze(2), causal=causal, scale=scale,
                            key_bias=z_bias, attn_bias=None if attn_bias is None else attn_bias.unsqueeze(1),
                            lengths=lengths)
        return o.squeeze(2).to(q.dtype)
    o, _ = _attn.attention_reference(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), causal, scale, key_bias=z_bias,
                                     attn_bias=attn_bias, lengths=lengths)
    return o.squeeze(2).to(q.dtype)
