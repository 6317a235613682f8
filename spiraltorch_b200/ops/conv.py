"""3x3 convolution (stride 1, padding 1) and pooling on NHWC bf16 activations
(``csrc/conv/conv.cu``: implicit GEMM on the tcgen05 kernel, bias + ReLU fused in the epilogue).

Weights live in the reference layout ``(out_channels, in_channels*kh*kw)`` with the K axis ordered
``[ic][kh][kw]`` (crates/st-nn/src/layers/conv.rs:951-969); the kernels want ``[tap][ic]`` (tap-major)
so :func:`to_tap_major` / :func:`from_tap_major` convert at the boundary (checkpoints keep the
reference layout).  CPU tensors use ``torch.nn.functional.conv2d`` on the same data (the oracle).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from . import native
from .gemm import gemm

launch_count = 0


class _ConvArgs(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("aux_in", ctypes.c_void_p)] + [(n, ctypes.c_int) for n in ("N", "H", "W", "C", "OC", "act")]


class _WgradArgs(ctypes.Structure):
    _fields_ = [("dy", ctypes.c_void_p), ("x", ctypes.c_void_p), ("dw", ctypes.c_void_p)] + \
               [(n, ctypes.c_int) for n in ("N", "H", "W", "C", "OC", "splits")]


def to_tap_major(w_ref: torch.Tensor, ic: int) -> torch.Tensor:
    """``[OC, IC*9]`` ([ic][kh][kw]) → ``[OC, 9*IC]`` ([kh][kw][ic])."""
    oc = w_ref.shape[0]
    return w_ref.reshape(oc, ic, 9).permute(0, 2, 1).reshape(oc, 9 * ic).contiguous()


def from_tap_major(w_tap: torch.Tensor, ic: int) -> torch.Tensor:
    oc = w_tap.shape[0]
    return w_tap.reshape(oc, 9, ic).permute(0, 2, 1).reshape(oc, ic * 9).contiguous()


def dgrad_weights(w_tap: torch.Tensor, ic: int) -> torch.Tensor:
    """Weights of the data-gradient convolution: ``Wt[ic][kh'][kw'][oc] = W[oc][2-kh'][2-kw'][ic]``."""
    oc = w_tap.shape[0]
    return w_tap.reshape(oc, 3, 3, ic).flip(1, 2).permute(3, 1, 2, 0).reshape(ic, 9 * oc).contiguous()


def implicit_ok(N: int, H: int, W: int, C: int, OC: int, pixels: int = 128) -> bool:
    """Whether the implicit-GEMM kernels take this geometry: channels in 64-blocks, and a pixel block of
    ``pixels`` output positions (128 forward / data gradient, 64 weight gradient) must be W columns x whole rows
    x whole images.  Other shapes go through the explicit im2col + GEMM path."""
    if C % 64 != 0 or OC % 8 != 0 or W <= 0 or W > pixels or pixels % W != 0:
        return False
    hb, nb = pixels // W, 1
    if hb > H:
        if hb % H != 0:
            return False
        nb, hb = hb // H, H
    return H % hb == 0 and N % nb == 0


def _conv_ref(x, w_tap, bias, act, aux_in):
    N, H, W, C = x.shape
    oc = w_tap.shape[0]
    w4 = w_tap.float().reshape(oc, 3, 3, C).permute(0, 3, 1, 2)
    y = F.conv2d(x.float().permute(0, 3, 1, 2), w4, None if bias is None else bias.float(), padding=1)
    y = y.permute(0, 2, 3, 1)
    if act == 1:
        y = torch.relu(y)
    elif act == 4:
        y = torch.where(aux_in.float().reshape(y.shape) > 0, y, torch.zeros_like(y))
    return y.to(x.dtype).contiguous()


def conv3x3(x: torch.Tensor, w_tap: torch.Tensor, bias: Optional[torch.Tensor] = None, *, relu: bool = False,
            relu_mask_of: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x`` NHWC ``[N,H,W,C]``, ``w_tap`` ``[OC, 9*C]`` → NHWC ``[N,H,W,OC]``.
    ``relu_mask_of`` (same shape as the output) zeroes the output where that tensor is <= 0
    (used by the data gradient)."""
    global launch_count
    N, H, W, C = x.shape
    OC = w_tap.shape[0]
    act = 4 if relu_mask_of is not None else (1 if relu else 0)
    if not native.use_native(x):
        return _conv_ref(x, w_tap, bias, act, relu_mask_of)
    native.require_cuda("conv3x3", x, w_tap, bias, relu_mask_of)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and w_tap.dtype == torch.bfloat16 and w_tap.is_contiguous()
    assert w_tap.shape[1] == 9 * C, "weights must be [OC, 9*C] (tap-major)"
    assert relu_mask_of is None or relu_mask_of.shape == (N, H, W, OC)
    if not implicit_ok(N, H, W, C, OC, 128):
        # few input channels (the RGB stem) or a geometry the 4-D TMA boxes cannot tile: explicit im2col
        # with K padded to a multiple of 32, then the plain GEMM
        kpad = (9 * C + 31) // 32 * 32
        col = torch.empty((N * H * W, kpad), dtype=torch.bfloat16, device=x.device)
        st = native.lib().st_im2col3x3_small(native.ptr(x), native.ptr(col), ctypes.c_int(N), ctypes.c_int(H),
                                             ctypes.c_int(W), ctypes.c_int(C), ctypes.c_int(kpad),
                                             native.stream_ptr(x.device))
        native.check(st, "st_im2col3x3_small")
        launch_count += 1
        wp = torch.zeros((OC, kpad), dtype=torch.bfloat16, device=x.device)
        wp[:, : 9 * C] = w_tap
        if relu_mask_of is not None:
            y = gemm(col, wp, bias=bias, act="relu_bwd", aux_in=relu_mask_of.reshape(N * H * W, OC))
        else:
            y = gemm(col, wp, bias=bias, act="relu" if relu else None)
        return y.view(N, H, W, OC)
    y = torch.empty((N, H, W, OC), dtype=torch.bfloat16, device=x.device)
    a = _ConvArgs()
    a.x, a.w, a.y = x.data_ptr(), w_tap.data_ptr(), y.data_ptr()
    a.bias = None if bias is None else bias.data_ptr()
    a.aux_in = None if relu_mask_of is None else relu_mask_of.data_ptr()
    a.N, a.H, a.W, a.C, a.OC, a.act = N, H, W, C, OC, act
    native.check(native.lib().st_conv3x3_fwd(ctypes.byref(a), native.stream_ptr(x.device)), "st_conv3x3_fwd")
    launch_count += 1
    return y


def conv3x3_wgrad(dy: torch.Tensor, x: torch.Tensor, dw_tap: torch.Tensor) -> None:
    """``dw_tap[oc, tap, ic] += sum_p dy[p, oc] * x[p + tap, ic]`` (fp32 accumulation)."""
    global launch_count
    N, H, W, C = x.shape
    OC = dy.shape[-1]
    if not native.use_native(x):
        xf = x.float().permute(0, 3, 1, 2)
        cols = F.unfold(xf, 3, padding=1).reshape(N, C, 9, H * W).permute(0, 3, 2, 1).reshape(N * H * W, 9 * C)
        dw_tap += dy.float().reshape(-1, OC).t() @ cols
        return
    native.require_cuda("conv3x3_wgrad", dy, x, dw_tap)
    assert dw_tap.dtype == torch.float32 and dw_tap.is_contiguous() and dw_tap.numel() == OC * 9 * C
    assert dy.shape[:3] == x.shape[:3] and dy.is_contiguous() and x.is_contiguous()
    if not implicit_ok(N, H, W, C, OC, 64):
        kpad = (9 * C + 31) // 32 * 32
        col = torch.empty((N * H * W, kpad), dtype=torch.bfloat16, device=x.device)
        st = native.lib().st_im2col3x3_small(native.ptr(x), native.ptr(col), ctypes.c_int(N), ctypes.c_int(H),
                                             ctypes.c_int(W), ctypes.c_int(C), ctypes.c_int(kpad),
                                             native.stream_ptr(x.device))
        native.check(st, "st_im2col3x3_small")
        launch_count += 1
        tmp = gemm(dy.reshape(-1, OC), col, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dw_tap += tmp[:, : 9 * C]
        return
    a = _WgradArgs()
    a.dy, a.x, a.dw = dy.data_ptr(), x.data_ptr(), dw_tap.data_ptr()
    # one CTA per (tap, tile) when the summation order must be fixed; 0 lets the launcher split the pixel loop
    a.N, a.H, a.W, a.C, a.OC, a.splits = N, H, W, C, OC, (1 if native.deterministic_reduction() else 0)
    native.check(native.lib().st_conv3x3_wgrad(ctypes.byref(a), native.stream_ptr(x.device)), "st_conv3x3_wgrad")
    launch_count += 1


def maxpool2(x: torch.Tensor):
    """2x2 max pool on NHWC; returns ``(y, argmax)``."""
    global launch_count
    N, H, W, C = x.shape
    if not native.use_native(x):
        xv = x.reshape(N, H // 2, 2, W // 2, 2, C).permute(0, 1, 3, 5, 2, 4).reshape(N, H // 2, W // 2, C, 4)
        y, idx = xv.float().max(-1)
        return y.to(x.dtype), idx.to(torch.uint8)
    y = torch.empty((N, H // 2, W // 2, C), dtype=x.dtype, device=x.device)
    idx = torch.empty((N, H // 2, W // 2, C), dtype=torch.uint8, device=x.device)
    st = native.lib().st_maxpool2_fwd(native.ptr(x), native.ptr(y), native.ptr(idx), ctypes.c_int(N), ctypes.c_int(H),
                                      ctypes.c_int(W), ctypes.c_int(C), native.stream_ptr(x.device))
    native.check(st, "st_maxpool2_fwd")
    launch_count += 1
    return y, idx


def maxpool2_backward(dy: torch.Tensor, idx: torch.Tensor, H: int, W: int) -> torch.Tensor:
    global launch_count
    N, OH, OW, C = dy.shape
    if not native.use_native(dy):
        onehot = F.one_hot(idx.long(), 4).to(dy.dtype) * dy[..., None]
        return onehot.reshape(N, OH, OW, C, 2, 2).permute(0, 1, 4, 2, 5, 3).reshape(N, H, W, C).contiguous()
    dx = torch.empty((N, H, W, C), dtype=dy.dtype, device=dy.device)
    st = native.lib().st_maxpool2_bwd(native.ptr(dy.contiguous()), native.ptr(idx), native.ptr(dx), ctypes.c_int(N),
                                      ctypes.c_int(H), ctypes.c_int(W), ctypes.c_int(C), native.stream_ptr(dy.device))
    native.check(st, "st_maxpool2_bwd")
    launch_count += 1
    return dx


def global_avgpool(x: torch.Tensor) -> torch.Tensor:
    global launch_count
    N, H, W, C = x.shape
    if not native.use_native(x):
        return x.float().mean((1, 2)).to(x.dtype)
    y = torch.empty((N, C), dtype=x.dtype, device=x.device)
    st = native.lib().st_avgpool_fwd(native.ptr(x), native.ptr(y), ctypes.c_int(N), ctypes.c_int(H * W), ctypes.c_int(C),
                                     native.stream_ptr(x.device))
    native.check(st, "st_avgpool_fwd")
    launch_count += 1
    return y


def global_avgpool_backward(dy: torch.Tensor, H: int, W: int) -> torch.Tensor:
    global launch_count
    N, C = dy.shape
    if not native.use_native(dy):
        return (dy.float() / (H * W))[:, None, None, :].expand(N, H, W, C).to(dy.dtype).contiguous()
    dx = torch.empty((N, H, W, C), dtype=dy.dtype, device=dy.device)
    st = native.lib().st_avgpool_bwd(native.ptr(dy.contiguous()), native.ptr(dx), ctypes.c_int(N), ctypes.c_int(H * W),
                                     ctypes.c_int(C), native.stream_ptr(dy.device))
    native.check(st, "st_avgpool_bwd")
    launch_count += 1
    return dx
