"""Fused optimizer kernels on flat buffers (``csrc/optim/optim.cu``): AdamW with fp32 master
weights, SGD-momentum, gradient sum of squares + clip coefficient, and the Amegagrad
hypergrad / realgrad tape operations.

Reference parity: ``AmegaHypergrad`` / ``AmegaRealgrad`` (crates/st-tensor/src/pure.rs:8452,
9847, 10585-10815), ``apply_adam_slice`` (crates/st-nn/src/zspace_coherence/vae.rs:303-334).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import native

launch_count = 0


def adamw_reference(grad, master, m, v, weight, lr, beta1, beta2, eps, wd, step, grad_scale, zero_grad):
    g = grad.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mhat = m / (1 - beta1 ** step)
    vhat = v / (1 - beta2 ** step)
    master.sub_(lr * (mhat / (vhat.sqrt() + eps) + wd * master))
    if weight is not None:
        weight.copy_(master.to(weight.dtype))
    if zero_grad:
        grad.zero_()


def adamw_step(grad: torch.Tensor, master: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
               weight: Optional[torch.Tensor], *, lr: float, beta1: float = 0.9, beta2: float = 0.95,
               eps: float = 1e-8, weight_decay: float = 0.0, step: int = 1, grad_scale: float = 1.0,
               scale_tensor: Optional[torch.Tensor] = None, zero_grad: bool = False) -> None:
    """One fused AdamW step over flat, equally sized buffers.

    ``grad`` fp32 or bf16; ``master``/``m``/``v`` fp32; ``weight`` bf16 working copy (optional).
    The gradient is multiplied by ``grad_scale * scale_tensor[0]`` (device scalar, e.g. the clip
    coefficient) so no host synchronisation is needed.
    """
    global launch_count
    n = grad.numel()
    if not native.use_native(grad):
        gs = grad_scale * (float(scale_tensor) if scale_tensor is not None else 1.0)
        adamw_reference(grad, master, m, v, weight, lr, beta1, beta2, eps, weight_decay, step, gs, zero_grad)
        return
    assert master.dtype == m.dtype == v.dtype == torch.float32
    assert grad.dtype in (torch.float32, torch.bfloat16)
    assert weight is None or weight.dtype == torch.bfloat16
    for t in (grad, master, m, v, weight):
        assert t is None or (t.is_contiguous() and t.numel() == n)
    st = native.lib().st_adamw(
        native.ptr(grad), ctypes.c_int(int(grad.dtype == torch.bfloat16)), native.ptr(master), native.ptr(m),
        native.ptr(v), native.ptr(weight), ctypes.c_longlong(n), ctypes.c_float(lr), ctypes.c_float(beta1),
        ctypes.c_float(beta2), ctypes.c_float(eps), ctypes.c_float(weight_decay), ctypes.c_int(step),
        ctypes.c_float(grad_scale), native.ptr(scale_tensor), ctypes.c_int(int(zero_grad)),
        native.stream_ptr(grad.device))
    native.check(st, "st_adamw")
    launch_count += 1


def sgd_step(grad, master, momentum_buf, weight, *, lr: float, momentum: float = 0.0,
             weight_decay: float = 0.0, nesterov: bool = False, grad_scale: float = 1.0,
             scale_tensor=None, zero_grad: bool = False) -> None:
    global launch_count
    n = grad.numel()
    if not native.use_native(grad):
        gs = grad_scale * (float(scale_tensor) if scale_tensor is not None else 1.0)
        g = grad.float() * gs + weight_decay * master
        if momentum_buf is not None:
            momentum_buf.mul_(momentum).add_(g)
            g = g + momentum * momentum_buf if nesterov else momentum_buf
        master.sub_(lr * g)
        if weight is not None:
            weight.copy_(master.to(weight.dtype))
        if zero_grad:
            grad.zero_()
        return
    st = native.lib().st_sgd(
        native.ptr(grad), ctypes.c_int(int(grad.dtype == torch.bfloat16)), native.ptr(master),
        native.ptr(momentum_buf), native.ptr(weight), ctypes.c_longlong(n), ctypes.c_float(lr),
        ctypes.c_float(momentum), ctypes.c_float(weight_decay), ctypes.c_float(grad_scale),
        native.ptr(scale_tensor), ctypes.c_int(int(nesterov)), ctypes.c_int(int(zero_grad)),
        native.stream_ptr(grad.device))
    native.check(st, "st_sgd")
    launch_count += 1


def sumsq(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[0] += sum(x^2)`` (fp32 device scalar)."""
    global launch_count
    if not native.use_native(x):
        out += x.float().pow(2).sum()
        return out
    st = native.lib().st_sumsq(native.ptr(x), ctypes.c_int(int(x.dtype == torch.bfloat16)),
                               ctypes.c_longlong(x.numel()), native.ptr(out), native.stream_ptr(x.device))
    native.check(st, "st_sumsq")
    launch_count += 1
    return out


def clip_coef(sumsq_t: torch.Tensor, norm_scale: float, max_norm: float, coef: torch.Tensor,
              norm_out: Optional[torch.Tensor] = None) -> None:
    """``coef[0] = min(1, max_norm / (sqrt(sumsq) * norm_scale + 1e-6))`` on the device."""
    global launch_count
    if not native.use_native(sumsq_t):
        nrm = math.sqrt(float(sumsq_t)) * norm_scale
        if norm_out is not None:
            norm_out.fill_(nrm)
        coef.fill_(min(1.0, max_norm / (nrm + 1e-6)) if max_norm > 0 else 1.0)
        return
    st = native.lib().st_clip_coef(native.ptr(sumsq_t), ctypes.c_float(norm_scale), ctypes.c_float(max_norm),
                                   native.ptr(coef), native.ptr(norm_out), native.stream_ptr(sumsq_t.device))
    native.check(st, "st_clip_coef")
    launch_count += 1


# ---- Amegagrad tapes ------------------------------------------------------------------

def porous_mix(x: torch.Tensor, saturation: float, porosity: float) -> torch.Tensor:
    """Topos saturation (crates/st-tensor/src/pure/topos.rs:169-188), vectorised."""
    x = torch.where(torch.isfinite(x), x, torch.zeros_like(x))
    if saturation <= 0:
        return torch.zeros_like(x)
    limit = abs(saturation)
    mag = x.abs()
    if porosity <= 1.1920929e-7:
        over = torch.sign(x) * limit
    else:
        bleed = (mag - limit) / (mag + limit)
        absorb = min(porosity * 0.25, 1.0)
        over = torch.sign(x) * (limit * (1.0 - absorb * bleed.clamp(max=1.0))).clamp(min=0.0)
    return torch.where(mag <= limit, x, over)


def hyper_accumulate(g: torch.Tensor, v: torch.Tensor, curvature: float, tol: float, saturation: float,
                     porosity: float, conformal: bool = True, scale: float = 1.0) -> None:
    global launch_count
    if not native.use_native(g):
        x = v.float() * scale
        upd = x / (1.0 - curvature * x * x).abs().clamp(min=tol) if conformal else x
        g.copy_(porous_mix(g + upd, saturation, porosity))
        return
    v = v.float().contiguous()
    native.same_device("hyper_accumulate", g, v)
    st = native.lib().st_hyper_accumulate(native.ptr(g), native.ptr(v), ctypes.c_longlong(g.numel()),
                                          ctypes.c_float(curvature), ctypes.c_float(tol),
                                          ctypes.c_float(saturation), ctypes.c_float(porosity),
                                          ctypes.c_int(int(conformal)), ctypes.c_float(scale),
                                          native.stream_ptr(g.device))
    native.check(st, "st_hyper_accumulate")
    launch_count += 1


def project_to_poincare(x: torch.Tensor, curvature: float) -> torch.Tensor:
    global launch_count
    if curvature >= 0:
        raise ValueError(f"curvature must be negative for the Poincare projection, got {curvature}")
    if not native.use_native(x):
        norm = x.float().pow(2).sum(-1, keepdim=True).sqrt()
        factor = torch.where(norm > 0, torch.tanh(norm / math.sqrt(-curvature)) / norm.clamp(min=1e-38),
                             torch.ones_like(norm))
        return (x.float() * factor).to(x.dtype)
    xf = x.float().contiguous()
    y = torch.empty_like(xf)
    st = native.lib().st_poincare_project(native.ptr(xf), native.ptr(y), ctypes.c_int(xf.shape[0]),
                                          ctypes.c_int(xf.shape[1]), ctypes.c_float(curvature),
                                          native.stream_ptr(x.device))
    native.check(st, "st_poincare_project")
    launch_count += 1
    return y


def hyper_apply(w: torch.Tensor, g: Optional[torch.Tensor], g_real: Optional[torch.Tensor], *,
                curvature: float, lr: float, lr_real: float, tol: float, saturation: float,
                porosity: float) -> None:
    """In-place Amegagrad step on fp32 ``w`` ``[rows, cols]``: hypergrad update + topos saturation
    + row-wise Poincaré projection, then the realgrad update on the projected weights; both
    accumulators are reset."""
    global launch_count
    rows, cols = w.shape
    if not native.use_native(w):
        if g is not None:
            step = lr / (1.0 - curvature * w * w).abs().clamp(min=tol)
            w.copy_(project_to_poincare(porous_mix(w - step * g, saturation, porosity), curvature))
            g.zero_()
        if g_real is not None:
            w.sub_(lr_real * g_real)
            g_real.zero_()
        return
    assert w.dtype == torch.float32 and w.is_contiguous()
    native.same_device("hyper_apply", w, g, g_real)
    st = native.lib().st_hyper_apply(native.ptr(w), native.ptr(g), native.ptr(g_real), ctypes.c_int(rows),
                                     ctypes.c_int(cols), ctypes.c_float(curvature), ctypes.c_float(lr),
                                     ctypes.c_float(lr_real), ctypes.c_float(tol), ctypes.c_float(saturation),
                                     ctypes.c_float(porosity), native.stream_ptr(w.device))
    native.check(st, "st_hyper_apply")
    launch_count += 1
