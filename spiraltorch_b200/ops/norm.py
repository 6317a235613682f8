"""LayerNorm / RMSNorm forward and backward (``csrc/norm/norm.cu``).

bf16 activations, fp32 statistics; parameter gradients are produced in fp32 and either
returned (cast to the parameter dtype) or accumulated into ``param.main_grad`` when that
attribute exists (fp32 gradient accumulation across micro-batches).

Reference parity: ``Tensor::layer_norm_affine`` / ``layer_norm_affine_add``
(crates/st-tensor/src/pure.rs:3702-4058), ``nn.LayerNorm`` (crates/st-nn/src/layers/normalization.rs:352).
RMSNorm has no counterpart in the reference.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

launch_count = 0
_scratch: dict = {}


def _get_scratch(device, elems: int) -> torch.Tensor:
    buf = _scratch.get(device)
    if buf is None or buf.numel() < elems:
        buf = torch.empty(max(elems, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def norm_reference(x, gamma, beta, eps, rms, residual=None):
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    if rms:
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        y = xf * rstd * gamma.float()
        mean = torch.zeros_like(rstd)
    else:
        mean = xf.mean(-1, keepdim=True)
        var = (xf - mean).pow(2).mean(-1, keepdim=True)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean) * rstd * gamma.float()
        if beta is not None:
            y = y + beta.float()
    return y, xf, mean.squeeze(-1), rstd.squeeze(-1)


def norm_forward(x2: torch.Tensor, gamma, beta, eps: float, rms: bool, residual=None, out=None):
    """x2: [rows, d] bf16.  Returns (y, summed_input_or_None, mean, rstd); ``out`` (contiguous, same shape and
    dtype) receives y when given."""
    global launch_count
    rows, d = x2.shape
    if out is not None:
        assert out.shape == x2.shape and out.dtype == x2.dtype and out.is_contiguous() and out.device == x2.device
    if not native.use_native(x2):
        y, xs, mean, rstd = norm_reference(x2, gamma, beta, eps, rms, residual)
        y = y.to(x2.dtype)
        if out is not None:
            y = out.copy_(y)
        return y, (xs.to(x2.dtype) if residual is not None else None), mean, rstd
    y = torch.empty_like(x2) if out is None else out
    s = torch.empty_like(x2) if residual is not None else None
    mean = torch.empty(rows, dtype=torch.float32, device=x2.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    st = native.lib().st_norm_fwd(
        ctypes.c_int(int(rms)), native.ptr(x2), native.ptr(residual), native.ptr(gamma), native.ptr(beta),
        native.ptr(y), native.ptr(s), native.ptr(mean), native.ptr(rstd), ctypes.c_int(rows),
        ctypes.c_int(d), ctypes.c_float(eps), native.stream_ptr(x2.device))
    native.check(st, "st_norm_fwd")
    launch_count += 1
    return y, s, mean, rstd


def norm_backward(dy2, x2, gamma, mean, rstd, rms: bool, dgamma: torch.Tensor,
                  dbeta: Optional[torch.Tensor], accumulate: bool, dres=None, out=None):
    """Writes dx (returned; into ``out`` when given) and fp32 dgamma/dbeta (in place, ``+=`` when ``accumulate``)."""
    global launch_count
    rows, d = x2.shape
    if out is not None:
        assert out.shape == x2.shape and out.dtype == x2.dtype and out.is_contiguous() and out.device == x2.device
    if not native.use_native(x2):
        xf, dyf, g = x2.float(), dy2.float(), gamma.float()
        xh = (xf - (0 if rms else mean.unsqueeze(-1))) * rstd.unsqueeze(-1)
        gy = dyf * g
        m1 = (gy * xh).mean(-1, keepdim=True)
        m2 = 0 if rms else gy.mean(-1, keepdim=True)
        dx = rstd.unsqueeze(-1) * (gy - m2 - xh * m1)
        if dres is not None:
            dx = dx + dres.float()
        dg = (dyf * xh).sum(0)
        dgamma.copy_(dgamma + dg if accumulate else dg)
        if dbeta is not None:
            db = dyf.sum(0)
            dbeta.copy_(dbeta + db if accumulate else db)
        dx = dx.to(x2.dtype)
        return dx if out is None else out.copy_(dx)
    dx = torch.empty_like(x2) if out is None else out
    lib = native.lib()
    lib.st_norm_bwd_scratch_elems.restype = ctypes.c_longlong
    need = lib.st_norm_bwd_scratch_elems(ctypes.c_int(rows), ctypes.c_int(d))
    scratch = _get_scratch(x2.device, int(need))
    st = lib.st_norm_bwd(
        ctypes.c_int(int(rms)), native.ptr(dy2), native.ptr(x2), native.ptr(gamma), native.ptr(mean),
        native.ptr(rstd), native.ptr(dres), native.ptr(dx), native.ptr(dgamma), native.ptr(dbeta),
        ctypes.c_int(int(accumulate)), native.ptr(scratch), ctypes.c_int(rows), ctypes.c_int(d),
        native.stream_ptr(x2.device))
    native.check(st, "st_norm_bwd")
    launch_count += 2 if rms or dbeta is None else 3
    return dx


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, _, mean, rstd = norm_forward(x2, gamma, beta, eps, rms)
        ctx.save_for_backward(x2, gamma, mean, rstd)
        ctx.rms = rms
        ctx.has_beta = beta is not None
        ctx.gamma_ref, ctx.beta_ref = gamma, beta
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, gamma, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape)
        if not dy2.is_contiguous() or dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype).contiguous()
        gamma_p, beta_p = ctx.gamma_ref, ctx.beta_ref
        mg = getattr(gamma_p, "main_grad", None)
        mb = getattr(beta_p, "main_grad", None) if ctx.has_beta else None
        if mg is not None and (not ctx.has_beta or mb is not None):
            dx = norm_backward(dy2, x2, gamma, mean, rstd, ctx.rms, mg, mb, True)
            return dx.reshape(dy.shape), None, None, None, None
        dg = torch.empty(x2.shape[1], dtype=torch.float32, device=x2.device)
        db = torch.empty_like(dg) if ctx.has_beta else None
        dx = norm_backward(dy2, x2, gamma, mean, rstd, ctx.rms, dg, db, False)
        return (dx.reshape(dy.shape), dg.to(gamma.dtype),
                db.to(gamma.dtype) if db is not None else None, None, None)


def layer_norm(x, gamma, beta=None, eps: float = 1e-5) -> torch.Tensor:
    return _NormFn.apply(x, gamma, beta, eps, False)


def rms_norm(x, gamma, eps: float = 1e-6) -> torch.Tensor:
    return _NormFn.apply(x, gamma, None, eps, True)
