"""Scaled-dot-product attention, forward and backward, on the tcgen05 kernels
(``csrc/attention/attn_fwd.cu``, ``csrc/attention/attn_bwd.cu``).

Tensors are ``[B, S, H, D]`` views (D contiguous, any B/S/H strides), so Q, K and V can be
slices of one fused QKV projection output and O feeds the output projection without a copy.
CPU tensors use an fp32 PyTorch statement of the same math (also the test oracle).

Reference parity: ``Tensor::scaled_dot_attention`` (crates/st-tensor/src/pure.rs:4061-4157,
online-softmax ``fused_attention_cpu`` :11845-11919); the backward has no counterpart in
the reference (its attention is forward-only).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import native

launch_count = 0


class _FwdArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("Q", "K", "V", "O", "lse")] + \
               [(n, ctypes.c_longlong) for n in ("q_sb", "q_ss", "q_sh", "k_sb", "k_ss", "k_sh",
                                                "v_sb", "v_ss", "v_sh", "o_sb", "o_ss", "o_sh")] + \
               [(n, ctypes.c_int) for n in ("B", "H", "Sq", "Sk", "D")] + \
               [("scale", ctypes.c_float), ("causal", ctypes.c_int)] + \
               [("key_bias", ctypes.c_void_p), ("kb_sb", ctypes.c_longlong), ("kb_sh", ctypes.c_longlong),
                ("attn_bias", ctypes.c_void_p), ("ab_sb", ctypes.c_longlong), ("ab_sh", ctypes.c_longlong),
                ("ab_sq", ctypes.c_longlong), ("lengths", ctypes.c_void_p)]


class _BwdArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("Q", "K", "V", "O", "dO", "lse", "delta", "dQ_acc",
                                               "dQ", "dK", "dV")] + \
               [(n, ctypes.c_longlong) for n in ("q_sb", "q_ss", "q_sh", "k_sb", "k_ss", "k_sh",
                                                "v_sb", "v_ss", "v_sh", "o_sb", "o_ss", "o_sh",
                                                "do_sb", "do_ss", "do_sh",
                                                "dq_sb", "dq_ss", "dq_sh", "dk_sb", "dk_ss", "dk_sh",
                                                "dv_sb", "dv_ss", "dv_sh")] + \
               [(n, ctypes.c_int) for n in ("B", "H", "Sq", "Sk", "D")] + \
               [("scale", ctypes.c_float), ("causal", ctypes.c_int)] + \
               [("key_bias", ctypes.c_void_p), ("kb_sb", ctypes.c_longlong), ("kb_sh", ctypes.c_longlong),
                ("attn_bias", ctypes.c_void_p), ("ab_sb", ctypes.c_longlong), ("ab_sh", ctypes.c_longlong),
                ("ab_sq", ctypes.c_longlong), ("lengths", ctypes.c_void_p)]


def attention_reference(q, k, v, causal: bool, scale: float, bias: Optional[torch.Tensor] = None,
                        key_bias: Optional[torch.Tensor] = None, attn_bias: Optional[torch.Tensor] = None,
                        lengths: Optional[torch.Tensor] = None):
    """fp32 reference: q,k,v ``[B,S,H,D]`` → (o ``[B,S,H,D]`` fp32, lse ``[B,H,S]``).

    ``key_bias`` ``[B, Sk]`` or ``[B, H, Sk]`` and ``attn_bias`` ``[B, Sq, Sk]`` or ``[B, H, Sq, Sk]`` are added
    to ``scale * q·kᵀ``; with ``lengths`` ``[B]`` keys at or beyond the length are masked and queries at or
    beyond it give zero rows (crates/st-core/src/backend/cuda_attention.cu:117-202)."""
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if bias is not None:
        s = s + bias
    if key_bias is not None:
        kb = key_bias.float()
        s = s + (kb[:, None, None, :] if kb.dim() == 2 else kb[:, :, None, :])
    if attn_bias is not None:
        ab = attn_bias.float()
        s = s + (ab[:, None] if ab.dim() == 3 else ab)
    sq, sk = s.shape[-2:]
    if causal:
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    if lengths is not None:
        ln = lengths.to(s.device).view(-1, 1, 1, 1)
        dead = (torch.arange(sk, device=s.device).view(1, 1, 1, sk) >= ln) | \
               (torch.arange(sq, device=s.device).view(1, 1, sq, 1) >= ln)
        s = s.masked_fill(dead, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.where(torch.isfinite(lse).unsqueeze(-1), p, torch.zeros_like(p))     # fully masked rows → zeros
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o, lse


def _bias_args(a, q, k, key_bias, attn_bias, lengths, keep: list) -> None:
    """Fill the bias / length fields of an argument block (fp32 biases, int32 lengths, keys contiguous)."""
    B, Sq, H, _ = q.shape
    Sk = k.shape[1]
    if key_bias is not None:
        kb = key_bias.to(torch.float32)
        if kb.shape not in ((B, Sk), (B, H, Sk)):
            raise ValueError(f"attention: key_bias must be [B, Sk] or [B, H, Sk], got {tuple(kb.shape)}")
        kb = kb.contiguous()
        keep.append(kb)
        a.key_bias = kb.data_ptr()
        a.kb_sb, a.kb_sh = kb.stride(0), (kb.stride(1) if kb.dim() == 3 else 0)
    if attn_bias is not None:
        ab = attn_bias.to(torch.float32)
        if ab.shape not in ((B, Sq, Sk), (B, H, Sq, Sk)):
            raise ValueError(f"attention: attn_bias must be [B, Sq, Sk] or [B, H, Sq, Sk], got {tuple(ab.shape)}")
        ab = ab.contiguous()
        keep.append(ab)
        a.attn_bias = ab.data_ptr()
        a.ab_sb, a.ab_sh, a.ab_sq = ab.stride(0), (ab.stride(1) if ab.dim() == 4 else 0), ab.stride(-2)
    if lengths is not None:
        ln = lengths.to(device=q.device, dtype=torch.int32).contiguous()
        if ln.shape != (B,):
            raise ValueError(f"attention: lengths must be [B], got {tuple(ln.shape)}")
        keep.append(ln)
        a.lengths = ln.data_ptr()


def set_pair_kernel(on: bool) -> None:
    """Plain (no bias, no lengths) forward attention runs the pair kernel by default: two 128-row query tiles per
    CTA share every K / V tile, with the probabilities and the output accumulator in tensor memory.  ``False``
    selects the single-tile kernel, which the biased / variable-length cases always use."""
    native.lib().st_attn_fwd_set_pair_kernel(1 if on else 0)


def pair_kernel_enabled() -> bool:
    return bool(native.lib().st_attn_fwd_get_pair_kernel())


_env_applied = False


def _apply_env_once() -> None:
    """``ST_ATTN_FWD_PAIR=0`` in the environment selects the single-tile forward kernel for the whole process."""
    global _env_applied
    if not _env_applied:
        _env_applied = True
        v = os.environ.get("ST_ATTN_FWD_PAIR")
        if v is not None:
            set_pair_kernel(v.strip().lower() not in ("0", "false", "off", ""))


def _check_layout(t: torch.Tensor, name: str) -> None:
    if t.dim() != 4 or t.stride(-1) != 1 or t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be a bf16 [B,S,H,D] view with contiguous D")


def _check_shapes(q, k, v) -> None:
    """K and V must agree with each other and with Q's batch, heads and head dimension: the kernel sizes every
    access from Q's B/H/D and K's length, so a smaller K or V would be read past its allocation."""
    if k.shape != v.shape:
        raise ValueError(f"attention: k {tuple(k.shape)} and v {tuple(v.shape)} differ")
    if k.dim() != 4 or q.dim() != 4 or (k.shape[0], k.shape[2], k.shape[3]) != (q.shape[0], q.shape[2], q.shape[3]):
        raise ValueError(f"attention: k/v {tuple(k.shape)} do not match q {tuple(q.shape)} in batch, heads or head_dim")


def attention_forward(q, k, v, causal: bool = True, scale: Optional[float] = None, *,
                      key_bias: Optional[torch.Tensor] = None, attn_bias: Optional[torch.Tensor] = None,
                      lengths: Optional[torch.Tensor] = None):
    """Returns ``(o, lse)``; ``o`` is contiguous ``[B,S,H,D]`` bf16, ``lse`` fp32 ``[B,H,S]``.
    Optional additive biases and valid lengths as in :func:`attention_reference`."""
    global launch_count
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if not native.use_native(q):
        o, lse = attention_reference(q, k, v, causal, scale, key_bias=key_bias, attn_bias=attn_bias, lengths=lengths)
        return o.to(q.dtype).contiguous(), lse
    native.require_cuda("attention_forward", q, k, v, key_bias, attn_bias, lengths)
    _apply_env_once()
    _check_shapes(q, k, v)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_layout(t, n)
    o = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    a = _FwdArgs()
    a.Q, a.K, a.V, a.O, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = q.stride(0), q.stride(1), q.stride(2)
    a.k_sb, a.k_ss, a.k_sh = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_ss, a.v_sh = v.stride(0), v.stride(1), v.stride(2)
    a.o_sb, a.o_ss, a.o_sh = o.stride(0), o.stride(1), o.stride(2)
    a.B, a.H, a.Sq, a.Sk, a.D = B, H, Sq, Sk, D
    a.scale, a.causal = float(scale), int(causal)
    keep: list = []
    _bias_args(a, q, k, key_bias, attn_bias, lengths, keep)
    native.check(native.lib().st_attn_fwd(ctypes.byref(a), native.stream_ptr(q.device)), "st_attn_fwd")
    launch_count += 1
    return o, lse


def attention_backward(q, k, v, o, lse, do, causal: bool = True, scale: Optional[float] = None,
                       dq=None, dk=None, dv=None, *, key_bias=None, attn_bias=None, lengths=None):
    """Returns ``(dq, dk, dv)`` (bf16, ``[B,S,H,D]``); outputs may be preallocated strided views."""
    global launch_count
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if not native.use_native(q):
        with torch.enable_grad():
            qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            of, _ = attention_reference(qf, kf, vf, causal, scale, key_bias=key_bias, attn_bias=attn_bias,
                                        lengths=lengths)
            g = torch.autograd.grad(of, (qf, kf, vf), do.float())
        outs = []
        for grad, given in zip(g, (dq, dk, dv)):
            if given is None:
                outs.append(grad.to(q.dtype))
            else:
                given.copy_(grad.to(given.dtype))
                outs.append(given)
        return tuple(outs)
    native.require_cuda("attention_backward", q, k, v, o, lse, do, dq, dk, dv, key_bias, attn_bias, lengths)
    _check_shapes(q, k, v)
    if o.shape != q.shape or do.shape != q.shape:
        raise ValueError(f"attention_backward: o {tuple(o.shape)} and do {tuple(do.shape)} must match q {tuple(q.shape)}")
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (do, "do")):
        _check_layout(t, n)
    dev = q.device
    dq = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=dev) if dq is None else dq
    dk = torch.empty((B, Sk, H, D), dtype=torch.bfloat16, device=dev) if dk is None else dk
    dv = torch.empty((B, Sk, H, D), dtype=torch.bfloat16, device=dev) if dv is None else dv
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
    a = _BwdArgs()
    a.Q, a.K, a.V, a.O, a.dO = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr()
    a.lse, a.delta, a.dQ_acc = lse.data_ptr(), delta.data_ptr(), None      # dQ accumulates in TMEM
    a.dQ, a.dK, a.dV = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    for pre, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", do), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(a, pre + "_sb", t.stride(0))
        setattr(a, pre + "_ss", t.stride(1))
        setattr(a, pre + "_sh", t.stride(2))
    a.B, a.H, a.Sq, a.Sk, a.D = B, H, Sq, Sk, D
    a.scale, a.causal = float(scale), int(causal)
    keep: list = []
    _bias_args(a, q, k, key_bias, attn_bias, lengths, keep)
    native.check(native.lib().st_attn_bwd(ctypes.byref(a), native.stream_ptr(dev)), "st_attn_bwd")
    launch_count += 3
    return dq, dk, dv


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, key_bias, attn_bias, lengths):
        o, lse = attention_forward(q, k, v, causal, scale, key_bias=key_bias, attn_bias=attn_bias, lengths=lengths)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        ctx.extras = (key_bias, attn_bias, lengths)     # biases are constants here: no gradient flows to them
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        if do.stride(-1) != 1 or do.dtype != q.dtype:
            do = do.to(q.dtype).contiguous()
        kb, ab, ln = ctx.extras
        dq, dk, dv = attention_backward(q, k, v, o, lse, do, ctx.causal, ctx.scale, key_bias=kb, attn_bias=ab,
                                        lengths=ln)
        return dq, dk, dv, None, None, None, None, None


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None, *,
              key_bias: Optional[torch.Tensor] = None, attn_bias: Optional[torch.Tensor] = None,
              lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable attention on ``[B,S,H,D]`` tensors (gradients for q, k, v; the biases are constants)."""
    return _AttentionFn.apply(q, k, v, causal, scale, key_bias, attn_bias, lengths)
