"""bf16 GEMM with fused epilogues on the tcgen05 kernel (``csrc/gemm/gemm_sm100.cu``).

``gemm`` computes ``C[M,N] = epilogue(alpha * A @ B^T)`` where each operand may be stored
K-major (``A`` is ``[M,K]``, ``B`` is ``[N,K]``) or MN-major (``A`` is ``[K,M]``, ``B`` is
``[K,N]``), so a linear layer's forward, data-gradient and weight-gradient all run without a
transposition pass.  CPU tensors take an fp32 PyTorch path with the same semantics (that is
the numerical oracle in the tests).

Reference parity: ``Tensor::matmul``, ``matmul_bias_relu/gelu``, ``matmul_bias_add_relu/gelu``
(crates/st-tensor/src/pure.rs:2013,4406,4637,4824,5084).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_BWD, ACT_RELU_BWD = 0, 1, 2, 3, 4
_ACT_NAMES = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_bwd": 3, "relu_bwd": 4}

#: number of native kernel launches issued through this module (for bench accounting)
launch_count = 0


class _GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
        ("aux_out", ctypes.c_void_p), ("aux_in", ctypes.c_void_p),
        ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong), ("ldc", ctypes.c_longlong),
        ("ldr", ctypes.c_longlong), ("ld_aux_out", ctypes.c_longlong), ("ld_aux_in", ctypes.c_longlong),
        ("batch_stride_a", ctypes.c_longlong), ("batch_stride_b", ctypes.c_longlong),
        ("batch_stride_c", ctypes.c_longlong),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("batch", ctypes.c_int),
        ("a_mn_major", ctypes.c_int), ("b_mn_major", ctypes.c_int),
        ("out_fp32", ctypes.c_int), ("accumulate", ctypes.c_int), ("act", ctypes.c_int),
        ("alpha", ctypes.c_float), ("max_ctas", ctypes.c_int),
    ]


#: split the K loop of weight-gradient GEMMs whose tile count fills the SMs badly (the partial
#: sums meet in fp32 atomics, so the summation order is not fixed); native.deterministic_reduction()
#: (SPIRAL_DETERMINISTIC_REDUCTION / SPIRAL_DETERMINISTIC) turns it off per call
SPLIT_K = True
_NUM_SMS = 148


def _split_k(M: int, N: int, K: int) -> int:
    tiles = ((M + 127) // 128) * ((N + 255) // 256 if N > 128 else 1)
    best, best_eff = 1, tiles / (-(-tiles // _NUM_SMS) * _NUM_SMS)
    for s in (2, 3, 4):
        if K % (s * 64) or K // s < 2048:
            continue
        work = tiles * s
        eff = work / (-(-work // _NUM_SMS) * _NUM_SMS)
        if eff > best_eff + 0.04:
            best, best_eff = s, eff
    return best


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def gelu_tanh_grad(x: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def _reference(a, b, a_mn, b_mn, out, out_dtype, bias, act, residual, aux_out, aux_in, alpha, accumulate):
    """fp32 PyTorch statement of the kernel's semantics (CPU path and test oracle)."""
    af = a.float().transpose(-1, -2) if a_mn else a.float()
    bf = b.float() if b_mn else b.float().transpose(-1, -2)
    v = alpha * (af @ bf)
    if bias is not None:
        v = v + bias.float()
    if aux_out is not None:
        aux_out.copy_(v.to(aux_out.dtype))
    if act == ACT_RELU:
        v = torch.relu(v)
    elif act == ACT_GELU:
        v = gelu_tanh(v)
    elif act == ACT_GELU_BWD:
        v = v * gelu_tanh_grad(aux_in.float())
    elif act == ACT_RELU_BWD:
        v = torch.where(aux_in.float() > 0, v, torch.zeros_like(v))
    if residual is not None:
        v = v + residual.float()
    if out is None:
        return v.to(out_dtype)
    if accumulate:
        v = v + out.float()
    out.copy_(v.to(out.dtype))
    return out


# bf16 copies of fp32 parameters: a weight is rounded once per optimizer step instead of once per forward.
# Entries are keyed by storage address and invalidated by the tensor's version counter; each entry also HOLDS its
# source tensor, so the address cannot be freed and handed to another tensor while the entry lives (a recycled
# address with an equal version would otherwise return another tensor's values).  Least-recently-used entries are
# dropped once the cache holds more than _BF16_CACHE_BYTES of sources and copies.
from collections import OrderedDict as _OrderedDict

_bf16_cache: "_OrderedDict" = _OrderedDict()
_bf16_cache_bytes = 0
_BF16_CACHE_BYTES = 1 << 30


def cached_bf16(t: torch.Tensor) -> torch.Tensor:
    """bf16 copy of ``t`` (itself when it already is bf16), reused until ``t`` is modified in place."""
    global _bf16_cache_bytes
    if t.dtype == torch.bfloat16:
        return t
    key = (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, t.device)
    hit = _bf16_cache.get(key)
    if hit is not None and hit[0] == t._version:
        _bf16_cache.move_to_end(key)
        return hit[1]
    out = t.detach().to(torch.bfloat16).contiguous()
    cost = t.numel() * (t.element_size() + 2)
    if cost > _BF16_CACHE_BYTES // 4:
        return out                                   # too large to be worth pinning
    if hit is not None:
        _bf16_cache_bytes -= hit[3]
    _bf16_cache[key] = (t._version, out, t.detach(), cost)      # the detached alias keeps the storage alive
    _bf16_cache.move_to_end(key)
    _bf16_cache_bytes += cost
    while _bf16_cache_bytes > _BF16_CACHE_BYTES and len(_bf16_cache) > 1:
        _, old = _bf16_cache.popitem(last=False)
        _bf16_cache_bytes -= old[3]
    return out


def clear_bf16_cache() -> None:
    """Drops every cached bf16 copy (CUDA-graph capture calls this so that the casts it needs are captured too)."""
    global _bf16_cache_bytes
    _bf16_cache.clear()
    _bf16_cache_bytes = 0


def _pad_to(t: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    if t.shape[-2] == rows and t.shape[-1] == cols and t.stride(-1) == 1 and t.stride(-2) % 8 == 0 \
            and t.data_ptr() % 16 == 0:
        return t
    out = t.new_zeros(*t.shape[:-2], rows, cols)
    out[..., : t.shape[-2], : t.shape[-1]] = t
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         bias: Optional[torch.Tensor] = None, act=None, residual: Optional[torch.Tensor] = None,
         aux_out: Optional[torch.Tensor] = None, aux_in: Optional[torch.Tensor] = None,
         alpha: float = 1.0, accumulate: bool = False, max_ctas: int = 0) -> torch.Tensor:
    """``C = epilogue(alpha * op(A) @ op(B)^T)``; 2-D or batched 3-D operands.

    ``a``: ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b``: ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    Epilogue order: ``+bias`` → store ``aux_out`` → activation (``relu``/``gelu``, or multiply
    by the derivative evaluated at ``aux_in`` for ``gelu_bwd``/``relu_bwd``) → ``+residual`` →
    ``+out`` when ``accumulate`` → cast to ``out``'s dtype (bf16 or fp32).
    """
    global launch_count
    act_id = _ACT_NAMES[act] if not isinstance(act, int) else act
    if out is not None:
        out_dtype = out.dtype
    if out_dtype is None:
        out_dtype = torch.bfloat16 if a.is_cuda else a.dtype
    if not native.use_native(a):
        return _reference(a, b, a_mn, b_mn, out, out_dtype, bias, act_id, residual, aux_out, aux_in,
                          alpha, accumulate)

    native.require_cuda("gemm", a, b, out, bias, residual, aux_out, aux_in)
    batched = a.dim() == 3
    if batched:
        assert b.dim() == 3 and a.shape[0] == b.shape[0]
    M = a.shape[-1] if a_mn else a.shape[-2]
    K = a.shape[-2] if a_mn else a.shape[-1]
    N = b.shape[-1] if b_mn else b.shape[-2]
    Kb = b.shape[-2] if b_mn else b.shape[-1]
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    if a.dtype != torch.bfloat16:
        a = a.to(torch.bfloat16)
    if b.dtype != torch.bfloat16:
        b = b.to(torch.bfloat16)
    # TMA needs 16-byte aligned rows: pad the contiguous dimension to a multiple of 8.
    def _fix(t):
        r, c = t.shape[-2], t.shape[-1]
        c8 = (c + 7) // 8 * 8
        if t.stride(-1) != 1 or t.stride(-2) % 8 != 0 or t.data_ptr() % 16 != 0 or c8 != c or \
                (t.dim() == 3 and t.stride(0) % 8 != 0):
            return _pad_to(t.contiguous() if t.stride(-1) != 1 else t, r, c8)
        return t
    a = _fix(a)
    b = _fix(b)
    batch = a.shape[0] if batched else 1
    if out is None:
        shape = (batch, M, N) if batched else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    else:
        assert out.stride(-1) == 1 and out.shape[-2] == M and out.shape[-1] == N
        assert out.dtype in (torch.bfloat16, torch.float32)
    for t in (bias, residual, aux_out, aux_in):
        if t is not None:
            assert t.dtype == torch.bfloat16 and t.stride(-1) == 1, "epilogue operands must be bf16"
    args = _GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.bias = 0 if bias is None else bias.data_ptr()
    args.residual = 0 if residual is None else residual.data_ptr()
    args.aux_out = 0 if aux_out is None else aux_out.data_ptr()
    args.aux_in = 0 if aux_in is None else aux_in.data_ptr()
    args.lda, args.ldb, args.ldc = a.stride(-2), b.stride(-2), out.stride(-2)
    args.ldr = 0 if residual is None else residual.stride(-2)
    args.ld_aux_out = 0 if aux_out is None else aux_out.stride(-2)
    args.ld_aux_in = 0 if aux_in is None else aux_in.stride(-2)
    args.batch_stride_a = a.stride(0) if batched else 0
    args.batch_stride_b = b.stride(0) if batched else 0
    args.batch_stride_c = out.stride(0) if batched else 0
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.a_mn_major, args.b_mn_major = int(a_mn), int(b_mn)
    args.out_fp32 = int(out.dtype == torch.float32)
    args.accumulate = int(accumulate)
    split = _split_k(M, N, K) if (SPLIT_K and not native.deterministic_reduction() and accumulate and a_mn and b_mn and not batched and
                                  out.dtype == torch.float32 and N % 32 == 0 and out.stride(0) % 4 == 0
                                  and bias is None and residual is None and act_id == 0) else 1
    if split > 1:
        # weight-gradient shape with a poor tile count: split the long reduction over `split`
        # CTAs per tile (expressed as a batch over K) and add the partials with fp32 atomics
        kc = K // split
        args.K, args.batch = kc, split
        args.batch_stride_a, args.batch_stride_b, args.batch_stride_c = kc * a.stride(0), kc * b.stride(0), 0
        args.accumulate = 2
    args.act = act_id
    args.alpha = float(alpha)
    args.max_ctas = int(max_ctas)
    st = native.lib().st_gemm_bf16(ctypes.byref(args), native.stream_ptr(a.device))
    native.check(st, "st_gemm_bf16")
    launch_count += 1
    return out


class _LinearFn(torch.autograd.Function):
    """``y = x @ W^T (+ bias)`` with W stored ``[out, in]``; dgrad and wgrad on the same kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != x2.dtype or not dy2.is_contiguous():
            dy2 = dy2.to(x2.dtype).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                # fp32 gradient accumulation straight from the epilogue
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable ``x @ weight^T + bias`` (weight ``[out, in]``)."""
    return _LinearFn.apply(x, weight, bias)
