"""RoPE, GELU/ReLU, column sums, embedding and row softmax (``csrc/elementwise/elementwise.cu``).

Reference parity: ``tensor_utils.wgsl`` entry points ``embedding_gather``,
``embedding_scatter_add``, ``relu``/``relu_backward``, ``sum_axis0``; ``fused_gelu_back.wgsl``;
``row_softmax`` / ``row_softmax_hardmax`` (crates/st-tensor/src/pure.rs:3277,11921);
RoPE cache util (crates/st-core/src/util/rope_lru.rs).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import native

launch_count = 0
_rope_cache: dict = {}


def rope_tables(seq_len: int, head_dim: int, base: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[seq_len, head_dim/2]`` fp32 (cached per device)."""
    key = (seq_len, head_dim, float(base), str(device))
    hit = _rope_cache.get(key)
    if hit is None:
        inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
        ang = torch.arange(seq_len, dtype=torch.float64)[:, None] * inv[None, :]
        hit = (ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous())
        _rope_cache[key] = hit
    return hit


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, backward: bool):
    """x: [T, heads, D]; rotate-half convention; position = t % seq_len."""
    T, Hh, D = x.shape
    half = D // 2
    pos = torch.arange(T, device=x.device) % seq_len
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :] * (-1.0 if backward else 1.0)
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def rope_(x: torch.Tensor, heads: int, head_dim: int, seq_len: int, base: float = 10000.0,
          backward: bool = False) -> torch.Tensor:
    """In-place RoPE on the first ``heads*head_dim`` columns of each row of ``x`` ``[T, ld]``."""
    global launch_count
    T = x.shape[0]
    cos, sin = rope_tables(seq_len, head_dim, base, x.device)
    if not native.use_native(x):
        view = x[:, : heads * head_dim].reshape(T, heads, head_dim)
        view.copy_(rope_reference(view, cos, sin, seq_len, backward))
        return x
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    st = native.lib().st_rope(native.ptr(x), native.ptr(cos), native.ptr(sin), ctypes.c_longlong(T),
                              ctypes.c_int(heads), ctypes.c_int(head_dim), ctypes.c_longlong(x.stride(0)),
                              ctypes.c_int(seq_len), ctypes.c_int(0), ctypes.c_int(int(backward)),
                              native.stream_ptr(x.device))
    native.check(st, "st_rope")
    launch_count += 1
    return x


def act_forward(x: torch.Tensor, kind: str) -> torch.Tensor:
    global launch_count
    if not native.use_native(x) or x.dtype != torch.bfloat16 or x.numel() % 8 or not x.is_contiguous():
        if x.is_cuda:
            x = x.contiguous()
        return torch.relu(x) if kind == "relu" else torch.nn.functional.gelu(x, approximate="tanh")
    y = torch.empty_like(x)
    st = native.lib().st_act_fwd(native.ptr(x), native.ptr(y), ctypes.c_longlong(x.numel()),
                                 ctypes.c_int(int(kind == "relu")), native.stream_ptr(x.device))
    native.check(st, "st_act_fwd")
    launch_count += 1
    return y


def act_backward(x: torch.Tensor, dy: torch.Tensor, kind: str) -> torch.Tensor:
    global launch_count
    if not native.use_native(x) or x.dtype != torch.bfloat16 or x.numel() % 8 or not x.is_contiguous() \
            or not dy.is_contiguous() or dy.dtype != x.dtype:
        from .gemm import gelu_tanh_grad
        g = (x > 0).to(dy.dtype) if kind == "relu" else gelu_tanh_grad(x.float()).to(dy.dtype)
        return dy * g
    dx = torch.empty_like(x)
    st = native.lib().st_act_bwd(native.ptr(x), native.ptr(dy), native.ptr(dx), ctypes.c_longlong(x.numel()),
                                 ctypes.c_int(int(kind == "relu")), native.stream_ptr(x.device))
    native.check(st, "st_act_bwd")
    launch_count += 1
    return dx


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        ctx.save_for_backward(x)
        ctx.kind = kind
        return act_forward(x, kind)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return act_backward(x, dy.contiguous(), ctx.kind), None


def gelu(x: torch.Tensor) -> torch.Tensor:
    return _ActFn.apply(x, "gelu")


def relu(x: torch.Tensor) -> torch.Tensor:
    return _ActFn.apply(x, "relu")


def colsum(x2: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """fp32 column sums of a bf16 ``[rows, cols]`` matrix (bias gradients)."""
    global launch_count
    rows, cols = x2.shape
    if out is None:
        out = torch.zeros(cols, dtype=torch.float32, device=x2.device)
    elif not accumulate:
        out.zero_()
    if not native.use_native(x2) or x2.dtype != torch.bfloat16 or x2.stride(-1) != 1 or \
            native.deterministic_reduction():      # the kernel joins its row chunks with fp32 atomics
        out += x2.float().sum(0)
        return out
    st = native.lib().st_colsum(native.ptr(x2), native.ptr(out), ctypes.c_longlong(rows), ctypes.c_int(cols),
                                ctypes.c_longlong(x2.stride(0)), native.stream_ptr(x2.device))
    native.check(st, "st_colsum")
    launch_count += 1
    return out


def embedding_forward(idx: torch.Tensor, weight: torch.Tensor, pos: Optional[torch.Tensor] = None,
                      seq_len: int = 0, vocab_start: int = 0) -> torch.Tensor:
    """``out[t] = weight[idx[t] - vocab_start]`` (zeros outside the shard) ``+ pos[t % seq_len]``."""
    global launch_count
    flat = idx.reshape(-1)
    T, d = flat.numel(), weight.shape[1]
    if not native.use_native(weight):
        local = flat - vocab_start
        ok = (local >= 0) & (local < weight.shape[0])
        out = weight[local.clamp(0, weight.shape[0] - 1)] * ok[:, None].to(weight.dtype)
        if pos is not None:
            out = out + pos[torch.arange(T, device=flat.device) % seq_len]
        return out
    assert weight.dtype == torch.bfloat16 and weight.is_contiguous()
    flat = flat.to(torch.int64).contiguous()
    out = torch.empty((T, d), dtype=torch.bfloat16, device=weight.device)
    st = native.lib().st_embedding_fwd(native.ptr(flat), native.ptr(weight), native.ptr(pos), native.ptr(out),
                                       ctypes.c_longlong(T), ctypes.c_int(d), ctypes.c_int(vocab_start),
                                       ctypes.c_int(weight.shape[0]), ctypes.c_int(seq_len),
                                       native.stream_ptr(weight.device))
    native.check(st, "st_embedding_fwd")
    launch_count += 1
    return out


def embedding_backward(idx: torch.Tensor, dy2: torch.Tensor, dweight: torch.Tensor,
                       dpos: Optional[torch.Tensor] = None, seq_len: int = 0, vocab_start: int = 0) -> None:
    """Scatter-add ``dy2`` (bf16 ``[T, d]``) into fp32 ``dweight`` (and ``dpos``)."""
    global launch_count
    flat = idx.reshape(-1)
    T, d = dy2.shape
    if not native.use_native(dy2):
        local = flat - vocab_start
        ok = (local >= 0) & (local < dweight.shape[0])
        dweight.index_add_(0, local[ok], dy2[ok].to(dweight.dtype))
        if dpos is not None:
            dpos.index_add_(0, torch.arange(T, device=flat.device) % seq_len, dy2.to(dpos.dtype))
        return
    assert dweight.dtype == torch.float32 and dy2.dtype == torch.bfloat16 and dy2.is_contiguous()
    flat = flat.to(torch.int64).contiguous()
    if native.deterministic_reduction():
        # fixed summation order: sort the positions by id (stable), one CTA per distinct id adds its rows in
        # position order; positions are summed over the batch with a plain (deterministic) reduction
        sorted_ids, perm = torch.sort(flat, stable=True)
        uniq, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
        starts = torch.cumsum(counts, 0) - counts
        st = native.lib().st_embedding_bwd_sorted(
            native.ptr(uniq), native.ptr(starts), native.ptr(counts), native.ptr(perm), native.ptr(dy2),
            native.ptr(dweight), ctypes.c_longlong(uniq.numel()), ctypes.c_int(d), ctypes.c_int(vocab_start),
            ctypes.c_int(dweight.shape[0]), native.stream_ptr(dy2.device))
        native.check(st, "st_embedding_bwd_sorted")
        launch_count += 1
        if dpos is not None:
            dpos += dy2.view(-1, seq_len, d).float().sum(0)
        return
    st = native.lib().st_embedding_bwd(native.ptr(flat), native.ptr(dy2), native.ptr(dweight), native.ptr(dpos),
                                       ctypes.c_longlong(T), ctypes.c_int(d), ctypes.c_int(vocab_start),
                                       ctypes.c_int(dweight.shape[0]), ctypes.c_int(seq_len),
                                       native.stream_ptr(dy2.device))
    native.check(st, "st_embedding_bwd")
    launch_count += 1


def row_softmax(x: torch.Tensor, hardmax: bool = False):
    """fp32 row softmax of a 2-D tensor; with ``hardmax`` also returns the one-hot arg-max mask
    (lowest index wins ties)."""
    global launch_count
    if not native.use_native(x):
        y = torch.softmax(x.float(), dim=-1)
        if not hardmax:
            return y
        idx = x.float().argmax(dim=-1, keepdim=True)
        return y, torch.zeros_like(y).scatter_(1, idx, 1.0)
    xf = x.float().contiguous()
    y = torch.empty_like(xf)
    h = torch.empty_like(xf) if hardmax else None
    st = native.lib().st_row_softmax_f32(native.ptr(xf), native.ptr(y), native.ptr(h), ctypes.c_int(xf.shape[0]),
                                         ctypes.c_int(xf.shape[1]), native.stream_ptr(x.device))
    native.check(st, "st_row_softmax_f32")
    launch_count += 1
    return (y, h) if hardmax else y


# ---- softmax + hardmax + spiral consensus + Z-space projection -------------------------------------------
def _ramanujan_pi(iterations: int) -> float:
    pref, base, factor, total, approx = (2.0 * math.sqrt(2.0)) / 9801.0, 396.0 ** 4, 1.0, 0.0, math.pi
    for k in range(max(1, iterations)):
        total += factor * (1103.0 + 26390.0 * k)
        approx = 1.0 / (pref * total)
        n = k + 1.0
        factor *= ((4 * n - 3) * (4 * n - 2) * (4 * n - 1) * (4 * n)) / (n ** 4 * base)
    return approx


GOLDEN_RATIO = (1.0 + math.sqrt(5.0)) / 2.0
GOLDEN_RATIO_CONJUGATE = 1.0 / GOLDEN_RATIO
GOLDEN_RATIO_BIAS = 1.0 - GOLDEN_RATIO_CONJUGATE
GOLDEN_ANGLE = math.pi * (3.0 - math.sqrt(5.0))
RAMANUJAN_PI = _ramanujan_pi(6)
RAMANUJAN_RATIO = math.pi / RAMANUJAN_PI
RAMANUJAN_DELTA = abs(RAMANUJAN_PI - math.pi)
LEECH_SCALE = 0.75 * 0.0019295743094039225 * math.sqrt(24.0) * RAMANUJAN_RATIO     # projector weight, packing density, rank


def row_softmax_spiral(x: torch.Tensor):
    """Row softmax, arg-max mask, spiral-consensus blend and per-row metrics in one kernel launch.

    Returns ``(soft, hard, spiral, metrics[rows, 4], zmetrics[rows, 4])`` with ``metrics`` columns
    (entropy, hardmass, enrichment, coherence) and ``zmetrics`` columns (focus, above, here, swirl).
    ``spiral = (1 + enrichment) * (phi_conj * soft + phi_bias * hard)`` with
    ``enrichment = leech_scale * (entropy * ramanujan_ratio + hardmass * phi)`` (the stub's
    ``_spiral_softmax_hardmax_consensus_python`` and softmax_spiral_consensus.wgsl /
    softmax_zspace_projection.wgsl of crates/st-backend-wgpu/src/shaders)."""
    global launch_count
    xf = x.float().contiguous()
    rows, cols = xf.shape
    if not native.use_native(x):
        soft = torch.softmax(xf, dim=-1)
        idx = xf.argmax(dim=-1, keepdim=True)
        hard = torch.zeros_like(soft).scatter_(1, idx, 1.0)
        entropy = -(torch.where(soft > 0, soft * torch.log(soft.clamp(min=1e-45)), torch.zeros_like(soft))).sum(-1)
        hardmass = hard.sum(-1)
        geodesic = entropy * RAMANUJAN_RATIO + hardmass * GOLDEN_RATIO
        enrichment = torch.where(geodesic > 1e-12, LEECH_SCALE * geodesic, torch.zeros_like(geodesic))
        spiral = (1.0 + enrichment)[:, None] * (GOLDEN_RATIO_CONJUGATE * soft + GOLDEN_RATIO_BIAS * hard)
        en = torch.where(entropy > 0, entropy / (entropy + 1.0), torch.zeros_like(entropy)).clamp(0, 1)
        hn = (hardmass / cols).clamp(0, 1)
        rn = torch.where(enrichment != 0, enrichment / (1.0 + enrichment.abs()), torch.zeros_like(enrichment)).clamp(0, 1)
        metrics = torch.stack([entropy, hardmass, enrichment, (en + hn + rn) / 3.0], dim=1)
        above_n = max(1, int(cols / GOLDEN_RATIO))
        here_n = max(1, int(cols / (GOLDEN_RATIO * GOLDEN_RATIO)))
        if above_n >= cols:
            above_n, here_n = cols, 0
        elif above_n + here_n >= cols:
            here_n = cols - above_n
        cidx = torch.arange(cols, device=xf.device, dtype=torch.float32)
        zmetrics = torch.stack([(soft * soft).sum(-1), soft[:, :above_n].sum(-1),
                                soft[:, above_n:above_n + here_n].sum(-1),
                                (soft * torch.sin(cidx * GOLDEN_ANGLE)).sum(-1)], dim=1)
        return soft, hard, spiral, metrics, zmetrics
    soft, hard, spiral = torch.empty_like(xf), torch.empty_like(xf), torch.empty_like(xf)
    metrics = torch.empty((rows, 4), dtype=torch.float32, device=xf.device)
    zmetrics = torch.empty((rows, 4), dtype=torch.float32, device=xf.device)
    st = native.lib().st_row_softmax_spiral_f32(
        native.ptr(xf), native.ptr(soft), native.ptr(hard), native.ptr(spiral), native.ptr(metrics),
        native.ptr(zmetrics), ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_float(GOLDEN_RATIO),
        ctypes.c_float(GOLDEN_RATIO_CONJUGATE), ctypes.c_float(GOLDEN_RATIO_BIAS), ctypes.c_float(LEECH_SCALE),
        ctypes.c_float(RAMANUJAN_RATIO), ctypes.c_float(GOLDEN_ANGLE), native.stream_ptr(xf.device))
    native.check(st, "st_row_softmax_spiral_f32")
    launch_count += 1
    return soft, hard, spiral, metrics, zmetrics


def nd_indexer(positions: torch.Tensor, dims, strides, segments: int, segment_stride: int):
    """Strided address and segment id of each logical element id (crates/st-backend-wgpu/src/shaders/nd_indexer.wgsl).

    ``dims`` / ``strides``: up to four entries, innermost last; a zero dimension is skipped.  The id is decoded
    against ``dims``, the coordinates are dotted with ``strides`` and the address falls into segment
    ``(address // segment_stride) % segments``.  Returns ``(addresses, segments)`` as int64 tensors (32-bit unsigned
    arithmetic inside, as the shader's)."""
    global launch_count
    dims, strides = list(dims), list(strides)
    if not 1 <= len(dims) <= 4 or len(dims) != len(strides):
        raise ValueError("nd_indexer takes between one and four dimensions with as many strides")
    if segments <= 0 or segment_stride <= 0:
        raise ValueError("segments and segment_stride must be positive")
    if any(d < 0 or d >= 1 << 32 for d in dims + strides):
        raise ValueError("dimensions and strides must fit an unsigned 32-bit integer")
    dims = [0] * (4 - len(dims)) + dims
    strides = [0] * (4 - len(strides)) + strides
    pos = positions.reshape(-1).to(torch.int64)
    if pos.numel() and (int(pos.min()) < 0 or int(pos.max()) >= 1 << 32):
        raise ValueError("logical ids must fit an unsigned 32-bit integer")
    if not (pos.is_cuda and native.available()):
        remaining, flat = pos.clone(), torch.zeros_like(pos)
        for d in range(3, -1, -1):
            if dims[d] == 0:
                continue
            flat = (flat + (remaining % dims[d]) * strides[d]) & 0xFFFFFFFF
            remaining = remaining // dims[d]
        return flat.reshape(positions.shape), ((flat // segment_stride) % segments).reshape(positions.shape)
    p32 = pos.to(torch.int32) if int(pos.max() if pos.numel() else 0) < 1 << 31 else (pos - (1 << 32) * (pos >= 1 << 31)).to(torch.int32)
    out_i, out_s = torch.empty_like(p32), torch.empty_like(p32)
    arr = ctypes.c_uint * 4
    st = native.lib().st_nd_indexer(native.ptr(p32), native.ptr(out_i), native.ptr(out_s), ctypes.c_longlong(p32.numel()),
                                    arr(*dims), arr(*strides), ctypes.c_uint(segments), ctypes.c_uint(segment_stride),
                                    native.stream_ptr(p32.device))
    native.check(st, "st_nd_indexer")
    launch_count += 1
    unsigned = lambda t: t.to(torch.int64) & 0xFFFFFFFF                       # noqa: E731
    return unsigned(out_i).reshape(positions.shape), unsigned(out_s).reshape(positions.shape)
