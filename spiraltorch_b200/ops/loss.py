"""Cross-entropy over bf16 logits with fused log-sum-exp (``st_ce_stats`` / ``st_ce_grad``).

The statistics pass produces, per row, the maximum, ``sum exp(l - max)`` and the target
logit of the local vocabulary shard.  With a tensor-parallel group the three per-row
vectors are combined across ranks (one small all-reduce of max, one of the rescaled sums
and target logits), which gives the vocab-parallel loss without ever gathering logits.
The gradient pass overwrites the logits buffer with ``(softmax - onehot) * coef``.

Reference parity: ``categorical_cross_entropy_{forward,backward}`` (tensor_utils.wgsl) and
``CategoricalCrossEntropy`` (crates/st-nn/src/loss/categorical_cross_entropy.rs:13-36); the
reference loss takes probabilities, this one takes logits and fuses the softmax.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import native

launch_count = 0
IGNORE_INDEX = -100


def _stats(logits2, target, vocab_start):
    global launch_count
    rows, V = logits2.shape
    if not native.use_native(logits2):
        lf = logits2.float()
        m = lf.max(dim=-1).values
        s = torch.exp(lf - m[:, None]).sum(-1)
        local = target - vocab_start
        ok = (local >= 0) & (local < V)
        t = torch.where(ok, lf.gather(1, local.clamp(0, V - 1)[:, None]).squeeze(1), torch.zeros_like(m))
        return m, s, t
    dev = logits2.device
    m = torch.empty(rows, dtype=torch.float32, device=dev)
    s = torch.empty_like(m)
    t = torch.empty_like(m)
    st = native.lib().st_ce_stats(native.ptr(logits2), native.ptr(target), native.ptr(m), native.ptr(s),
                                  native.ptr(t), ctypes.c_longlong(rows), ctypes.c_longlong(logits2.stride(0)),
                                  ctypes.c_int(V), ctypes.c_int(vocab_start), native.stream_ptr(dev))
    native.check(st, "st_ce_stats")
    launch_count += 1
    return m, s, t


def _grad_(logits2, target, lse, coef_tensor, coef, vocab_start):
    """Overwrite ``logits2`` with dlogits."""
    global launch_count
    rows, V = logits2.shape
    if not native.use_native(logits2):
        p = torch.exp(logits2.float() - lse[:, None])
        local = target - vocab_start
        ok = (local >= 0) & (local < V)
        onehot = torch.zeros_like(p)
        onehot[ok, local[ok]] = 1.0
        k = coef * (coef_tensor if coef_tensor is not None else 1.0)
        g = (p - onehot) * k
        g[target == IGNORE_INDEX] = 0
        logits2.copy_(g.to(logits2.dtype))
        return logits2
    st = native.lib().st_ce_grad(native.ptr(logits2), native.ptr(target), native.ptr(lse), native.ptr(coef_tensor),
                                 ctypes.c_float(coef), native.ptr(logits2), ctypes.c_longlong(rows),
                                 ctypes.c_longlong(logits2.stride(0)), ctypes.c_int(V), ctypes.c_int(vocab_start),
                                 ctypes.c_longlong(IGNORE_INDEX), native.stream_ptr(logits2.device))
    native.check(st, "st_ce_grad")
    launch_count += 1
    return logits2


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, vocab_start, group, scale):
        V = logits.shape[-1]
        logits2 = logits.reshape(-1, V)
        tgt = target.reshape(-1).to(torch.int64).contiguous()
        m, s, t = _stats(logits2, tgt, vocab_start)
        if group is not None and dist.get_world_size(group) > 1:
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack([s * torch.exp(m - gm), t])
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
            m, s, t = gm, packed[0], packed[1]
        lse = m + torch.log(s)
        valid = tgt != IGNORE_INDEX
        n_valid = valid.sum().clamp(min=1).to(torch.float32)
        loss = ((lse - t) * valid).sum() / n_valid * scale
        ctx.save_for_backward(logits2, tgt, lse, n_valid)
        ctx.vocab_start, ctx.scale, ctx.shape = vocab_start, scale, logits.shape
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits2, tgt, lse, n_valid = ctx.saved_tensors
        coef = (dloss.to(torch.float32) * ctx.scale / n_valid).reshape(1).contiguous()
        # the logits buffer is dead after this op: reuse it for the gradient
        g = _grad_(logits2, tgt, lse, coef, 1.0, ctx.vocab_start)
        return g.reshape(ctx.shape), None, None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, *, vocab_start: int = 0,
                  group: Optional[dist.ProcessGroup] = None, scale: float = 1.0) -> torch.Tensor:
    """Mean token cross-entropy (times ``scale``).  **Consumes** ``logits``: backward writes the
    gradient into the same buffer."""
    return _CrossEntropyFn.apply(logits, target, vocab_start, group, scale)
