"""Cross-rank InfoNCE: fused all-gather + similarity GEMM + row softmax (``csrc/comm/contrastive.cu``).

``FusedInfoNCE.apply(anchors, positives)`` returns this rank's mean loss over its anchors against
the positives of *all* ranks.  Forward is one kernel launch (the logits matrix ``[R, W*R]`` is
never written); backward recomputes the logits with the GEMM kernel, turns them into
``softmax - onehot`` in place with the cross-entropy gradient kernel, and runs the two gradient
GEMMs; the positive gradients of all ranks are reduce-scattered back to their owners (fused
GEMM → reduce-scatter when a :class:`FusedTPContext` is given, NCCL otherwise).

Reference: ``info_nce_loss`` (crates/spiral-selfsup/src/contrastive.rs:96-153) — single rank.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops
from ..ops import loss as loss_ops
from ..ops import native
from .symm import MAX_RANKS, PeerSignals, SymmetricHeap, _PeerGroup

launch_count = 0


class _NceArgs(ctypes.Structure):
    _fields_ = [("g", _PeerGroup), ("anchors", ctypes.c_ulonglong), ("positives", ctypes.c_ulonglong),
                ("gather_peers", ctypes.c_ulonglong * MAX_RANKS), ("gather_mc", ctypes.c_ulonglong),
                ("partial", ctypes.c_ulonglong), ("counters", ctypes.c_ulonglong),
                ("row_loss", ctypes.c_ulonglong), ("row_lse", ctypes.c_ulonglong),
                ("R", ctypes.c_int), ("D", ctypes.c_int), ("inv_temperature", ctypes.c_float),
                ("slot_enter", ctypes.c_int), ("slot_arrive", ctypes.c_int), ("comm_ctas", ctypes.c_int),
                ("arrive_target", ctypes.c_uint)]


class FusedInfoNCE:
    def __init__(self, heap: SymmetricHeap, signals: PeerSignals, rows: int, dim: int, temperature: float = 0.1,
                 comm_ctas: int = 4, tp=None):
        self.heap, self.signals, self.R, self.D, self.temperature = heap, signals, rows, dim, temperature
        self.comm_ctas, self.tp = comm_ctas, tp
        W, dev = heap.world, heap.device
        self.gather = heap.empty(W * rows * dim, torch.bfloat16)
        groups = (W * rows) // 512
        self.partial = torch.empty(groups * rows * 3, dtype=torch.float32, device=dev)
        self.counters = torch.zeros(rows // 128, dtype=torch.int32, device=dev)
        self.slot_enter = signals.alloc(MAX_RANKS)
        self.slot_arrive = signals.alloc(MAX_RANKS)
        self.launches = 0

    def gathered(self) -> torch.Tensor:
        return self.gather.tensor.view(self.heap.world * self.R, self.D)

    def forward_stats(self, anchors: torch.Tensor, positives: torch.Tensor):
        """One fused launch → ``(row_loss [R], row_lse [R])``."""
        global launch_count
        assert anchors.shape == positives.shape == (self.R, self.D)
        a_ = anchors.to(torch.bfloat16).contiguous()
        p_ = positives.to(torch.bfloat16).contiguous()
        row_loss = torch.empty(self.R, dtype=torch.float32, device=a_.device)
        row_lse = torch.empty_like(row_loss)
        self.launches += 1
        args = _NceArgs()
        args.g = self.signals.next_group()
        args.anchors, args.positives = a_.data_ptr(), p_.data_ptr()
        args.gather_peers = self.gather.peers_array()
        args.gather_mc = self.gather.mc()
        args.partial, args.counters = self.partial.data_ptr(), self.counters.data_ptr()
        args.row_loss, args.row_lse = row_loss.data_ptr(), row_lse.data_ptr()
        args.R, args.D = self.R, self.D
        args.inv_temperature = 1.0 / self.temperature
        args.slot_enter, args.slot_arrive, args.comm_ctas = self.slot_enter, self.slot_arrive, self.comm_ctas
        args.arrive_target = (self.launches * self.comm_ctas) & 0xFFFFFFFF
        native.check(native.lib().st_info_nce_fwd(ctypes.byref(args), native.stream_ptr(a_.device)), "st_info_nce_fwd")
        launch_count += 1
        self._saved = (a_, p_)
        return row_loss, row_lse

    def apply(self, anchors: torch.Tensor, positives: torch.Tensor) -> torch.Tensor:
        native.poll()   # an earlier launch that gave up a bounded wait leaves the arrival counters out of step
        return _InfoNceFn.apply(anchors, positives, self)


def info_nce_grad(logits: torch.Tensor, row_lse: torch.Tensor, coef: torch.Tensor, target_offset: int):
    """``(exp(logits - lse) - onehot) * coef`` in bf16 as ``[R, C]`` and as ``[C, R]``; the positive of row ``r`` is
    column ``r + target_offset``.  One kernel pass over the fp32 logits on CUDA, plain tensor ops on CPU."""
    global launch_count
    R, C = logits.shape
    if not (logits.is_cuda and native.available()):
        prob = torch.exp(logits.float() - row_lse[:, None])
        idx = torch.arange(R, device=logits.device)
        prob[idx, idx + target_offset] -= 1.0
        dl = (prob * coef.float()).to(torch.bfloat16)
        return dl, dl.t().contiguous()
    lg = logits.float().contiguous()
    dl = torch.empty(R, C, dtype=torch.bfloat16, device=lg.device)
    dl_t = torch.empty(C, R, dtype=torch.bfloat16, device=lg.device)
    st = native.lib().st_info_nce_grad(native.ptr(lg), native.ptr(row_lse.float().contiguous()), native.ptr(coef.float().contiguous()),
                                       native.ptr(dl), native.ptr(dl_t), ctypes.c_int(R), ctypes.c_int(C),
                                       ctypes.c_int(target_offset), native.stream_ptr(lg.device))
    native.check(st, "st_info_nce_grad")
    launch_count += 1
    return dl, dl_t


class _InfoNceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchors, positives, op: FusedInfoNCE):
        row_loss, row_lse = op.forward_stats(anchors, positives)
        a_, _ = op._saved
        ctx.op = op
        ctx.save_for_backward(a_, row_lse)
        ctx.in_dtype = anchors.dtype
        return row_loss.mean()

    @staticmethod
    def backward(ctx, dloss):
        op = ctx.op
        a_, row_lse = ctx.saved_tensors
        W, R, rank = op.heap.world, op.R, op.heap.rank
        p_all = op.gathered()
        inv_t = 1.0 / op.temperature
        # fp32 logits: for a confident positive, softmax - 1 is a difference of nearly equal numbers
        # and bf16 logits (spacing 0.06 near 10) would lose most of its digits
        logits = gemm_ops.gemm(a_, p_all, alpha=inv_t, out_dtype=torch.float32)      # [R, W*R]
        coef = (dloss.float() / R).reshape(1).contiguous()
        dl, dl_t = info_nce_grad(logits, row_lse, coef, rank * R)                    # softmax - onehot, scaled; and its transpose
        d_anchor = gemm_ops.gemm(dl, p_all, b_mn=True, alpha=inv_t)
        if W == 1:
            d_pos = gemm_ops.gemm(dl_t, a_, b_mn=True, alpha=inv_t)
        elif op.tp is not None:
            d_pos = op.tp.gemm_rs(dl_t, a_, b_mn=True, alpha=inv_t)
        else:
            partial = gemm_ops.gemm(dl_t, a_, b_mn=True, alpha=inv_t)
            d_pos = torch.empty((R, op.D), dtype=partial.dtype, device=partial.device)
            dist.reduce_scatter_tensor(d_pos, partial.contiguous(), group=op.heap.group)
        return d_anchor.to(ctx.in_dtype), d_pos.to(ctx.in_dtype), None
