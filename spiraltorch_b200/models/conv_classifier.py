"""Conv-pool image classifier: 4 stages of [conv3x3+bias+ReLU x2, max-pool 2x2] with channels
64/128/256/512, global average pool, Linear(512, classes) — with a hand-scheduled backward.

Images arrive NCHW fp32/bf16 (the public API layout) and are converted once to NHWC bf16; all
convolutions run as implicit GEMMs with bias+ReLU fused in the epilogue, data gradients fuse the
ReLU mask, weight gradients accumulate in fp32.  Parameters live in one flat buffer (bf16 weights +
fp32 ``main_grad``) so the flat optimizers and the fused data-parallel step apply directly.
Checkpoint keys follow the reference: ``conv{s}_{i}::weight`` of shape ``(OC, IC*3*3)`` with K ordered
``[ic][kh][kw]``, ``conv{s}_{i}::bias`` ``(1, OC)``, ``head::weight`` ``(512, classes)`` stored (in, out).

The reference's conv-pool model is a single 1→4 channel conv on 8x8 images
(models/python/vision_conv_pool_classification.py:183-197); this is the scaled-up family member.
"""
from __future__ import annotations

import math
import zlib
from typing import Optional

import torch
import torch.nn as nn

from ..ops import conv as C
from ..ops import elementwise as ew
from ..ops import gemm as gemm_ops
from ..ops import loss as loss_ops

STAGES = (64, 128, 256, 512)


class ConvClassifier(nn.Module):
    def __init__(self, num_classes: int = 100, in_channels: int = 3, image: int = 64, device="cuda",
                 dtype=torch.bfloat16, seed: int = 0, allocator=None):
        super().__init__()
        self.num_classes, self.in_channels, self.image, self.dtype = num_classes, in_channels, image, dtype
        self.classes_pad = (num_classes + 7) // 8 * 8
        self.grad_ready_hook = None
        shapes = []
        ic = in_channels
        for s, oc in enumerate(STAGES):
            for i in range(2):
                shapes.append((f"conv{s}_{i}.weight", (oc, 9 * ic)))
                shapes.append((f"conv{s}_{i}.bias", (oc,)))
                ic = oc
        shapes += [("head.weight", (self.classes_pad, 512)), ("head.bias", (self.classes_pad,))]
        offsets, off = {}, 0
        for name, shp in shapes:
            n = math.prod(shp)
            offsets[name] = (off, n, shp)
            off += (n + 127) // 128 * 128
        self.flat_elems = off
        self.decay_elems = off
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat_w = alloc(off, dtype)
        self.flat_grad = alloc(off, torch.float32)
        self._offsets = offsets
        self.p = {}
        for name, (o, n, shp) in offsets.items():
            view = self.flat_w[o:o + n].view(shp)
            if name.endswith("weight"):
                fan_in = shp[1]
                g = torch.Generator().manual_seed(zlib.crc32(f"{seed}/{name}".encode()) & 0x7FFFFFFF)
                view.copy_((torch.randn(shp, generator=g) * math.sqrt(2.0 / fan_in)).to(dtype))
                if name == "head.weight":
                    view[num_classes:].zero_()
            p = nn.Parameter(view, requires_grad=True)
            p.main_grad = self.flat_grad[o:o + n].view(shp)
            self.p[name] = p
            self.register_parameter(name.replace(".", "_"), p)

    # ------------------------------------------------------------------------------------------
    def forward_backward(self, images, labels, loss_scale: float = 1.0, backward: bool = True, layer_done=None):
        with torch.no_grad():
            return self._forward_backward(images, labels, loss_scale, backward, layer_done or self.grad_ready_hook)

    def _forward_backward(self, images: torch.Tensor, labels: Optional[torch.Tensor], loss_scale: float = 1.0,
                          backward: bool = True, layer_done=None):
        """``images`` NCHW; ``labels`` int64 ``[N]``.  Returns the mean loss (and accumulates gradients
        into ``main_grad``), or the logits when ``labels`` is None.  ``layer_done(name)`` is called as
        soon as the gradient of a parameter tensor is final (hook for overlapping the all-reduce)."""
        P = self.p
        x = images.to(self.flat_w.device, self.dtype).permute(0, 2, 3, 1).contiguous()
        acts, pools = [x], []
        for s in range(4):
            for i in range(2):
                x = C.conv3x3(x, P[f"conv{s}_{i}.weight"], P[f"conv{s}_{i}.bias"], relu=True)
                acts.append(x)
            x, idx = C.maxpool2(x)
            pools.append((idx, acts[-1].shape[1], acts[-1].shape[2]))
            acts.append(x)
        N, H, W, Cc = x.shape
        feat = C.global_avgpool(x)
        logits = gemm_ops.gemm(feat, P["head.weight"], bias=P["head.bias"])
        if labels is None:
            return logits[:, : self.num_classes]
        if self.classes_pad != self.num_classes:
            logits[:, self.num_classes:] = -30000.0
        tgt = labels.to(logits.device, torch.int64).contiguous()
        m, sm, t = loss_ops._stats(logits, tgt, 0)
        lse = m + torch.log(sm)
        loss = (lse - t).mean() * loss_scale
        if not backward:
            return loss
        coef = torch.full((1,), loss_scale / N, dtype=torch.float32, device=logits.device)
        dlogits = loss_ops._grad_(logits, tgt, lse, coef, 1.0, 0)
        gemm_ops.gemm(dlogits, feat, a_mn=True, b_mn=True, out=P["head.weight"].main_grad, accumulate=True)
        ew.colsum(dlogits, P["head.bias"].main_grad, accumulate=True)
        dfeat = gemm_ops.gemm(dlogits, P["head.weight"], b_mn=True)
        if layer_done:
            layer_done("head")          # only after the last read of the head weights
        d = C.global_avgpool_backward(dfeat, H, W)
        k = len(acts) - 1                           # index of the pooled output of the last stage
        for s in reversed(range(4)):
            idx, ph, pw = pools[s]
            d = C.maxpool2_backward(d, idx, ph, pw)         # gradient w.r.t. the (post-ReLU) conv output
            k -= 1                                          # acts[k] = output of conv s_1
            for i in (1, 0):
                y, xin = acts[k], acts[k - 1]
                if i == 1:
                    # the pooled gradient is already zero where the ReLU was inactive only by chance: mask it
                    d = torch.where(y > 0, d, torch.zeros_like(d))
                w = P[f"conv{s}_{i}.weight"]
                ic = xin.shape[-1]
                C.conv3x3_wgrad(d, xin, w.main_grad)
                ew.colsum(d.reshape(-1, d.shape[-1]), P[f"conv{s}_{i}.bias"].main_grad, accumulate=True)
                if k - 1 > 0:
                    d = C.conv3x3(d, C.dgrad_weights(w, ic), relu_mask_of=xin)
                if layer_done:
                    layer_done(f"conv{s}_{i}")   # after the data gradient has read the weights
                k -= 1
        return loss

    def forward(self, images, labels=None, loss_scale: float = 1.0):
        with torch.no_grad():
            return self.forward_backward(images, labels, loss_scale, backward=False)

    def zero_grad_buffers(self):
        self.flat_grad.zero_()

    def reference_state_dict(self) -> list:
        """``(name, Tensor)`` pairs in the reference checkpoint layout."""
        from ..tensor import Tensor
        out = []
        for name, p in self.p.items():
            mod, kind = name.split(".")
            t = p.detach().float().cpu()
            if mod == "head":
                t = t[: self.num_classes].t().contiguous() if kind == "weight" else t[: self.num_classes].reshape(1, -1)
            elif kind == "weight":
                t = C.from_tap_major(t, t.shape[1] // 9)
            else:
                t = t.reshape(1, -1)
            out.append((f"{mod}::{kind}", Tensor._wrap(t)))
        return sorted(out, key=lambda kv: kv[0])
