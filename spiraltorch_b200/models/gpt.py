"""GPT-style decoder-only language model (RMSNorm, RoPE, GELU MLP, tied embedding) with a
hand-scheduled forward/backward over the sm_100a kernels and optional tensor parallelism.

Design
------
* All weights live in ONE flat bf16 buffer with fp32 master / Adam moments / fp32 gradient
  buffers of the same length; every ``nn.Parameter`` is a view and carries ``main_grad``
  (a view of the flat fp32 gradient).  Weight gradients are accumulated in fp32 directly by
  the GEMM epilogue, so micro-batches need no extra pass.
* The step is written out by hand (no autograd graph): each layer's backward re-uses the
  saved activations and the fused epilogues (GELU + pre-activation store in FC1, GELU'
  multiply in the FC2 data-gradient, residual adds inside the norm kernels).
  :class:`GPTModel.forward` wraps the same code in one ``autograd.Function`` so
  ``loss.backward()`` works for API users.
* Tensor parallelism follows the sequence-parallel scheme: activations between sub-blocks
  are row shards, QKV/FC1 are column-parallel (all-gather → GEMM), out-proj/FC2 are
  row-parallel (GEMM → reduce-scatter), attention is head-parallel, the embedding and the
  tied LM head are vocab-parallel with a vocab-parallel cross-entropy.

The reference has no transformer LM with a backward pass (its ViT attention is forward-only,
crates/st-vision/src/models/vit.rs:133-189); the configuration follows the benchmark
description: d_model 2048, 24 layers, 16 heads, FFN 8192, vocab 50304, sequence 2048.
"""
from __future__ import annotations

import math
import os
import zlib
from dataclasses import dataclass, asdict
from typing import Optional

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm as gemm_ops
from ..ops import loss as loss_ops
from ..ops import native
from ..ops import norm as norm_ops
from ..parallel.tp import TPContext


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    d_model: int = 2048
    n_layers: int = 24
    n_heads: int = 16
    ffn: int = 8192
    seq_len: int = 2048
    rope_base: float = 10000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    norm: str = "rms"            # "rms" | "layer"
    positional: str = "rope"     # "rope" | "learned"
    bias: bool = False

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def param_count(self) -> int:
        per_layer = 4 * self.d_model ** 2 + 2 * self.d_model * self.ffn + 2 * self.d_model
        n = self.n_layers * per_layer + self.vocab_size * self.d_model + self.d_model
        if self.positional == "learned":
            n += self.seq_len * self.d_model
        return n

    def flops_per_token(self) -> float:
        """Training FLOPs per token (fwd+bwd), causal attention counted at half density."""
        dense = 6.0 * (self.n_layers * (4 * self.d_model ** 2 + 2 * self.d_model * self.ffn)
                       + self.vocab_size * self.d_model)
        attn = 6.0 * self.n_layers * 2 * self.seq_len * self.d_model / 2
        return dense + attn


GPT_1P3B = GPTConfig()
CHAR_LM = GPTConfig(vocab_size=256, d_model=768, n_layers=12, n_heads=12, ffn=3072, seq_len=512,
                    norm="layer", positional="learned")


class _Act:
    """Activations one layer keeps for its backward."""
    __slots__ = ("h1", "stat1", "y1_full", "qkv", "o", "lse", "h2", "stat2", "y2_full", "u", "a")


class GPTModel(nn.Module):
    def __init__(self, cfg: GPTConfig, device="cuda", dtype=torch.bfloat16,
                 tp: Optional[TPContext] = None, seed: int = 0, allocator=None):
        super().__init__()
        self.cfg = cfg
        self.grad_ready_hook = None   # called with a parameter-group name once its gradient is final
        self.tp = tp or TPContext()
        # fused collectives wait (bounded) on peers: poll their error record between layers
        self._fused_tp = type(self.tp).__name__ == "FusedTPContext" and torch.device(device).type == "cuda"
        W = self.tp.world
        assert cfg.n_heads % W == 0 and cfg.ffn % W == 0 and cfg.vocab_size % W == 0
        # Weight-gradient GEMMs need no communication.  When the fused linears are link-bound (many ranks, thin
        # per-rank GEMMs) they can run beside them: the backward pass launches its fused kernels on a grid that
        # leaves `_wgrad_ctas` SMs free and queues the weight gradients on a second stream, limited to those SMs.
        # ST_TP_WGRAD_OVERLAP=0/1 forces it off / on; ST_TP_WGRAD_CTAS sets the share (default 40 of 148).
        self._wgrad_ctas, self._wgrad_stream, self._wgrad_guard = 0, None, {}
        if self._fused_tp:
            env = os.environ.get("ST_TP_WGRAD_OVERLAP")
            if (W >= 6) if env is None else env == "1":
                self._wgrad_ctas = int(os.environ.get("ST_TP_WGRAD_CTAS", "40"))
                self._wgrad_stream = torch.cuda.Stream(torch.device(device))
        assert cfg.head_dim in (64, 128), "attention kernels support head_dim 64 and 128"
        self.heads_local = cfg.n_heads // W
        self.ffn_local = cfg.ffn // W
        self.vocab_local = cfg.vocab_size // W
        self.vocab_start = self.vocab_local * self.tp.rank
        self.dtype = dtype
        d, hl, D = cfg.d_model, self.heads_local, cfg.head_dim

        # ---- flat storage -------------------------------------------------------------------
        shapes = [("embed.weight", (self.vocab_local, d), True)]
        if cfg.positional == "learned":
            shapes.append(("pos.weight", (cfg.seq_len, d), False))
        for l in range(cfg.n_layers):
            shapes += [
                (f"h{l}.norm1.gamma", (d,), False),
                (f"h{l}.qkv.weight", (3 * hl * D, d), True),
                (f"h{l}.proj.weight", (d, hl * D), True),
                (f"h{l}.norm2.gamma", (d,), False),
                (f"h{l}.fc1.weight", (self.ffn_local, d), True),
                (f"h{l}.fc2.weight", (d, self.ffn_local), True),
            ]
            if cfg.norm == "layer":
                shapes += [(f"h{l}.norm1.beta", (d,), False), (f"h{l}.norm2.beta", (d,), False)]
        shapes.append(("norm_f.gamma", (d,), False))
        if cfg.norm == "layer":
            shapes.append(("norm_f.beta", (d,), False))
        # decayed (matrix) parameters first so that weight decay applies to one contiguous range
        shapes.sort(key=lambda s: not s[2])
        offsets, off = {}, 0
        for name, shp, _ in shapes:
            n = math.prod(shp)
            offsets[name] = (off, n, shp)
            off += (n + 127) // 128 * 128  # keep every tensor 256-byte aligned
        last_decayed = [s[0] for s in shapes if s[2]][-1]
        self.decay_elems = (offsets[last_decayed][0] + offsets[last_decayed][1] + 127) // 128 * 128
        self.flat_elems = off
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat_w = alloc(off, dtype)
        self.flat_grad = alloc(off, torch.float32)
        self._offsets = offsets
        self._names = [s[0] for s in shapes]

        params = {}
        for name, (o, n, shp) in offsets.items():
            view = self.flat_w[o:o + n].view(shp)
            if name.endswith("gamma"):
                view.fill_(1.0)
            elif name.endswith("beta"):
                view.zero_()
            else:
                # every rank draws the full tensor's stream position deterministically from the name
                key = zlib.crc32(f"{seed}/{name}/{self.tp.rank}".encode()) & 0x7FFFFFFF
                gdev = "cuda" if self.flat_w.is_cuda else "cpu"
                g = torch.Generator(device=self.flat_w.device if gdev == "cuda" else "cpu").manual_seed(key)
                view.copy_((torch.randn(shp, generator=g, device=self.flat_w.device) * cfg.init_std).to(dtype))
            p = nn.Parameter(view, requires_grad=True)
            p.main_grad = self.flat_grad[o:o + n].view(shp)
            params[name] = p
            self.register_parameter(name.replace(".", "_"), p)
        self.p = params
        self.last_loss: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------
    def named_flat_views(self):
        for name in self._names:
            o, n, shp = self._offsets[name]
            yield name, o, n, shp

    def _norm_fwd(self, x, name, residual=None, gather_key=None):
        """``gather_key``: the all-gather this output feeds; the context may offer the shard's place inside its
        gather buffer, which saves the fused all-gather the local copy."""
        rms = self.cfg.norm == "rms"
        beta = None if rms else self.p[name + ".beta"]
        out = None if gather_key is None else self.tp.shard_slot(gather_key, x.shape[0], x.shape[1])
        return norm_ops.norm_forward(x, self.p[name + ".gamma"], beta, self.cfg.norm_eps, rms, residual, out=out)

    def _norm_bwd(self, dy, x, stat, name, dres=None, gather_key=None):
        rms = self.cfg.norm == "rms"
        mean, rstd = stat
        beta_g = None if rms else self.p[name + ".beta"].main_grad
        out = None if gather_key is None else self.tp.shard_slot(gather_key, x.shape[0], x.shape[1])
        return norm_ops.norm_backward(dy, x, self.p[name + ".gamma"], mean, rstd, rms,
                                      self.p[name + ".gamma"].main_grad, beta_g, True, dres, out=out)

    # ------------------------------------------------------------------------------------------
    def _layer_forward(self, l: int, resid, x, B: int, S: int, keep: bool):
        cfg, tp, hl, D = self.cfg, self.tp, self.heads_local, self.cfg.head_dim
        P = self.p
        act = _Act()
        if x is None:
            y1, _, m1, r1 = self._norm_fwd(resid, f"h{l}.norm1", gather_key=(l, "y1"))
            h1 = resid
        else:
            y1, h1, m1, r1 = self._norm_fwd(x, f"h{l}.norm1", residual=resid, gather_key=(l, "y1"))
        qkv, y1_full = tp.ag_gemm(y1, P[f"h{l}.qkv.weight"], key=(l, "y1"))
        if cfg.positional == "rope":
            ew.rope_(qkv, 2 * hl, D, S, cfg.rope_base)
        qkv5 = qkv.view(B, S, 3, hl, D)
        o, lse = attn_ops.attention_forward(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], True)
        attn_out = tp.gemm_rs(o.view(B * S, hl * D), P[f"h{l}.proj.weight"])
        y2, h2, m2, r2 = self._norm_fwd(attn_out, f"h{l}.norm2", residual=h1, gather_key=(l, "y2"))
        u = torch.empty((y2.shape[0] * tp.world, self.ffn_local), dtype=y2.dtype, device=y2.device)
        a, y2_full = tp.ag_gemm(y2, P[f"h{l}.fc1.weight"], key=(l, "y2"), act="gelu", aux_out=u)
        mlp_out = tp.gemm_rs(a, P[f"h{l}.fc2.weight"])
        if keep:
            act.h1, act.stat1, act.y1_full, act.qkv, act.o, act.lse = h1, (m1, r1), y1_full, qkv, o, lse
            act.h2, act.stat2, act.y2_full, act.u, act.a = h2, (m2, r2), y2_full, u, a
        return h2, mlp_out, act

    def _wgrads(self, jobs, gather_keys=()):
        """``out += a^T b`` for every ``(a, b, out)``.  With the overlap on, the products are queued on the side stream
        (after everything the main stream has launched so far) and `gather_keys` names the gather buffers they read:
        the next all-gather into one of those waits for them."""
        g = gemm_ops.gemm
        if not self._wgrad_ctas:
            for a, b, out in jobs:
                g(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
            return
        side, main = self._wgrad_stream, torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for a, b, out in jobs:
                g(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, max_ctas=self._wgrad_ctas)
                a.record_stream(side)
                b.record_stream(side)
            done = torch.cuda.Event()
            done.record(side)
        for k in gather_keys:
            self._wgrad_guard[k] = done

    def _wgrad_wait(self, key) -> None:
        """Before the gather buffer `key` is written again: the weight gradients that still read it must be done."""
        ev = self._wgrad_guard.pop(key, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _wgrad_join(self) -> None:
        if self._wgrad_stream is not None:
            torch.cuda.current_stream().wait_stream(self._wgrad_stream)
            self._wgrad_guard.clear()

    def _layer_backward(self, l: int, act: _Act, d_out, B: int, S: int):
        """``d_out`` is the gradient w.r.t. both outputs (h2 and mlp_out) of the layer.  Its gather buffers alternate
        with the layer's parity, so that the weight gradients of one layer may still read theirs while the next
        layer's all-gathers already fill the other pair."""
        cfg, tp, hl, D = self.cfg, self.tp, self.heads_local, self.cfg.head_dim
        P = self.p
        w1, w2 = P[f"h{l}.fc1.weight"], P[f"h{l}.fc2.weight"]
        wqkv, wo = P[f"h{l}.qkv.weight"], P[f"h{l}.proj.weight"]
        k_mlp, k_attn = ("bwd_mlp", l & 1), ("bwd_attn", l & 1)
        self._wgrad_wait(k_mlp)
        du, dmlp_full = tp.ag_gemm(d_out, w2, b_mn=True, key=k_mlp, act="gelu_bwd", aux_in=act.u)
        self._wgrads([(dmlp_full, act.a, w2.main_grad), (du, act.y2_full, w1.main_grad)], (k_mlp,))
        dy2 = tp.gemm_rs(du, w1, b_mn=True)
        self._wgrad_wait(k_attn)
        d_h2 = self._norm_bwd(dy2, act.h2, act.stat2, f"h{l}.norm2", dres=d_out, gather_key=k_attn)
        o2 = act.o.view(B * S, hl * D)
        do, dh2_full = tp.ag_gemm(d_h2, wo, b_mn=True, key=k_attn)
        self._wgrads([(dh2_full, o2, wo.main_grad)], (k_attn,))
        dqkv = torch.empty_like(act.qkv)
        qkv5, dqkv5 = act.qkv.view(B, S, 3, hl, D), dqkv.view(B, S, 3, hl, D)
        attn_ops.attention_backward(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], act.o, act.lse,
                                    do.view(B, S, hl, D), True, None,
                                    dq=dqkv5[:, :, 0], dk=dqkv5[:, :, 1], dv=dqkv5[:, :, 2])
        if cfg.positional == "rope":
            ew.rope_(dqkv, 2 * hl, D, S, cfg.rope_base, backward=True)
        self._wgrads([(dqkv, act.y1_full, wqkv.main_grad)])
        dy1 = tp.gemm_rs(dqkv, wqkv, b_mn=True)
        # the result is the next layer's `d_out`, which its first all-gather pushes
        nxt = ("bwd_mlp", (l - 1) & 1)
        if l > 0:
            self._wgrad_wait(nxt)
        return self._norm_bwd(dy1, act.h1, act.stat1, f"h{l}.norm1", dres=d_h2, gather_key=nxt if l > 0 else None)

    # ------------------------------------------------------------------------------------------
    def _forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor], loss_scale: float,
                 keep: bool):
        cfg, tp = self.cfg, self.tp
        B, S = tokens.shape
        T = B * S
        assert T % tp.world == 0
        emb = self.p["embed.weight"]
        pos = self.p.get("pos.weight")
        assert pos is None or tp.world == 1, "learned positions are only used by the data-parallel models"
        h_full = ew.embedding_forward(tokens, emb, pos, S, self.vocab_start)
        resid = tp.reduce_scatter_rows(h_full)
        x = None
        acts = []
        for l in range(cfg.n_layers):
            resid, x, act = self._layer_forward(l, resid, x, B, S, keep=keep)
            acts.append(act)
            if self._fused_tp and native.error_pending():
                native.raise_on_device_error()     # a bounded wait ran out: stop now, not 2 s per kernel later
        yf, hf, mf, rf = self._norm_fwd(x, "norm_f", residual=resid, gather_key="head")
        logits, yf_full = tp.ag_gemm(yf, emb, key="head")
        if targets is None:
            return logits, None
        tgt = targets.reshape(-1).to(torch.int64).contiguous()
        m, s, t = loss_ops._stats(logits, tgt, self.vocab_start)
        if tp.world > 1:
            gm = m.clone()
            tp.all_reduce_(gm, op=torch.distributed.ReduceOp.MAX)
            packed = torch.stack([s * torch.exp(m - gm), t])
            tp.all_reduce_(packed)
            m, s, t = gm, packed[0], packed[1]
        lse = m + torch.log(s)
        valid = tgt != loss_ops.IGNORE_INDEX
        n_valid = valid.sum().clamp(min=1).to(torch.float32)
        loss = ((lse - t) * valid).sum() / n_valid * loss_scale
        self.last_loss = loss
        state = (tokens, tgt, logits, lse, n_valid, loss_scale, yf_full, hf, (mf, rf), acts, B, S) if keep else None
        return loss, state

    def _backward(self, state, dloss: Optional[torch.Tensor] = None) -> None:
        tokens, tgt, logits, lse, n_valid, loss_scale, yf_full, hf, statf, acts, B, S = state
        cfg, tp = self.cfg, self.tp
        emb = self.p["embed.weight"]
        pos = self.p.get("pos.weight")
        coef = (loss_scale / n_valid).reshape(1).to(torch.float32)
        if dloss is not None:
            coef = coef * dloss.to(torch.float32).reshape(1)
        dlogits = loss_ops._grad_(logits, tgt, lse, coef.contiguous(), 1.0, self.vocab_start)
        overlap = self._wgrad_ctas > 0
        if overlap:
            tp.max_ctas = max(torch.cuda.get_device_properties(dlogits.device).multi_processor_count - self._wgrad_ctas, 1)
        try:
            self._wgrads([(dlogits, yf_full, emb.main_grad)])
            dyf = tp.gemm_rs(dlogits, emb, b_mn=True)
            d = self._norm_bwd(dyf, hf, statf, "norm_f", gather_key=("bwd_mlp", (cfg.n_layers - 1) & 1))
            for l in reversed(range(cfg.n_layers)):
                d = self._layer_backward(l, acts[l], d, B, S)
                acts[l] = None
                if self._fused_tp and native.error_pending():
                    native.raise_on_device_error()
                if self.grad_ready_hook is not None:
                    self._wgrad_join()
                    self.grad_ready_hook(f"h{l}")
        finally:
            if overlap:
                tp.max_ctas = 0
        self._wgrad_join()              # the embedding gradient below and the optimizer read what the side stream wrote
        d_full = tp.all_gather_rows(d)
        dpos = pos.main_grad if pos is not None else None
        ew.embedding_backward(tokens, d_full.contiguous(), emb.main_grad, dpos, S, self.vocab_start)
        if self.grad_ready_hook is not None:
            self.grad_ready_hook("embed")

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor,
                         loss_scale: float = 1.0) -> torch.Tensor:
        """One micro-batch: returns the (scaled) mean token loss and accumulates every parameter
        gradient into ``main_grad`` (fp32).  ``tokens``/``targets`` are ``[B, S]`` int64 and
        identical on every tensor-parallel rank."""
        with torch.no_grad():
            loss, state = self._forward(tokens, targets, loss_scale, keep=True)
            self._backward(state)
        return loss

    def forward(self, tokens, targets=None, loss_scale: float = 1.0):
        """``model(tokens)`` → logits; ``model(tokens, targets)`` → loss.  Under autograd the loss
        is differentiable: ``loss.backward()`` accumulates into each parameter's ``main_grad``."""
        if targets is None or not torch.is_grad_enabled():
            with torch.no_grad():
                out, _ = self._forward(tokens, targets, loss_scale, keep=False)
            return out
        return _GPTLossFn.apply(self, tokens, targets, loss_scale, self.p["norm_f.gamma"])

    # ------------------------------------------------------------------------------------------
    def sync_replicated_grads(self) -> None:
        """Norm gains (and the learned positions) are replicated across tensor-parallel ranks
        but see only their sequence shard: sum their gradients over the group."""
        if self.tp.world == 1:
            return
        self.tp.all_reduce_(self.flat_grad[self.decay_elems:])

    def zero_grad_buffers(self) -> None:
        self.flat_grad.zero_()

    def state_dict_unsharded(self) -> dict:
        """Gather tensor-parallel shards into full ``[out, in]`` matrices (for checkpoints)."""
        import torch.distributed as dist
        out = {}
        W = self.tp.world
        for name, p in self.p.items():
            t = p.detach()
            if W > 1 and (name.endswith("qkv.weight") or name.endswith("fc1.weight") or name == "embed.weight"):
                parts = [torch.empty_like(t) for _ in range(W)]
                dist.all_gather(parts, t.contiguous(), group=self.tp.group)
                if name.endswith("qkv.weight"):
                    hl, D = self.heads_local, self.cfg.head_dim
                    parts = [x.view(3, hl, D, -1) for x in parts]
                    t = torch.cat(parts, dim=1).reshape(3 * self.cfg.n_heads * D, -1)
                else:
                    t = torch.cat(parts, dim=0)
            elif W > 1 and (name.endswith("proj.weight") or name.endswith("fc2.weight")):
                parts = [torch.empty_like(t) for _ in range(W)]
                dist.all_gather(parts, t.contiguous(), group=self.tp.group)
                t = torch.cat(parts, dim=1)
            out[name] = t.float().cpu()
        return out

    def load_unsharded(self, full: dict) -> None:
        """Load full (tensor-parallel-free) tensors, keeping this rank's shard of each."""
        W, r = self.tp.world, self.tp.rank
        hl, D, H = self.heads_local, self.cfg.head_dim, self.cfg.n_heads
        with torch.no_grad():
            for name, p in self.p.items():
                t = full[name]
                if W > 1:
                    if name.endswith("qkv.weight"):
                        t = t.view(3, H, D, -1)[:, r * hl:(r + 1) * hl].reshape(3 * hl * D, -1)
                    elif name.endswith("fc1.weight") or name == "embed.weight":
                        t = t.chunk(W, dim=0)[r]
                    elif name.endswith("proj.weight") or name.endswith("fc2.weight"):
                        t = t.chunk(W, dim=1)[r]
                p.copy_(t.to(p.dtype))

    def describe(self) -> dict:
        d = asdict(self.cfg)
        d.update(params=self.cfg.param_count(), tp=self.tp.world, flat_elems_per_rank=self.flat_elems)
        return d


class _GPTLossFn(torch.autograd.Function):
    """Autograd façade over the hand-scheduled step.  Gradients are accumulated into the
    parameters' fp32 ``main_grad`` buffers by the kernels themselves; autograd only carries
    the scalar ``dloss`` into the scheduled backward."""

    @staticmethod
    def forward(ctx, model: GPTModel, tokens, targets, loss_scale, anchor):
        loss, state = model._forward(tokens, targets, loss_scale, keep=True)
        ctx.model, ctx.state = model, state
        return loss.clone()

    @staticmethod
    def backward(ctx, dloss):
        with torch.no_grad():
            ctx.model._backward(ctx.state, dloss)
        ctx.state = None
        return None, None, None, None, None
