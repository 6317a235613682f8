#!/usr/bin/env python
"""Secondary benchmarks: the data-parallel configurations (byte-level char LM, conv-pool classifier,
contrastive encoder) at N GPUs, fused data-parallel step vs the NCCL all-reduce baseline.

    python benchmarks/dp_models.py --model charlm|conv|contrastive [--mode fused|nccl] [--steps K]
    python -m torch.distributed.run --nproc-per-node N ... benchmarks/dp_models.py --model conv

Prints one JSON line per run (rank 0): samples or tokens per second over the whole job, device-timed
(CUDA events, max over ranks), after 3 warm-up steps.  Weak scaling: the per-GPU batch is fixed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from spiraltorch_b200.models.conv_classifier import ConvClassifier  # noqa: E402
from spiraltorch_b200.models.contrastive import ContrastiveEncoder, make_views  # noqa: E402
from spiraltorch_b200.models.gpt import CHAR_LM, GPTModel  # noqa: E402
from spiraltorch_b200.optim.flat import FlatAdamW, FlatSGD  # noqa: E402
from spiraltorch_b200.parallel.dp import FusedDataParallel, NcclDataParallel  # noqa: E402
from spiraltorch_b200.selfsup import info_nce_torch  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="charlm", choices=["charlm", "conv", "contrastive"])
    ap.add_argument("--mode", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="replay the forward/backward pass from a CUDA graph (the step is launch-bound otherwise); the "
                         "data-parallel step stays outside the graph and is not overlapped with the backward pass")
    ap.add_argument("--clip", type=float, default=0.0,
                    help="global-norm clipping threshold applied in BOTH arms (0 = off): the fused step then runs its "
                         "two-phase form, the NCCL arm clips in the flat optimizer")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD if world > 1 else None
    torch.manual_seed(1000 + rank)

    fused = args.mode == "fused"
    if args.graph:
        args.no_overlap = True        # hooks fire at capture time only
    hyper = dict(lr=3e-4, weight_decay=0.0) if args.model != "conv" else dict(lr=0.005, momentum=0.9, weight_decay=0.0)
    kind = "sgd" if args.model == "conv" else "adamw"
    dp = FusedDataParallel(group, dev, kind=kind, overlap=not args.no_overlap, max_grad_norm=args.clip, **hyper) \
        if fused else None
    alloc = dp.allocator if fused else None

    if args.model == "charlm":
        model = GPTModel(CHAR_LM, device=dev, seed=7, allocator=alloc)
        probs = 1.0 / torch.arange(1, 257, dtype=torch.float64) ** 1.1          # Zipf(s=1.1) over byte ids
        toks = torch.multinomial(probs / probs.sum(), 32 * 513 * 2, replacement=True).view(2, 32, 513).to(dev)
        unit, per_step = "tokens/s", 32 * 512

        def fwd_bwd(i):
            return model.forward_backward(toks[i % 2, :, :-1].contiguous(), toks[i % 2, :, 1:].contiguous())
    elif args.model == "conv":
        model = ConvClassifier(num_classes=100, device=dev, seed=7, allocator=alloc)
        imgs = torch.randn(2, 256, 3, 64, 64, device=dev).bfloat16()
        labels = torch.randint(0, 100, (2, 256), device=dev)
        unit, per_step = "images/s", 256

        def fwd_bwd(i):
            return model.forward_backward(imgs[i % 2], labels[i % 2])
    else:
        model = None
        enc = ContrastiveEncoder(device=dev, seed=7)
        base = torch.randn(1024, 512, device=dev)
        unit, per_step = "samples/s", 1024
        from spiraltorch_b200.parallel.contrastive import FusedInfoNCE
        from spiraltorch_b200.parallel.symm import PeerSignals, SymmetricHeap
        heap = dp.heap if fused else SymmetricHeap(group, dev)
        sig = dp.signals if fused else PeerSignals(heap)
        nce = FusedInfoNCE(heap, sig, 1024, 256, 0.1) if fused else None
        opt_t = torch.optim.AdamW(enc.parameters(), lr=3e-4, fused=True)

        def fwd_bwd(i):
            opt_t.zero_grad(set_to_none=True)
            v1, v2 = make_views(base, 0.1)
            za, zp = enc(v1), enc(v2)
            if fused:
                loss = nce.apply(za, zp)
            else:
                gathered = [torch.empty_like(zp) for _ in range(world)] if world > 1 else [zp]
                if world > 1:
                    dist.all_gather(gathered, zp.contiguous())
                    gathered[rank] = zp
                allp = torch.cat(gathered, 0)
                logits = za @ allp.t() / 0.1
                idx = torch.arange(1024, device=dev) + rank * 1024
                loss = (torch.logsumexp(logits, -1) - logits[torch.arange(1024, device=dev), idx]).mean()
            loss.backward()
            if world > 1:
                flat = torch.cat([p.grad.reshape(-1) for p in enc.parameters()])
                dist.all_reduce(flat)
                flat /= world
                off = 0
                for p in enc.parameters():
                    p.grad.copy_(flat[off:off + p.numel()].view_as(p))
                    off += p.numel()
            opt_t.step()
            return loss.detach()

    if model is not None:
        if fused:
            dp.attach(model)
        else:
            opt = (FlatSGD(model, lr=0.005, momentum=0.9, max_grad_norm=args.clip) if kind == "sgd" else
                   FlatAdamW(model, lr=3e-4, weight_decay=0.0, max_grad_norm=args.clip))
            nccl = NcclDataParallel(model, opt, group)

    if args.graph and model is not None:
        from spiraltorch_b200.training import GraphedForwardBackward
        if args.model == "charlm":
            graphed = GraphedForwardBackward(model, (toks[0, :, :-1].contiguous(), toks[0, :, 1:].contiguous()))

            def fwd_bwd(i):   # noqa: F811
                return graphed(toks[i % 2, :, :-1], toks[i % 2, :, 1:])
        else:
            graphed = GraphedForwardBackward(model, (imgs[0], labels[0]))

            def fwd_bwd(i):   # noqa: F811
                return graphed(imgs[i % 2], labels[i % 2])

    def step(i):
        if model is None:
            return fwd_bwd(i)
        if fused:
            dp.arm()
            loss = fwd_bwd(i)
            dp.finish_step()
        else:
            loss = fwd_bwd(i)
            nccl.finish_step()
        return loss

    for i in range(args.warmup):
        loss = step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(i)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    from spiraltorch_b200.ops import native
    native.raise_on_device_error()
    if rank == 0:
        print(json.dumps({"model": args.model, "mode": args.mode, "n_gpus": world, "unit": unit,
                          "value": per_step * world * args.steps / (ms.item() / 1e3),
                          "ms_per_step": ms.item() / args.steps, "loss": float(loss), "scaling": "weak",
                          "overlap": not args.no_overlap, "clip": args.clip, "cuda_graph": bool(args.graph)}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
