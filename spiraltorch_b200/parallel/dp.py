"""Data parallelism over flat parameter buffers.

``FusedDataParallel`` keeps a model's flat bf16 weights and fp32 gradient buffer in symmetric
memory and runs the data-parallel step bucket by bucket with the fused kernel of
``csrc/comm/dp_step.cu`` (reduce-scatter + 1/world + optimizer on the owned shard + all-gather
of the new weights, one launch per bucket).  Optimizer state is sharded across the ranks.
With ``overlap=True`` a bucket is launched on a side stream as soon as the backward pass has
finalised every gradient it contains (the models call ``grad_ready_hook``), so communication
and the optimizer overlap the remaining backward kernels.

``NcclDataParallel`` is the baseline: NCCL all-reduce of the flat gradient + the unfused flat
optimizer.

Reference semantics: all-reduce **mean** of every accumulator, then the optimizer step
(crates/st-nn/src/trainer.rs:7259-7268, :9035-9062); no bucketing or overlap exists there.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from .symm import FusedDPStep, PeerSignals, SymmetricHeap


class SymmetricAllocator:
    """Allocator for model flat buffers: symmetric memory, length padded to ``8 * world * 128``."""

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.buffers: dict = {}

    def __call__(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        gran = 8 * self.heap.world * 128
        padded = (numel + gran - 1) // gran * gran
        buf = self.heap.empty(padded, dtype, zero=True)
        self.buffers[dtype] = buf
        return buf.tensor[:numel]


class FusedDataParallel:
    def __init__(self, group, device, kind: str = "adamw", bucket_mb: float = 32.0, overlap: bool = True,
                 comm_ctas: int = 32, max_grad_norm: float = 0.0, **hyper):
        """``max_grad_norm > 0``: clip by the global norm of the averaged gradient.  The reductions still overlap
        the backward pass bucket by bucket; the clipped update and the weight broadcast of every bucket follow
        once the backward pass has ended (same optimizer as the single-GPU and NCCL paths)."""
        self.max_grad_norm = float(max_grad_norm)
        self.heap = SymmetricHeap(group, device)
        self.signals = PeerSignals(self.heap)
        self.allocator = SymmetricAllocator(self.heap)
        self.kind, self.hyper, self.overlap = kind, hyper, overlap
        self.bucket_elems = int(bucket_mb * (1 << 20) / 4)
        if self.heap.world == 1:
            # nothing to overlap with: one launch over the whole gradient buffer on the compute stream (per-bucket
            # launches on a side stream only add launch and stream-switch latency to a launch-bound step)
            self.overlap = False
            self.bucket_elems = 1 << 40
        self.comm_ctas = comm_ctas
        self.model = None
        self.dp: Optional[FusedDPStep] = None
        self.stream = torch.cuda.Stream(device) if torch.device(device).type == "cuda" else None
        self._armed = False

    def attach(self, model) -> None:
        """Call after constructing the model with ``allocator=self.allocator``."""
        self.model = model
        grad, w = self.allocator.buffers[torch.float32], self.allocator.buffers[model.flat_w.dtype]
        self.dp = FusedDPStep(self.heap, self.signals, grad, w, kind=self.kind, bucket_elems=self.bucket_elems,
                              max_ctas=self.comm_ctas if self.overlap else 0, max_grad_norm=self.max_grad_norm)
        # which parameter groups does each bucket need?
        spans = {}
        for name, (o, n, _) in model._offsets.items():
            group = name.split(".")[0]
            lo, hi = spans.get(group, (o, o + n))
            spans[group] = (min(lo, o), max(hi, o + n))
        self._bucket_needs = []
        for (off, ln, *_r) in self.dp.buckets:
            self._bucket_needs.append({g for g, (lo, hi) in spans.items() if lo < off + ln and hi > off})
        self._done: set = set()
        self._launched: set = set()
        if hasattr(model, "grad_ready_hook"):
            model.grad_ready_hook = self._on_ready

    def arm(self) -> None:
        """Enable bucket launches for the coming backward pass (the last micro-batch of a step)."""
        self._armed = True
        self._done.clear()
        self._launched.clear()
        self.dp.begin_step()

    def _launch(self, i: int) -> None:
        if self.stream is not None and self.overlap:
            self.stream.wait_stream(torch.cuda.current_stream(self.heap.device))
            with torch.cuda.stream(self.stream):
                self._bucket_kernel(i)
        else:
            self._bucket_kernel(i)
        self._launched.add(i)

    def _bucket_kernel(self, i: int) -> None:
        if self.max_grad_norm > 0:
            self.dp.reduce_bucket(i, **self.hyper)
        else:
            self.dp.step_bucket(i, **self.hyper)

    def _on_ready(self, group: str) -> None:
        if not self._armed or not self.overlap:
            return
        self._done.add(group)
        # buckets are launched in a fixed order on every rank (highest index first)
        for i in reversed(range(len(self._bucket_needs))):
            if i in self._launched:
                continue
            if self._bucket_needs[i] <= self._done:
                self._launch(i)
            else:
                break

    def finish_step(self) -> None:
        """Launch whatever is left and make the main stream wait for the new weights."""
        if not self._armed:
            self.dp.begin_step()
        for i in reversed(range(len(self.dp.buckets))):
            if i not in self._launched:
                self._launch(i)
        if self.max_grad_norm > 0:
            # every reduction is queued: now the clipped update + weight broadcast, bucket by bucket
            if self.stream is not None and self.overlap:
                with torch.cuda.stream(self.stream):
                    for i in reversed(range(len(self.dp.buckets))):
                        self.dp.update_bucket(i, **self.hyper)
            else:
                for i in reversed(range(len(self.dp.buckets))):
                    self.dp.update_bucket(i, **self.hyper)
        if self.stream is not None and self.overlap:
            torch.cuda.current_stream(self.heap.device).wait_stream(self.stream)
        self._armed = False
        self._launched.clear()
        self._done.clear()
        native.poll()


class NcclDataParallel:
    """Baseline: all-reduce the flat gradient with NCCL, then the (unfused-with-comm) optimizer."""

    def __init__(self, model, optimizer, group=None):
        self.model, self.optimizer, self.group = model, optimizer, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def finish_step(self) -> None:
        if self.world > 1:
            dist.all_reduce(self.model.flat_grad, group=self.group)
        self.optimizer.step(grad_scale=1.0 / self.world)
