"""User-facing training loop for the language models: host batches in, loss out.

``LMTrainer.train_step`` takes one global batch of token ids that lives in (pinned) host
memory, stages it to the device on a copy stream, runs every micro-batch through the
model's scheduled forward/backward, applies the fused optimizer step and returns the mean
loss as a Python float (one 4-byte device→host read).  This is the call the end-to-end
benchmark times.

Reference parity: plays the role of ``ModuleTrainer::train_epoch`` for the transformer
configurations (crates/st-nn/src/trainer.rs:7271); events use the same names
(``EpochStart``/``EpochEnd``/``TrainerStep``) on :mod:`spiraltorch_b200.plugin`.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from .models.gpt import GPTModel
from .ops import native
from .optim.flat import FlatAdamW


class LMTrainer:
    def __init__(self, model: GPTModel, optimizer: Optional[FlatAdamW] = None, micro_batch: int = 8,
                 publish_events: bool = False):
        self.model = model
        self.optimizer = optimizer or FlatAdamW(model)
        self.micro_batch = micro_batch
        self.device = model.flat_w.device
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._loss_acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory() if self.device.type == "cuda" \
            else torch.zeros(1)
        self.publish_events = publish_events
        self.steps = 0
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0

    def _stage(self, t: torch.Tensor) -> torch.Tensor:
        if self.copy_stream is None:
            return t.to(self.device)
        with torch.cuda.stream(self.copy_stream):
            out = t.to(self.device, non_blocking=True)
        return out

    def device_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step on device-resident ``[B, S]`` token ids; returns the mean loss as a
        device scalar (no host synchronisation)."""
        B = tokens.shape[0]
        mb = min(self.micro_batch, B)
        assert B % mb == 0, "global batch must be a multiple of the micro-batch"
        n_micro = B // mb
        self._loss_acc.zero_()
        for i in range(n_micro):
            loss = self.model.forward_backward(tokens[i * mb:(i + 1) * mb], targets[i * mb:(i + 1) * mb],
                                               loss_scale=1.0 / n_micro)
            self._loss_acc += loss
        self.optimizer.step()
        self.steps += 1
        if self.device.type == "cuda":
            native.poll()     # a kernel that gave up a bounded wait left its outputs unwritten: stop here
        return self._loss_acc

    def train_step(self, tokens_host: torch.Tensor, targets_host: torch.Tensor) -> float:
        """Host → device copy of the batch, one optimizer step, device → host read of the loss."""
        t0 = time.perf_counter()
        tok = self._stage(tokens_host)
        tgt = self._stage(targets_host)
        if self.copy_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
        self.h2d_bytes_last = tokens_host.numel() * tokens_host.element_size() + \
            targets_host.numel() * targets_host.element_size()
        loss_dev = self.device_step(tok, tgt)
        if self.device.type == "cuda":
            self._loss_host.copy_(loss_dev, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            loss = float(self._loss_host[0])
            native.poll()
        else:
            loss = float(loss_dev[0])
        self.d2h_bytes_last = 4
        if self.publish_events:
            from . import plugin
            plugin.publish("TrainerStep", {"step": self.steps, "loss": loss,
                                           "step_time_ms": (time.perf_counter() - t0) * 1e3})
        return loss


class GraphedForwardBackward:
    """``model.forward_backward`` captured once in a CUDA graph and replayed per micro-batch.

    The small models (85 M char-LM, conv classifier) launch about a thousand kernels of a few microseconds per
    step, so the step time is the host's launch rate; a replay issues them from the device side instead.  Inputs
    live in static buffers (``tokens`` / ``targets`` are copied in before each replay), the loss comes back as a
    static device scalar, and gradients accumulate into the model's ``flat_grad`` exactly as in the eager call.

    Only single-rank tensor-parallel contexts can be captured: the fused collectives take their epoch and arrival
    targets by value, which a captured graph would freeze.  Gradient hooks (``grad_ready_hook``) run at capture
    time only, so bucket overlap of the data-parallel step is not available under a graph; the data-parallel step
    itself stays outside the graph.
    """

    def __init__(self, model, example_inputs: tuple, warmup: int = 2, **kwargs):
        if getattr(getattr(model, "tp", None), "world", 1) != 1:
            raise ValueError("CUDA-graph capture needs a single-rank tensor-parallel context")
        dev = model.flat_w.device
        if dev.type != "cuda":
            raise ValueError("CUDA-graph capture needs a CUDA model")
        self.model, self.kwargs = model, kwargs
        self.static_in = tuple(t.to(dev).clone() for t in example_inputs)
        hook, model.grad_ready_hook = getattr(model, "grad_ready_hook", None), None
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        grads = model.flat_grad.clone()
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):             # first calls allocate scratch, tables and opt into shared memory
                model.forward_backward(*self.static_in, **kwargs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        native.poll()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_loss = model.forward_backward(*self.static_in, **kwargs)
        model.flat_grad.copy_(grads)                    # the warm-up and capture passes must not count as gradients
        model.grad_ready_hook = hook
        self.replays = 0

    def __call__(self, *inputs) -> torch.Tensor:
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_loss
