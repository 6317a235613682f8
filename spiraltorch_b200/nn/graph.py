"""A whole ``st.nn`` training step (forward, loss, backward, parameter step) captured once in a CUDA graph.

The small reference models (WaveRnn mixer, GNN regressor, MLPs) launch a few dozen kernels of a few microseconds per
step, so an eager step costs what the host needs to issue them.  A replay issues the same launches from the device:
the step time drops to the kernels' own duration.  The captured step is exactly the eager one — the same module
code runs once under capture — with two differences that capture forces:

* inputs live in static buffers that ``__call__`` copies into, and the loss comes back as a static device scalar
  (read it with ``float(...)`` only when a number is needed: that read is the step's only host synchronisation);
* finite-checks cannot stop a replay, so they OR into a device flag that ``check()`` reads and turns into the same
  ``TensorError`` the eager step would have raised.
"""
from __future__ import annotations

import torch

from ..ops import gemm as _gemm
from ..ops import native
from ..tensor import Tensor, TensorError
from . import modules as _modules


class GraphedTrainStep:
    def __init__(self, module, loss, x, y, learning_rate: float = 1e-2, warmup: int = 3):
        xt, yt = (x.torch() if isinstance(x, Tensor) else x), (y.torch() if isinstance(y, Tensor) else y)
        if xt.device.type != "cuda":
            raise ValueError("CUDA-graph capture needs CUDA inputs (move the module and the batch to the GPU first)")
        dev = xt.device
        self.module, self.loss, self.learning_rate = module, loss, float(learning_rate)
        self.static_x, self.static_y = Tensor._wrap(xt.detach().clone()), Tensor._wrap(yt.detach().clone())
        self.nonfinite = torch.zeros((), dtype=torch.bool, device=dev)
        self._params = [p for p in module.parameters()]
        saved = [(p.value.clone(), None if p.gradient is None else p.gradient.clone()) for p in self._params]
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):          # first calls build descriptor tables, scratch and shared-memory opt-ins
                self._step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        native.poll()
        for p, (v, _) in zip(self._params, saved):   # warm-up steps must not count as training
            p.value.copy_(v)
        _gemm.clear_bf16_cache()                     # every cast a replay depends on has to be part of the graph
        self.graph = torch.cuda.CUDAGraph()
        prev, _modules._capture_flag = _modules._capture_flag, self.nonfinite
        try:
            with torch.cuda.graph(self.graph):
                self.static_loss = self._step()
        finally:
            _modules._capture_flag = prev
        for p, (v, g) in zip(self._params, saved):   # capture executes nothing, but keep the accumulators as they were
            p.gradient = g
        _gemm.clear_bf16_cache()
        self.replays = 0

    def _step(self) -> torch.Tensor:
        pred = self.module.forward(self.static_x)
        value = self.loss.forward(pred, self.static_y)
        self.module.backward(self.static_x, self.loss.backward(pred, self.static_y))
        self.module.apply_step(self.learning_rate)
        return value.torch().reshape(())

    def __call__(self, x, y) -> torch.Tensor:
        """Runs one training step on ``(x, y)``; returns the loss as a device scalar (valid until the next call)."""
        self.static_x.torch().copy_(x.torch() if isinstance(x, Tensor) else x, non_blocking=True)
        self.static_y.torch().copy_(y.torch() if isinstance(y, Tensor) else y, non_blocking=True)
        self.graph.replay()
        # a replay writes the parameters without passing through the autograd version counters that the bf16
        # weight cache keys on: bump them so an eager forward after graphed training re-casts the weights
        torch.autograd.graph.increment_version([p.value for p in self._params])
        self.replays += 1
        return self.static_loss

    def check(self) -> None:
        """One host read: raises if any replay so far met a non-finite loss input or gradient, or a kernel gave up a wait."""
        native.poll()
        if bool(self.nonfinite):
            self.nonfinite.zero_()
            raise TensorError("non-finite loss input or gradient inside a graphed training step")
