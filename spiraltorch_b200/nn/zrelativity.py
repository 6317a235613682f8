"""`ZRelativityModule`: exposes the tensors of an assembled `ZRelativityModel` (block metric, gauge field, scalar moduli,
warp factor) as trainable parameters of an `st.nn` module, so that an optimiser can move the geometry.

Parity: crates/st-nn/src/layers/zrelativity.rs — `ZRelativityModule::from_model` (:148-179), `forward` (:289-294: the
input is ignored, the output is the ``1 x parameter_dimension`` concatenation block | gauge | moduli | warp), `backward`
(:296-355: the matching slices of ``grad_output`` accumulate into the learnable segments; the input gradient is zero).
The segments whose `learnable` flag is off stay in the vector as constants.
"""
from __future__ import annotations

import torch

from .. import observability
from ..relativity import ZRelativityModel
from ..tensor import Tensor, TensorError
from .modules import Module, _t


class ZRelativityModule(Module):
    def __init__(self, model: ZRelativityModel):
        super().__init__()
        bundle, flags = model.tensor_bundle(), model.learnable_flags()
        self.model = model
        self.block = self._register("block_metric", bundle.block_metric.clone())
        self.gauge = self._register("gauge_field", bundle.gauge_field.clone(), trainable=flags.mixed)
        self.scalar = self._register("scalar_moduli", bundle.scalar_moduli.clone(), trainable=flags.internal)
        self.warp = None if bundle.warp is None else self._register("warp_factor", bundle.warp.clone(), trainable=flags.warp)
        self._segments = [p for p in (self.block, self.gauge, self.scalar, self.warp) if p is not None]
        self.vector_length = sum(p.value.numel() for p in self._segments)

    from_model = classmethod(lambda cls, model: cls(model))

    def parameter_dimension(self) -> int:
        return self.vector_length

    def learnable_segments(self) -> int:
        return sum(1 for p in self._segments if p.trainable)

    def _meta(self, kind: str, values: torch.Tensor, prefix: str) -> dict:
        fin = torch.isfinite(values)
        v = values[fin].abs()
        flags = self.model.learnable_flags()
        return {"backend": "parameter_adapter", "kind": kind, "parameter_dimension": self.vector_length,
                "total_dim": self.model.geometry.total_dimension(), "internal_dim": self.model.geometry.internal.dimension(),
                "has_warp": self.warp is not None, "learnable_segments": self.learnable_segments(), "learnable_warp": flags.warp,
                "learnable_mixed": flags.mixed, "learnable_internal": flags.internal, "block_len": self.block.value.numel(),
                "gauge_len": self.gauge.value.numel(), "scalar_len": self.scalar.value.numel(),
                "warp_len": 0 if self.warp is None else self.warp.value.numel(), f"{prefix}_finite": int(fin.sum()),
                f"{prefix}_non_finite": int((~fin).sum()), f"{prefix}_abs_mean": float(v.mean()) if v.numel() else 0.0,
                f"{prefix}_abs_max": float(v.max()) if v.numel() else 0.0}

    def forward(self, x: Tensor = None) -> Tensor:
        out = torch.cat([p.value.reshape(-1) for p in self._segments]).reshape(1, -1)
        shape = tuple(_t(x).shape) if x is not None else (0, 0)
        observability.emit_tensor_op("zrelativity_module_forward", shape, tuple(out.shape))
        observability.emit_tensor_op_meta("zrelativity_module_forward", lambda: self._meta("zrelativity_module_forward", out, "value"))
        return Tensor._wrap(out)

    __call__ = forward

    def backward(self, x: Tensor, grad_output: Tensor) -> Tensor:
        g = _t(grad_output)
        if tuple(g.shape) != (1, self.vector_length):
            raise TensorError(f"backward: grad_output shape {tuple(g.shape)} != (1, {self.vector_length})")
        offset = 0
        for p in self._segments:
            n = p.value.numel()
            p.accumulate(g[0, offset:offset + n].to(p.value.device))
            offset += n
        xt = _t(x)
        observability.emit_tensor_op("zrelativity_module_backward", tuple(g.shape), tuple(xt.shape))
        observability.emit_tensor_op_meta("zrelativity_module_backward", lambda: self._meta("zrelativity_module_backward", g, "grad"))
        return Tensor._wrap(torch.zeros_like(xt))
