"""Modules of the public ``nn`` API with the reference's explicit two-call training protocol.

Every module offers ``forward(x)``, ``backward(x, grad_output)`` (needs the input again: no
activation cache is kept, exactly like the reference — ``Sequential.backward`` recomputes the
forward), ``attach_hypergrad / attach_realgrad``, ``zero_accumulators``, ``apply_step(lr)``
and ``state_dict()`` (a name-sorted list of ``(name, Tensor)``) / ``load_state_dict``.

Each layer states its math once as a pure PyTorch function ``_fwd(x, params)``; ``backward``
differentiates that function with ``torch.autograd`` and applies the reference's gradient
convention: parameter gradients are divided by the batch size (rows of the input) before they
are accumulated (crates/st-nn/src/layers/linear.rs:109-170, conv.rs:567, embedding.rs:449,
normalization.rs:116).  On CUDA tensors the heavy math of ``Linear``, ``LayerNorm``, ``Embedding``, ``ZConv``
and 2x2 max ``Pool2d`` - forward, data gradient and parameter gradients - runs on the sm_100a kernels through
:mod:`spiraltorch_b200.nn.functional`, so neither call reaches a library GEMM or convolution.

Parameter naming and layouts follow the reference: ``Linear`` has ``{name}::weight`` of shape
``(in, out)`` and ``{name}::bias`` ``(1, out)``; convolutions keep ``(out_channels,
in_channels*kh*kw)``; norms use ``::gamma`` / ``::beta`` (crates/st-nn/src/layers/*.rs).
"""
from __future__ import annotations

import math
from typing import Callable, Iterable, Optional, Sequence

import torch
import torch.nn.functional as F

from ..optim.amegagrad import AmegaHypergrad, AmegaRealgrad
from ..tensor import Tensor, TensorError


from ..ops import recurrent as _rec  # noqa: E402
from . import functional as _fn  # noqa: E402


def _t(x) -> torch.Tensor:
    return x.torch() if isinstance(x, Tensor) else torch.as_tensor(x, dtype=torch.float32)


_capture_flag: Optional[torch.Tensor] = None      # device flag that collects finite-checks while a CUDA graph is captured


def assert_finite(tensors, describe) -> None:
    """Raises ``TensorError(describe(i))`` for the first non-finite tensor ``i``.  All tensors are reduced to one
    device flag first, so the check costs one host read however many tensors it covers; under CUDA-graph capture
    (no host read possible) the flag is OR-ed into the capturing step's error word instead, which its owner polls."""
    tensors = [t for t in tensors if t is not None]
    if not tensors:
        return
    oks = [torch.isfinite(t).all() for t in tensors]
    ok = oks[0] if len(oks) == 1 else torch.stack(oks).all()
    if ok.is_cuda and torch.cuda.is_current_stream_capturing():
        if _capture_flag is None:
            raise TensorError("finite-check reached under CUDA-graph capture without a capture flag")
        _capture_flag.logical_or_(~ok)
        return
    if not bool(ok):
        bad = next(i for i, o in enumerate(oks) if not bool(o))
        raise TensorError(describe(bad))


class Parameter:
    """Named 2-D parameter with Euclidean, hypergrad and realgrad accumulators
    (crates/st-nn/src/module.rs:44-52)."""

    def __init__(self, name: str, value: torch.Tensor, trainable: bool = True):
        self.name = name
        self.value = value.to(torch.float32).contiguous()
        self.gradient: Optional[torch.Tensor] = None
        self.hypergrad: Optional[AmegaHypergrad] = None
        self.realgrad: Optional[AmegaRealgrad] = None
        self.trainable = trainable

    def accumulate(self, grad: torch.Tensor) -> None:
        if not self.trainable:
            return
        grad = grad.reshape(self.value.shape)
        if self.hypergrad is not None:
            self.hypergrad.accumulate_wave(grad)
        if self.realgrad is not None:
            self.realgrad.accumulate(grad)
        if self.hypergrad is None and self.realgrad is None:
            self.gradient = grad.clone() if self.gradient is None else self.gradient + grad

    def accumulators(self) -> list[torch.Tensor]:
        out = []
        if self.hypergrad is not None:
            out.append(self.hypergrad.gradient)
        if self.realgrad is not None:
            out.append(self.realgrad.gradient)
        if self.gradient is not None:
            out.append(self.gradient)
        return out

    def scale_accumulators(self, factor: float) -> None:
        for a in self.accumulators():
            a.mul_(factor)

    def zero(self) -> None:
        self.gradient = None
        if self.hypergrad is not None:
            self.hypergrad.reset()
        if self.realgrad is not None:
            self.realgrad.reset()

    def apply_step(self, fallback_lr: float) -> None:
        if not self.trainable:
            return
        if self.hypergrad is not None or self.realgrad is not None:
            if self.hypergrad is not None:
                self.hypergrad.apply(self.value)
            if self.realgrad is not None:
                self.realgrad.apply(self.value)
        elif self.gradient is not None:
            self.value.sub_(fallback_lr * self.gradient)
            self.gradient = None


class _MovedModule:
    """What a Python handle turns into after ``Sequential.add`` took the layer."""

    def __getattr__(self, item):
        raise ValueError("this module was moved into a Sequential and can no longer be used directly")


class Module:
    def __init__(self):
        self._params: list[Parameter] = []
        self.training = True

    # ---- parameters ---------------------------------------------------------------------
    def _register(self, name: str, value: torch.Tensor, trainable: bool = True) -> Parameter:
        p = Parameter(name, value, trainable)
        self._params.append(p)
        return p

    def parameters(self) -> list[Parameter]:
        return list(self._params)

    def _param_map(self) -> dict[str, torch.Tensor]:
        return {p.name: p.value for p in self.parameters()}

    def to(self, device) -> "Module":
        for p in self.parameters():
            p.value = p.value.to(device)
            if p.hypergrad is not None:
                p.hypergrad.to(device)
            if p.realgrad is not None:
                p.realgrad.to(device)
            p.zero()
        return self

    # ---- math ---------------------------------------------------------------------------
    def _fwd(self, x: torch.Tensor, params: dict[str, torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, x: Tensor) -> Tensor:
        with torch.no_grad():
            return Tensor._wrap(self._fwd(_t(x), self._param_map()))

    __call__ = forward

    def backward(self, x: Tensor, grad_output: Tensor) -> Tensor:
        xt = _t(x).detach().requires_grad_(True)
        plist = [p for p in self.parameters() if p.trainable]
        # leaves alias the parameter storage (no copy): the values are only read here, and the bf16 copies
        # cached per storage stay valid from the forward to the backward call
        leaves = {p.name: p.value.detach().requires_grad_(True) for p in plist}
        pmap = dict(self._param_map())
        pmap.update(leaves)
        with torch.enable_grad():
            y = self._fwd(xt, pmap)
            g = _t(grad_output)
            if y.shape != g.shape:
                raise TensorError(f"backward: grad_output shape {tuple(g.shape)} != output shape {tuple(y.shape)}")
            grads = torch.autograd.grad(y, [xt] + [leaves[p.name] for p in plist], g, allow_unused=True)
        batch = max(1, xt.shape[0])
        live = [(p, gp) for p, gp in zip(plist, grads[1:]) if gp is not None]
        assert_finite([gp for _, gp in live], lambda i: f"non-finite gradient for parameter {live[i][0].name}")
        for p, gp in live:
            p.accumulate(gp / batch)
        gx = grads[0] if grads[0] is not None else torch.zeros_like(xt)
        return Tensor._wrap(gx.detach())

    # ---- optimizer plumbing ----------------------------------------------------------------
    def attach_hypergrad(self, curvature: float = -1.0, learning_rate: float = 1e-2, *, topos=None) -> None:
        for p in self.parameters():
            if p.trainable:
                p.hypergrad = AmegaHypergrad(curvature, learning_rate, *p.value.shape, topos=topos,
                                             device=p.value.device)

    def attach_realgrad(self, learning_rate: float = 1e-2) -> None:
        for p in self.parameters():
            if p.trainable:
                p.realgrad = AmegaRealgrad(learning_rate, *p.value.shape, device=p.value.device)

    def zero_accumulators(self) -> None:
        for p in self.parameters():
            p.zero()

    def apply_step(self, fallback_lr: float = 1e-2) -> None:
        for p in self.parameters():
            p.apply_step(fallback_lr)

    def train(self) -> None:
        self.training = True

    def eval(self) -> None:
        self.training = False

    def infuse_text(self, text: str) -> None:
        """Text infusion hook of the reference trainer; a no-op for plain layers."""

    # ---- state ----------------------------------------------------------------------------
    def state_dict(self) -> list[tuple[str, Tensor]]:
        return sorted(((p.name, Tensor._wrap(p.value.clone())) for p in self.parameters()), key=lambda kv: kv[0])

    def load_state_dict(self, state) -> None:
        entries = dict(state.items() if hasattr(state, "items") else state)
        for p in self.parameters():
            if p.name not in entries:
                raise KeyError(f"missing parameter '{p.name}' in state dict")
            v = _t(entries[p.name])
            if tuple(v.shape) != tuple(p.value.shape):
                raise TensorError(f"shape mismatch for '{p.name}': {tuple(v.shape)} vs {tuple(p.value.shape)}")
        for p in self.parameters():
            p.value.copy_(_t(entries[p.name]).to(p.value.device))

    def state_dict_compatibility(self, state) -> dict:
        entries = dict(state.items() if hasattr(state, "items") else state)
        own = {p.name: tuple(p.value.shape) for p in self.parameters()}
        missing = sorted(k for k in own if k not in entries)
        unexpected = sorted(k for k in entries if k not in own)
        mismatch = sorted(k for k in own if k in entries and tuple(_t(entries[k]).shape) != own[k])
        return {"compatible": not (missing or unexpected or mismatch), "missing": missing,
                "unexpected": unexpected, "shape_mismatch": mismatch}

    def load_state_dict_checked(self, state) -> dict:
        report = self.state_dict_compatibility(state)
        if report["compatible"]:
            self.load_state_dict(state)
        return report

    # ---- checkpoints with renamed / reshaped keys (bindings/st-py/src/nn.rs:5277-5653) ------
    @staticmethod
    def _transform_state(source: torch.Tensor, transform: str, target_shape) -> torch.Tensor:
        def overlap(t):
            out = torch.zeros(target_shape, dtype=t.dtype, device=t.device)
            r, c = min(t.shape[0], target_shape[0]), min(t.shape[1], target_shape[1])
            out[:r, :c] = t[:r, :c]
            return out
        if transform == "identity":
            return source
        if transform == "transpose":
            return source.t().contiguous()
        if transform in ("copy_overlap_zeros", "copy_overlap"):
            return overlap(source)
        if transform in ("transpose_copy_overlap_zeros", "transpose_copy_overlap"):
            return overlap(source.t())
        raise ValueError(f"unsupported state_dict transform '{transform}'")

    def _mapped_report(self, checkpoint, key_map):
        import hashlib
        if not isinstance(key_map, dict):
            raise TypeError("key_map must be a dict mapping source keys to target keys or rule dicts")
        ckpt = {k: _t(v) for k, v in dict(checkpoint.items() if hasattr(checkpoint, "items") else checkpoint).items()}
        expected = {p.name: p.value for p in self.parameters()}
        entries, adapted, seen, mapped_sources = [], {}, set(), set()
        matched = missing = shape_mismatched = unknown_targets = 0
        for source_name, rule in key_map.items():
            if isinstance(rule, str):
                target, transform = rule, "identity"
            elif isinstance(rule, dict):
                if "target" not in rule:
                    raise ValueError("key_map rule missing 'target'")
                target, transform = rule["target"], rule.get("transform", "identity")
            else:
                raise TypeError("key_map values must be target strings or dicts with target/transform fields")
            mapped_sources.add(source_name)
            src = ckpt.get(source_name)
            entry = {"name": target, "source_name": source_name, "transform": transform, "expected_shape": None,
                     "source_shape": tuple(src.shape) if src is not None else None,
                     "original_source_shape": tuple(src.shape) if src is not None else None}
            if target not in expected:
                unknown_targets += 1
                entries.append({**entry, "status": "unexpected_target"})
                continue
            seen.add(target)
            want = tuple(expected[target].shape)
            entry["expected_shape"] = want
            if src is None:
                missing += 1
                entries.append({**entry, "status": "missing_source"})
                continue
            out = self._transform_state(src, transform, want)
            entry["source_shape"] = tuple(out.shape)
            if tuple(out.shape) == want:
                matched += 1
                adapted[target] = out
                entries.append({**entry, "status": "matched"})
            else:
                shape_mismatched += 1
                entries.append({**entry, "status": "shape_mismatch"})
        for name, value in expected.items():
            if name not in seen:
                missing += 1
                entries.append({"name": name, "status": "missing_rule", "source_name": "", "transform": "identity",
                                "expected_shape": tuple(value.shape), "source_shape": None,
                                "original_source_shape": None})

        def state_hash(state):
            h = hashlib.sha256()
            for k in sorted(state):
                v = state[k].detach().to(torch.float32).cpu().contiguous()
                h.update(k.encode())
                h.update(str(tuple(v.shape)).encode())
                h.update(v.numpy().tobytes())
            return h.hexdigest()
        report = {"compatible": missing == 0 and shape_mismatched == 0 and matched > 0, "matched": matched,
                  "missing": missing, "shape_mismatched": shape_mismatched,
                  "extra": sum(1 for k in ckpt if k not in mapped_sources) + unknown_targets, "entries": entries,
                  "source_hash": state_hash(ckpt), "matched_subset_hash": state_hash(adapted)}
        return report, adapted

    def state_dict_compatibility_with_key_map(self, checkpoint, key_map) -> dict:
        """Report of how a foreign checkpoint maps onto this module under ``key_map``:
        ``{source: target}`` or ``{source: {"target": ..., "transform": identity | transpose |
        copy_overlap_zeros | transpose_copy_overlap_zeros}}``."""
        return self._mapped_report(checkpoint, key_map)[0]

    def load_state_dict_subset_mapped_checked(self, checkpoint, key_map) -> dict:
        """Loads every matched entry (and only those); parameters without a usable source keep their values."""
        report, adapted = self._mapped_report(checkpoint, key_map)
        for p in self.parameters():
            if p.name in adapted:
                p.value.copy_(adapted[p.name].to(p.value.device, torch.float32))
        return report


# ------------------------------------------------------------------------------------------------
def _linear_args(args, kwargs, what: str):
    """``Layer("name", a, b)`` or ``Layer(a, b, name="...")`` (bindings/st-py/src/nn.rs:185-260)."""
    name = kwargs.pop("name", None)
    args = list(args)
    if args and isinstance(args[0], str):
        name = args.pop(0)
    if len(args) != 2:
        raise TypeError(f"{what} expects (name, a, b) or (a, b, name=...)")
    if name is None:
        name = what.lower()
    return name, int(args[0]), int(args[1])


def _mm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x @ w with w stored (in, out); on CUDA the tcgen05 GEMM, forward and both gradients."""
    return _fn.linear(x, w, None)


class Identity(Module):
    def _fwd(self, x, params):
        return x * 1.0


class Linear(Module):
    def __init__(self, *args, **kwargs):
        super().__init__()
        self.name, self.input_dim, self.output_dim = _linear_args(args, kwargs, "Linear")
        n = self.input_dim * self.output_dim
        w = (torch.arange(1, n + 1, dtype=torch.float32) * 0.01).reshape(self.input_dim, self.output_dim)
        self.weight = self._register(f"{self.name}::weight", w)
        self.bias = self._register(f"{self.name}::bias", torch.zeros(1, self.output_dim))

    def init_normal(self, std: float = 0.02, seed: Optional[int] = None) -> "Linear":
        g = torch.Generator().manual_seed(0 if seed is None else seed)
        self.weight.value.copy_(torch.randn(self.weight.value.shape, generator=g) * std)
        return self

    def _fwd(self, x, params):
        if x.shape[1] != self.input_dim:
            raise TensorError(f"Linear {self.name}: expected {self.input_dim} input columns, got {x.shape[1]}")
        return _fn.linear(x, params[f"{self.name}::weight"], params[f"{self.name}::bias"])


class LoraLinear(Module):
    def __init__(self, input_dim: int, output_dim: int, rank: int, *, alpha: float = 1.0, name: str = "lora"):
        super().__init__()
        if not (alpha > 0 and math.isfinite(alpha)):
            raise ValueError("lora_alpha must be positive and finite")
        if rank < 1 or rank > min(input_dim, output_dim):
            raise ValueError("lora_rank must be in [1, min(input_dim, output_dim)]")
        self.name, self.rank, self.alpha = name, rank, float(alpha)
        self.scale = self.alpha / rank
        n = input_dim * output_dim
        w = (torch.arange(1, n + 1, dtype=torch.float32) * 0.01).reshape(input_dim, output_dim)
        self._register(f"{name}::weight", w, trainable=False)
        self._register(f"{name}::bias", torch.zeros(1, output_dim), trainable=False)
        a = (torch.arange(1, input_dim * rank + 1, dtype=torch.float32) * 0.01).reshape(input_dim, rank)
        self._register(f"{name}::lora_a", a)
        self._register(f"{name}::lora_b", torch.zeros(rank, output_dim))

    def _fwd(self, x, p):
        n = self.name
        base = _fn.linear(x, p[f"{n}::weight"], p[f"{n}::bias"])
        return base + self.scale * _mm(_mm(x, p[f"{n}::lora_a"]), p[f"{n}::lora_b"])

    def state_dict(self):
        return sorted(((p.name, Tensor._wrap(p.value.clone())) for p in self.parameters() if p.trainable),
                      key=lambda kv: kv[0])

    def base_state_dict(self):
        return sorted(((p.name, Tensor._wrap(p.value.clone())) for p in self.parameters() if not p.trainable),
                      key=lambda kv: kv[0])


class Embedding(Module):
    """Input: float token ids ``(batch, steps)``; output ``(batch, steps*dim)``."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        self.name, self.vocab, self.dim = _linear_args(args, kwargs, "Embedding")
        g = torch.Generator().manual_seed(17)
        self._register(f"{self.name}::weight", torch.randn(self.vocab, self.dim, generator=g) * 0.02)

    def _fwd(self, x, p):
        ids = x.detach().round().long().clamp(0, self.vocab - 1)
        return _fn.embedding(ids, p[f"{self.name}::weight"]).reshape(x.shape[0], -1)


class Relu(Module):
    def _fwd(self, x, p):
        return torch.relu(x)


class Gelu(Module):
    def _fwd(self, x, p):
        return F.gelu(x, approximate="tanh")


class Dropout(Module):
    def __init__(self, probability: float, *, seed: Optional[int] = None, training: bool = True):
        super().__init__()
        if not 0.0 <= probability < 1.0:
            raise ValueError("dropout probability must be in [0, 1)")
        self.probability, self.training = probability, training
        self._gen = torch.Generator().manual_seed(0 if seed is None else seed)
        self._mask: Optional[torch.Tensor] = None

    def _fwd(self, x, p):
        if not self.training or self.probability == 0.0:
            return x * 1.0
        if self._mask is None or self._mask.shape != x.shape or not torch.is_grad_enabled():
            keep = 1.0 - self.probability
            self._mask = (torch.rand(x.shape, generator=self._gen) < keep).to(x.dtype).to(x.device) / keep
        return x * self._mask


class Scaler(Module):
    def __init__(self, name: str, features: int):
        super().__init__()
        self.name = name
        self._register(f"{name}::gain", torch.ones(1, features))

    def _fwd(self, x, p):
        return x * p[f"{self.name}::gain"]


class ZSpaceMixer(Scaler):
    """Per-feature mixing gain (crates/st-nn/src/layers/zspace_mixer.rs:69)."""


class NonLiner(Module):
    """``gain * act(slope * x + bias)`` with per-feature parameters
    (crates/st-nn/src/layers/non_liner.rs:356)."""

    def __init__(self, name: str, features: int, *, activation: str = "tanh", slope: float = 1.0,
                 gain: float = 1.0, bias: float = 0.0, curvature: Optional[float] = None, **_ignored):
        super().__init__()
        self.name, self.activation, self.curvature = name, activation, curvature
        self._register(f"{name}::gain", torch.full((1, features), float(gain)))
        self._register(f"{name}::slope", torch.full((1, features), float(slope)))
        self._register(f"{name}::bias", torch.full((1, features), float(bias)))

    def _fwd(self, x, p):
        z = x * p[f"{self.name}::slope"] + p[f"{self.name}::bias"]
        act = {"tanh": torch.tanh, "sigmoid": torch.sigmoid, "softsign": F.softsign,
               "relu": torch.relu, "gelu": lambda v: F.gelu(v, approximate="tanh")}.get(self.activation, torch.tanh)
        return act(z) * p[f"{self.name}::gain"]


def _project_rows(x: torch.Tensor, curvature: float) -> torch.Tensor:
    norm = x.pow(2).sum(-1, keepdim=True).clamp(min=1e-24).sqrt()
    return x * torch.tanh(norm / math.sqrt(-curvature)) / norm


class LayerNorm(Module):
    def __init__(self, name: str, features: int, curvature: float = -1.0, epsilon: float = 1e-5):
        super().__init__()
        self.name, self.features, self.curvature, self.epsilon = name, features, curvature, epsilon
        self._register(f"{name}::gamma", torch.ones(1, features))
        self._register(f"{name}::beta", torch.zeros(1, features))

    def _fwd(self, x, p):
        return _fn.layer_norm(x, p[f"{self.name}::gamma"], p[f"{self.name}::beta"], self.epsilon)


class ZSpaceLayerNorm(LayerNorm):
    """Layer norm followed by a blend towards the Poincaré projection of the normalised row."""

    def __init__(self, name, features, curvature=-1.0, epsilon=1e-5, *, projector_gain: float = 1.0):
        super().__init__(name, features, curvature, epsilon)
        self.projector_gain = projector_gain

    def _fwd(self, x, p):
        y = super()._fwd(x, p)
        g = max(0.0, min(1.0, self.projector_gain))
        return (1 - g) * y + g * _project_rows(y, self.curvature) * math.sqrt(self.features)


class BatchNorm1d(Module):
    def __init__(self, name: str, features: int, momentum: float = 0.1, epsilon: float = 1e-5, *, training=True):
        super().__init__()
        self.name, self.features, self.momentum, self.epsilon, self.training = name, features, momentum, epsilon, training
        self._register(f"{name}::gamma", torch.ones(1, features))
        self._register(f"{name}::beta", torch.zeros(1, features))
        self.running_mean = torch.zeros(features)
        self.running_var = torch.ones(features)

    def _fwd(self, x, p):
        if self.training:
            mean, var = x.mean(0), x.var(0, unbiased=False)
            if not torch.is_grad_enabled():
                self.running_mean = (1 - self.momentum) * self.running_mean.to(x.device) + self.momentum * mean.detach()
                self.running_var = (1 - self.momentum) * self.running_var.to(x.device) + self.momentum * var.detach()
        else:
            mean, var = self.running_mean.to(x.device), self.running_var.to(x.device)
        return (x - mean) * torch.rsqrt(var + self.epsilon) * p[f"{self.name}::gamma"] + p[f"{self.name}::beta"]


class ZSpaceBatchNorm1d(BatchNorm1d):
    def __init__(self, name, features, curvature=-1.0, momentum=0.1, epsilon=1e-5, *, projector_gain=1.0,
                 training=True):
        super().__init__(name, features, momentum, epsilon, training=training)
        self.curvature, self.projector_gain = curvature, projector_gain

    def _fwd(self, x, p):
        y = super()._fwd(x, p)
        g = max(0.0, min(1.0, self.projector_gain))
        return (1 - g) * y + g * _project_rows(y, self.curvature) * math.sqrt(self.features)


class ZSpaceSoftmax(Module):
    """Row softmax with a curvature-scaled temperature (crates/st-nn/src/layers/softmax.rs:254)."""

    def __init__(self, curvature: float = -1.0, temperature: float = 1.0, **_ignored):
        super().__init__()
        if curvature >= 0 or temperature <= 0:
            raise ValueError("ZSpaceSoftmax needs curvature < 0 and temperature > 0")
        self.curvature, self.temperature = curvature, temperature

    def _fwd(self, x, p):
        return torch.softmax(x * math.sqrt(-self.curvature) / self.temperature, dim=-1)


class WaveGate(Module):
    """Sigmoid gate with temperature, output projected onto the Poincaré ball
    (crates/st-nn/src/layers/wave_gate.rs:227)."""

    def __init__(self, name: str, features: int, curvature: float = -1.0, temperature: float = 1.0):
        super().__init__()
        self.name, self.curvature, self.temperature = name, curvature, temperature
        self._register(f"{name}::gain", torch.ones(1, features))
        self._register(f"{name}::bias", torch.zeros(1, features))

    def _fwd(self, x, p):
        gate = torch.sigmoid((x * p[f"{self.name}::gain"] + p[f"{self.name}::bias"]) / self.temperature)
        return _project_rows(x * gate, self.curvature)


class _Recurrent(Module):
    def __init__(self, name: str, input_dim: int, hidden_dim: int, steps: int, gates: int):
        super().__init__()
        self.name, self.input_dim, self.hidden_dim, self.steps, self.gates = name, input_dim, hidden_dim, steps, gates
        g = torch.Generator().manual_seed(23)
        k = 1.0 / math.sqrt(hidden_dim)
        self._register(f"{name}::w_ih", (torch.rand(input_dim, gates * hidden_dim, generator=g) * 2 - 1) * k)
        self._register(f"{name}::w_hh", (torch.rand(hidden_dim, gates * hidden_dim, generator=g) * 2 - 1) * k)
        self._register(f"{name}::bias", torch.zeros(1, gates * hidden_dim))

    def _split(self, x):
        if x.shape[1] != self.steps * self.input_dim:
            raise TensorError(f"{self.name}: expected {self.steps}*{self.input_dim} input columns")
        return x.reshape(x.shape[0], self.steps, self.input_dim)


class SpiralRnn(_Recurrent):
    """Elman-style recurrence over ``steps`` slices of the input; returns the last hidden state
    (crates/st-nn/src/layers/spiral_rnn.rs:168)."""

    def __init__(self, name, input_dim, hidden_dim, steps):
        super().__init__(name, input_dim, hidden_dim, steps, 1)

    def _fwd(self, x, p):
        # one launch for the whole sequence on CUDA (csrc/recurrent/scan.cu); the step loop on CPU
        return _rec.rnn_sequence(self._split(x), p[f"{self.name}::w_ih"], p[f"{self.name}::w_hh"],
                                 p[f"{self.name}::bias"], "tanh")


class Lstm(_Recurrent):
    """LSTM over ``steps`` slices, returns the last hidden state (crates/st-nn/src/layers/lstm.rs:555)."""

    def __init__(self, name, input_dim, hidden_dim, steps):
        super().__init__(name, input_dim, hidden_dim, steps, 4)

    def _fwd(self, x, p):
        return _rec.rnn_sequence(self._split(x), p[f"{self.name}::w_ih"], p[f"{self.name}::w_hh"],
                                 p[f"{self.name}::bias"], "lstm")


class WaveRnn(_Recurrent):
    """Gated recurrence with a dilated skip (crates/st-nn/src/layers/wave_rnn.rs:62)."""

    def __init__(self, name, input_dim, hidden_dim, steps, *, dilation: int = 2, **_ignored):
        super().__init__(name, input_dim, hidden_dim, steps, 2)
        self.dilation = max(1, dilation)

    def _fwd(self, x, p):
        return _rec.rnn_sequence(self._split(x), p[f"{self.name}::w_ih"], p[f"{self.name}::w_hh"],
                                 p[f"{self.name}::bias"], "wave", self.dilation)


class ZSpaceCoherenceScan(Module):
    """Attention-free causal scan: every step mixes the previous ``memory`` steps with softmax
    weights of their coherence (dot product) at the given temperature
    (crates/st-nn/src/layers/coherence_scan.rs:163)."""

    def __init__(self, dim: int, steps: int, memory: int, curvature: float = -1.0, temperature: float = 1.0):
        super().__init__()
        self.dim, self.steps, self.memory, self.curvature, self.temperature = dim, steps, memory, curvature, temperature

    def _fwd(self, x, p):
        b = x.shape[0]
        xs = x.reshape(b, self.steps, self.dim)
        scores = torch.matmul(xs, xs.transpose(1, 2)) * (math.sqrt(-self.curvature) / self.temperature)
        idx = torch.arange(self.steps, device=x.device)
        mask = (idx[None, :] <= idx[:, None]) & (idx[None, :] > idx[:, None] - self.memory)
        scores = scores.masked_fill(~mask, float("-inf"))
        return torch.matmul(torch.softmax(scores, -1), xs).reshape(b, -1)


class ZSpaceCoherenceWaveBlock(ZSpaceCoherenceScan):
    """Coherence scan followed by dilated causal averaging (crates/st-nn/src/layers/coherence_wave.rs:91)."""

    def __init__(self, dim, steps, memory, curvature=-1.0, temperature=1.0, *, kernel_size: int = 3,
                 dilations: Optional[Sequence[int]] = None):
        super().__init__(dim, steps, memory, curvature, temperature)
        self.kernel_size, self.dilations = kernel_size, list(dilations or [1, 2])

    def _fwd(self, x, p):
        y = super()._fwd(x, p).reshape(x.shape[0], self.steps, self.dim)
        out = y
        for d in self.dilations:
            acc = y.clone()
            for k in range(1, self.kernel_size):
                shifted = F.pad(y, (0, 0, k * d, 0))[:, : self.steps]
                acc = acc + shifted
            out = out + acc / self.kernel_size
        return (out / (1 + len(self.dilations))).reshape(x.shape[0], -1)


_DIRECTIONS = {"to_canonical": True, "to": True, "from_canonical": False, "from": False}


def _reorder_rows(x: torch.Tensor, channels: int, spatial: tuple, layout: str, direction: str) -> torch.Tensor:
    """Rows of flattened feature maps between channel-last and the canonical channel-first order: one strided copy."""
    layout = layout.upper()
    first, last = ("NCHW", "NHWC") if len(spatial) == 2 else ("NCDHW", "NDHWC")
    if layout not in (first, last):
        raise ValueError(f"unsupported layout '{layout}', expected '{first}' or '{last}'")
    if direction.lower() not in _DIRECTIONS:
        raise ValueError(f"unknown direction '{direction}', expected 'to_canonical' or 'from_canonical'")
    size = channels * math.prod(spatial)
    if x.dim() != 2 or x.shape[1] != size:
        raise TensorError(f"feature tensor has {tuple(x.shape)} values per row, expected (*, {size})")
    if layout == first:
        return x * 1.0
    b, nd = x.shape[0], len(spatial)
    if _DIRECTIONS[direction.lower()]:                 # channel-last rows -> channel-first rows
        return x.reshape(b, *spatial, channels).permute(0, nd + 1, *range(1, nd + 1)).reshape(b, -1)
    return x.reshape(b, channels, *spatial).permute(0, *range(2, nd + 2), 1).reshape(b, -1)


def reorder_feature_tensor(tensor: Tensor, channels: int, height: int, width: int, layout: str = "NHWC",
                           direction: str = "to_canonical") -> Tensor:
    """``(batch, C*H*W)`` rows between ``NHWC`` and the canonical ``NCHW`` order (``NCHW`` is the identity);
    ``direction`` is ``to_canonical`` / ``to`` or ``from_canonical`` / ``from`` (bindings/st-py/src/nn.rs:900-931, 1250-1264)."""
    return Tensor._wrap(_reorder_rows(_t(tensor), channels, (height, width), layout, direction).contiguous())


def reorder_feature_tensor_3d(tensor: Tensor, channels: int, depth: int, height: int, width: int, layout: str = "NDHWC",
                              direction: str = "to_canonical") -> Tensor:
    """The same for volumes: ``NDHWC`` rows against the canonical ``NCDHW`` order (bindings/st-py/src/nn.rs:977-1010)."""
    return Tensor._wrap(_reorder_rows(_t(tensor), channels, (depth, height, width), layout, direction).contiguous())


class FeatureReorder2d(Module):
    def __init__(self, channels: int, height: int, width: int, *, layout: str = "NCHW", direction: str = "to_canonical"):
        super().__init__()
        self.c, self.h, self.w, self.layout, self.direction = channels, height, width, layout.upper(), direction
        _reorder_rows(torch.zeros(1, channels * height * width), channels, (height, width), layout, direction)   # validates the labels

    def _fwd(self, x, p):
        return _reorder_rows(x, self.c, (self.h, self.w), self.layout, self.direction)


def conv_output_shape(input_hw, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> tuple[int, int]:
    oh = (input_hw[0] + 2 * padding[0] - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1
    ow = (input_hw[1] + 2 * padding[1] - dilation[1] * (kernel[1] - 1) - 1) // stride[1] + 1
    return oh, ow


def pool_output_shape(input_hw, kernel, stride=None, padding=(0, 0)) -> tuple[int, int]:
    stride = stride or kernel
    return conv_output_shape(input_hw, kernel, stride, padding)


class ZConv(Module):
    """2-D convolution on NCHW-flattened rows ``(batch, C*H*W)``; weight ``(OC, IC*kh*kw)``
    (bindings/st-py/src/nn.rs:8127, crates/st-nn/src/layers/conv.rs:607)."""

    def __init__(self, name: str, in_channels: int, out_channels: int, input_hw, kernel, *, stride=None,
                 padding=(0, 0), dilation=(1, 1), layout: str = "NCHW"):
        super().__init__()
        self.name, self.ic, self.oc = name, in_channels, out_channels
        self.input_hw, self.kernel = tuple(input_hw), tuple(kernel)
        self.stride = tuple(stride) if stride else (1, 1)
        self.padding, self.dilation, self.layout = tuple(padding), tuple(dilation), layout.upper()
        n = out_channels * in_channels * self.kernel[0] * self.kernel[1]
        w = (torch.arange(1, n + 1, dtype=torch.float32) * (0.01 / max(1, n) ** 0.5)).reshape(out_channels, -1)
        self._register(f"{name}::weight", w)
        self._register(f"{name}::bias", torch.zeros(1, out_channels))

    def output_hw(self):
        return conv_output_shape(self.input_hw, self.kernel, self.stride, self.padding, self.dilation)

    def _fwd(self, x, p):
        b = x.shape[0]
        img = x.reshape(b, self.ic, *self.input_hw)
        y = _fn.conv2d(img, p[f"{self.name}::weight"], p[f"{self.name}::bias"], self.kernel, self.stride,
                       self.padding, self.dilation)
        return y.reshape(b, -1)


class Pool2d(Module):
    def __init__(self, mode: str, channels: int, height: int, width: int, kernel, *, stride=None, padding=None,
                 layout: str = "NCHW"):
        super().__init__()
        if mode not in ("max", "avg"):
            raise ValueError("Pool2d mode must be 'max' or 'avg'")
        self.mode, self.c, self.h, self.w = mode, channels, height, width
        self.kernel = tuple(kernel)
        self.stride = tuple(stride) if stride else self.kernel
        self.padding = tuple(padding) if padding else (0, 0)

    def _fwd(self, x, p):
        img = x.reshape(x.shape[0], self.c, self.h, self.w)
        if self.mode == "max" and self.kernel == (2, 2) and self.stride == (2, 2) and self.padding == (0, 0):
            return _fn.max_pool2x2(img).reshape(x.shape[0], -1)
        f = F.max_pool2d if self.mode == "max" else F.avg_pool2d
        return f(img, self.kernel, self.stride, self.padding).reshape(x.shape[0], -1)


ZPooling = Pool2d


class Sequential(Module):
    def __init__(self, layers: Optional[Iterable[Module]] = None):
        super().__init__()
        self.layers: list[Module] = []
        for l in layers or []:
            self.add(l)

    def add(self, layer: Module) -> None:
        """Takes ownership of ``layer``: the caller's handle becomes unusable
        (bindings/st-py/src/nn.rs:1369-1384)."""
        if isinstance(layer, _MovedModule):
            raise ValueError("module was already moved into a Sequential")
        owned = object.__new__(layer.__class__)
        owned.__dict__ = layer.__dict__
        layer.__dict__ = {}
        layer.__class__ = _MovedModule
        self.layers.append(owned)

    push = add

    def len(self) -> int:
        return len(self.layers)

    def __len__(self) -> int:
        return len(self.layers)

    def parameters(self) -> list[Parameter]:
        out = []
        for l in self.layers:
            out.extend(l.parameters())
        return out

    def _fwd(self, x, params):
        for l in self.layers:
            x = l._fwd(x, params)
        return x

    def train(self):
        self.training = True
        for l in self.layers:
            l.train()

    def eval(self):
        self.training = False
        for l in self.layers:
            l.eval()

    def infuse_text(self, text: str) -> None:
        for l in self.layers:
            l.infuse_text(text)
