"""``Tensor``: the 2-D, row-major, float32 tensor of the public API, device-resident.

The reference tensor lives on the host and every accelerated op uploads, dispatches and
reads back (crates/st-tensor/src/pure.rs:1404-1411, :2126-2137).  Here the storage is a
``torch.Tensor`` that stays on its device (``cpu`` or ``cuda``); CUDA ops run on the
sm_100a kernels (bf16 tensor-core inputs, fp32 accumulation) and CPU ops are plain fp32.

Method names, argument conventions and error behaviour follow the reference Python
binding (bindings/st-py/src/tensor.rs:280-1440): constructors ``Tensor(rows, cols[, data])``,
``Tensor((rows, cols), data=[...])``, ``Tensor(data=[[...], ...])``; ``shape()`` is a method;
``tolist()`` returns a list of rows; every op validates shapes and (optionally) finiteness.
"""
from __future__ import annotations

import math
import os
from typing import Any, Iterable, Optional, Sequence

import torch

from .ops import attention as _attn
from .ops import elementwise as _ew
from .ops import gemm as _gemm
from .ops import native as _native
from .ops import norm as _norm
from .ops import optim as _optim

_DEFAULT_DEVICE = [torch.device("cpu")]
_CHECK_FINITE = [os.environ.get("SPIRALTORCH_CHECK_FINITE", "0") == "1"]

MATMUL_BACKENDS = {"auto", "faer", "cpu-simd", "simd", "naive", "cpu", "wgpu", "hip", "cuda", "gpu"}


class TensorError(ValueError):
    """Shape, value or backend error raised by tensor operations."""


class NonFiniteValue(TensorError):
    def __init__(self, label: str, value: float):
        super().__init__(f"non-finite value in {label}: {value}")
        self.label, self.value = label, value


def set_default_device(device) -> None:
    """Device new tensors are created on (``"cpu"`` or ``"cuda"``)."""
    _DEFAULT_DEVICE[0] = torch.device(device)


def default_device() -> torch.device:
    return _DEFAULT_DEVICE[0]


def set_finite_checks(enabled: bool) -> None:
    """Validate op inputs/outputs for NaN/Inf (forces a device synchronisation per op)."""
    _CHECK_FINITE[0] = bool(enabled)


def _emit(op: str, in_shape, out_shape, **fields) -> None:
    from . import observability
    observability.emit_tensor_op(op, in_shape, out_shape, **fields)


class Tensor:
    __slots__ = ("_t",)

    # ---------------------------------------------------------------- construction
    def __init__(self, *args: Any, shape: Optional[Sequence[int]] = None, rows: Optional[int] = None,
                 cols: Optional[int] = None, data: Any = None, backend: Optional[str] = None, device=None):
        if len(args) > 3:
            raise TypeError("Tensor() takes at most 3 positional arguments")
        if len(args) >= 1 and isinstance(args[0], torch.Tensor):
            t = args[0]
            if t.dim() != 2:
                raise TensorError(f"Tensor wraps 2-D data only, got {tuple(t.shape)}")
            self._t = t.detach().to(torch.float32)
            return
        if len(args) >= 1 and isinstance(args[0], (tuple, list)) and len(args[0]) == 2 and \
                all(isinstance(v, int) for v in args[0]) and (len(args) == 1 or data is None):
            shape = tuple(args[0])
            if len(args) >= 2:
                data = args[1]
        elif len(args) >= 2 and isinstance(args[0], int):
            rows, cols = int(args[0]), int(args[1])
            if len(args) == 3:
                data = args[2]
        elif len(args) == 1 and data is None:
            data = args[0]
        if shape is not None:
            rows, cols = int(shape[0]), int(shape[1])
        dev = torch.device(device) if device is not None else default_device()
        if data is None:
            if rows is None or cols is None:
                raise TypeError("Tensor() needs a shape or data")
            self._t = torch.zeros(rows, cols, dtype=torch.float32, device=dev)
            return
        if isinstance(data, Tensor):
            data = data._t
        flat = torch.as_tensor(data, dtype=torch.float32)
        if rows is None or cols is None:
            if flat.dim() != 2:
                raise TensorError("nested row data (list of rows) is required when no shape is given")
            rows, cols = flat.shape
        if flat.numel() != rows * cols:
            raise TensorError(f"data length {flat.numel()} does not match shape ({rows}, {cols})")
        self._t = flat.reshape(rows, cols).contiguous().to(dev)

    @classmethod
    def _wrap(cls, t: torch.Tensor) -> "Tensor":
        out = cls.__new__(cls)
        out._t = t if t.dtype == torch.float32 else t.float()
        return out

    @staticmethod
    def zeros(rows: int, cols: int, device=None) -> "Tensor":
        return Tensor._wrap(torch.zeros(rows, cols, device=device or default_device()))

    @staticmethod
    def _generator(seed: Optional[int], label: str) -> torch.Generator:
        from .config import determinism
        g = torch.Generator(device="cpu")
        g.manual_seed(determinism.resolve_seed(seed, label))
        return g

    @staticmethod
    def randn(rows: int, cols: int, mean: float = 0.0, std: float = 1.0, seed: Optional[int] = None,
              device=None) -> "Tensor":
        g = Tensor._generator(seed, f"randn/{rows}x{cols}")
        t = torch.randn(rows, cols, generator=g) * std + mean
        return Tensor._wrap(t.to(device or default_device()))

    @staticmethod
    def rand(rows: int, cols: int, min: float = 0.0, max: float = 1.0, seed: Optional[int] = None,
             device=None) -> "Tensor":
        if not max > min:
            raise TensorError("rand() needs max > min")
        g = Tensor._generator(seed, f"rand/{rows}x{cols}")
        t = torch.rand(rows, cols, generator=g) * (max - min) + min
        return Tensor._wrap(t.to(device or default_device()))

    # ---------------------------------------------------------------- basics
    @property
    def rows(self) -> int:
        return self._t.shape[0]

    @property
    def cols(self) -> int:
        return self._t.shape[1]

    @property
    def device(self) -> torch.device:
        return self._t.device

    def shape(self) -> tuple[int, int]:
        return (self._t.shape[0], self._t.shape[1])

    def _host(self) -> torch.Tensor:
        """Host copy of the data.  The copy synchronises with the device, so this is also where a kernel
        that gave up (bounded wait, refused access) is reported instead of handing back unwritten memory."""
        if not self._t.is_cuda:
            return self._t.detach()
        out = self._t.detach().cpu()
        _native.poll()
        return out

    def tolist(self) -> list[list[float]]:
        return self._host().tolist()

    def data(self) -> list[float]:
        return self._host().reshape(-1).tolist()

    def torch(self) -> torch.Tensor:
        """The underlying ``torch.Tensor`` (shares storage)."""
        return self._t

    def to(self, device) -> "Tensor":
        out = Tensor._wrap(self._t.to(device))
        if self._t.is_cuda and not out._t.is_cuda:
            _native.poll()
        return out

    def cuda(self) -> "Tensor":
        return self.to("cuda")

    def cpu(self) -> "Tensor":
        return self.to("cpu")

    def clone(self) -> "Tensor":
        return Tensor._wrap(self._t.clone())

    def __repr__(self) -> str:
        return f"Tensor(rows={self.rows}, cols={self.cols}, device='{self._t.device}')"

    def __len__(self) -> int:
        return self.rows

    def _check(self, label: str, *tensors: torch.Tensor) -> None:
        if _CHECK_FINITE[0]:
            for t in tensors:
                if not torch.isfinite(t).all():
                    bad = t[~torch.isfinite(t)][0].item()
                    raise NonFiniteValue(label, bad)

    def _same_shape(self, other: "Tensor", op: str) -> None:
        if self.shape() != other.shape():
            raise TensorError(f"{op}: shape mismatch {self.shape()} vs {other.shape()}")

    # ---------------------------------------------------------------- matmul family
    def _mm(self, other: "Tensor", backend: Optional[str], *, bias=None, act=None, residual=None,
            label="matmul") -> torch.Tensor:
        if backend is not None and backend not in MATMUL_BACKENDS:
            raise TensorError(f"unknown matmul backend '{backend}'")
        if self.cols != other.rows:
            raise TensorError(f"{label}: inner dimensions differ {self.shape()} x {other.shape()}")
        self._check(label + "_input", self._t, other._t)
        use_cuda = self._t.is_cuda and backend not in ("cpu", "naive", "faer", "simd", "cpu-simd")
        if use_cuda:
            a = self._t.to(torch.bfloat16)
            b = _gemm.cached_bf16(other._t)      # weights are rounded once, not on every call
            out = _gemm.gemm(a, b, b_mn=True, out_dtype=torch.float32 if (act is None and bias is None and residual is None) else torch.bfloat16,
                             bias=None if bias is None else bias.to(torch.bfloat16).reshape(-1),
                             act=act, residual=None if residual is None else residual.to(torch.bfloat16))
            out = out.float()
        else:
            a, b = self._t.cpu() if backend in ("cpu", "naive", "faer", "simd", "cpu-simd") else self._t, \
                other._t.cpu() if backend in ("cpu", "naive", "faer", "simd", "cpu-simd") else other._t
            out = a @ b
            if bias is not None:
                out = out + bias.to(out.device).reshape(1, -1)
            if act == "relu":
                out = torch.relu(out)
            elif act == "gelu":
                out = torch.nn.functional.gelu(out, approximate="tanh")
            if residual is not None:
                out = out + residual.to(out.device)
            out = out.to(self._t.device)
        self._check(label + "_output", out)
        from . import observability as _obs
        _obs.record_receipt(_obs.TensorExecutionReceipt(
            label, backend or "auto", "cuda" if self._t.is_cuda and backend not in ("cpu", "naive", "faer", "simd", "cpu-simd") else "cpu",
            "cuda" if use_cuda else "cpu", None,
            {"kind": "dense_matmul", "rows": self.rows, "inner": self.cols, "cols": other.cols}))
        _emit(label, self.shape(), tuple(out.shape), backend="cuda" if use_cuda else "cpu")
        return out

    def matmul(self, other: "Tensor", *, backend: Optional[str] = None, out: Optional["Tensor"] = None) -> "Tensor":
        res = self._mm(other, backend)
        if out is not None:
            if out.shape() != tuple(res.shape):
                raise TensorError("matmul: out has the wrong shape")
            out._t.copy_(res)
            return out
        return Tensor._wrap(res)

    __matmul__ = lambda self, other: self.matmul(other)  # noqa: E731

    def matmul_bias_relu(self, other: "Tensor", bias: "Tensor", *, backend=None) -> "Tensor":
        return Tensor._wrap(self._mm(other, backend, bias=bias._t, act="relu", label="matmul_bias_relu"))

    def matmul_bias_gelu(self, other: "Tensor", bias: "Tensor", *, backend=None) -> "Tensor":
        return Tensor._wrap(self._mm(other, backend, bias=bias._t, act="gelu", label="matmul_bias_gelu"))

    def matmul_bias_add_relu(self, other: "Tensor", bias: "Tensor", residual: "Tensor", *, backend=None) -> "Tensor":
        # reference order: activation(acc + bias + residual)
        pre = self._mm(other, backend, bias=bias._t, label="matmul_bias_add_relu") + residual._t
        return Tensor._wrap(torch.relu(pre))

    def matmul_bias_add_gelu(self, other: "Tensor", bias: "Tensor", residual: "Tensor", *, backend=None) -> "Tensor":
        pre = self._mm(other, backend, bias=bias._t, label="matmul_bias_add_gelu") + residual._t
        return Tensor._wrap(torch.nn.functional.gelu(pre, approximate="tanh"))

    # ---------------------------------------------------------------- softmax / attention / norm
    def row_softmax(self, *, backend=None) -> "Tensor":
        self._check("row_softmax_input", self._t)
        return Tensor._wrap(_ew.row_softmax(self._t))

    def row_softmax_hardmax(self, *, backend=None) -> tuple["Tensor", "Tensor"]:
        y, h = _ew.row_softmax(self._t, hardmax=True)
        return Tensor._wrap(y), Tensor._wrap(h)

    def row_hardmax(self, *, backend=None) -> "Tensor":
        return self.row_softmax_hardmax()[1]

    def row_softmax_hardmax_spiral(self, *, backend=None) -> tuple["Tensor", "Tensor", "Tensor", dict]:
        """Softmax, arg-max mask, their spiral-consensus blend and the consensus metrics (one kernel on CUDA)."""
        self._check("row_softmax_input", self._t)
        soft, hard, spiral, metrics, _ = _ew.row_softmax_spiral(self._t)
        means = metrics.mean(dim=0).tolist() if metrics.shape[0] else [0.0, 0.0, 0.0, 0.0]
        report = {"phi": _ew.GOLDEN_RATIO, "phi_conjugate": _ew.GOLDEN_RATIO_CONJUGATE, "phi_bias": _ew.GOLDEN_RATIO_BIAS,
                  "ramanujan_ratio": _ew.RAMANUJAN_RATIO, "ramanujan_delta": _ew.RAMANUJAN_DELTA,
                  "average_enrichment": means[2], "mean_entropy": means[0], "mean_hardmass": means[1],
                  "spiral_coherence": means[3]}
        return Tensor._wrap(soft), Tensor._wrap(hard), Tensor._wrap(spiral), report

    def row_softmax_zspace_projection(self, *, backend=None) -> "Tensor":
        """Per-row Z-space summary of the softmax: columns (focus, above, here, swirl) over golden-ratio bands
        (crates/st-backend-wgpu/src/shaders/softmax_zspace_projection.wgsl)."""
        return Tensor._wrap(_ew.row_softmax_spiral(self._t)[4])

    def scaled_dot_attention(self, keys: "Tensor", values: "Tensor", *, contexts: int, sequence: int,
                             scale: Optional[float] = None, z_bias: Optional["Tensor"] = None,
                             attn_bias: Optional["Tensor"] = None, backend=None) -> "Tensor":
        """``self`` (queries), ``keys``, ``values``: ``(contexts*sequence, head_dim)``.  ``z_bias`` is
        ``(contexts, sequence)`` added per key; ``attn_bias`` is ``(contexts*sequence, sequence)`` added
        per (query, key).  No causal flag: causality is expressed through ``attn_bias``."""
        d = self.cols
        if self.rows != contexts * sequence or keys.shape() != self.shape() or values.rows != self.rows:
            raise TensorError("scaled_dot_attention: operands must be (contexts*sequence, head_dim)")
        scale = 1.0 / math.sqrt(d) if scale is None else scale
        q = self._t.view(contexts, sequence, d)
        k = keys._t.view(contexts, sequence, d)
        v = values._t.view(contexts, sequence, values.cols)
        fast = self._t.is_cuda and d in (64, 128) and values.cols == d
        if fast:
            # contexts map onto the batch axis of the kernel (one head); z_bias is its per-key bias and
            # attn_bias its per-(query, key) bias, both added to scale * q·k before the softmax
            o, _ = _attn.attention_forward(
                q.to(torch.bfloat16).unsqueeze(2), k.to(torch.bfloat16).unsqueeze(2),
                v.to(torch.bfloat16).unsqueeze(2), causal=False, scale=scale,
                key_bias=None if z_bias is None else z_bias._t.reshape(contexts, sequence),
                attn_bias=None if attn_bias is None else attn_bias._t.reshape(contexts, sequence, sequence))
            out = o.float().reshape(contexts * sequence, d)
            self._check("scaled_dot_attention_output", out)
            return Tensor._wrap(out)
        s = torch.matmul(q, k.transpose(1, 2)) * scale
        if z_bias is not None:
            s = s + z_bias._t.view(contexts, 1, sequence)
        if attn_bias is not None:
            s = s + attn_bias._t.view(contexts, sequence, sequence)
        p = torch.softmax(s, dim=-1)
        out = torch.matmul(p, v).reshape(contexts * sequence, values.cols)
        self._check("scaled_dot_attention_output", out)
        return Tensor._wrap(out)

    def layer_norm_affine(self, gamma: "Tensor", beta: "Tensor", *, epsilon: float = 1e-5, backend=None) -> "Tensor":
        if gamma.cols != self.cols or beta.cols != self.cols:
            raise TensorError("layer_norm_affine: gamma/beta must be (1, cols)")
        return Tensor._wrap(self._layer_norm(None, gamma, beta, epsilon))

    def _layer_norm(self, residual, gamma, beta, epsilon) -> torch.Tensor:
        x = self._t
        if x.is_cuda and self.cols % 8 == 0:
            # LayerNorm kernel (bf16 in / out, fp32 statistics); the residual add is fused into it
            y, _, _, _ = _norm.norm_forward(
                x.to(torch.bfloat16).contiguous(), _gemm.cached_bf16(gamma._t).reshape(-1),
                _gemm.cached_bf16(beta._t).reshape(-1), float(epsilon), False,
                None if residual is None else residual._t.to(torch.bfloat16).contiguous())
            return y.float()
        v = x if residual is None else x + residual._t
        return torch.nn.functional.layer_norm(v, (self.cols,), gamma._t.reshape(-1), beta._t.reshape(-1), epsilon)

    def layer_norm_affine_add(self, residual: "Tensor", gamma: "Tensor", beta: "Tensor", *,
                              epsilon: float = 1e-5, backend=None) -> "Tensor":
        self._same_shape(residual, "layer_norm_affine_add")
        if gamma.cols != self.cols or beta.cols != self.cols:
            raise TensorError("layer_norm_affine_add: gamma/beta must be (1, cols)")
        return Tensor._wrap(self._layer_norm(residual, gamma, beta, epsilon))

    def gelu(self) -> "Tensor":
        return Tensor._wrap(torch.nn.functional.gelu(self._t, approximate="tanh"))

    def relu(self) -> "Tensor":
        return Tensor._wrap(torch.relu(self._t))

    # ---------------------------------------------------------------- element-wise
    def add(self, other: "Tensor") -> "Tensor":
        self._same_shape(other, "add")
        return Tensor._wrap(self._t + other._t)

    def sub(self, other: "Tensor") -> "Tensor":
        self._same_shape(other, "sub")
        return Tensor._wrap(self._t - other._t)

    def scale(self, factor: float) -> "Tensor":
        return Tensor._wrap(self._t * float(factor))

    def hadamard(self, other: "Tensor") -> "Tensor":
        self._same_shape(other, "hadamard")
        return Tensor._wrap(self._t * other._t)

    def add_scaled_inplace(self, other: "Tensor", scale: float) -> None:
        self._same_shape(other, "add_scaled")
        self._t.add_(other._t, alpha=float(scale))

    def add_row_inplace(self, row: "Tensor | Sequence[float]") -> None:
        r = row._t.reshape(-1) if isinstance(row, Tensor) else torch.as_tensor(row, dtype=torch.float32)
        if r.numel() != self.cols:
            raise TensorError("add_row_inplace: row length must equal cols")
        self._t.add_(r.to(self._t.device).reshape(1, -1))

    def mul_row(self, row: "Tensor") -> "Tensor":
        return Tensor._wrap(self._t * row._t.reshape(1, -1))

    def transpose(self) -> "Tensor":
        return Tensor._wrap(self._t.t().contiguous())

    def reshape(self, rows: int, cols: int) -> "Tensor":
        if rows * cols != self._t.numel():
            raise TensorError(f"reshape: cannot view {self.shape()} as ({rows}, {cols})")
        return Tensor._wrap(self._t.reshape(rows, cols))

    def sum_axis0(self) -> list[float]:
        return self._t.sum(0).cpu().tolist()

    def sum_axis1(self) -> list[float]:
        return self._t.sum(1).cpu().tolist()

    def sum_axis0_tensor(self) -> "Tensor":
        return Tensor._wrap(self._t.sum(0, keepdim=True))

    def squared_l2_norm(self) -> float:
        return float(self._t.pow(2).sum())

    def max_axis0(self) -> "Tensor":
        return Tensor._wrap(self._t.max(0, keepdim=True).values)

    def cat_rows(self, other: "Tensor") -> "Tensor":
        if self.cols != other.cols:
            raise TensorError("cat_rows: column counts differ")
        return Tensor._wrap(torch.cat([self._t, other._t], 0))

    @staticmethod
    def cat_rows_many(tensors: Iterable["Tensor"]) -> "Tensor":
        return Tensor._wrap(torch.cat([t._t for t in tensors], 0))

    # ---------------------------------------------------------------- hyperbolic helpers
    def project_to_poincare(self, curvature: float) -> "Tensor":
        """Row-wise ``row * tanh(|row| / sqrt(-c)) / |row|`` (crates/st-tensor/src/pure.rs:7528-7621)."""
        if curvature >= 0:
            raise TensorError(f"non-hyperbolic curvature {curvature}")
        return Tensor._wrap(_optim.project_to_poincare(self._t, curvature))

    def hyperbolic_distance(self, other: "Tensor", curvature: float) -> float:
        """Poincaré-ball distance between the two tensors viewed as single points."""
        if curvature >= 0:
            raise TensorError(f"non-hyperbolic curvature {curvature}")
        self._same_shape(other, "hyperbolic_distance")
        scale = math.sqrt(-curvature)
        u, v = self._t.reshape(-1) / scale, other._t.reshape(-1) / scale
        du, dv = 1 - u.pow(2).sum(), 1 - v.pow(2).sum()
        diff = (u - v).pow(2).sum()
        arg = 1 + 2 * diff / (du * dv).clamp(min=1e-12)
        return float(scale * torch.acosh(arg.clamp(min=1.0)))

    # ---------------------------------------------------------------- DLPack
    def __dlpack__(self, stream=None):
        return self._t.__dlpack__(stream=stream) if stream is not None else self._t.__dlpack__()

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()

    def to_dlpack(self):
        return torch.utils.dlpack.to_dlpack(self._t)

    @staticmethod
    def from_dlpack(capsule) -> "Tensor":
        t = torch.utils.dlpack.from_dlpack(capsule)
        if t.dim() == 1:
            t = t.reshape(1, -1)
        if t.dim() != 2:
            raise TensorError("from_dlpack: only 1-D and 2-D tensors are supported")
        return Tensor._wrap(t.to(torch.float32))


def _instrument(names) -> None:
    """Every public op publishes a tensor-op event (input shape, output shape, device) when somebody listens."""
    import functools

    def wrap(name, fn):
        @functools.wraps(fn)
        def inner(self, *args, **kwargs):
            out = fn(self, *args, **kwargs)
            from . import observability
            if observability.has_observers() or _plugin_listening():
                first = out[0] if isinstance(out, tuple) else out
                shape = first.shape() if isinstance(first, Tensor) else ()
                _emit(name, self.shape(), shape, backend="cuda" if self._t.is_cuda else "cpu")
            return out
        return inner
    for n in names:
        setattr(Tensor, n, wrap(n, getattr(Tensor, n)))


def _plugin_listening() -> bool:
    from . import plugin
    return plugin.has_listeners("TensorOp")


_instrument(["row_softmax", "row_softmax_hardmax", "scaled_dot_attention", "layer_norm_affine", "layer_norm_affine_add",
             "gelu", "relu", "add", "sub", "scale", "hadamard", "mul_row", "transpose", "reshape", "sum_axis0_tensor",
             "max_axis0", "cat_rows", "project_to_poincare"])
