"""Z-space specific models: RBF-kernel attention over (band, sheet, echo) indices with uncertainty
propagation, an attention-free coherence sequencer, and the Z-space VAE with its own optimisers.

Restated from crates/st-nn/src/z_rba/attention.rs:51-640 (``ZIndex``, ``ZMetricWeights``,
``ArdParameters``, product RBF kernel added to the scaled dot-product logits, variance output
``Σ_j p_ij² |σ_j|``), crates/st-nn/src/zspace_coherence/sequencer.rs (coherence-weighted mixing
instead of attention) and crates/st-nn/src/zspace_coherence/vae.rs:296-1100 (linear encoder to
``(mu, logvar)``, reparameterised sample, linear decoder, reconstruction + KL, SGD / Adam /
RMSprop updates).  Everything is batched tensor math on the caller's device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..tensor import Tensor, TensorError
from .modules import _mm, _t


@dataclass(frozen=True)
class ZIndex:
    band: int
    sheet: int
    echo: int


@dataclass
class ZMetricWeights:
    w_band: float = 1.0
    w_sheet: float = 0.7
    w_echo: float = 0.5

    def normalised(self) -> "ZMetricWeights":
        s = self.w_band + self.w_sheet + self.w_echo
        if not math.isfinite(s) or s <= 1.1920929e-07:
            return ZMetricWeights()
        return ZMetricWeights(self.w_band / s, self.w_sheet / s, self.w_echo / s)

    def validate(self) -> None:
        for v in (self.w_band, self.w_sheet, self.w_echo):
            if not math.isfinite(v) or v < 0:
                raise TensorError("zrba_metric_weight must be finite and non-negative")


@dataclass
class ArdParameters:
    ell_band: float = 1.0
    ell_sheet: float = 1.0
    ell_echo: float = 1.0
    sigma2: float = 1.0

    def __post_init__(self):
        self.ell_band, self.ell_sheet, self.ell_echo = (max(v, 1e-2) for v in (self.ell_band, self.ell_sheet, self.ell_echo))


class ZFrame:
    """Geometry of the index grid: linear band / sheet distances, circular echo distance."""

    def __init__(self, echoes: int = 8, band_step: float = 1.0, sheet_step: float = 1.0):
        self.echoes, self.band_step, self.sheet_step = max(1, echoes), band_step, sheet_step

    def distances(self, idx: Sequence[ZIndex], device) -> tuple:
        b = torch.tensor([i.band for i in idx], dtype=torch.float32, device=device)
        s = torch.tensor([i.sheet for i in idx], dtype=torch.float32, device=device)
        e = torch.tensor([i.echo for i in idx], dtype=torch.float32, device=device)
        db = (b[:, None] - b[None, :]).abs() * self.band_step
        ds = (s[:, None] - s[None, :]).abs() * self.sheet_step
        de = (e[:, None] - e[None, :]).abs() % self.echoes
        return db, ds, torch.minimum(de, self.echoes - de)


@dataclass
class ZTensor:
    mu: Tensor
    sigma: Tensor
    indices: list

    def __post_init__(self):
        if self.mu.shape() != self.sigma.shape():
            raise TensorError(f"mu {self.mu.shape()} and sigma {self.sigma.shape()} must have the same shape")
        if len(self.indices) != self.mu.shape()[0]:
            raise TensorError("one ZIndex per row is required")


@dataclass
class AttentionTelemetry:
    entropy: list = field(default_factory=list)
    dominant_probability: list = field(default_factory=list)
    kernel_mass: list = field(default_factory=list)


@dataclass
class ZRBFAttentionOutput:
    mean: Tensor
    variance: Tensor
    telemetry: AttentionTelemetry


class ZRBFAttention:
    def __init__(self, d_model: int, n_heads: int, metric: Optional[ZMetricWeights] = None, ard: bool = False, device="cpu"):
        if d_model <= 0 or n_heads <= 0 or d_model % n_heads:
            raise TensorError(f"d_model {d_model} must be a positive multiple of n_heads {n_heads}")
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, d_model // n_heads
        self.metric = metric or ZMetricWeights()
        self.metric.validate()
        self.ard = ard
        seed = torch.arange(d_model * d_model, dtype=torch.float32).reshape(d_model, d_model)
        init = torch.tanh(torch.sin(seed) * 0.02 + 0.02 * torch.cos(seed)).to(device)
        self.query, self.key, self.value, self.output = (init.clone() for _ in range(4))
        self.head_params = [ArdParameters(1.0 * (1 + 0.1 * h), 0.8 * (1 + 0.1 * h), 0.6 * (1 + 0.1 * h), 1.0) if ard
                            else ArdParameters() for h in range(n_heads)]

    def forward(self, inp: ZTensor, frame: ZFrame) -> ZRBFAttentionOutput:
        mu, sigma = _t(inp.mu).float(), _t(inp.sigma).float()
        rows, cols = mu.shape
        if cols != self.d_model:
            raise TensorError(f"input has {cols} columns, expected {self.d_model}")
        if not bool(torch.isfinite(mu).all() and torch.isfinite(sigma).all()):
            raise TensorError("zrba_attention input is not finite")
        tel = AttentionTelemetry()
        if rows == 0:
            z = torch.zeros(0, self.d_model, device=mu.device)
            return ZRBFAttentionOutput(Tensor._wrap(z), Tensor._wrap(z.clone()), tel)
        with torch.no_grad():
            q, k, v = (_mm(mu, w.to(mu.device)) for w in (self.query, self.key, self.value))
            H, D = self.n_heads, self.head_dim
            qh, kh, vh = (t.reshape(rows, H, D).transpose(0, 1) for t in (q, k, v))          # [H, rows, D]
            logits = qh @ kh.transpose(1, 2) / math.sqrt(D)
            w = self.metric.normalised()
            db, ds, de = frame.distances(inp.indices, mu.device)
            kern = torch.stack([p.sigma2 * torch.exp(-0.5 * (db * max(w.w_band, 1e-6) / max(p.ell_band, 1e-3)) ** 2)
                                * torch.exp(-0.5 * (ds * max(w.w_sheet, 1e-6) / max(p.ell_sheet, 1e-3)) ** 2)
                                * torch.exp(-0.5 * (de * max(w.w_echo, 1e-6) / max(p.ell_echo, 1e-3)) ** 2)
                                for p in self.head_params])
            prob = torch.softmax(logits + kern, -1)
            heads = (prob @ vh).transpose(0, 1).reshape(rows, self.d_model)
            sig = sigma.abs().reshape(rows, H, D).transpose(0, 1)
            var = ((prob ** 2) @ sig).transpose(0, 1).reshape(rows, self.d_model)
            mean = _mm(heads, self.output.to(mu.device))
            ent = -(prob * torch.log(prob.clamp(min=1e-30))).sum(-1).mean(-1)
            tel.entropy = ent.tolist()
            tel.dominant_probability = prob.amax(dim=(1, 2)).tolist()
            tel.kernel_mass = kern.mean(dim=(1, 2)).tolist()
        if not bool(torch.isfinite(mean).all() and torch.isfinite(var).all()):
            raise TensorError("zrba_attention_output is not finite")
        return ZRBFAttentionOutput(Tensor._wrap(mean), Tensor._wrap(var), tel)


class MellinBasis:
    """Per-coordinate exponents: ``project(x) = sign(x) |x|^s / ||.||`` with ``|x|`` floored at 1e-9 and exponent 1
    for coordinates past the table (crates/st-nn/src/zspace_coherence/vae.rs:15-74)."""

    def __init__(self, exponents):
        self.exponents = torch.as_tensor(list(exponents), dtype=torch.float64)

    @classmethod
    def constant(cls, dimension: int, exponent: float) -> "MellinBasis":
        return cls([exponent] * dimension)

    @classmethod
    def ramp(cls, dimension: int, start: float, end: float) -> "MellinBasis":
        if dimension <= 1:
            return cls([start])
        return cls([start + (end - start) * i / (dimension - 1) for i in range(dimension)])

    def dimension(self) -> int:
        return int(self.exponents.numel())

    def project(self, x) -> torch.Tensor:
        t = _t(x).double()
        flat = t.reshape(-1, t.shape[-1])
        e = torch.ones(flat.shape[-1], dtype=torch.float64, device=t.device)
        n = min(self.dimension(), flat.shape[-1])
        e[:n] = self.exponents[:n].to(t.device)
        warped = torch.sign(flat) * flat.abs().clamp(min=1e-9) ** e
        warped = torch.where(flat == 0, flat.abs().clamp(min=1e-9) ** e, warped)          # +0 keeps the positive branch
        norm = warped.norm(dim=-1, keepdim=True)
        return (warped / torch.where(norm > 0, norm, torch.ones_like(norm))).reshape(t.shape).to(_t(x).dtype if _t(x).is_floating_point() else torch.float32)


@dataclass
class ZSpaceVaeStats:
    """Per-call losses: mean squared reconstruction error over the input dimensions, KL summed over the latent
    dimensions, ELBO = -(recon + kl); batch calls report the mean over rows."""
    recon_loss: float
    kl_loss: float
    evidence_lower_bound: float
    target: torch.Tensor


@dataclass
class ZSpaceVaeState:
    mu: torch.Tensor
    logvar: torch.Tensor
    latent: torch.Tensor
    reconstruction: torch.Tensor
    stats: ZSpaceVaeStats

    recon_loss = property(lambda self: self.stats.recon_loss)
    kl_loss = property(lambda self: self.stats.kl_loss)
    evidence_lower_bound = property(lambda self: self.stats.evidence_lower_bound)


@dataclass
class ZSpaceVaeBatchStats:
    batch_size: int
    recon_loss: float
    kl_loss: float
    evidence_lower_bound: float
    weighted_loss: float
    kl_weight: float
    learning_rate: float
    gradient_l2: float
    clipped_gradient_l2: float
    update_l2: float
    optimizer_step: int
    optimizer: str

    def __getitem__(self, key: str):
        return self.batch_size if key == "samples" else getattr(self, key)


class ZSpaceVae:
    """Linear-Gaussian VAE over Z-space coordinates with its own SGD / Adam / RMSprop state
    (crates/st-nn/src/zspace_coherence/vae.rs:296-1044).

    Training uses the latent mean (no sampling noise in the gradient) and closed-form gradients:
    ``d_rec = 2 (rec - x) / input_dim``, ``dW_dec = d_rec^T z``, ``d_mu = d_rec W_dec + beta mu``,
    ``d_logvar = beta (exp(logvar) - 1) / 2``, encoder gradients are the outer products with the input, all averaged
    over the batch — five GEMMs per step on the parameters' device instead of a per-sample loop.  The summed gradient
    is clipped to ``grad_clip`` (L2 over all six tensors) before the optimizer step."""

    OPTIMIZERS = ("sgd", "adam", "rmsprop")

    def __init__(self, input_dim: int, latent_dim: int, seed: int = 0, device="cpu"):
        if input_dim <= 0 or latent_dim <= 0:
            raise TensorError(f"invalid dimensions ({input_dim}, {latent_dim})")
        g = torch.Generator().manual_seed(seed)
        s = 1.0 / math.sqrt(input_dim)
        mk = lambda r, c, sc: (torch.randn(r, c, generator=g) * sc).to(device)  # noqa: E731
        self.p = {"enc_mu": mk(input_dim, latent_dim, s), "enc_logvar": mk(input_dim, latent_dim, s * 0.1),
                  "dec": mk(latent_dim, input_dim, 1.0 / math.sqrt(latent_dim)),
                  "b_mu": torch.zeros(latent_dim, device=device), "b_logvar": torch.zeros(latent_dim, device=device),
                  "b_dec": torch.zeros(input_dim, device=device)}
        self.input_dim, self.latent_dim = input_dim, latent_dim
        self._gen = torch.Generator().manual_seed(seed + 1)
        self._kind, self._step = "sgd", 0
        self._m = {k: torch.zeros_like(v) for k, v in self.p.items()}
        self._v = {k: torch.zeros_like(v) for k, v in self.p.items()}
        self._hyper = {"beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "decay": 0.99, "grad_clip": None}

    def optimizer_kind(self) -> str:
        return self._kind

    def optimizer_step(self) -> int:
        return self._step

    def configure_optimizer_by_name(self, name: str, **hyper) -> None:
        """``beta1`` / ``beta2`` in [0, 1), ``eps`` > 0, ``decay`` in [0, 1), ``grad_clip`` positive or ``None``."""
        name = name.lower()
        if name not in self.OPTIMIZERS:
            raise TensorError(f"unknown optimiser '{name}'")
        aliases = {"epsilon": "eps", "rms_decay": "decay"}
        hyper = {aliases.get(k, k): v for k, v in hyper.items()}
        for k, v in hyper.items():
            if k not in self._hyper:
                raise TensorError(f"unknown optimiser setting '{k}'")
            if k == "grad_clip":
                if v is not None and not (math.isfinite(v) and v > 0):
                    raise TensorError("invalid value: zspace_vae_grad_clip")
            elif not math.isfinite(v) or (k == "eps" and v <= 0) or (k != "eps" and not 0.0 <= v < 1.0):
                raise TensorError(f"invalid value: zspace_vae_{k}")
        self._kind = name
        self._hyper.update(hyper)
        self.reset_optimizer()

    configure_optimizer = configure_optimizer_by_name

    def reset_optimizer(self) -> None:
        self._step = 0
        for d in (self._m, self._v):
            for t in d.values():
                t.zero_()

    def _rows(self, x, label: str = "zspace_vae_input") -> torch.Tensor:
        x = _t(x).float().reshape(-1, self.input_dim).to(self.p["dec"].device)
        if x.shape[0] == 0:
            raise TensorError(f"empty input: {label}")
        if not bool(torch.isfinite(x).all()):
            raise TensorError(f"non-finite value for {label}")
        return x

    def encode(self, x: torch.Tensor):
        return x @ self.p["enc_mu"] + self.p["b_mu"], x @ self.p["enc_logvar"] + self.p["b_logvar"]

    def encode_with_mellin(self, x, basis: MellinBasis):
        return self.encode(basis.project(x).float())

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return z @ self.p["dec"] + self.p["b_dec"]

    def decode_with_mellin(self, z, basis: MellinBasis) -> torch.Tensor:
        return basis.project(self.decode(z)).float()

    def _state(self, x, mu, logvar, z) -> ZSpaceVaeState:
        rec = self.decode(z)
        recon = ((rec - x) ** 2).mean(-1)
        kl = -0.5 * (1 + logvar - mu ** 2 - logvar.exp()).sum(-1)
        r, k = float(recon.mean()), float(kl.mean())
        return ZSpaceVaeState(mu, logvar, z, rec, ZSpaceVaeStats(r, k, -(r + k), x))

    def forward(self, x, sample: bool = True) -> ZSpaceVaeState:
        x = self._rows(x)
        mu, logvar = self.encode(x)
        z = mu
        if sample:
            z = mu + torch.exp(0.5 * logvar) * torch.randn(x.shape[0], self.latent_dim, generator=self._gen).to(x.device)
        return self._state(x, mu, logvar, z)

    def forward_mean(self, x) -> ZSpaceVaeState:
        return self.forward(x, sample=False)

    @staticmethod
    def _hyperparams(learning_rate: float, kl_weight: float):
        if not math.isfinite(learning_rate):
            raise TensorError("non-finite value for zspace_vae_learning_rate")
        if learning_rate <= 0:
            raise TensorError(f"non-positive learning rate {learning_rate}")
        if not math.isfinite(kl_weight):
            raise TensorError("non-finite value for zspace_vae_kl_weight")
        if kl_weight < 0:
            raise TensorError("invalid value: zspace_vae_kl_weight")
        return float(learning_rate), float(kl_weight)

    def _gradients(self, x, beta: float):
        mu, logvar = self.encode(x)
        st = self._state(x, mu, logvar, mu)
        n = x.shape[0]
        d_rec = (st.reconstruction - x) * (2.0 / self.input_dim)
        d_mu = d_rec @ self.p["dec"].T
        d_lv = torch.zeros_like(logvar)
        if beta > 0:
            d_mu = d_mu + beta * mu
            d_lv = beta * 0.5 * (logvar.exp() - 1.0)
        g = {"enc_mu": x.T @ d_mu / n, "enc_logvar": x.T @ d_lv / n, "dec": mu.T @ d_rec / n,
             "b_mu": d_mu.mean(0), "b_logvar": d_lv.mean(0), "b_dec": d_rec.mean(0)}
        return st, g

    def _apply(self, grads: dict, lr: float) -> float:
        self._step += 1
        h, sq = self._hyper, 0.0
        for k, w in self.p.items():
            g = grads[k]
            if self._kind == "sgd":
                upd = lr * g
            elif self._kind == "adam":
                self._m[k].mul_(h["beta1"]).add_(g, alpha=1 - h["beta1"])
                self._v[k].mul_(h["beta2"]).addcmul_(g, g, value=1 - h["beta2"])
                upd = lr * (self._m[k] / (1 - h["beta1"] ** self._step)) / \
                    ((self._v[k] / (1 - h["beta2"] ** self._step)).sqrt() + h["eps"])
            else:
                self._v[k].mul_(h["decay"]).addcmul_(g, g, value=1 - h["decay"])
                upd = lr * g / (self._v[k].sqrt() + h["eps"])
            w.sub_(upd)
            sq += float(upd.pow(2).sum())
        return math.sqrt(sq)

    def _clip(self, grads: dict):
        norm = math.sqrt(sum(float(g.pow(2).sum()) for g in grads.values()))
        limit = self._hyper["grad_clip"]
        if limit is not None and norm > limit and norm > 0:
            for g in grads.values():
                g.mul_(limit / norm)
            return norm, limit
        return norm, norm

    def train_batch(self, x, learning_rate: float = 1e-2, beta: float = 1.0) -> ZSpaceVaeBatchStats:
        x = self._rows(x, "zspace_vae_train_batch")
        lr, beta = self._hyperparams(learning_rate, beta)
        st, grads = self._gradients(x, beta)
        norm, clipped = self._clip(grads)
        upd = self._apply(grads, lr)
        s = st.stats
        return ZSpaceVaeBatchStats(x.shape[0], s.recon_loss, s.kl_loss, s.evidence_lower_bound, s.recon_loss + beta * s.kl_loss, beta, lr,
                                   norm, clipped, upd, self._step, self._kind)

    def train_step(self, x, learning_rate: float = 1e-2, beta: float = 1.0) -> ZSpaceVaeState:
        """One update from a single input (or a batch treated as one averaged sample); returns the pre-update state."""
        x = self._rows(x)
        lr, beta = self._hyperparams(learning_rate, beta)
        st, grads = self._gradients(x, beta)
        self._clip(grads)
        self._apply(grads, lr)
        return st

    def evaluate_batch(self, x, beta: float = 1.0) -> ZSpaceVaeBatchStats:
        x = self._rows(x, "zspace_vae_evaluate_batch")
        _, beta = self._hyperparams(1.0, beta)
        s = self.forward_mean(x).stats
        return ZSpaceVaeBatchStats(x.shape[0], s.recon_loss, s.kl_loss, s.evidence_lower_bound, s.recon_loss + beta * s.kl_loss, beta, 0.0,
                                   0.0, 0.0, 0.0, self._step, self._kind)

    def refine_decoder(self, state: ZSpaceVaeState, learning_rate: float) -> None:
        """One plain gradient step of the decoder alone towards the state's target, rate clamped to [1e-6, 0.1]."""
        lr = min(max(learning_rate, 1e-6), 1e-1)
        err = state.reconstruction - state.stats.target
        self.p["dec"].sub_(lr * (state.latent.T @ err) / err.shape[0])
        self.p["b_dec"].sub_(lr * err.mean(0))

    def state_dict(self) -> dict:
        return {k: v.detach().cpu().clone() for k, v in self.p.items()}

    def load_state_dict(self, state: dict) -> None:
        for k, v in state.items():
            if k not in self.p or self.p[k].shape != v.shape:
                raise TensorError(f"unexpected VAE parameter '{k}' with shape {tuple(v.shape)}")
            self.p[k].copy_(v)

    def save(self, path) -> None:
        import json
        from ..config import atomic_write
        atomic_write(path, json.dumps({"version": 1, "input_dim": self.input_dim, "latent_dim": self.latent_dim, "optimizer": self._kind,
                                       "optimizer_step": self._step, "hyper": self._hyper,
                                       "parameters": {k: {"shape": list(v.shape), "data": v.flatten().tolist()}
                                                      for k, v in self.state_dict().items()}}))

    @classmethod
    def load(cls, path) -> "ZSpaceVae":
        import json
        blob = json.load(open(path))
        if blob.get("version", 1) != 1:
            raise TensorError(f"unsupported VAE checkpoint version {blob.get('version')}")
        vae = cls(blob["input_dim"], blob["latent_dim"])
        vae.load_state_dict({k: torch.tensor(v["data"]).reshape(v["shape"]) for k, v in blob["parameters"].items()})
        vae._kind = blob.get("optimizer", "sgd")
        vae._step = int(blob.get("optimizer_step", 0))
        vae._hyper.update(blob.get("hyper", {}))
        return vae


class LanguageWaveEncoder:
    """Text → complex spectrum → Poincaré-ball coordinates (crates/st-tensor/src/pure.rs:8296-8360).

    Each character contributes ``(ord mod 1024)/1024 + |sin((i+1)/n)|`` scaled by the temperature;
    the DFT of that signal gives ``n`` complex values, each mapped to the disc with radius
    ``tanh(|z|·sqrt(-c))`` and interleaved as ``(x, y)`` pairs; the row is then projected to the ball."""

    def __init__(self, curvature: float = -1.0, temperature: float = 1.0):
        if not (math.isfinite(curvature) and curvature < 0):
            raise TensorError(f"curvature must be negative, got {curvature}")
        if not (math.isfinite(temperature) and temperature > 0):
            raise TensorError(f"temperature must be positive, got {temperature}")
        self.curvature, self.temperature = curvature, temperature

    def encode_wave(self, text: str) -> torch.Tensor:
        n = len(text)
        if n == 0:
            raise TensorError("text is empty")
        idx = torch.arange(1, n + 1, dtype=torch.float32)
        bucket = torch.tensor([(ord(ch) % 1024) / 1024.0 for ch in text], dtype=torch.float32)
        signal = (bucket + torch.sin(idx / n).abs()) * self.temperature
        return torch.fft.fft(signal.to(torch.complex64))

    def encode_z_space(self, text: str) -> torch.Tensor:
        wave = self.encode_wave(text)
        radius = torch.tanh(wave.abs() * math.sqrt(-self.curvature))
        angle = torch.angle(wave)
        coords = torch.stack([radius * torch.cos(angle), radius * torch.sin(angle)], dim=1).reshape(1, -1)
        from .modules import _project_rows
        return _project_rows(coords, self.curvature)


class ZSpaceTextVae:
    """Z-space VAE over fixed character windows: text is cut or space-padded to ``window_chars``,
    encoded by :class:`LanguageWaveEncoder` into ``2·window_chars`` features and fed to
    :class:`ZSpaceVae` (crates/st-nn/src/zspace_coherence/text_vae.rs:22-330)."""

    def __init__(self, window_chars: int, latent_dim: int, curvature: float = -1.0, temperature: float = 1.0,
                 seed: int = 0):
        if window_chars <= 0:
            raise TensorError("zspace_text_vae_window_chars must be positive")
        if latent_dim <= 0:
            raise TensorError("zspace_text_vae_latent_dim must be positive")
        self.window_chars, self.input_dim = window_chars, 2 * window_chars
        self.encoder = LanguageWaveEncoder(curvature, temperature)
        self.vae = ZSpaceVae(self.input_dim, latent_dim, seed)

    latent_dim = property(lambda self: self.vae.latent_dim)
    curvature = property(lambda self: self.encoder.curvature)
    temperature = property(lambda self: self.encoder.temperature)

    def optimizer_kind(self) -> str:
        return self.vae.optimizer_kind()

    def configure_optimizer_by_name(self, name: str, **hyper) -> None:
        self.vae.configure_optimizer_by_name(name, **hyper)

    def reset_optimizer(self) -> None:
        self.vae.reset_optimizer()

    def _window(self, text: str) -> str:
        return text[: self.window_chars].ljust(self.window_chars)

    def encode_text(self, text: str) -> torch.Tensor:
        return self.encoder.encode_z_space(self._window(text)).reshape(-1)

    def encode_text_with_mellin(self, text: str, basis) -> torch.Tensor:
        """Warps the encoding by a :class:`MellinBasis`, or projects it onto an ``(input_dim, input_dim)`` matrix."""
        enc = self.encode_text(text)
        if isinstance(basis, MellinBasis):
            return basis.project(enc).float()
        if basis.shape != (self.input_dim, self.input_dim):
            raise TensorError(f"Mellin basis must be {self.input_dim}x{self.input_dim}, got {tuple(basis.shape)}")
        return basis.to(enc.dtype) @ enc

    def _batch(self, texts, basis=None) -> torch.Tensor:
        if not texts:
            raise TensorError("text batch is empty")
        enc = (lambda t: self.encode_text_with_mellin(t, basis)) if basis is not None else self.encode_text
        return torch.stack([enc(t) for t in texts])

    def forward_text(self, text: str, basis=None) -> ZSpaceVaeState:
        return self.vae.forward(self._batch([text], basis))

    def forward_mean_text(self, text: str, basis=None) -> ZSpaceVaeState:
        return self.vae.forward_mean(self._batch([text], basis))

    def train_text(self, text: str, learning_rate: float = 1e-2, beta: float = 1.0, basis=None) -> ZSpaceVaeState:
        return self.vae.train_step(self._batch([text], basis), learning_rate, beta)

    def train_text_batch(self, texts, learning_rate: float = 1e-2, beta: float = 1.0, basis=None) -> ZSpaceVaeBatchStats:
        return self.vae.train_batch(self._batch(list(texts), basis), learning_rate, beta)

    def evaluate_text_batch(self, texts, basis=None, beta: float = 1.0) -> ZSpaceVaeBatchStats:
        return self.vae.evaluate_batch(self._batch(list(texts), basis), beta)

    def save(self, path) -> None:
        import json
        from ..config import atomic_write
        atomic_write(path, json.dumps({"version": 1, "window_chars": self.window_chars, "curvature": self.curvature,
                                       "temperature": self.temperature, "latent_dim": self.latent_dim,
                                       "optimizer": self.vae.optimizer_kind(),
                                       "vae": {k: {"shape": list(v.shape), "data": v.flatten().tolist()}
                                               for k, v in self.vae.state_dict().items()}}))

    @classmethod
    def load(cls, path) -> "ZSpaceTextVae":
        import json
        blob = json.load(open(path))
        if blob.get("version") != 1:
            raise TensorError(f"unsupported text VAE checkpoint version {blob.get('version')}")
        m = cls(blob["window_chars"], blob["latent_dim"], blob["curvature"], blob["temperature"])
        m.vae.load_state_dict({k: torch.tensor(v["data"]).reshape(v["shape"]) for k, v in blob["vae"].items()})
        m.vae._kind = blob.get("optimizer", "sgd")
        return m
