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


@dataclass
class ZSpaceVaeState:
    mu: torch.Tensor
    logvar: torch.Tensor
    latent: torch.Tensor
    reconstruction: torch.Tensor
    recon_loss: float
    kl_loss: float


class ZSpaceVae:
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
        self._hyper = {"beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "decay": 0.99}

    def optimizer_kind(self) -> str:
        return self._kind

    def optimizer_step(self) -> int:
        return self._step

    def configure_optimizer_by_name(self, name: str, **hyper) -> None:
        name = name.lower()
        if name not in self.OPTIMIZERS:
            raise TensorError(f"unknown optimiser '{name}'")
        self._kind = name
        self._hyper.update(hyper)
        self.reset_optimizer()

    def reset_optimizer(self) -> None:
        self._step = 0
        for d in (self._m, self._v):
            for t in d.values():
                t.zero_()

    def encode(self, x: torch.Tensor):
        return x @ self.p["enc_mu"] + self.p["b_mu"], x @ self.p["enc_logvar"] + self.p["b_logvar"]

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return z @ self.p["dec"] + self.p["b_dec"]

    def _losses(self, x, p, eps):
        mu = x @ p["enc_mu"] + p["b_mu"]
        logvar = (x @ p["enc_logvar"] + p["b_logvar"]).clamp(-10.0, 10.0)
        z = mu + torch.exp(0.5 * logvar) * eps
        rec = z @ p["dec"] + p["b_dec"]
        recon = ((rec - x) ** 2).sum(-1).mean()
        kl = (-0.5 * (1 + logvar - mu ** 2 - logvar.exp()).sum(-1)).mean()
        return mu, logvar, z, rec, recon, kl

    def forward(self, x, sample: bool = True) -> ZSpaceVaeState:
        x = _t(x).float().reshape(-1, self.input_dim)
        eps = torch.randn(x.shape[0], self.latent_dim, generator=self._gen).to(x.device) if sample else \
            torch.zeros(x.shape[0], self.latent_dim, device=x.device)
        with torch.no_grad():
            mu, logvar, z, rec, recon, kl = self._losses(x, self.p, eps)
        return ZSpaceVaeState(mu, logvar, z, rec, float(recon), float(kl))

    def forward_mean(self, x) -> ZSpaceVaeState:
        return self.forward(x, sample=False)

    def train_batch(self, x, learning_rate: float = 1e-2, beta: float = 1.0) -> ZSpaceVaeState:
        x = _t(x).float().reshape(-1, self.input_dim)
        if not bool(torch.isfinite(x).all()):
            raise TensorError("non-finite VAE input")
        eps = torch.randn(x.shape[0], self.latent_dim, generator=self._gen).to(x.device)
        leaves = {k: v.detach().clone().requires_grad_(True) for k, v in self.p.items()}
        with torch.enable_grad():
            mu, logvar, z, rec, recon, kl = self._losses(x, leaves, eps)
            grads = torch.autograd.grad(recon + beta * kl, list(leaves.values()))
        self._step += 1
        h = self._hyper
        for (k, w), g in zip(self.p.items(), grads):
            if self._kind == "sgd":
                upd = g
            elif self._kind == "adam":
                self._m[k].mul_(h["beta1"]).add_(g, alpha=1 - h["beta1"])
                self._v[k].mul_(h["beta2"]).addcmul_(g, g, value=1 - h["beta2"])
                upd = (self._m[k] / (1 - h["beta1"] ** self._step)) / \
                      ((self._v[k] / (1 - h["beta2"] ** self._step)).sqrt() + h["eps"])
            else:
                self._v[k].mul_(h["decay"]).addcmul_(g, g, value=1 - h["decay"])
                upd = g / (self._v[k].sqrt() + h["eps"])
            w.sub_(learning_rate * upd)
        return ZSpaceVaeState(mu.detach(), logvar.detach(), z.detach(), rec.detach(), float(recon.detach()), float(kl.detach()))

    train_step = train_batch

    def evaluate_batch(self, x) -> dict:
        st = self.forward_mean(x)
        return {"recon_loss": st.recon_loss, "kl_loss": st.kl_loss, "samples": st.mu.shape[0]}

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
        atomic_write(path, json.dumps({"input_dim": self.input_dim, "latent_dim": self.latent_dim, "optimizer": self._kind,
                                       "parameters": {k: {"shape": list(v.shape), "data": v.flatten().tolist()}
                                                      for k, v in self.state_dict().items()}}))

    @classmethod
    def load(cls, path) -> "ZSpaceVae":
        import json
        blob = json.load(open(path))
        vae = cls(blob["input_dim"], blob["latent_dim"])
        vae.load_state_dict({k: torch.tensor(v["data"]).reshape(v["shape"]) for k, v in blob["parameters"].items()})
        vae._kind = blob.get("optimizer", "sgd")
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

    def encode_text_with_mellin(self, text: str, basis: torch.Tensor) -> torch.Tensor:
        """Projects the encoding onto a ``(input_dim, input_dim)`` Mellin basis matrix."""
        enc = self.encode_text(text)
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
        return self.vae.train_batch(self._batch([text], basis), learning_rate, beta)

    def train_text_batch(self, texts, learning_rate: float = 1e-2, beta: float = 1.0, basis=None) -> ZSpaceVaeState:
        return self.vae.train_batch(self._batch(list(texts), basis), learning_rate, beta)

    def evaluate_text_batch(self, texts, basis=None) -> dict:
        return self.vae.evaluate_batch(self._batch(list(texts), basis))

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
