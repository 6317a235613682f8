"""Psi synchronisation: samples the phase of a driven branch stroboscopically, identifies the circle-map coupling from
the samples, and scans an Arnold-tongue map (rotation-number lock strength over forcing strength x drive frequency).

Parity: crates/st-core/src/theory/psi_sync.rs — `SyncState` (:26-56), `MetaMembModel::phi_sample` (:58-100),
`PsiBranchConfig` (:102-131), `RationalLock` (:149-178), `PsiSynchroConfig` (:191-212),
`PsiSynchroMonolith::{synchronise_branches, run_branch, sample_branch, heatmap_for_branch}` (:215-345),
`identify_kappa` (:452-497), `rotation_number` (:498-516), `nearest_rational` (:517-528).

The tongue map iterates the circle map ``phi <- phi + Omega - K/2pi sin(2 pi phi)`` for every grid cell; here all cells
advance together as one tensor (on the GPU when asked), instead of a doubly nested host loop, and the nearest-rational
search is a single reduction over the denominators.  The reference draws the map with a plotting crate; `render_heatmap`
writes the same colour ramp as a PNG with the standard library.
"""
from __future__ import annotations

import math
import struct
import zlib
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import torch

from . import observability

TWO_PI = 2.0 * math.pi


@dataclass
class SyncState:
    tau: float = 0.0
    step: float = 0.01
    seed: int = 42
    epoch: int = 0
    gamma: float = 1.3
    lam: float = 1.0
    wd: float = 0.7
    omega0: float = 0.72
    drift_coupled: float = 1.05
    poincare: bool = True


@dataclass
class PsiBranchConfig:
    branch_id: str
    gamma: float
    lam: float
    wd: float
    omega0: float
    drift_coupled: float
    phase0: float = 0.0
    samples: int = 64
    step: float = 0.01
    z_coordinate: float = 0.0

    @classmethod
    def with_state(cls, branch_id: str, state: SyncState, samples: int) -> "PsiBranchConfig":
        return cls(branch_id, state.gamma, state.lam, state.wd, state.omega0, state.drift_coupled, 0.0, samples, state.step, 0.0)


@dataclass
class MetaMembModel:
    """Three slow sinusoids whose sum ("bloom") modulates the branch phase."""
    delta: Sequence[float] = (0.03, 0.05, 0.02)
    omega: Sequence[float] = (1.2, 0.9, 1.6)
    theta: Sequence[float] = (0.0, 1.0, 2.5)

    def bloom(self, t: torch.Tensor) -> torch.Tensor:
        d, w, th = (torch.tensor(v, dtype=torch.float64, device=t.device) for v in (self.delta, self.omega, self.theta))
        return (d * torch.sin(w * t[..., None] + th)).sum(-1)

    def phi(self, t: torch.Tensor, branch: PsiBranchConfig) -> torch.Tensor:
        psi = branch.omega0 * t + branch.lam * branch.drift_coupled ** branch.gamma * torch.tanh(5.0 * self.bloom(t))
        return torch.remainder((psi - (branch.wd * t + branch.phase0)) / TWO_PI, 1.0)

    def phi_sample(self, t: float, branch: PsiBranchConfig) -> float:
        return float(self.phi(torch.tensor([t], dtype=torch.float64), branch)[0])


@dataclass(frozen=True)
class RationalLock:
    p: int = 0
    q: int = 1
    error: float = float("inf")
    lam: float = 0.0
    wd: float = 0.0

    def __str__(self) -> str:
        return f"{self.p}/{self.q} @ λ={self.lam:.4f} ω_d={self.wd:.4f} (ε={self.error:.3e})"


class PsiSyncError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass
class PsiSynchroConfig:
    lam_range: Tuple[float, float, int] = (0.0, 2.0, 60)
    wd_range: Tuple[float, float, int] = (0.3, 1.2, 80)
    burn: int = 200
    sample: int = 300
    qmax: int = 8
    out_dir: Optional[str] = None
    device: str = "cpu"


@dataclass
class PsiBranchReport:
    branch: PsiBranchConfig
    phi_samples: List[float]
    omega_hat: float
    kappa_hat: float
    rmse: float
    lam_grid: List[float]
    wd_grid: List[float]
    heatmap: torch.Tensor                 # [lam, wd] lock strength 1 / (error + 1e-6)
    best_lock: RationalLock
    heatmap_path: Optional[Path] = None


def wrap_unit(x: torch.Tensor) -> torch.Tensor:
    return torch.remainder(x + 0.5, 1.0) - 0.5


def identify_kappa(phi: Sequence[float], lam: float) -> Tuple[float, float, float]:
    """Least squares of the wrapped increments on ``(1, sin 2 pi phi)``: returns ``(Omega_hat, kappa_hat, rmse)`` with
    ``kappa_hat = -2 pi a_hat / lam``."""
    x = torch.as_tensor(phi, dtype=torch.float64)
    if x.numel() < 2:
        return 0.0, 0.0, 0.0
    d = wrap_unit(x[1:] - x[:-1])
    s = torch.sin(TWO_PI * x[:-1])
    s11, s12, s22, y1, y2 = float(d.numel()), float(s.sum()), float((s * s).sum()), float(d.sum()), float((s * d).sum())
    det = s11 * s22 - s12 * s12
    omega, a = (0.0, 0.0) if abs(det) < 1e-12 else ((s22 * y1 - s12 * y2) / det, (s11 * y2 - s12 * y1) / det)
    rmse = float(((d - (omega + a * s)) ** 2).mean().sqrt())
    return omega, -TWO_PI * a / max(lam, 1e-9), rmse


def rotation_number(omega, kappa, burn: int, sample: int) -> torch.Tensor:
    """Mean advance per iteration of the circle map after `burn` iterations, for every element of the (broadcast)
    ``omega`` / ``kappa`` tensors."""
    omega = torch.as_tensor(omega, dtype=torch.float64)
    kappa = torch.as_tensor(kappa, dtype=torch.float64, device=omega.device)
    omega, kappa = torch.broadcast_tensors(omega, kappa)
    scale = kappa / TWO_PI
    phi = torch.zeros_like(omega)
    for _ in range(burn):
        phi = torch.remainder(phi + omega - scale * torch.sin(TWO_PI * phi), 1.0)
    total = torch.zeros_like(omega)
    for _ in range(sample):
        nxt = torch.remainder(phi + omega - scale * torch.sin(TWO_PI * phi), 1.0)
        total += torch.remainder(nxt - phi, 1.0)
        phi = nxt
    return total / sample if sample else total


def nearest_rational(x, qmax: int):
    """``(p, q, error)`` of the closest ``p / q`` with ``q <= qmax`` (the smallest such ``q`` on ties), elementwise."""
    x = torch.as_tensor(x, dtype=torch.float64)
    q = torch.arange(1, max(qmax, 1) + 1, dtype=torch.float64, device=x.device)
    xq = x[..., None] * q
    p = torch.where(xq >= 0, torch.floor(xq + 0.5), -torch.floor(-xq + 0.5))            # round half away from zero
    err = (x[..., None] - p / q).abs()
    best = err.argmin(-1, keepdim=True)                                                  # first minimum: smallest q
    return p.gather(-1, best).squeeze(-1).to(torch.int64), q[best.squeeze(-1)].to(torch.int64), err.gather(-1, best).squeeze(-1)


def linspace(lo: float, hi: float, bins: int) -> List[float]:
    return [lo] if bins <= 1 else [lo + (hi - lo) / (bins - 1) * i for i in range(bins)]


def gradient_color(norm: float) -> Tuple[int, int, int]:
    c = min(max(norm, 0.0), 1.0)
    return int(255.0 * c), int(255.0 * max(1.0 - abs(c - 0.5) * 2.0, 0.0)), int(255.0 * (1.0 - c))


def write_png(path, rgb: torch.Tensor) -> None:
    """``rgb``: uint8 ``[H, W, 3]``."""
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + bytes(rgb[y].reshape(-1).tolist()) for y in range(h))

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    Path(path).write_bytes(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) +
                           chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


class PsiSynchroMonolith:
    def __init__(self, base_state: Optional[SyncState] = None, config: Optional[PsiSynchroConfig] = None,
                 model: Optional[MetaMembModel] = None):
        self.base_state, self.config, self.model = base_state or SyncState(), config or PsiSynchroConfig(), model or MetaMembModel()

    with_model = classmethod(lambda cls, base_state, config, model: cls(base_state, config, model))

    def synchronise_branches(self, branches: Sequence[PsiBranchConfig]) -> List[PsiBranchReport]:
        return [self.run_branch(b) for b in branches]

    def sample_branch(self, branch: PsiBranchConfig) -> List[float]:
        """Stroboscopic samples once per drive period ``2 pi / wd``, taken at the first integration step at or after
        each period mark."""
        td = TWO_PI / branch.wd
        marks = self.base_state.tau + td * torch.arange(branch.samples, dtype=torch.float64)
        steps = torch.ceil((marks - self.base_state.tau - 1e-12) / branch.step).clamp(min=0)
        return self.model.phi(self.base_state.tau + steps * branch.step, branch).tolist()

    def heatmap_for_branch(self, branch: PsiBranchConfig, kappa_hat: float):
        cfg = self.config
        lam_grid, wd_grid = linspace(*cfg.lam_range), linspace(*cfg.wd_range)
        dev = torch.device(cfg.device)
        lam = torch.tensor(lam_grid, dtype=torch.float64, device=dev)[:, None]
        wd = torch.tensor(wd_grid, dtype=torch.float64, device=dev)[None, :]
        rho = rotation_number(branch.omega0 / wd - 1.0, kappa_hat * lam, cfg.burn, cfg.sample)
        p, q, err = nearest_rational(rho, cfg.qmax)
        flat = int(err.reshape(-1).argmin())                               # first minimum in row-major order, as a scan would find
        i, j = divmod(flat, len(wd_grid))
        lock = RationalLock(int(p[i, j]), int(q[i, j]), float(err[i, j]), lam_grid[i], wd_grid[j])
        return lam_grid, wd_grid, (1.0 / (err + 1e-6)).cpu(), lock

    def render_heatmap(self, out_dir, branch: PsiBranchConfig, lam_grid, wd_grid, matrix: torch.Tensor, cell: int = 8) -> Path:
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        path = out / f"heatmap_{branch.branch_id.replace(':', '-')}_gamma_{branch.gamma:.2f}.png"
        norm = matrix / max(float(matrix.max()), 1.0)
        img = torch.tensor([[gradient_color(float(v)) for v in row] for row in norm.flip(0)], dtype=torch.uint8)   # lambda grows upwards
        write_png(path, img.repeat_interleave(cell, 0).repeat_interleave(cell, 1))
        return path

    def run_branch(self, branch: PsiBranchConfig) -> PsiBranchReport:
        if branch.samples < 2:
            raise PsiSyncError("insufficient_samples", f"branch '{branch.branch_id}' requires at least two samples (requested {branch.samples})")
        branch = replace(branch, gamma=max(branch.gamma, 1e-9), lam=max(branch.lam, 1e-9), wd=max(branch.wd, 1e-9), step=max(branch.step, 1e-6))
        phi = self.sample_branch(branch)
        omega_hat, kappa_hat, rmse = identify_kappa(phi, branch.lam)
        lam_grid, wd_grid, matrix, lock = self.heatmap_for_branch(branch, kappa_hat)
        path = None
        if self.config.out_dir:
            try:
                path = self.render_heatmap(self.config.out_dir, branch, lam_grid, wd_grid, matrix)
            except OSError as exc:
                raise PsiSyncError("plot", f"unable to render heatmap for branch '{branch.branch_id}': {exc}")
        report = PsiBranchReport(branch, phi, omega_hat, kappa_hat, rmse, lam_grid, wd_grid, matrix, lock, path)
        observability.emit_tensor_op("psi_sync_branch", (len(phi), 1), tuple(matrix.shape))
        observability.emit_tensor_op_meta("psi_sync_branch", lambda: {
            "backend": "torch", "kind": "psi_sync_branch", "branch_id": branch.branch_id, "samples": len(phi), "omega_hat": omega_hat,
            "kappa_hat": kappa_hat, "rmse": rmse, "lam_bins": len(lam_grid), "wd_bins": len(wd_grid), "best_lock_p": lock.p,
            "best_lock_q": lock.q, "best_lock_error": lock.error, "heatmap_peak": float(matrix.max()), "heatmap_mean": float(matrix.mean()),
            "rendered": path is not None})
        return report
