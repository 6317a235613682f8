"""The qubit-lattice "quantum reality" model: a layered superconducting hardware record, N qubits whose Bloch angles
follow given trajectories, a bloom signature on top of them, the interference kernel between every pair of qubits and
the row-stochastic transport it induces, collapse redistribution of a probability vector, entropies and pressures per
qubit and per cluster, the interference atlas (PSD projection, diffusion coordinates, within / between cluster ratio,
stability under a noise model) and the auto-tuned dual-local collapse drive (k-nearest-neighbour graph scored by
connectivity, algebraic connectivity and cluster ratio).

Reference parity: crates/st-logic/src/quantum_reality.rs (hardware records :34-96, clusters and the taxicab layout
:98-206, trajectories / states / fidelity :208-283, bloom :285-345, drift :348-427, kernels and transport :429-477,
pressures and entropies :479-542, collapse and drift mixing :544-590, atlas :592-907, auto-tune :909-962, engine
:1029-1188).  The lattice is held as tensors over all qubits, so every pairwise quantity is one broadcast [N, N]
expression and every spectral step one `torch.linalg.eigh`, on whichever device the lattice lives.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch

from .meta_narrative import ZSpace

TimeFn = Union[float, torch.Tensor, Callable[[float], Union[float, torch.Tensor]]]


# ---------------------------------------------------------------------------------------------------------------
# hardware and simulation records
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class QubitLayer:
    material: str = "NbTiN"
    geometry: str = "planar"


@dataclass
class JosephsonJunction:
    barrier_material: str = "AlOx"
    barrier_thickness_nm: float = 1.8


@dataclass
class OnChipLines:
    topology: str = "coplanar"
    center_width_microns: float = 10.0
    impedance_ohms: float = 50.0


@dataclass
class GroundPlane:
    material: str = "Nb"
    shielded: bool = True


@dataclass
class CryoEnclosure:
    temperature_mk: float = 10.0
    shields: str = "mu-metal"


@dataclass
class HardwareStack:
    qubit_layer: QubitLayer = field(default_factory=QubitLayer)
    junction: JosephsonJunction = field(default_factory=JosephsonJunction)
    on_chip_lines: OnChipLines = field(default_factory=OnChipLines)
    ground_plane: GroundPlane = field(default_factory=GroundPlane)
    cryo_enclosure: CryoEnclosure = field(default_factory=CryoEnclosure)


@dataclass
class SubstratePhysicalModel:
    lattice_a_angstrom: float = 4.76
    lattice_c_angstrom: float = 12.99
    die_dims_mm: Tuple[float, float, float] = (8.0, 8.0, 0.5)
    epsilon_r: float = 9.4
    thermal_conductivity_w_mk: float = 35.0
    cte_per_k: float = 5.6e-6


@dataclass
class SimulationParameters:
    qubit_frequency_ghz: float = 5.0
    anharmonicity_mhz: float = -300.0
    coupling_mhz: float = 20.0
    t1_microseconds: float = 30.0
    t2_microseconds: float = 40.0
    pi_pulse_ns: float = 25.0


# ---------------------------------------------------------------------------------------------------------------
# clusters and layout
# ---------------------------------------------------------------------------------------------------------------
class ClusterStructure:
    """Consecutive index ranges: cluster k holds ``segments[k]`` qubits."""

    def __init__(self, segments: Sequence[int]):
        if not segments:
            raise ValueError("cluster structure requires segments")
        self.segments = [int(s) for s in segments]

    def cluster_count(self) -> int:
        return len(self.segments)

    def total_qubits(self) -> int:
        return sum(self.segments)

    def cluster_bounds(self, k: int) -> Optional[Tuple[int, int]]:
        if not 0 <= k < len(self.segments):
            return None
        start = sum(self.segments[:k])
        return start, start + self.segments[k]

    def cluster_indices(self, k: int) -> range:
        b = self.cluster_bounds(k)
        return range(*b) if b else range(0)

    def cluster_of(self, n: int) -> Optional[int]:
        start = 0
        for k, ln in enumerate(self.segments):
            if start <= n < start + ln:
                return k
            start += ln
        return None

    def labels(self, n: Optional[int] = None, device=None) -> torch.Tensor:
        """Cluster id per qubit index (-1 beyond the last cluster), as an int64 tensor of length ``n``."""
        lab = torch.repeat_interleave(torch.arange(len(self.segments)), torch.tensor(self.segments))
        n = lab.numel() if n is None else n
        out = torch.full((n,), -1, dtype=torch.int64)
        out[:min(n, lab.numel())] = lab[:n]
        return out.to(device) if device is not None else out


class TaxicabLayout:
    """Integer grid coordinates per qubit; qubits beyond the stored ones sit on the x axis at their own index."""

    def __init__(self, coordinates: Sequence[Tuple[int, int]]):
        self.coordinates = [(int(x), int(y)) for x, y in coordinates]

    @classmethod
    def from_cluster(cls, cluster: ClusterStructure) -> "TaxicabLayout":
        return cls([(i, k) for k, ln in enumerate(cluster.segments) for i in range(ln)])

    def coordinate_of(self, index: int) -> Tuple[int, int]:
        return self.coordinates[index] if index < len(self.coordinates) else (index, 0)

    def ensure_capacity(self, n: int) -> None:
        self.coordinates.extend((i, 0) for i in range(len(self.coordinates), n))

    def tensor(self, n: int, device=None) -> torch.Tensor:
        return torch.tensor([self.coordinate_of(i) for i in range(n)], dtype=torch.float64, device=device).reshape(n, 2)

    def manhattan(self, n: int, device=None) -> torch.Tensor:
        c = self.tensor(n, device)
        return (c[:, None, :] - c[None, :, :]).abs().sum(-1)


# ---------------------------------------------------------------------------------------------------------------
# lattice state, bloom, drift
# ---------------------------------------------------------------------------------------------------------------
def _at(fn: TimeFn, t: float, n: int, device) -> torch.Tensor:
    v = fn(t) if callable(fn) else fn
    v = torch.as_tensor(v, dtype=torch.float64, device=device)
    return v.expand(n) if v.dim() == 0 else v


class QubitLattice:
    """All qubits at once: ``omega`` [N] and the Bloch angles / their rates as constants, [N] tensors or functions of t."""

    def __init__(self, omega, theta: TimeFn, phi: TimeFn, theta_dot: TimeFn = 0.0, phi_dot: TimeFn = 0.0):
        self.omega = torch.as_tensor(omega, dtype=torch.float64).flatten()
        self._fns = (theta, phi, theta_dot, phi_dot)

    def __len__(self) -> int:
        return self.omega.numel()

    @property
    def device(self):
        return self.omega.device

    def to(self, device) -> "QubitLattice":
        mv = lambda f: f if callable(f) or not torch.is_tensor(f) else f.to(device)             # noqa: E731
        out = QubitLattice(self.omega.to(device), *(mv(f) for f in self._fns))
        return out

    def theta(self, t: float) -> torch.Tensor:
        return _at(self._fns[0], t, len(self), self.device)

    def phi(self, t: float) -> torch.Tensor:
        return _at(self._fns[1], t, len(self), self.device)

    def theta_dot(self, t: float) -> torch.Tensor:
        return _at(self._fns[2], t, len(self), self.device)

    def phi_dot(self, t: float) -> torch.Tensor:
        return _at(self._fns[3], t, len(self), self.device)

    def indices(self) -> torch.Tensor:
        return torch.arange(len(self), dtype=torch.float64, device=self.device)

    def bloch_vectors(self, t: float) -> torch.Tensor:
        th, ph = self.theta(t), self.phi(t)
        return torch.stack([th.sin() * ph.cos(), th.sin() * ph.sin(), th.cos()], -1)

    def bloch_velocities(self, t: float) -> torch.Tensor:
        th, ph, thd, phd = self.theta(t), self.phi(t), self.theta_dot(t), self.phi_dot(t)
        return torch.stack([thd * th.cos() * ph.cos() - th.sin() * ph.sin() * phd, thd * th.cos() * ph.sin() + th.sin() * ph.cos() * phd,
                            -thd * th.sin()], -1)

    def fidelity_matrix(self, t: float) -> torch.Tensor:
        """|<psi_m | psi_n>|^2 = (1 + n_m . n_n) / 2 for every pair."""
        b = self.bloch_vectors(t)
        return 0.5 * (1.0 + b @ b.T)


@dataclass
class BloomSignature:
    """B_n(t) = varphi0^4 sin(theta_n) ln(1 + n + epsilon_t t)^psi(t)."""
    varphi0: float
    epsilon_t: float
    psi: TimeFn = 1.0

    def _envelope(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        psi = float(self.psi(t) if callable(self.psi) else self.psi)
        return self.varphi0 ** 4 * torch.log(1.0 + lattice.indices() + self.epsilon_t * t) ** psi

    def amplitude(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        return lattice.theta(t).sin() * self._envelope(lattice, t)

    def d_theta(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        return lattice.theta(t).cos() * self._envelope(lattice, t)

    def d_phi(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        return torch.zeros(len(lattice), dtype=torch.float64, device=lattice.device)


@dataclass
class DriftField:
    """Azimuthal drift phi(t) Re(zeta_n) cos(omega t + phi_n) / sin(theta_n); qubits without a zeta use 1."""
    phi: TimeFn
    omega: float
    zeta: Optional[torch.Tensor] = None

    def phi_component(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        n = len(lattice)
        z = torch.ones(n, dtype=torch.float64, device=lattice.device)
        if self.zeta is not None:
            zr = torch.as_tensor(self.zeta).real.to(torch.float64).flatten().to(lattice.device)
            z[:min(n, zr.numel())] = zr[:n]
        amp = float(self.phi(t) if callable(self.phi) else self.phi)
        d = amp * z * torch.cos(self.omega * t + lattice.phi(t))
        s = lattice.theta(t).sin()
        return torch.where(s.abs() < 1e-9, torch.zeros_like(d), d / torch.where(s.abs() < 1e-9, torch.ones_like(s), s))

    def drift_vectors(self, lattice: QubitLattice, t: float) -> torch.Tensor:
        """[N, 2]: (theta component, phi component); the field is purely azimuthal."""
        p = self.phi_component(lattice, t)
        return torch.stack([torch.zeros_like(p), p], -1)


@dataclass
class NoiseModel:
    t2_drift: float = 0.0
    phi_drift: float = 0.0
    omega_variation: float = 0.0

    def is_active(self) -> bool:
        return self.t2_drift > 0.0 or abs(self.phi_drift) > 0.0 or abs(self.omega_variation) > 0.0


# ---------------------------------------------------------------------------------------------------------------
# pairwise kernels and what follows from them
# ---------------------------------------------------------------------------------------------------------------
def fidelity(lattice: QubitLattice, m: int, n: int, t: float) -> float:
    return float(lattice.fidelity_matrix(t)[m, n])


def wavelet_modulation(cluster: ClusterStructure, cluster_index: int, omega: float, t: float, bloom: BloomSignature, lattice: QubitLattice) -> complex:
    idx = [i for i in cluster.cluster_indices(cluster_index) if i < len(lattice)]
    if not idx:
        return 0j
    ii = torch.tensor(idx, device=lattice.device)
    amp = bloom.amplitude(lattice, t)[ii]
    return complex((amp * torch.exp(-1j * omega * ii.to(torch.float64))).sum())


def spiral_phase_affinity(lattice: QubitLattice, t: float, bloom: BloomSignature) -> torch.Tensor:
    """sqrt|B_m B_n| F_mn exp(i (omega_m - omega_n) t) for every pair (complex128 [N, N])."""
    b = bloom.amplitude(lattice, t)
    mag = (b[:, None] * b[None, :]).abs().sqrt() * lattice.fidelity_matrix(t)
    return torch.polar(mag, (lattice.omega[:, None] - lattice.omega[None, :]) * t)


def interference_kernel(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, sigma_d: float, sigma_bloom: float) -> torch.Tensor:
    """Gaussian in the drift difference times a normalised Gaussian ("soft delta") in the bloom difference."""
    d = drift.phi_component(lattice, t)
    b = bloom.amplitude(lattice, t)
    sb = max(sigma_bloom, 1e-12)
    drift_k = torch.exp(-(d[:, None] - d[None, :]) ** 2 / (2.0 * sigma_d ** 2))
    bloom_k = torch.exp(-(b[:, None] - b[None, :]) ** 2 / (2.0 * sb * sb)) / (math.sqrt(2.0 * math.pi) * sb)
    return drift_k * bloom_k


def _row_normalise(m: torch.Tensor) -> torch.Tensor:
    s = m.sum(-1, keepdim=True)
    return torch.where(s > 0.0, m / torch.where(s > 0.0, s, torch.ones_like(s)), torch.zeros_like(m))


def row_normalised_transport(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, sigma_d: float, sigma_bloom: float) -> torch.Tensor:
    k = interference_kernel(lattice, t, bloom, drift, sigma_d, sigma_bloom)
    s = k.sum(-1, keepdim=True)
    return torch.where(s > 0.0, k / torch.where(s > 0.0, s, torch.ones_like(s)), k)


def thermo_pressure(lattice: QubitLattice, t: float, bloom: BloomSignature, alpha_th: float) -> torch.Tensor:
    return torch.exp(-alpha_th * (bloom.d_theta(lattice, t) ** 2 + bloom.d_phi(lattice, t) ** 2))


def _delta_log(lattice: QubitLattice, t: float, bloom: BloomSignature) -> torch.Tensor:
    return torch.log1p((bloom.amplitude(lattice, t) - bloom.d_theta(lattice, t)).abs())


def shadow_entropy(lattice: QubitLattice, t: float, bloom: BloomSignature) -> float:
    w = (1.0 + lattice.theta(t).cos()) / 2.0
    return float((w * _delta_log(lattice, t, bloom)).sum() / max(len(lattice), 1))


def degeneracy_counts(lattice: QubitLattice, t: float, bloom: BloomSignature, epsilon: float) -> torch.Tensor:
    b = bloom.amplitude(lattice, t)
    close = (b[:, None] - b[None, :]).abs() < epsilon
    close.fill_diagonal_(False)
    return close.sum(-1)


def taxicab_entropies(cluster: ClusterStructure, lattice: QubitLattice, t: float, bloom: BloomSignature, degeneracy: torch.Tensor) -> torch.Tensor:
    """sum over the cluster of ln(1 + |B - dB/dtheta|) x degeneracy, for every cluster at once."""
    lab = cluster.labels(len(lattice), lattice.device)
    vals = _delta_log(lattice, t, bloom) * degeneracy.to(torch.float64)
    out = torch.zeros(cluster.cluster_count(), dtype=torch.float64, device=lattice.device)
    ok = lab >= 0
    return out.index_add(0, lab[ok], vals[ok])


def taxicab_entropy(cluster: ClusterStructure, cluster_index: int, lattice: QubitLattice, t: float, bloom: BloomSignature, degeneracy: torch.Tensor) -> float:
    return float(taxicab_entropies(cluster, lattice, t, bloom, degeneracy)[cluster_index])


def collapse_redistribution(lam: torch.Tensor, probability, mu: float) -> torch.Tensor:
    """p <- (1 - mu) p + mu Lambda p."""
    p = torch.as_tensor(probability, dtype=torch.float64, device=lam.device)
    mu = min(max(mu, 0.0), 1.0)
    n = lam.shape[1]
    padded = torch.zeros(n, dtype=torch.float64, device=lam.device)
    padded[:min(n, p.numel())] = p[:n]
    mixed = lam @ padded
    out = (1.0 - mu) * p
    out[:min(p.numel(), mixed.numel())] += mu * mixed[:p.numel()]
    return out


def superposed_drift(lam: torch.Tensor, lattice: QubitLattice, t: float, drift: DriftField) -> torch.Tensor:
    return lam @ drift.drift_vectors(lattice, t)


# ---------------------------------------------------------------------------------------------------------------
# atlas
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class AtlasResult:
    kernel: torch.Tensor
    diffusion_coordinates: torch.Tensor
    pseudo_cluster_ratio: float


@dataclass
class AtlasAnalysis:
    base: AtlasResult
    noisy: Optional[AtlasResult]
    stability: float


def _pseudo_ratio(matrix: torch.Tensor, clusters: ClusterStructure) -> float:
    lab = clusters.labels(matrix.shape[0], matrix.device)     # qubits beyond the last cluster share the label -1
    same = lab[:, None] == lab[None, :]
    w = matrix.clamp_min(0.0).clone()
    w.fill_diagonal_(0.0)
    return float(w[same].sum() / (w[~same].sum() + 1e-9))


def _project_to_psd(m: torch.Tensor) -> torch.Tensor:
    vals, vecs = torch.linalg.eigh(0.5 * (m + m.T))
    return (vecs * vals.clamp_min(0.0)) @ vecs.T


def _diffusion_map(kernel: torch.Tensor, components: int) -> torch.Tensor:
    n = kernel.shape[0]
    if n == 0:
        return kernel.new_zeros(0, 0)
    deg = kernel.sum(-1).clamp_min(1e-9)
    norm = kernel / (deg[:, None] * deg[None, :]).sqrt()
    vals, vecs = torch.linalg.eigh(0.5 * (norm + norm.T))
    order = torch.argsort(vals.abs(), descending=True)[:min(components, n)]
    return vecs[:, order]


def _interference_matrix(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, layout: TaxicabLayout, bandwidth: float,
                         noise: Optional[NoiseModel]) -> torch.Tensor:
    n = len(lattice)
    sigma = max(bandwidth, 1e-6)
    b = bloom.amplitude(lattice, t)
    amp = 0.5 * (b[:, None] + b[None, :])
    phase = (lattice.omega[:, None] - lattice.omega[None, :]) * t
    spatial = torch.exp(-layout.manhattan(n, lattice.device) ** 2 / (sigma * sigma))
    if noise is not None:
        if noise.t2_drift > 0.0:
            amp = amp * math.exp(-abs(t) / max(noise.t2_drift, 1e-9))
        ph, idx = lattice.phi(t), lattice.indices()
        phase = phase + noise.phi_drift * (ph[:, None] - ph[None, :]) + noise.omega_variation * t * (idx[:, None] - idx[None, :])
    d = drift.phi_component(lattice, t)
    return amp * torch.cos(phase + d[:, None] - d[None, :]) * spatial


def interference_atlas(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, layout: TaxicabLayout, bandwidth: float,
                       clusters: ClusterStructure, noise: Optional[NoiseModel] = None) -> AtlasAnalysis:
    def analyse(model: Optional[NoiseModel]) -> AtlasResult:
        psd = _project_to_psd(_interference_matrix(lattice, t, bloom, drift, layout, bandwidth, model))
        return AtlasResult(psd, _diffusion_map(psd, 3), _pseudo_ratio(psd, clusters))
    base = analyse(None)
    noisy = analyse(noise) if noise is not None and noise.is_active() else None
    stability = 1.0
    if noisy is not None:
        stability = 1.0 - abs(base.pseudo_cluster_ratio - noisy.pseudo_cluster_ratio) / (abs(base.pseudo_cluster_ratio) + 1e-9)
    return AtlasAnalysis(base, noisy, min(max(stability, 0.0), 1.0))


# ---------------------------------------------------------------------------------------------------------------
# auto-tuned dual-local drive
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class AutoTuneResult:
    k_nn: int
    k_scale: float
    bandwidth: float
    objective: float
    connectivity: int
    lambda2: float
    pseudo_ratio: float


def dual_local_kernel(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, layout: TaxicabLayout, k_scale: float,
                      bandwidth: float) -> torch.Tensor:
    """exp(-(feature distance^2 + spatial distance) / sigma^2) with features (bloom, drift, omega / k_scale) and the spatial part
    twice the taxicab distance (coordinate differences plus the Manhattan term)."""
    n = len(lattice)
    sigma, fs = max(bandwidth, 1e-9), max(abs(k_scale), 1e-9)
    b, d, w = bloom.amplitude(lattice, t), drift.phi_component(lattice, t), lattice.omega / fs
    feat = (b[:, None] - b[None, :]) ** 2 + (d[:, None] - d[None, :]) ** 2 + (w[:, None] - w[None, :]) ** 2
    return torch.exp(-(feat + 2.0 * layout.manhattan(n, lattice.device)) / (sigma * sigma))


def knn_adjacency(kernel: torch.Tensor, k: int) -> torch.Tensor:
    """Symmetric graph keeping, for every node, its k strongest off-diagonal weights (max of the two directions)."""
    n = kernel.shape[0]
    k = min(k, max(n - 1, 0))
    if n == 0 or k == 0:
        return torch.zeros_like(kernel)
    off = kernel.clone()
    off.fill_diagonal_(-math.inf)
    vals, idx = torch.topk(off, k, dim=-1)
    adj = torch.zeros_like(kernel).scatter_(1, idx, vals.clamp_min(0.0))
    return torch.maximum(adj, adj.T)


def _laplacian_spectrum(adj: torch.Tensor) -> torch.Tensor:
    return torch.linalg.eigvalsh(torch.diag(adj.sum(-1)) - adj)


def connected_components(adj: torch.Tensor) -> int:
    """Number of connected components (label propagation by repeated neighbourhood minima)."""
    n = adj.shape[0]
    if n == 0:
        return 0
    link = (adj > 0.0) | torch.eye(n, dtype=torch.bool, device=adj.device)
    lab = torch.arange(n, device=adj.device)
    big = torch.full((n, n), n, device=adj.device)
    for _ in range(n):
        new = torch.where(link, lab[None, :].expand(n, n), big).min(-1).values
        if torch.equal(new, lab):
            break
        lab = new
    return int(torch.unique(lab).numel())


def laplacian_lambda2(adj: torch.Tensor) -> float:
    return max(float(_laplacian_spectrum(adj)[1]), 0.0) if adj.shape[0] > 1 else 0.0


def auto_tune_collapse_drive(lattice: QubitLattice, t: float, bloom: BloomSignature, drift: DriftField, layout: TaxicabLayout,
                             clusters: ClusterStructure, k_nn_candidates: Sequence[int], k_scale_candidates: Sequence[float],
                             bandwidth_candidates: Sequence[float]) -> Optional[AutoTuneResult]:
    """Grid search: objective = (1 / components) x exp(-(lambda2 - 0.5)^2 / 0.25) x ratio / (1 + ratio); the first best wins."""
    layout.ensure_capacity(len(lattice))
    best: Optional[AutoTuneResult] = None
    for k_nn in k_nn_candidates:
        if k_nn == 0:
            continue
        for k_scale in k_scale_candidates:
            for bw in bandwidth_candidates:
                adj = knn_adjacency(dual_local_kernel(lattice, t, bloom, drift, layout, k_scale, bw), k_nn)
                comps = connected_components(adj)
                lam2 = laplacian_lambda2(adj)
                ratio = _pseudo_ratio(adj, clusters)
                obj = (min(max(1.0 / comps, 0.0), 1.0) if comps else 0.0) * math.exp(-((lam2 - 0.5) ** 2) / 0.25) * ratio / (1.0 + ratio)
                if best is None or obj > best.objective:
                    best = AutoTuneResult(int(k_nn), float(k_scale), float(bw), obj, comps, lam2, ratio)
    return best


# ---------------------------------------------------------------------------------------------------------------
# engine
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class MonadBiome:
    weights: List[float]


@dataclass
class ZMonadBridge:
    probability: torch.Tensor
    shadow_entropy: float
    coherence: float


@dataclass
class CollapseManifold:
    cluster_entropies: torch.Tensor
    degeneracy: torch.Tensor
    pressure_map: torch.Tensor
    average_entropy: float


@dataclass
class QuantumRealityEngine:
    clusters: ClusterStructure
    lattice: QubitLattice
    bloom: BloomSignature
    drift: DriftField
    sigma_d: float
    sigma_bloom: float
    hardware: HardwareStack = field(default_factory=HardwareStack)
    substrate: SubstratePhysicalModel = field(default_factory=SubstratePhysicalModel)
    simulation: SimulationParameters = field(default_factory=SimulationParameters)

    def lambda_(self, t: float) -> torch.Tensor:
        return row_normalised_transport(self.lattice, t, self.bloom, self.drift, self.sigma_d, self.sigma_bloom)

    def lambda_with_dual_locality(self, t: float, layout: TaxicabLayout, params: AutoTuneResult) -> torch.Tensor:
        layout.ensure_capacity(len(self.lattice))
        return _row_normalise(knn_adjacency(dual_local_kernel(self.lattice, t, self.bloom, self.drift, layout, params.k_scale, params.bandwidth),
                                            params.k_nn))

    def tuned_collapse_drive(self, t: float, layout: TaxicabLayout, k_nn_candidates, k_scale_candidates, bandwidth_candidates):
        params = auto_tune_collapse_drive(self.lattice, t, self.bloom, self.drift, layout, self.clusters, k_nn_candidates, k_scale_candidates,
                                          bandwidth_candidates)
        return None if params is None else (params, self.lambda_with_dual_locality(t, layout, params))

    def connect_zspace_monad(self, z_space: ZSpace, biome: MonadBiome, t: float, mu: float) -> ZMonadBridge:
        sig = torch.tensor(z_space.signature, dtype=torch.float64, device=self.lattice.device)
        total = float(sig[torch.isfinite(sig)].sum()) if sig.numel() else 0.0
        if not (total > 0.0 and math.isfinite(total)):
            total = 1.0
        p = collapse_redistribution(self.lambda_(t), sig.clamp_min(0.0) / total, mu)
        w = torch.zeros_like(p)
        bw = torch.tensor(biome.weights, dtype=torch.float64, device=p.device)
        w[:min(p.numel(), bw.numel())] = bw[:p.numel()]
        return ZMonadBridge(p, shadow_entropy(self.lattice, t, self.bloom), float((p * w).sum()))

    def collapse_manifold(self, t: float, degeneracy_epsilon: float, alpha_th: float) -> CollapseManifold:
        deg = degeneracy_counts(self.lattice, t, self.bloom, max(degeneracy_epsilon, 1e-9))
        ent = taxicab_entropies(self.clusters, self.lattice, t, self.bloom, deg)
        return CollapseManifold(ent, deg, thermo_pressure(self.lattice, t, self.bloom, alpha_th), float(ent.mean()) if ent.numel() else 0.0)
