"""Logic-side utilities: contextual observation, temporal volume dynamics, SoftLogic feedback
events, a key/value store with the Redis helper surface, sparse-problem tuning profiles and the
signal-capture studio.

Reference components and where their behaviour is defined:

* contextual observation of A/B arrangements — crates/st-logic/src/contextual_observation.rs:35-260
* temporal interpolation / integration of volumes — crates/st-logic/src/temporal_dynamics.rs:63-160
* feedback metric events — crates/st-zeta/src/lib.rs:16-90
* key/value helpers and the tuning ``Choice`` record — crates/st-kv/src/lib.rs:35-440
* problem profile and Wilson bound — crates/st-amg/src/profile.rs:28-275, src/sr_learn.rs:180-192
* signal capture, overlay frames, storyboard — crates/st-qr-studio/src/lib.rs:43-460,831-1180

Everything here is host-side bookkeeping (the reference runs it on the CPU as well); tensors that
appear are torch tensors on whatever device the caller uses.
"""
from __future__ import annotations

import json
import logging
import math
import threading
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Deque, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

# ----------------------------------------------------------------------------------------------
# Contextual observation
# ----------------------------------------------------------------------------------------------

A, B = "A", "B"


class Arrangement:
    """Placement of the two pure atoms on a support given as an undirected edge list."""

    def __init__(self, placements: Sequence[str], edges: Iterable[Tuple[int, int]] = ()):
        self.placements = [str(p) for p in placements]
        for p in self.placements:
            if p not in (A, B):
                raise ValueError(f"atom must be 'A' or 'B', got {p!r}")
        n = len(self.placements)
        seen = set()
        for u, v in edges:
            if u == v or not (0 <= u < n and 0 <= v < n):
                continue
            seen.add((min(u, v), max(u, v)))
        self.edges = sorted(seen)
        self.adjacency: List[List[int]] = [[] for _ in range(n)]
        for u, v in self.edges:
            self.adjacency[u].append(v)
            self.adjacency[v].append(u)

    @classmethod
    def from_line(cls, placements: Sequence[str]) -> "Arrangement":
        return cls(placements, [(i, i + 1) for i in range(len(placements) - 1)])

    def __len__(self) -> int:
        return len(self.placements)

    def boundary_edges(self) -> int:
        return sum(1 for u, v in self.edges if self.placements[u] != self.placements[v])

    def is_pure(self) -> bool:
        return self.boundary_edges() == 0

    def flipped(self) -> "Arrangement":
        return Arrangement([B if p == A else A for p in self.placements], self.edges)

    def population(self) -> Tuple[int, int]:
        a = sum(1 for p in self.placements if p == A)
        return a, len(self.placements) - a

    def cluster_counts(self) -> Tuple[int, int]:
        visited = [False] * len(self.placements)
        counts = [0, 0]
        for start in range(len(self.placements)):
            if visited[start]:
                continue
            atom = self.placements[start]
            counts[0 if atom == A else 1] += 1
            queue = deque([start])
            visited[start] = True
            while queue:
                node = queue.popleft()
                for nbr in self.adjacency[node]:
                    if not visited[nbr] and self.placements[nbr] == atom:
                        visited[nbr] = True
                        queue.append(nbr)
        return counts[0], counts[1]

    def cluster_imbalance(self) -> int:
        a, b = self.cluster_counts()
        return b - a


@dataclass(frozen=True)
class ContextualSignature:
    boundary_edges: int
    absolute_population_imbalance: int
    cluster_imbalance: int

    def meaning_weight(self) -> float:
        if not (self.boundary_edges or self.absolute_population_imbalance or self.cluster_imbalance):
            return 0.0
        return (self.boundary_edges + 0.5 * self.absolute_population_imbalance
                + 0.25 * abs(self.cluster_imbalance))


class ContextObserver:
    """Observes only label-swap-invariant quantities of an arrangement."""

    @staticmethod
    def observe(arrangement: Arrangement) -> Optional[Tuple[int, int]]:
        boundary = arrangement.boundary_edges()
        if boundary == 0:
            return None                                    # undetermined: a pure arrangement carries no context
        a, b = arrangement.population()
        return boundary, abs(b - a)

    @staticmethod
    def is_swap_invariant(arrangement: Arrangement) -> bool:
        return ContextObserver.observe(arrangement) == ContextObserver.observe(arrangement.flipped())

    @staticmethod
    def signature(arrangement: Arrangement) -> Optional[ContextualSignature]:
        obs = ContextObserver.observe(arrangement)
        if obs is None:
            return None
        return ContextualSignature(obs[0], obs[1], arrangement.cluster_imbalance())


def lift_to_label(arrangement: Arrangement, prefer_b: bool = True) -> Optional[str]:
    """Picks a label for the majority atom under an orientation gauge; ``None`` when the
    arrangement is pure or balanced (the gauge cannot be fixed from swap-invariant data)."""
    if ContextObserver.observe(arrangement) is None:
        return None
    a, b = arrangement.population()
    if a == b:
        return None
    majority_is_b = b > a
    return "b" if majority_is_b == prefer_b else "a"


class MeaningBasis:
    """±1 signal of an arrangement and its magnitude spectrum."""

    def __init__(self, arrangement: Arrangement):
        if len(arrangement) == 0:
            raise ValueError("empty arrangement")
        self.signal = torch.tensor([1.0 if p == B else -1.0 for p in arrangement.placements])
        self.spectrum = torch.fft.rfft(self.signal).abs()

    def dominant_frequency(self) -> Optional[Tuple[int, float]]:
        if self.spectrum.numel() <= 1:
            return None
        idx = int(torch.argmax(self.spectrum[1:]).item()) + 1
        return idx, float(self.spectrum[idx])


# ----------------------------------------------------------------------------------------------
# Temporal dynamics of volumes
# ----------------------------------------------------------------------------------------------


@dataclass
class TemporalPropagationConfig:
    steps: int = 4
    delta_time: float = 1.0 / 24.0
    harmonic_blend: float = 0.5
    decay_gain: float = 1.0


@dataclass
class TemporalVolumeState:
    """Voxels ``(D, H, W)``, per-voxel harmonic channels ``(D, H, W, C)`` and resonance decay."""

    voxels: torch.Tensor
    harmonics: torch.Tensor
    resonance_decay: torch.Tensor

    @classmethod
    def zeros(cls, depth: int, height: int, width: int, channels: int = 0, device=None) -> "TemporalVolumeState":
        return cls(torch.zeros(depth, height, width, device=device),
                   torch.zeros(depth, height, width, channels, device=device),
                   torch.zeros(depth, height, width, device=device))

    def _with_channels(self, channels: int) -> torch.Tensor:
        c = self.harmonics.shape[-1]
        if c >= channels:
            return self.harmonics
        pad = torch.zeros(*self.harmonics.shape[:-1], channels - c, device=self.harmonics.device)
        return torch.cat([self.harmonics, pad], dim=-1)


def _check_pair(a: TemporalVolumeState, b: TemporalVolumeState) -> None:
    if a.voxels.shape != b.voxels.shape:
        raise ValueError(f"volume shape mismatch: {tuple(a.voxels.shape)} vs {tuple(b.voxels.shape)}")


def interpolate_temporal_sequence(start: TemporalVolumeState, end: TemporalVolumeState,
                                  config: TemporalPropagationConfig = TemporalPropagationConfig()
                                  ) -> List[TemporalVolumeState]:
    """``start``, ``steps`` linear in-betweens at t = k / (steps + 1), ``end``."""
    _check_pair(start, end)
    steps = max(1, config.steps)
    channels = max(start.harmonics.shape[-1], end.harmonics.shape[-1])
    hs, he = start._with_channels(channels), end._with_channels(channels)
    frames = [start]
    for k in range(1, steps + 1):
        t = k / (steps + 1.0)
        frames.append(TemporalVolumeState(torch.lerp(start.voxels, end.voxels, t), torch.lerp(hs, he, t),
                                          torch.lerp(start.resonance_decay, end.resonance_decay, t)))
    frames.append(end)
    return frames


def integrate_volume(state: TemporalVolumeState, drive: TemporalVolumeState,
                     config: TemporalPropagationConfig = TemporalPropagationConfig()) -> None:
    """Relaxes ``state`` toward ``drive`` in place: per sub-step the voxel keeps ``1 - decay·dt`` of
    itself, the decay field follows the same blend and harmonics move by ``harmonic_blend``."""
    _check_pair(state, drive)
    if not math.isfinite(config.delta_time) or config.delta_time <= 0:
        raise ValueError("temporal_delta_time must be positive and finite")
    steps = max(1, config.steps)
    dt = config.delta_time / steps
    blend = min(max(config.harmonic_blend, 0.0), 1.0)
    gain = max(config.decay_gain, 0.0)
    channels = drive.harmonics.shape[-1]
    state.harmonics = state._with_channels(channels)
    src = drive._with_channels(state.harmonics.shape[-1])
    drive_decay = drive.resonance_decay.clamp_min(0.0) * gain
    decay = (drive_decay * dt).clamp_max(1.0)
    retain = 1.0 - decay
    for _ in range(steps):
        state.voxels = state.voxels * retain + drive.voxels * decay
        state.resonance_decay = state.resonance_decay * retain + drive_decay * decay
        state.harmonics = state.harmonics * (1.0 - blend) + src * blend


# ----------------------------------------------------------------------------------------------
# Feedback events (zeta)
# ----------------------------------------------------------------------------------------------

_zeta_log = logging.getLogger("spiraltorch.softlogic.zeta")


class ZetaFeedback:
    """Emits SoftLogic feedback metrics as structured log events and keeps them for export."""

    def __init__(self, run_id: str, export_path: str, metrics: Sequence[str] = ()):
        self.run_id, self.export_path, self.metrics = run_id, export_path, list(metrics)
        self.events: List[Dict[str, Any]] = []

    @classmethod
    def from_block(cls, run_id: str, block) -> "ZetaFeedback":
        return cls(run_id, getattr(block, "export_path", ""), getattr(block, "metrics", ()))

    def _emit(self, record: Dict[str, Any]) -> None:
        record = {"run": self.run_id, "export": self.export_path, **record}
        self.events.append(record)
        _zeta_log.info(json.dumps(record, sort_keys=True))

    def emit_numeric(self, metric_name: str, value: float) -> None:
        self._emit({"metric": metric_name, "value": float(value)})

    def emit_pattern(self, metric_name: str, pattern: str) -> None:
        self._emit({"metric": metric_name, "pattern": str(pattern)})

    def emit_phase_deviation(self, value: float) -> None:
        self.emit_numeric("phase_deviation", value)

    def emit_collapse_resonance(self, pattern: str) -> None:
        self.emit_pattern("collapse_resonance", pattern)

    def emit_kernel_cache_hits(self, hits: int) -> None:
        self.emit_numeric("kernel_cache_hits", float(hits))

    def flush(self) -> None:
        """Appends buffered events as JSON lines to ``export_path`` when one is set."""
        if self.export_path and self.events:
            with open(self.export_path, "a", encoding="utf-8") as fh:
                for e in self.events:
                    fh.write(json.dumps(e, sort_keys=True) + "\n")
        self.events.clear()


# ----------------------------------------------------------------------------------------------
# Key/value store with the Redis helper surface
# ----------------------------------------------------------------------------------------------


@dataclass
class Choice:
    """Rank-k kernel choice shared between tuners (same fields as the reference record)."""

    use_2ce: bool = False
    wg: int = 256
    kl: int = 32
    ch: int = 8192
    algo_topk: int = 0
    ctile: int = 0
    mode_midk: int = 0
    mode_bottomk: int = 0
    tile_cols: int = 0
    radix: int = 0
    segments: int = 0


class KvError(RuntimeError):
    pass


class MemoryKv:
    """Thread-safe in-process key/value store implementing the commands the framework's heuristics
    use (strings with TTL and NX, counters, lists, hashes, JSON helpers, pipelines).  A ``redis://``
    URL is accepted by :func:`connect` only when the ``redis`` client package is importable."""

    def __init__(self, clock: Callable[[], float] = time.monotonic):
        self._d: Dict[str, Any] = {}
        self._exp: Dict[str, float] = {}
        self._lock = threading.RLock()
        self._clock = clock

    def _live(self, key: str) -> bool:
        t = self._exp.get(key)
        if t is not None and self._clock() >= t:
            self._d.pop(key, None)
            self._exp.pop(key, None)
        return key in self._d

    # strings
    def get(self, key: str):
        with self._lock:
            return self._d[key] if self._live(key) else None

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value
            self._exp.pop(key, None)

    def set_ex(self, key: str, value, seconds: float) -> None:
        with self._lock:
            self._d[key] = value
            self._exp[key] = self._clock() + seconds

    def set_nx(self, key: str, value) -> bool:
        with self._lock:
            if self._live(key):
                return False
            self.set(key, value)
            return True

    def getset(self, key: str, value):
        with self._lock:
            old = self.get(key)
            self.set(key, value)
            return old

    def delete(self, key: str) -> int:
        with self._lock:
            live = self._live(key)
            self._d.pop(key, None)
            self._exp.pop(key, None)
            return int(live)

    del_ = delete

    def exists(self, key: str) -> bool:
        with self._lock:
            return self._live(key)

    def expire(self, key: str, seconds: float) -> bool:
        with self._lock:
            if not self._live(key):
                return False
            self._exp[key] = self._clock() + seconds
            return True

    def ttl(self, key: str) -> int:
        """-2 for a missing key, -1 for a key without expiry, else whole seconds left."""
        with self._lock:
            if not self._live(key):
                return -2
            t = self._exp.get(key)
            return -1 if t is None else max(0, int(math.ceil(t - self._clock())))

    def incr_by(self, key: str, amount):
        with self._lock:
            cur = self.get(key) or 0
            if not isinstance(cur, (int, float)):
                raise KvError(f"value at {key!r} is not numeric")
            self._d[key] = cur + amount
            return self._d[key]

    # lists
    def _list(self, key: str) -> list:
        if not self._live(key):
            self._d[key] = []
        v = self._d[key]
        if not isinstance(v, list):
            raise KvError(f"value at {key!r} is not a list")
        return v

    def lpush(self, key: str, *values) -> int:
        with self._lock:
            lst = self._list(key)
            for v in values:
                lst.insert(0, v)
            return len(lst)

    def rpush(self, key: str, *values) -> int:
        with self._lock:
            lst = self._list(key)
            lst.extend(values)
            return len(lst)

    @staticmethod
    def _range(n: int, start: int, stop: int) -> slice:
        s = start + n if start < 0 else start
        e = stop + n if stop < 0 else stop
        return slice(max(s, 0), max(e + 1, 0))

    def lrange(self, key: str, start: int, stop: int) -> list:
        with self._lock:
            lst = self._list(key) if self._live(key) else []
            return list(lst[self._range(len(lst), start, stop)])

    def ltrim(self, key: str, start: int, stop: int) -> None:
        with self._lock:
            if self._live(key):
                lst = self._list(key)
                self._d[key] = lst[self._range(len(lst), start, stop)]

    # hashes
    def _hash(self, key: str) -> dict:
        if not self._live(key):
            self._d[key] = {}
        v = self._d[key]
        if not isinstance(v, dict):
            raise KvError(f"value at {key!r} is not a hash")
        return v

    def hset(self, key: str, field_name: str, value) -> bool:
        with self._lock:
            h = self._hash(key)
            new = field_name not in h
            h[field_name] = value
            return new

    def hget(self, key: str, field_name: str):
        with self._lock:
            return self._hash(key).get(field_name) if self._live(key) else None

    def hdel(self, key: str, field_name: str) -> int:
        with self._lock:
            return int(self._hash(key).pop(field_name, None) is not None) if self._live(key) else 0

    def hgetall(self, key: str) -> dict:
        with self._lock:
            return dict(self._hash(key)) if self._live(key) else {}

    # JSON helpers
    def set_json(self, key: str, value, *, ex: Optional[float] = None, nx: bool = False) -> bool:
        payload = json.dumps(value, sort_keys=True)
        with self._lock:
            if nx and self._live(key):
                return False
            if ex is not None:
                self.set_ex(key, payload, ex)
            else:
                self.set(key, payload)
            return True

    def get_json(self, key: str):
        raw = self.get(key)
        if raw is None:
            return None
        try:
            return json.loads(raw)
        except (TypeError, ValueError) as exc:
            raise KvError(f"value at {key!r} is not JSON: {exc}") from exc

    def get_or_set_json(self, key: str, default: Callable[[], Any], *, ex: Optional[float] = None):
        with self._lock:
            cur = self.get_json(key)
            if cur is not None:
                return cur
            value = default()
            self.set_json(key, value, ex=ex)
            return value

    def lpush_json(self, key: str, value) -> int:
        return self.lpush(key, json.dumps(value, sort_keys=True))

    def rpush_json(self, key: str, value) -> int:
        return self.rpush(key, json.dumps(value, sort_keys=True))

    def lrange_json(self, key: str, start: int, stop: int) -> list:
        return [json.loads(v) for v in self.lrange(key, start, stop)]

    # tuning choices
    def set_choice(self, key: str, choice: Choice, *, ex: Optional[float] = None, nx: bool = False) -> bool:
        return self.set_json(key, asdict(choice), ex=ex, nx=nx)

    def get_choice(self, key: str) -> Optional[Choice]:
        d = self.get_json(key)
        return None if d is None else Choice(**d)

    def get_or_set_choice(self, key: str, default: Callable[[], Choice]) -> Choice:
        return Choice(**self.get_or_set_json(key, lambda: asdict(default())))

    def push_choice(self, key: str, choice: Choice, *, left: bool = True, keep: Optional[int] = None) -> int:
        n = (self.lpush_json if left else self.rpush_json)(key, asdict(choice))
        if keep is not None:
            self.ltrim(key, 0, keep - 1) if left else self.ltrim(key, -keep, -1)
            n = min(n, keep)
        return n

    def lrange_choice(self, key: str, start: int, stop: int) -> List[Choice]:
        return [Choice(**d) for d in self.lrange_json(key, start, stop)]

    def pipeline(self, build: Callable[["MemoryKv"], Any]):
        """Runs ``build(self)`` atomically with respect to other users of the store."""
        with self._lock:
            return build(self)


_stores: Dict[str, MemoryKv] = {}
_stores_lock = threading.Lock()


def connect(url: str = "memory://default") -> MemoryKv:
    """``memory://<name>`` returns the process-wide store of that name.  Other schemes need a client
    package that is not part of this build and raise :class:`KvError`."""
    if not url.startswith("memory://"):
        raise KvError(f"no client for {url.split(':', 1)[0]!r} URLs in this build; use memory://<name>")
    with _stores_lock:
        return _stores.setdefault(url, MemoryKv())


# ----------------------------------------------------------------------------------------------
# Sparse-problem tuning profile
# ----------------------------------------------------------------------------------------------


def wilson_lower_bound(wins: int, trials: int, z: float = 1.96) -> float:
    if trials <= 0:
        return 0.0
    n = float(trials)
    p = wins / n
    z2 = z * z
    denom = 1.0 + z2 / n
    center = p + z2 / (2.0 * n)
    margin = math.sqrt(p * (1.0 - p) / n + z2 / (4.0 * n * n)) * z
    return (center - margin) / denom


class ProblemProfile:
    """Derived statistics of a sparse linear problem and the launch hints computed from them."""

    def __init__(self, rows: int, cols: int, nnz: int, subgroup: bool = True):
        self.rows, self.cols, self.nnz, self.subgroup = max(rows, 1), max(cols, 1), max(nnz, 1), subgroup
        self.density = min(max(self.nnz / float(self.rows * self.cols), 1e-6), 1.0)
        self.aspect = max(self.rows, self.cols) / float(min(self.rows, self.cols))
        self.curvature = max(math.log2(max(self.rows, self.cols)), 1.0)
        self.diag_ratio = 1.0
        self.mean_row_nnz = max(self.nnz / float(self.rows), 1.0)
        self.row_nnz_stddev = max(math.sqrt(self.mean_row_nnz), 0.5)
        self.max_row_nnz = int(math.ceil(self.mean_row_nnz))
        self.min_row_nnz = int(max(math.floor(self.mean_row_nnz), 1))
        self.bandwidth_hint = max(min(self.rows, self.cols), 1)
        self.bandwidth_peak = self.bandwidth_hint
        self.bandwidth_stddev = max(self.bandwidth_hint * 0.35, 1.0)

    @classmethod
    def from_sparse(cls, matrix: torch.Tensor, subgroup: bool = True) -> "ProblemProfile":
        """Measures a dense or sparse-COO matrix: per-row counts, diagonal hits and bandwidths."""
        dense = matrix.to_dense() if matrix.is_sparse else matrix
        nz = dense != 0
        rows, cols = dense.shape
        prof = cls(rows, cols, int(nz.sum()), subgroup)
        per_row = nz.sum(dim=1).float()
        if per_row.numel():
            prof.mean_row_nnz = max(float(per_row.mean()), 1.0)
            prof.row_nnz_stddev = max(float(per_row.std(unbiased=False)), 0.5) if rows > 1 else 0.5
            prof.max_row_nnz, prof.min_row_nnz = int(per_row.max()), int(per_row.min())
            idx = torch.arange(cols, device=dense.device).expand(rows, cols)
            lo = torch.where(nz, idx, torch.full_like(idx, cols)).min(dim=1).values
            hi = torch.where(nz, idx, torch.full_like(idx, -1)).max(dim=1).values
            bw = (hi - lo + 1).clamp_min(0).float()[per_row > 0]
            if bw.numel():
                prof.bandwidth_hint = max(int(bw.mean().round()), 1)
                prof.bandwidth_peak = int(bw.max())
                prof.bandwidth_stddev = max(float(bw.std(unbiased=False)), 1.0) if bw.numel() > 1 else 1.0
            d = min(rows, cols)
            prof.diag_ratio = float(nz[torch.arange(d), torch.arange(d)].float().mean()) if d else 1.0
        return prof

    def sparsity_index(self) -> float:
        return 1.0 - self.density

    def bandwidth_spread(self) -> float:
        return self.bandwidth_stddev / max(float(self.bandwidth_hint), 1.0)

    def row_nnz_spread(self) -> float:
        return self.row_nnz_stddev / max(self.mean_row_nnz, 1.0)

    def row_nnz_imbalance(self) -> float:
        return (self.max_row_nnz - self.min_row_nnz) / max(self.mean_row_nnz, 1.0)

    def density_class(self) -> str:
        d = self.density
        return "ultra_sparse" if d < 0.03 else "sparse" if d < 0.10 else "moderate" if d < 0.30 else "dense"

    def aspect_class(self) -> str:
        if self.rows == self.cols or self.aspect < 1.2:
            return "square"
        return "wide" if self.cols > self.rows else "tall"

    def jacobi_hint(self) -> int:
        return {"ultra_sparse": 0, "sparse": 1, "moderate": 2, "dense": 3}[self.density_class()]

    def lane_hint(self) -> int:
        """Threads per block for a row kernel over this problem."""
        if self.bandwidth_peak >= 14_000 or self.bandwidth_hint >= 8_000:
            return 512
        if self.bandwidth_hint <= 2_000 and self.mean_row_nnz < 12.0:
            return 128
        if self.bandwidth_spread() > 0.4:
            return 512
        if self.subgroup:
            return 512 if self.cols >= 8192 else 256
        if self.rows <= 16:
            return 128
        return 256 if self.cols <= 4096 else 512

    def tile_hint(self) -> int:
        c, bw = self.cols, self.bandwidth_hint
        if c <= 4096 and bw <= 4096:
            tile = 4096 if self.subgroup else 2048
        elif 4097 <= c <= 16384 and bw <= 8192:
            tile = 8192 if self.subgroup else 4096
        elif bw <= 4096:
            tile = 8192
        elif 16385 <= c <= 65536 and bw <= 12_000:
            tile = 8192
        else:
            tile = 16384
        if self.bandwidth_peak >= 14_000:
            tile = max(tile, 8192)
        spread = self.bandwidth_spread()
        if spread > 0.4:
            tile = max(tile, 8192)
        elif spread < 0.25 and self.bandwidth_peak < 4000:
            tile = min(max(tile, 4096), 8192)
        return tile

    def fractional_alpha(self) -> float:
        alpha = (math.sqrt(self.density) * 0.65 + 0.25) * (1.0 - 0.05 / self.curvature)
        return min(max(alpha, 0.15), 0.95)


class SoftRuleLearner:
    """Keeps win/trial counts per soft rule and accepts a rule into the rule book once the Wilson
    lower bound of its win rate clears a threshold (crates/st-amg/src/sr_learn.rs:194-292)."""

    def __init__(self, z: float = 1.96, threshold: float = 0.55):
        self.z, self.threshold = z, threshold
        self.stats: Dict[str, List[int]] = {}
        self.accepted: List[str] = []

    def observe(self, rule: str, won: bool) -> float:
        s = self.stats.setdefault(rule, [0, 0])
        s[0] += int(won)
        s[1] += 1
        lb = wilson_lower_bound(s[0], s[1], self.z)
        if lb >= self.threshold and rule not in self.accepted:
            self.accepted.append(rule)
        return lb

    def on_conversation(self, consensus_rules: Sequence[str], other_proposals: Sequence[Sequence[str]],
                        won: bool) -> List[str]:
        """Consensus rules take the outcome; rules that were proposed but outvoted take the opposite."""
        for r in consensus_rules:
            self.observe(r, won)
        for proposal in other_proposals:
            for r in proposal:
                if r not in consensus_rules:
                    self.observe(r, not won)
        return list(self.accepted)


# ----------------------------------------------------------------------------------------------
# Signal-capture studio
# ----------------------------------------------------------------------------------------------


class StudioError(RuntimeError):
    pass


@dataclass
class SignalCaptureConfig:
    sample_rate_hz: float
    channels: List[str] = field(default_factory=list)
    history_limit: int = 512

    def __post_init__(self):
        self.sample_rate_hz = max(float(self.sample_rate_hz), 1.0)
        self.history_limit = max(int(self.history_limit), 1)

    def allows(self, channel: str) -> bool:
        return not self.channels or channel in self.channels


@dataclass
class PulseSnapshot:
    blocks: int
    mean: float
    standard_error: float
    z_score: float
    band_energy: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    z_bias: float = 0.0

    def magnitude(self) -> float:
        return abs(self.z_score)

    @classmethod
    def from_samples(cls, samples: torch.Tensor, block: int = 16) -> "PulseSnapshot":
        """Block-mean z statistic of a 1-D signal and its low / mid / high spectral energy thirds."""
        x = samples.detach().flatten().float()
        n = (x.numel() // block) * block
        if n == 0:
            raise StudioError("not enough samples for one block")
        means = x[:n].view(-1, block).mean(dim=1)
        mean = float(means.mean())
        se = float(means.std(unbiased=True) / math.sqrt(means.numel())) if means.numel() > 1 else 0.0
        z = mean / se if se > 0 else 0.0
        power = torch.fft.rfft(x[:n]).abs().square()[1:]
        thirds = [float(c.sum()) for c in torch.tensor_split(power, 3)] if power.numel() >= 3 else [0.0] * 3
        total = sum(thirds) or 1.0
        bands = tuple(t / total for t in thirds)
        return cls(int(means.numel()), mean, se, z, bands, float(bands[0] - bands[2]))


@dataclass
class RecordedPulse:
    channel: str
    pulse: PulseSnapshot
    timestamp: float


@dataclass
class OverlayGlyph:
    glyph: str
    intensity: float

    def __post_init__(self):
        self.intensity = max(float(self.intensity), 0.0)


@dataclass
class OverlayFrame:
    channel: str
    timestamp: float
    glyphs: List[OverlayGlyph] = field(default_factory=list)

    @classmethod
    def from_pairs(cls, channel: str, timestamp: float, pairs: Iterable[Tuple[str, float]]) -> "OverlayFrame":
        return cls(channel, timestamp, [OverlayGlyph(g, i) for g, i in pairs])

    def push_glyph(self, glyph: OverlayGlyph) -> None:
        self.glyphs.append(glyph)

    def extend_tags(self, tags: Iterable[str], base_intensity: float) -> None:
        have = {g.glyph for g in self.glyphs}
        for t in tags:
            if t not in have:
                self.glyphs.append(OverlayGlyph(t, base_intensity))
                have.add(t)


class SignalCaptureSession:
    def __init__(self, config: SignalCaptureConfig):
        self.config = config
        self.history: Deque[RecordedPulse] = deque(maxlen=config.history_limit)

    def ingest(self, channel: str, pulse: PulseSnapshot, timestamp: Optional[float] = None) -> RecordedPulse:
        if not self.config.allows(channel):
            raise StudioError(f"unknown channel {channel!r}")
        rec = RecordedPulse(channel, pulse, time.time() if timestamp is None else timestamp)
        self.history.append(rec)
        return rec

    def records(self) -> List[RecordedPulse]:
        return list(self.history)


class QuantumRealityStudio:
    """Captures pulses per channel, composes an overlay frame for each (dominant narrative tag, else
    the channel's fallback tag, else the channel name; intensity = narrative intensity or |z|), hands
    frames to sinks and exports a storyboard."""

    def __init__(self, config: SignalCaptureConfig, fallback_tags: Optional[Dict[str, List[str]]] = None):
        self.session = SignalCaptureSession(config)
        self.fallback_tags = dict(fallback_tags or {})
        self.frames: Deque[Tuple[RecordedPulse, OverlayFrame]] = deque(maxlen=config.history_limit)
        self.sinks: List[Callable[[RecordedPulse, OverlayFrame], None]] = []

    def register_sink(self, sink: Callable[[RecordedPulse, OverlayFrame], None]) -> None:
        self.sinks.append(sink)

    def sink_count(self) -> int:
        return len(self.sinks)

    def ingest(self, channel: str, pulse: PulseSnapshot, narrative: Optional[Dict[str, float]] = None,
               timestamp: Optional[float] = None) -> OverlayFrame:
        rec = self.session.ingest(channel, pulse, timestamp)
        fallback = self.fallback_tags.get(channel)
        if narrative:
            glyph, intensity = max(narrative.items(), key=lambda kv: kv[1])
            intensity = max(float(intensity), rec.pulse.magnitude()) if intensity <= 0 else float(intensity)
        else:
            glyph = fallback[0] if fallback else channel
            intensity = rec.pulse.magnitude()
        frame = OverlayFrame.from_pairs(channel, rec.timestamp, [(glyph, intensity)])
        self.frames.append((rec, frame))
        for sink in self.sinks:
            try:
                sink(rec, frame)
            except Exception as exc:                       # a failing sink must not lose the capture
                raise StudioError(f"sink failed: {exc}") from exc
        return frame

    def stitch_narrative_tags(self, overlay: OverlayFrame, tags: Iterable[str]) -> OverlayFrame:
        base = max((g.intensity for g in overlay.glyphs), default=0.0)
        overlay.extend_tags(tags, base)
        return overlay

    def export_storyboard(self) -> Dict[str, Any]:
        frames = []
        for ordinal, (rec, frame) in enumerate(self.frames):
            frames.append({"ordinal": ordinal, "channel": rec.channel, "timestamp": rec.timestamp,
                           "z_score": rec.pulse.z_score, "band_energy": list(rec.pulse.band_energy),
                           "glyphs": [asdict(g) for g in frame.glyphs]})
        return {"frames": frames, "channels": sorted({f["channel"] for f in frames})}

    def export_storyboard_grouped(self) -> Dict[str, Any]:
        grouped: Dict[str, list] = {}
        for f in self.export_storyboard()["frames"]:
            grouped.setdefault(f["channel"], []).append(f)
        return {"channels": grouped}

    def export_storyboard_ndjson(self) -> str:
        return "\n".join(json.dumps(f, sort_keys=True) for f in self.export_storyboard()["frames"])
