"""Device capability record and the launch-shape heuristics derived from it.

Parity: crates/st-core/src/backend/device_caps.rs:45-600 (`BackendKind`, `DeviceCaps`,
`align_workgroup`, `occupancy_score`, `preferred_tile`, `recommended_workgroup`,
`recommended_tiles`, `prefers_two_stage_with_rows`).

Only two backends exist in this build — `cuda` (one B200, sm_100a) and `cpu` (the oracle).  The
reference's other labels (`wgpu`, `mps`, `hip`) parse, so configuration files written for it are
reported clearly, and resolve to an error that says the backend is not part of this build.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

B200_SM_COUNT = 148
B200_SMEM_PER_CTA = 227 * 1024
B200_TMEM_COLUMNS = 512

_KNOWN = ("wgpu", "mps", "cuda", "hip", "cpu")
_ALIASES = {"gpu": "cuda", "nvidia": "cuda", "b200": "cuda", "auto": "cuda", "webgpu": "wgpu", "metal": "mps", "rocm": "hip"}


class DeviceCapsError(ValueError):
    pass


def parse_backend(label: str) -> str:
    """Normalise a backend label; unknown labels raise, known-but-absent ones are kept so the
    caller can report them (`DeviceCaps.for_backend` refuses them)."""
    l = _ALIASES.get(label.strip().lower(), label.strip().lower())
    if l not in _KNOWN:
        raise DeviceCapsError(f"unknown backend kind {label!r}; expected one of {', '.join(_KNOWN)}")
    return l


def _align_up(v: int, a: int) -> int:
    return -(-v // a) * a


@dataclass(frozen=True)
class DeviceCaps:
    backend: str = "cpu"
    subgroup: bool = False
    lane_width: int = 1
    max_workgroup: int = 1
    shared_mem_per_workgroup: Optional[int] = None
    sm_count: int = 1

    # -- constructors ---------------------------------------------------------------------------
    @classmethod
    def cuda(cls, lane_width: int = 32, max_block: int = 1024, shared_mem_per_block: Optional[int] = B200_SMEM_PER_CTA,
             sm_count: int = B200_SM_COUNT) -> "DeviceCaps":
        return cls("cuda", True, max(lane_width, 1), max(max_block, 1), shared_mem_per_block, sm_count).validate()

    b200 = cuda

    @classmethod
    def cpu(cls) -> "DeviceCaps":
        return cls("cpu", False, 1, 256, None, 1)

    @classmethod
    def for_backend(cls, label: str) -> "DeviceCaps":
        b = parse_backend(label)
        if b == "cuda":
            return cls.cuda()
        if b == "cpu":
            return cls.cpu()
        raise DeviceCapsError(f"backend {b!r} is not part of this build (sm_100a CUDA and the CPU oracle only)")

    @classmethod
    def probe(cls, device=None) -> "DeviceCaps":
        """Caps of a live CUDA device (lane width, block limit, opt-in shared memory, SM count); CPU
        caps when no GPU is visible."""
        import torch
        if not torch.cuda.is_available():
            return cls.cpu()
        p = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
        smem = getattr(p, "shared_memory_per_block_optin", None) or B200_SMEM_PER_CTA
        return cls.cuda(p.warp_size, p.max_threads_per_block if hasattr(p, "max_threads_per_block") else 1024, int(smem),
                        p.multi_processor_count)

    def validate(self) -> "DeviceCaps":
        if self.lane_width <= 0:
            raise DeviceCapsError("lane_width must be positive")
        if self.max_workgroup < self.lane_width:
            raise DeviceCapsError(f"max_workgroup {self.max_workgroup} is below the lane width {self.lane_width}")
        if self.shared_mem_per_workgroup is not None and self.shared_mem_per_workgroup <= 0:
            raise DeviceCapsError("shared memory budget must be positive when given")
        return self

    def with_subgroup(self, subgroup: bool) -> "DeviceCaps":
        return replace(self, subgroup=subgroup)

    def with_max_workgroup(self, n: int) -> "DeviceCaps":
        return replace(self, max_workgroup=max(n, 1))

    def with_shared_mem(self, nbytes: Optional[int]) -> "DeviceCaps":
        return replace(self, shared_mem_per_workgroup=nbytes)

    # -- block shapes ---------------------------------------------------------------------------
    def _align(self, value: int, ceiling: int) -> int:
        lanes = max(self.lane_width, 1)
        top = max(ceiling, lanes)
        a = _align_up(min(max(value, lanes), top), lanes)
        if a > top:
            a = top - top % lanes
        return max(a, lanes)

    def align_workgroup(self, requested: int) -> int:
        """Round a requested block size to whole warps inside `[lane_width, max_workgroup]`."""
        return self._align(requested, self.max_workgroup)

    def occupancy_score(self, requested: int) -> float:
        if requested == 0:
            return 0.0
        lanes = max(self.lane_width, 1)
        top = max(self.max_workgroup, lanes)
        a = self.align_workgroup(requested)
        score = 0.6 * min(a, top) / top + 0.4 * (1.0 - min(abs(a - requested) / max(a, 1), 0.6))
        if self.subgroup:
            score *= min(max(a // lanes, 1) / 4.0, 1.25)
        return min(max(score, 0.0), 1.25)

    def recommended_workgroup(self, rows: int = 0) -> int:
        lanes = max(self.lane_width, 1)
        top = max(self.max_workgroup, lanes)
        target = min(max(lanes * (8 if self.subgroup else 4), min(64, top)), top)
        if 0 < rows < target:
            return min(max(_align_up(rows, lanes), lanes), target)
        return target

    # -- tiles ----------------------------------------------------------------------------------
    def preferred_tile(self, cols: int, hint: int = 0) -> int:
        seed = hint or (4096 if cols > 131072 else 2048 if cols > 65536 else 1024 if cols > 8192 else 512 if cols > 4096 else 256)
        return self._align(seed, 1024 if self.backend == "cpu" else 8192)

    def preferred_compaction_tile(self, cols: int, hint: int = 0) -> int:
        seed = hint or (1024 if cols > 65536 else 512 if cols > 8192 else 256)
        return self._align(seed, 1024 if self.backend == "cpu" else 4096)

    def recommended_tiles(self, cols: int) -> tuple:
        """(sweep tile, compaction tile): the largest power-of-two option not above `cols`, bounded
        by block limits and by shared memory at about two fp32 values per lane."""
        lanes = max(self.lane_width, 1)
        floor = _align_up(128, lanes)
        tile = next((o for o in (16384, 8192, 4096, 2048, 1024, 512, 256) if cols >= o), 256)
        tile = max(min(_align_up(tile, lanes), max(self.max_workgroup, lanes) * lanes), floor)
        if self.shared_mem_per_workgroup is not None:
            cap = max(self.shared_mem_per_workgroup // (8 * lanes), lanes)
            tile = max(min(tile, max(_align_up(cap, lanes), lanes)), floor)
        ctile = min(1024 if cols > 65536 else 512 if cols > 8192 else 256, tile)
        if self.shared_mem_per_workgroup is not None and self.shared_mem_per_workgroup < 48 * 1024:
            ctile = min(ctile, 512)
        return tile, min(_align_up(max(ctile, 128), lanes), max(tile, lanes))

    @staticmethod
    def default_lane_quota(k: int) -> int:
        return 32 if k >= 64 else 16 if k >= 16 else 8

    def prefers_two_stage(self, cols: int, k: int, rows: int = 0) -> bool:
        """Whether a rank-k selection should split into per-tile candidates + merge."""
        lanes = max(self.lane_width, 1)
        col_heavy, k_heavy = cols > 32768, k > lanes * 4
        if rows == 0:
            return col_heavy or k_heavy
        if self.backend == "cpu":
            return col_heavy and rows > 512
        return col_heavy or (k_heavy and rows > lanes * 8)

    def persistent_grid(self, items: int, ctas_per_sm: int = 1) -> int:
        """Grid of a persistent kernel: one CTA (or `ctas_per_sm`) per SM, never more than the work."""
        return max(1, min(items, self.sm_count * max(ctas_per_sm, 1)))
