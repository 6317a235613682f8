"""Probabilistic lane selection and cross-rank lane consensus.

A *lane* is a launch-width choice in ``[1, 4096]``.  Ranks (or tuners) vote with weights; the votes
form a validated distribution from which one lane is drawn deterministically from a seed, or reduced
to a consensus lane (weighted mean rounded half up, or weighted median).  Invalid inputs are
rejected, never clamped or repaired.  Sample and report records carry the reference's kind /
contract-version strings and SHA-256 commitments, so they can be compared across implementations:
crates/st-core/src/distributed/prob_params.rs:20-40 (constants), :98-183 (construction),
:231-348 (sampling), :435-650 (consensus), :1003-1016 (tolerance, splitmix64 draw), :1122-1145 (digests).
"""
from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

LANE_MIN, LANE_MAX = 1, 4096
LANE_SAMPLE_KIND = "spiraltorch.distributed_lane_sample"
LANE_SAMPLE_CONTRACT_VERSION = "spiraltorch.distributed_lane_sample.v1"
LANE_CONSENSUS_REPORT_KIND = "spiraltorch.lane_consensus_report"
LANE_CONSENSUS_REPORT_CONTRACT_VERSION = "spiraltorch.lane_consensus_report.v1"
LANE_SAMPLE_RNG_ALGORITHM = "splitmix64_u53_v1"
SEMANTIC_OWNER = "spiraltorch_b200.distributed.lanes"
_DIST_DOMAIN = b"spiraltorch.lane_distribution.v1\0"
_OUT_DOMAIN = b"spiraltorch.lane_consensus.output.v1\0"
_M64 = (1 << 64) - 1


class LaneProbabilityError(ValueError):
    pass


def probability_sum_tolerance(n: int) -> float:
    return 1.0e-12 + n * 2.220446049250313e-16 * 8.0


def canonical_lane_draw(seed: int) -> float:
    """splitmix64 finaliser of ``seed``; the top 53 bits become a double in [0, 1)."""
    v = (seed + 0x9E3779B97F4A7C15) & _M64
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & _M64
    v ^= v >> 31
    return (v >> 11) * (1.0 / float(1 << 53))


def _check_lane(lane: int) -> int:
    if not isinstance(lane, int) or isinstance(lane, bool) or not LANE_MIN <= lane <= LANE_MAX:
        raise LaneProbabilityError(f"lane {lane!r} is outside [{LANE_MIN}, {LANE_MAX}]")
    return lane


def _check_positive(field: str, position: int, value: float) -> None:
    if not (isinstance(value, (int, float)) and math.isfinite(value) and value > 0):
        raise LaneProbabilityError(f"{field}[{position}] must be positive and finite, got {value!r}")


def _ksum(values: Iterable[float]) -> float:
    total, comp = 0.0, 0.0
    for v in values:
        y = v - comp
        t = total + y
        comp = (t - total) - y
        total = t
    return total


class LaneDistribution:
    """Validated, lane-sorted, normalised distribution over lanes."""

    def __init__(self, entries: List[Tuple[int, float]]):
        self.entries = entries

    @classmethod
    def from_probabilities(cls, entries: Sequence[Tuple[int, float]]) -> "LaneDistribution":
        entries = list(entries)
        if not entries:
            raise LaneProbabilityError("distribution support is empty")
        if len(entries) > LANE_MAX:
            raise LaneProbabilityError(f"support of {len(entries)} lanes exceeds {LANE_MAX}")
        seen = set()
        for pos, (lane, p) in enumerate(entries):
            _check_lane(lane)
            if lane in seen:
                raise LaneProbabilityError(f"duplicate lane {lane}")
            seen.add(lane)
            _check_positive("probability", pos, p)
        entries.sort(key=lambda e: e[0])
        mass = _ksum(p for _, p in entries)
        tol = probability_sum_tolerance(len(entries))
        if abs(mass - 1.0) > tol:
            raise LaneProbabilityError(f"probability mass {mass!r} differs from 1 by more than {tol:.3e}")
        return cls([(lane, p / mass) for lane, p in entries])

    @classmethod
    def from_weights(cls, entries: Iterable[Tuple[int, float]]) -> "LaneDistribution":
        entries = list(entries)
        if not entries:
            raise LaneProbabilityError("distribution support is empty")
        seen = set()
        for pos, (lane, w) in enumerate(entries):
            _check_lane(lane)
            if lane in seen:
                raise LaneProbabilityError(f"duplicate lane {lane}")
            seen.add(lane)
            _check_positive("weight", pos, w)
        entries.sort(key=lambda e: e[0])
        wmax = max(w for _, w in entries)
        scaled = [w / wmax for _, w in entries]
        total = _ksum(scaled)
        return cls.from_probabilities([(lane, s / total) for (lane, _), s in zip(entries, scaled)])

    def mass(self) -> float:
        return _ksum(p for _, p in self.entries)

    def entropy(self) -> float:
        return _ksum(-p * math.log(p) for _, p in self.entries)

    def effective_sample_size(self) -> float:
        return 1.0 / _ksum(p * p for _, p in self.entries)

    def sha256(self) -> str:
        h = hashlib.sha256()
        h.update(_DIST_DOMAIN)
        h.update(struct.pack("<Q", len(self.entries)))
        for lane, p in self.entries:
            h.update(struct.pack("<i", lane))
            h.update(struct.pack("<d", p))                 # IEEE-754 bits, little endian
        return h.hexdigest()

    def _index_for_draw(self, draw: float) -> int:
        if not (math.isfinite(draw) and 0.0 <= draw < 1.0):
            raise LaneProbabilityError("draw must be finite in [0, 1)")
        threshold = draw * self.mass()
        cumulative = 0.0
        for i, (_, p) in enumerate(self.entries):
            cumulative += p
            if threshold < cumulative:
                return i
        return len(self.entries) - 1

    def sample(self, seed: int) -> Dict[str, object]:
        if not 0 <= seed <= _M64:
            raise LaneProbabilityError("seed must fit in 64 unsigned bits")
        draw = canonical_lane_draw(seed)
        idx = self._index_for_draw(draw)
        lane, p = self.entries[idx]
        return {"kind": LANE_SAMPLE_KIND, "contract_version": LANE_SAMPLE_CONTRACT_VERSION,
                "semantic_owner": SEMANTIC_OWNER, "semantic_backend": "python",
                "rng_algorithm": LANE_SAMPLE_RNG_ALGORITHM, "seed": str(seed), "support_size": str(len(self.entries)),
                "support_index": str(idx), "draw": draw, "params": {"lane": lane}, "probability": p,
                "distribution_sha256": self.sha256(), "committed": True}

    def validate_sample(self, sample: Dict[str, object]) -> None:
        """Recomputes the draw and the selection; any mismatch raises."""
        if sample.get("kind") != LANE_SAMPLE_KIND or sample.get("contract_version") != LANE_SAMPLE_CONTRACT_VERSION:
            raise LaneProbabilityError("sample kind / contract version mismatch")
        if sample.get("distribution_sha256") != self.sha256():
            raise LaneProbabilityError("sample was drawn from a different distribution")
        expect = self.sample(int(sample["seed"]))
        for key in ("support_size", "support_index", "draw", "params", "probability"):
            if sample.get(key) != expect[key]:
                raise LaneProbabilityError(f"sample field {key!r} does not match the recomputed draw")


def parse_policy(value: str) -> str:
    v = value.strip().lower()
    if v in ("mean", "weighted_mean"):
        return "weighted_mean"
    if v in ("median", "weighted_median"):
        return "weighted_median"
    raise LaneProbabilityError(f"unknown lane consensus policy {value!r}")


def consensus_lane_params(dist: LaneDistribution, policy: str = "weighted_median") -> Dict[str, object]:
    """Returns ``{"params": {"lane": L}, "report": {...}}`` for the chosen policy."""
    policy = parse_policy(policy)
    if policy == "weighted_mean":
        mean = _ksum(lane * p for lane, p in dist.entries) / dist.mass()
        if not LANE_MIN <= mean <= LANE_MAX:
            raise LaneProbabilityError(f"derived lane {mean} is out of range")
        lane = int(math.floor(mean + 0.5))
    else:
        midpoint, cumulative, lane = dist.mass() * 0.5, 0.0, dist.entries[-1][0]
        for ln, p in dist.entries:
            cumulative += p
            if cumulative >= midpoint:
                lane = ln
                break
    _check_lane(lane)
    input_sha = dist.sha256()
    h = hashlib.sha256()
    h.update(_OUT_DOMAIN)
    h.update(policy.encode())
    h.update(b"\0")
    h.update(struct.pack("<i", lane))
    h.update(input_sha.encode())
    report = {"kind": LANE_CONSENSUS_REPORT_KIND, "contract_version": LANE_CONSENSUS_REPORT_CONTRACT_VERSION,
              "semantic_owner": SEMANTIC_OWNER, "semantic_backend": "python", "policy": policy,
              "support_size": str(len(dist.entries)), "probability_mass": dist.mass(), "entropy": dist.entropy(),
              "effective_sample_size": dist.effective_sample_size(), "selected_lane": lane,
              "input_sha256": input_sha, "output_sha256": h.hexdigest(), "committed": True}
    return {"params": {"lane": lane}, "report": report}


def merge_votes(votes: Iterable[Tuple[int, float]]) -> LaneDistribution:
    """Sums the weights of repeated lanes (several ranks voting for the same lane) and normalises."""
    acc: Dict[int, float] = {}
    for pos, (lane, w) in enumerate(votes):
        _check_lane(lane)
        _check_positive("vote_weight", pos, w)
        acc[lane] = acc.get(lane, 0.0) + w
    return LaneDistribution.from_weights(acc.items())


def distributed_consensus(local_votes: Sequence[Tuple[int, float]], group=None, policy: str = "weighted_median",
                          max_votes: int = 16) -> Dict[str, object]:
    """Every rank contributes up to ``max_votes`` (lane, weight) pairs; the pairs are all-gathered
    through ``torch.distributed`` (any backend) and every rank derives the same consensus, which the
    matching output digests prove.  Without an initialised process group the local votes decide."""
    import torch
    import torch.distributed as dist
    votes = list(local_votes)[:max_votes]
    if dist.is_available() and dist.is_initialized():
        world = dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
        buf = torch.zeros(max_votes, 2, dtype=torch.float64, device=dev)
        for i, (lane, w) in enumerate(votes):
            buf[i, 0], buf[i, 1] = float(lane), float(w)
        gathered = [torch.zeros_like(buf) for _ in range(world)]
        dist.all_gather(gathered, buf, group=group)
        votes = [(int(l), float(w)) for g in gathered for l, w in g.cpu().tolist() if w > 0]
    return consensus_lane_params(merge_votes(votes), policy)
