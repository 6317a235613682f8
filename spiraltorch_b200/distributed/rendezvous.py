"""In-process rendezvous with an all-reduce that fails consistently on every rank.

Semantics restated from crates/spiral-selfsup/src/trainer/distributed.rs:18-430:

* a named group (``memory://<id>``) of ``world_size`` ranks; joining twice with the same rank →
  ``DuplicateRank``; a different world size → ``WorldSizeMismatch``;
* ``all_reduce_sum(values)``: the first arrival of a round opens a new *generation* and zero-fills
  the shared buffer; every contributor adds its values; the last arrival publishes the completed
  round; the others wait on a condition variable with the remaining timeout (default 30 s);
* a contributor that runs out of time fails the round **for every rank** (``CollectiveTimeout``);
  non-finite inputs (``NonFiniteInput{rank,index}``), a non-finite sum (``NonFiniteReduction``), a
  length mismatch (``BufferLengthMismatch``) and a member that leaves during a round
  (``ParticipantLeft{rank,generation}``) are reported to every rank of that round;
* the caller's buffer is only overwritten when the round completed — never partially;
* after a failed round the group stays usable, and a rank may re-join.
"""
from __future__ import annotations

import math
import threading
import time
from typing import Optional

DEFAULT_COLLECTIVE_TIMEOUT = 30.0


class DistributedError(RuntimeError):
    kind = "DistributedError"

    def __init__(self, message: str = "", **fields):
        super().__init__(message or f"{self.kind}{fields}")
        self.fields = fields
        for k, v in fields.items():
            setattr(self, k, v)


class EmptyWorldSize(DistributedError):
    kind = "EmptyWorldSize"


class RankOutOfBounds(DistributedError):
    kind = "RankOutOfBounds"


class WorldSizeMismatch(DistributedError):
    kind = "WorldSizeMismatch"


class DuplicateRank(DistributedError):
    kind = "DuplicateRank"


class UnknownRank(DistributedError):
    kind = "UnknownRank"


class DuplicateContribution(DistributedError):
    kind = "DuplicateContribution"


class BufferLengthMismatch(DistributedError):
    kind = "BufferLengthMismatch"


class NonFiniteInput(DistributedError):
    kind = "NonFiniteInput"


class NonFiniteReduction(DistributedError):
    kind = "NonFiniteReduction"


class ParticipantLeft(DistributedError):
    kind = "ParticipantLeft"


class CollectiveTimeout(DistributedError):
    kind = "CollectiveTimeout"


class PeerTensorFailure(DistributedError):
    kind = "PeerTensorFailure"


class _Round:
    __slots__ = ("generation", "buffer", "contributors", "error", "done", "result")

    def __init__(self, generation: int, length: int):
        self.generation = generation
        self.buffer = [0.0] * length
        self.contributors: set[int] = set()
        self.error: Optional[DistributedError] = None
        self.done = False
        self.result: Optional[list[float]] = None


class _Group:
    def __init__(self, group_id: str, world_size: int):
        self.group_id, self.world_size = group_id, world_size
        self.lock = threading.Lock()
        self.cond = threading.Condition(self.lock)
        self.members: set[int] = set()
        self.generation = 0
        self.round: Optional[_Round] = None


_registry: dict[str, _Group] = {}
_registry_lock = threading.Lock()


def registry_size() -> int:
    with _registry_lock:
        return len(_registry)


class RendezvousSession:
    """One rank's membership of a group; ``close()`` (or garbage collection) leaves the group and
    fails an in-flight round for the remaining ranks."""

    def __init__(self, group: _Group, rank: int):
        self._group, self.rank = group, rank
        self._closed = False

    @property
    def world_size(self) -> int:
        return self._group.world_size

    @property
    def group_id(self) -> str:
        return self._group.group_id

    def generation(self) -> int:
        with self._group.lock:
            return self._group.generation

    def in_flight(self) -> bool:
        g = self._group
        with g.lock:
            return g.round is not None and not g.round.done and self.rank in g.round.contributors

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        g = self._group
        with g.cond:
            g.members.discard(self.rank)
            rnd = g.round
            if rnd is not None and not rnd.done:
                rnd.error = ParticipantLeft(rank=self.rank, generation=rnd.generation)
                rnd.done = True
                g.cond.notify_all()
            empty = not g.members
        if empty:
            with _registry_lock:
                if _registry.get(g.group_id) is g and not g.members:
                    del _registry[g.group_id]

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    # ------------------------------------------------------------------------------------------
    def all_reduce_sum(self, values: list[float], timeout: float = DEFAULT_COLLECTIVE_TIMEOUT) -> list[float]:
        """Returns the element-wise sum over all ranks; raises the same error on every rank of a
        failed round.  ``values`` is never modified."""
        if self._closed:
            raise UnknownRank(rank=self.rank)
        g = self._group
        deadline = time.monotonic() + timeout
        started = time.monotonic()
        with g.cond:
            if self.rank not in g.members:
                raise UnknownRank(rank=self.rank)
            # wait for a previous, still-draining round to be collected by all of its contributors
            while g.round is not None and g.round.done and self.rank in g.round.contributors:
                # this rank already collected the old round (contributors are removed on collect)
                break
            rnd = g.round
            if rnd is None or rnd.done:
                g.generation += 1
                rnd = _Round(g.generation, len(values))
                g.round = rnd
            if self.rank in rnd.contributors:
                # rejected without aborting the round for the others
                raise DuplicateContribution(rank=self.rank, generation=rnd.generation)
            if len(values) != len(rnd.buffer):
                rnd.error = BufferLengthMismatch(expected=len(rnd.buffer), got=len(values), rank=self.rank)
                rnd.done = True
                rnd.contributors.add(self.rank)
                g.cond.notify_all()
                return self._collect(g, rnd)
            bad = next((i for i, v in enumerate(values) if not math.isfinite(v)), None)
            if bad is not None:
                rnd.error = NonFiniteInput(rank=self.rank, index=bad)
                rnd.done = True
                rnd.contributors.add(self.rank)
                g.cond.notify_all()
                return self._collect(g, rnd)
            for i, v in enumerate(values):
                rnd.buffer[i] += v
            rnd.contributors.add(self.rank)
            if len(rnd.contributors) == g.world_size:
                bad = next((i for i, v in enumerate(rnd.buffer) if not math.isfinite(v)), None)
                if bad is not None:
                    rnd.error = NonFiniteReduction(index=bad)
                else:
                    rnd.result = list(rnd.buffer)
                rnd.done = True
                g.cond.notify_all()
                return self._collect(g, rnd)
            while not rnd.done:
                remaining = deadline - time.monotonic()
                if remaining <= 0:
                    rnd.error = CollectiveTimeout(generation=rnd.generation,
                                                  waited_ms=int((time.monotonic() - started) * 1000))
                    rnd.done = True
                    g.cond.notify_all()
                    break
                g.cond.wait(remaining)
            return self._collect(g, rnd)

    def _collect(self, g: _Group, rnd: _Round) -> list[float]:
        # called with the lock held
        rnd.contributors.discard(self.rank)
        if not rnd.contributors and g.round is rnd:
            g.round = None
        if rnd.error is not None:
            raise type(rnd.error)(**rnd.error.fields)
        assert rnd.result is not None
        return list(rnd.result)


def join(group_id: str, rank: int, world_size: int) -> RendezvousSession:
    """Join (or create) the in-memory group ``group_id``."""
    if world_size <= 0:
        raise EmptyWorldSize()
    if rank < 0 or rank >= world_size:
        raise RankOutOfBounds(rank=rank, world_size=world_size)
    with _registry_lock:
        g = _registry.get(group_id)
        if g is None:
            g = _Group(group_id, world_size)
            _registry[group_id] = g
    with g.lock:
        if g.world_size != world_size:
            raise WorldSizeMismatch(expected=g.world_size, got=world_size)
        if rank in g.members:
            raise DuplicateRank(rank=rank)
        g.members.add(rank)
    return RendezvousSession(g, rank)
