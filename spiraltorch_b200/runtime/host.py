"""ctypes bindings of the CUDA-free host runtime (``csrc/host/host_runtime.cpp``).

* :class:`WorkerPool` — native worker threads that run Python callables (the callable's
  exception is captured and returned, like the panic capture of
  crates/st-core/src/runtime/golden.rs:237-400);
* :class:`NativeRendezvous` — in-process all-reduce over ``float32`` buffers with the uniform error
  vocabulary of crates/spiral-selfsup/src/trainer/distributed.rs (the waiting happens in C++ with
  the GIL released, so rank threads really overlap);
* :class:`PrefetchLoader` — a worker thread that gathers shuffled mini-batches ahead of the
  consumer (crates/st-nn/src/dataset.rs:287-360);
* :func:`atomic_write` — tmp file + fsync + rename + directory fsync
  (crates/st-core/src/runtime/persistence.rs:21-62).
"""
from __future__ import annotations

import ctypes
import threading
import traceback
from typing import Any, Callable, Optional

import numpy as np
import torch

from ..distributed import rendezvous as rdv
from ..utils import build

_lib = None
_lib_lock = threading.Lock()
_TASK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)


def lib() -> ctypes.CDLL:
    global _lib
    with _lib_lock:
        if _lib is None:
            path = build.build_host()
            L = ctypes.CDLL(str(path))
            L.st_host_pool_create.restype = ctypes.c_void_p
            L.st_host_pool_create.argtypes = [ctypes.c_int]
            L.st_host_pool_destroy.argtypes = [ctypes.c_void_p]
            L.st_host_pool_workers.argtypes = [ctypes.c_void_p]
            L.st_host_pool_submit.restype = ctypes.c_uint64
            L.st_host_pool_submit.argtypes = [ctypes.c_void_p, _TASK, ctypes.c_void_p]
            L.st_host_pool_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int64,
                                            ctypes.POINTER(ctypes.c_int)]
            L.st_host_pool_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]
            L.st_host_rdv_join.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int64)]
            L.st_host_rdv_leave.argtypes = [ctypes.c_void_p]
            L.st_host_rdv_generation.restype = ctypes.c_uint64
            L.st_host_rdv_generation.argtypes = [ctypes.c_void_p]
            L.st_host_rdv_all_reduce_sum.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                                     ctypes.c_int64, ctypes.POINTER(ctypes.c_int64)]
            L.st_host_loader_create.restype = ctypes.c_void_p
            L.st_host_loader_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_int, ctypes.c_int]
            L.st_host_loader_next.restype = ctypes.c_int64
            L.st_host_loader_next.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
            L.st_host_loader_destroy.argtypes = [ctypes.c_void_p]
            L.st_host_atomic_write.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64]
            _lib = L
    return _lib


# --------------------------------------------------------------------------------------------------
class TaskHandle:
    def __init__(self, pool: "WorkerPool", ticket: int, slot: dict):
        self._pool, self._ticket, self._slot = pool, ticket, slot

    def join(self, timeout: Optional[float] = None):
        """Returns the callable's result; re-raises :class:`WorkerFailure` if it raised."""
        status = ctypes.c_int(0)
        ms = -1 if timeout is None else int(timeout * 1000)
        rc = lib().st_host_pool_wait(self._pool._h, self._ticket, ms, ctypes.byref(status))
        if rc == 1:
            raise TimeoutError(f"task {self._ticket} still running after {timeout}s")
        if rc == 2:
            raise KeyError(f"unknown task {self._ticket}")
        self._pool._release(self._ticket)
        if status.value != 0:
            raise WorkerFailure(self._slot.get("error", "worker failed"), self._slot.get("traceback", ""))
        return self._slot.get("result")


class WorkerFailure(RuntimeError):
    def __init__(self, message: str, tb: str = ""):
        super().__init__(message)
        self.worker_traceback = tb


class WorkerPool:
    """``spawn(fn, *args)`` runs ``fn`` on a native worker thread; failures are captured, never
    propagate into the pool, and are counted (``stats()['failed']``)."""

    def __init__(self, workers: int = 0, name: str = "golden"):
        self._h = lib().st_host_pool_create(workers)
        self.name = name
        self._live: dict[int, tuple] = {}
        self._lock = threading.Lock()

    @property
    def workers(self) -> int:
        return lib().st_host_pool_workers(self._h)

    def spawn(self, fn: Callable[..., Any], *args, **kwargs) -> TaskHandle:
        slot: dict = {}

        def tramp(_arg):
            try:
                slot["result"] = fn(*args, **kwargs)
                return 0
            except BaseException as exc:  # noqa: BLE001 - the pool must survive any failure
                slot["error"] = f"{type(exc).__name__}: {exc}"
                slot["traceback"] = traceback.format_exc()
                return 1

        cb = _TASK(tramp)
        with self._lock:
            ticket = lib().st_host_pool_submit(self._h, cb, None)
            self._live[ticket] = (cb, slot)           # keep the trampoline alive until joined
        return TaskHandle(self, ticket, slot)

    def _release(self, ticket: int) -> None:
        with self._lock:
            self._live.pop(ticket, None)

    def map(self, fn, items, timeout: Optional[float] = None) -> list:
        return [h.join(timeout) for h in [self.spawn(fn, it) for it in items]]

    def stats(self) -> dict:
        out = (ctypes.c_uint64 * 3)()
        lib().st_host_pool_stats(self._h, out)
        return {"submitted": int(out[0]), "completed": int(out[1]), "failed": int(out[2])}

    def close(self) -> None:
        if self._h:
            lib().st_host_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


# --------------------------------------------------------------------------------------------------
_RDV_ERRORS = {
    1: (rdv.EmptyWorldSize, ()),
    2: (rdv.RankOutOfBounds, ("rank", "world_size")),
    3: (rdv.WorldSizeMismatch, ("expected", "got")),
    4: (rdv.DuplicateRank, ("rank",)),
    5: (rdv.UnknownRank, ()),
    6: (rdv.DuplicateContribution, ("rank", "generation")),
    7: (rdv.BufferLengthMismatch, ("expected", "got", "rank")),
    8: (rdv.NonFiniteInput, ("rank", "index")),
    9: (rdv.NonFiniteReduction, ("index",)),
    10: (rdv.ParticipantLeft, ("rank", "generation")),
    11: (rdv.CollectiveTimeout, ("generation", "waited_ms")),
}


def _raise_rdv(code: int, detail) -> None:
    cls, names = _RDV_ERRORS[code]
    raise cls(**{n: int(detail[i]) for i, n in enumerate(names)})


class NativeRendezvous:
    """One rank's membership of an in-process group, reducing ``float32`` tensors in place."""

    def __init__(self, group_id: str, rank: int, world_size: int):
        self.group_id, self.rank, self.world_size = group_id, rank, world_size
        h = ctypes.c_void_p()
        detail = (ctypes.c_int64 * 3)()
        code = lib().st_host_rdv_join(group_id.encode(), rank, world_size, ctypes.byref(h), detail)
        if code:
            _raise_rdv(code, detail)
        self._h = h

    def generation(self) -> int:
        return int(lib().st_host_rdv_generation(self._h))

    def all_reduce_sum_(self, values: torch.Tensor, timeout: float = rdv.DEFAULT_COLLECTIVE_TIMEOUT) -> torch.Tensor:
        """In-place sum over ranks of a contiguous CPU ``float32`` tensor.  On failure every rank of
        the round raises the same error and ``values`` is left untouched."""
        if self._h is None:
            raise rdv.UnknownRank(rank=self.rank)
        if values.device.type != "cpu" or values.dtype != torch.float32 or not values.is_contiguous():
            raise TypeError("all_reduce_sum_ expects a contiguous CPU float32 tensor")
        detail = (ctypes.c_int64 * 3)()
        code = lib().st_host_rdv_all_reduce_sum(self._h, values.data_ptr(), values.numel(), int(timeout * 1000), detail)
        if code:
            _raise_rdv(code, detail)
        return values

    def close(self) -> None:
        if self._h is not None:
            h, self._h = self._h, None
            lib().st_host_rdv_leave(h)

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


def native_registry_size() -> int:
    return int(lib().st_host_rdv_registry_size())


# --------------------------------------------------------------------------------------------------
class PrefetchLoader:
    """Iterates ``(x, y)`` float32 mini-batches gathered by a native worker thread ``depth``
    batches ahead of the consumer.  ``order`` is the (already shuffled) row permutation."""

    def __init__(self, features: torch.Tensor, targets: Optional[torch.Tensor], order, batch_size: int,
                 depth: int = 2, drop_last: bool = False, pin_memory: bool = False):
        self.features = features.detach().to(torch.float32).contiguous().cpu()
        self.targets = None if targets is None else targets.detach().to(torch.float32).contiguous().cpu()
        if self.features.dim() != 2 or (self.targets is not None and self.targets.dim() != 2):
            raise ValueError("PrefetchLoader expects 2-D feature / target matrices")
        self.order = np.ascontiguousarray(np.asarray(order, dtype=np.int64))
        self.batch_size, self.depth, self.drop_last, self.pin_memory = batch_size, depth, drop_last, pin_memory

    def __len__(self) -> int:
        n = len(self.order)
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def __iter__(self):
        rows, fc = self.features.shape
        tc = 0 if self.targets is None else self.targets.shape[1]
        h = lib().st_host_loader_create(self.features.data_ptr(), 0 if self.targets is None else self.targets.data_ptr(),
                                        rows, fc, tc, self.order.ctypes.data, len(self.order), self.batch_size,
                                        self.depth, int(self.drop_last))
        if not h:
            raise ValueError("invalid loader configuration (batch size, depth or row index out of range)")
        try:
            while True:
                x = torch.empty((self.batch_size, fc), dtype=torch.float32, pin_memory=self.pin_memory)
                y = torch.empty((self.batch_size, tc), dtype=torch.float32, pin_memory=self.pin_memory) if tc else None
                n = lib().st_host_loader_next(h, x.data_ptr(), 0 if y is None else y.data_ptr())
                if n == 0:
                    return
                yield (x[:n], None if y is None else y[:n])
        finally:
            lib().st_host_loader_destroy(h)


def atomic_write(path: str, data: bytes) -> None:
    buf = ctypes.create_string_buffer(data, len(data))
    rc = lib().st_host_atomic_write(str(path).encode(), buf, len(data))
    if rc:
        raise OSError(f"atomic_write({path!r}) failed at stage {rc}")
