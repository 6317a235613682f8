"""``Dataset`` / ``DataLoader`` of the public API (crates/st-nn/src/dataset.rs:287-360):
``shuffle(seed)``, ``batched(n)``, ``dynamic_batch_by_rows(max_rows)`` and ``prefetch(depth)``
(a worker thread that stages batches ahead; on CUDA the staging is a pinned-memory copy on a
side stream)."""
from __future__ import annotations

import queue
import threading
from typing import Iterable, Iterator, Optional, Sequence

import torch

from ..tensor import Tensor


class Dataset:
    def __init__(self, samples: Optional[Iterable[tuple[Tensor, Tensor]]] = None):
        self._samples: list[tuple[Tensor, Tensor]] = list(samples or [])

    @staticmethod
    def from_samples(samples) -> "Dataset":
        return Dataset(samples)

    def push(self, x: Tensor, y: Tensor) -> None:
        self._samples.append((x, y))

    def __len__(self) -> int:
        return len(self._samples)

    def len(self) -> int:
        return len(self._samples)

    def __getitem__(self, i: int):
        return self._samples[i]

    def __iter__(self):
        return iter(self._samples)

    def loader(self) -> "DataLoader":
        return DataLoader(self)


def from_samples(samples) -> Dataset:
    return Dataset(samples)


class DataLoader:
    def __init__(self, dataset: Dataset, *, order: Optional[Sequence[int]] = None, batch: int = 1,
                 max_rows: Optional[int] = None, prefetch_depth: int = 0, device=None):
        self.dataset, self._order = dataset, list(order) if order is not None else list(range(len(dataset)))
        self._batch, self._max_rows, self._prefetch, self._device = batch, max_rows, prefetch_depth, device

    def _clone(self, **kw) -> "DataLoader":
        args = dict(order=self._order, batch=self._batch, max_rows=self._max_rows,
                    prefetch_depth=self._prefetch, device=self._device)
        args.update(kw)
        return DataLoader(self.dataset, **args)

    def shuffle(self, seed: int) -> "DataLoader":
        g = torch.Generator().manual_seed(int(seed))
        perm = torch.randperm(len(self._order), generator=g).tolist()
        return self._clone(order=[self._order[i] for i in perm])

    def batched(self, batch: int) -> "DataLoader":
        if batch < 1:
            raise ValueError("batch must be >= 1")
        return self._clone(batch=batch, max_rows=None)

    def dynamic_batch_by_rows(self, max_rows: int) -> "DataLoader":
        if max_rows < 1:
            raise ValueError("max_rows must be >= 1")
        return self._clone(max_rows=max_rows)

    def prefetch(self, depth: int) -> "DataLoader":
        return self._clone(prefetch_depth=max(0, depth))

    def to(self, device) -> "DataLoader":
        return self._clone(device=device)

    def __len__(self) -> int:
        return sum(1 for _ in self._groups())

    def _groups(self) -> Iterator[list[int]]:
        if self._max_rows is not None:
            cur, rows = [], 0
            for i in self._order:
                r = self.dataset[i][0].rows
                if cur and rows + r > self._max_rows:
                    yield cur
                    cur, rows = [], 0
                cur.append(i)
                rows += r
            if cur:
                yield cur
        else:
            for s in range(0, len(self._order), self._batch):
                yield self._order[s:s + self._batch]

    def _make(self, idxs: list[int]) -> tuple[Tensor, Tensor]:
        xs = Tensor.cat_rows_many(self.dataset[i][0] for i in idxs)
        ys = Tensor.cat_rows_many(self.dataset[i][1] for i in idxs)
        if self._device is not None:
            dev = torch.device(self._device)
            if dev.type == "cuda":
                xs = Tensor._wrap(xs.torch().pin_memory().to(dev, non_blocking=True))
                ys = Tensor._wrap(ys.torch().pin_memory().to(dev, non_blocking=True))
            else:
                xs, ys = xs.to(dev), ys.to(dev)
        return xs, ys

    def __iter__(self) -> "DataLoaderIter":
        return DataLoaderIter(self._batches())

    iter = __iter__

    def _batches(self) -> Iterator[tuple[Tensor, Tensor]]:
        if self._prefetch <= 0:
            for g in self._groups():
                yield self._make(g)
            return
        q: "queue.Queue" = queue.Queue(maxsize=self._prefetch)
        sentinel = object()

        def worker():
            try:
                for g in self._groups():
                    q.put(self._make(g))
                q.put(sentinel)
            except BaseException as exc:  # noqa: BLE001 - re-raised in the consumer
                q.put(exc)

        threading.Thread(target=worker, daemon=True).start()
        while True:
            item = q.get()
            if item is sentinel:
                return
            if isinstance(item, BaseException):
                raise item
            yield item


class DataLoaderIter:
    """One pass over a loader's batches (bindings/st-py/src/nn.rs:8915-8940: ``iter(loader)`` returns this object; it is its
    own iterator and raises `StopIteration` when the pass is over)."""

    def __init__(self, batches: Iterator[tuple[Tensor, Tensor]]):
        self._batches = batches

    def __iter__(self) -> "DataLoaderIter":
        return self

    def __next__(self) -> tuple[Tensor, Tensor]:
        return next(self._batches)
