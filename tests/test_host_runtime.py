"""Native host runtime: worker pool, rendezvous all-reduce, prefetch loader, durable writes, and the
multi-trainer driver with dropout tolerance built on them.  All CPU."""
import os
import threading
import time

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200.distributed import rendezvous as rdv
from spiraltorch_b200.runtime import golden, host


def test_worker_pool_runs_and_captures_failures():
    pool = host.WorkerPool(3)
    assert pool.workers == 3
    hs = [pool.spawn(lambda i=i: i * i) for i in range(8)]
    assert [h.join() for h in hs] == [i * i for i in range(8)]

    def boom():
        raise ValueError("bad worker")

    h = pool.spawn(boom)
    with pytest.raises(host.WorkerFailure, match="ValueError: bad worker") as ei:
        h.join()
    assert "boom" in ei.value.worker_traceback
    # the pool survives a failure
    assert pool.spawn(lambda: 7).join() == 7
    s = pool.stats()
    assert s["submitted"] == 10 and s["completed"] == 10 and s["failed"] == 1
    slow = pool.spawn(time.sleep, 0.3)
    with pytest.raises(TimeoutError):
        slow.join(timeout=0.01)
    slow.join()
    pool.close()


def test_worker_pool_threads_overlap():
    pool = host.WorkerPool(4)
    t0 = time.monotonic()
    pool.map(lambda _: time.sleep(0.2), range(4))
    assert time.monotonic() - t0 < 0.6
    pool.close()


def _ranks(world, fn):
    out, errs = [None] * world, [None] * world

    def run(r):
        try:
            out[r] = fn(r)
        except Exception as exc:  # noqa: BLE001
            errs[r] = exc

    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out, errs


def test_native_rendezvous_sum_and_uniform_errors():
    world = 4
    sessions = [host.NativeRendezvous("memory://native-a", r, world) for r in range(world)]

    def ok(r):
        v = torch.full((1000,), float(r + 1))
        sessions[r].all_reduce_sum_(v)
        return v

    out, errs = _ranks(world, ok)
    assert all(e is None for e in errs)
    for v in out:
        assert torch.equal(v, torch.full((1000,), 10.0))
    assert sessions[0].generation() == 1

    # a non-finite contribution fails the round for every rank and leaves buffers untouched
    def bad(r):
        v = torch.full((8,), float(r))
        if r == 2:
            v[5] = float("nan")
            time.sleep(0.3)            # arrive last: the failure reaches every rank of the round
        keep = v.clone()
        try:
            sessions[r].all_reduce_sum_(v)
        finally:
            assert torch.equal(torch.nan_to_num(v), torch.nan_to_num(keep))

    _, errs = _ranks(world, bad)
    assert all(isinstance(e, rdv.NonFiniteInput) for e in errs)
    assert {e.rank for e in errs} == {2} and {e.index for e in errs} == {5}

    # the group is usable afterwards
    out, errs = _ranks(world, ok)
    assert all(e is None for e in errs)

    # length mismatch
    def mism(r):
        if r == 1:
            time.sleep(0.3)
        sessions[r].all_reduce_sum_(torch.zeros(4 if r != 1 else 5))

    _, errs = _ranks(world, mism)
    assert all(isinstance(e, rdv.BufferLengthMismatch) for e in errs)
    for s_ in sessions:
        s_.close()
    assert host.native_registry_size() == 0


def test_native_rendezvous_timeout_and_leave():
    world = 3
    sessions = [host.NativeRendezvous("memory://native-b", r, world) for r in range(world)]

    # rank 2 never joins the round: the others time out with the same error
    def late(r):
        if r == 2:
            return None
        sessions[r].all_reduce_sum_(torch.ones(4), timeout=0.2)

    t0 = time.monotonic()
    _, errs = _ranks(world, late)
    assert time.monotonic() - t0 < 2.0
    assert isinstance(errs[0], rdv.CollectiveTimeout) and isinstance(errs[1], rdv.CollectiveTimeout)
    assert errs[0].generation == errs[1].generation

    # a member that leaves during a round fails it for the waiting ranks
    def leave(r):
        if r == 2:
            time.sleep(0.1)
            sessions[2].close()
            return None
        sessions[r].all_reduce_sum_(torch.ones(4), timeout=5.0)

    _, errs = _ranks(world, leave)
    assert isinstance(errs[0], rdv.ParticipantLeft) and errs[0].rank == 2
    assert isinstance(errs[1], rdv.ParticipantLeft)
    with pytest.raises(rdv.DuplicateRank):
        host.NativeRendezvous("memory://native-b", 0, world)
    with pytest.raises(rdv.WorldSizeMismatch):
        host.NativeRendezvous("memory://native-b", 2, world + 1)
    for s_ in sessions[:2]:
        s_.close()


def test_prefetch_loader_matches_direct_gather():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(103, 7, generator=g)
    y = torch.randn(103, 2, generator=g)
    order = torch.randperm(103, generator=g).tolist()
    batches = list(host.PrefetchLoader(x, y, order, batch_size=16, depth=3))
    assert len(batches) == 7 and batches[-1][0].shape[0] == 103 - 96
    assert torch.equal(torch.cat([b[0] for b in batches]), x[order])
    assert torch.equal(torch.cat([b[1] for b in batches]), y[order])
    dropped = list(host.PrefetchLoader(x, None, order, batch_size=16, drop_last=True))
    assert len(dropped) == 6 and dropped[0][1] is None
    with pytest.raises(ValueError):
        list(host.PrefetchLoader(x, y, [0, 500], batch_size=2))


def test_atomic_write_replaces_file(tmp_path):
    p = tmp_path / "state.json"
    host.atomic_write(str(p), b"one")
    host.atomic_write(str(p), b"two-longer")
    assert p.read_bytes() == b"two-longer"
    assert [f.name for f in tmp_path.iterdir()] == ["state.json"]
    with pytest.raises(OSError):
        host.atomic_write(str(tmp_path / "missing" / "x"), b"z")


# ---- GoldenRetriever ---------------------------------------------------------------------------
def _make_worker(seed):
    model = st.nn.Sequential()
    model.add(st.nn.Linear("fc", 4, 1))
    g = torch.Generator().manual_seed(seed)
    batches = [(st.Tensor._wrap(torch.randn(8, 4, generator=g)), st.Tensor._wrap(torch.randn(8, 1, generator=g)))
               for _ in range(3)]
    trainer = st.nn.ModuleTrainer(backend="cpu", fallback_learning_rate=1e-2)
    return model, st.nn.MeanSquaredError(), batches, trainer


class _Exploding(st.nn.MeanSquaredError):
    def forward(self, prediction, target):
        raise RuntimeError("loss exploded")


def test_golden_retriever_epoch_and_dropout_tolerance():
    workers = [_make_worker(s) for s in range(3)]
    trainers = [w[3] for w in workers]
    sched = [t.roundtable(8, 1) for t in trainers]
    gr = golden.GoldenRetriever(golden.GoldenRetrieverConfig(coordinate_blackcat=True), trainers)
    digest = gr.subscribe_digest()
    rep = gr.run_epoch([w[0] for w in workers], [w[1] for w in workers], [w[2] for w in workers], sched)
    assert rep.workers == 3 and rep.batches == 9 and not rep.dropouts
    assert abs(rep.average_loss - rep.total_loss / 9) < 1e-6
    assert rep.cooperative_pulse.worker_count == 3
    assert digest.get_nowait().workers == 3

    # one worker fails: fatal without dropout tolerance ...
    losses = [w[1] for w in workers]
    losses[1] = _Exploding()
    with pytest.raises(st.TensorError, match="worker 1"):
        gr.run_epoch([w[0] for w in workers], losses, [w[2] for w in workers], sched)
    gr.close()

    # ... recorded and survived with it
    gr2 = golden.GoldenRetriever(golden.GoldenRetrieverConfig(allow_dropout=True, min_successful_workers=2), trainers)
    rep = gr2.run_epoch([w[0] for w in workers], losses, [w[2] for w in workers], sched)
    assert rep.workers == 2 and rep.batches == 6
    assert [d.worker for d in rep.dropouts] == [1] and "loss exploded" in rep.dropouts[0].error
    assert [d.worker for d in gr2.last_dropouts()] == [1]
    # too many failures
    losses[0] = _Exploding()
    with pytest.raises(st.TensorError, match="completed 1 of 3 workers"):
        gr2.run_epoch([w[0] for w in workers], losses, [w[2] for w in workers], sched)
    gr2.close()


def test_golden_barycenter():
    gr = golden.GoldenRetriever(golden.GoldenRetrieverConfig(), [_make_worker(0)[3]])
    a = st.Tensor._wrap(torch.ones(2, 8))
    b = st.Tensor._wrap(torch.full((2, 8), 3.0))
    out = gr.sync_z_barycenter([a, b], rank=2)
    vals = torch.tensor(out.tolist())
    assert vals.shape == (2, 8)
    assert torch.allclose(vals, vals[0, 0].expand_as(vals)) and 2.0 < vals[0, 0].item() < 4.0
    with pytest.raises(st.TensorError):
        gr.sync_z_barycenter([a, st.Tensor._wrap(torch.ones(3, 8))], rank=1)
    gr.close()
