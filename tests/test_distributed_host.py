"""Failure detection and consistency of the host-side collectives (thread ranks, no GPU).

Mirrors the reference's strategy (crates/spiral-selfsup/src/trainer/distributed.rs:432-670): ranks are
threads joined through a named in-memory group; failures are injected on the host (a rank that never
joins, a rank that leaves, non-finite inputs, a closure that fails on one rank)."""
import threading
import time

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200.distributed import (BufferLengthMismatch, CollectiveTimeout, CpuDevice, DistributedDevice, NativeDistributedDevice,
                                          DuplicateContribution, DuplicateRank, EmptyWorldSize, MetricReduce,
                                          NonFiniteInput, NonFiniteReduction, ParticipantLeft, PeerTensorFailure,
                                          RankOutOfBounds, WorldSizeMismatch, join)
from spiraltorch_b200.distributed import rendezvous as rdv


def _run(world, fn):
    out, errs = [None] * world, [None] * world

    def target(r):
        try:
            out[r] = fn(r)
        except BaseException as exc:  # noqa: BLE001
            errs[r] = exc

    threads = [threading.Thread(target=target, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
        assert not t.is_alive()
    return out, errs


def test_join_validation_and_registry_cleanup():
    with pytest.raises(EmptyWorldSize):
        join("g-val", 0, 0)
    with pytest.raises(RankOutOfBounds):
        join("g-val", 2, 2)
    a = join("g-val", 0, 2)
    with pytest.raises(DuplicateRank):
        join("g-val", 0, 2)
    with pytest.raises(WorldSizeMismatch):
        join("g-val", 1, 3)
    b = join("g-val", 1, 2)
    before = rdv.registry_size()
    a.close()
    b.close()
    assert rdv.registry_size() == before - 1


def test_repeated_rounds_four_ranks_mean():
    sessions = [join("g-rounds", r, 4) for r in range(4)]

    def work(r):
        acc = []
        for i in range(64):
            acc.append(sessions[r].all_reduce_sum([float(r + i), 1.0], timeout=10))
        return acc

    out, errs = _run(4, work)
    assert not any(errs)
    for r in range(4):
        for i in range(64):
            assert out[r][i] == [float(0 + 1 + 2 + 3 + 4 * i), 4.0]
    for s in sessions:
        s.close()


def test_non_finite_input_and_overflow_reported_to_every_rank():
    sessions = [join("g-nan", r, 2) for r in range(2)]
    _, errs = _run(2, lambda r: sessions[r].all_reduce_sum([float("nan") if r == 1 else 1.0], timeout=5))
    assert all(isinstance(e, NonFiniteInput) for e in errs) and errs[0].rank == 1 and errs[0].index == 0
    _, errs = _run(2, lambda r: sessions[r].all_reduce_sum([1.7e308], timeout=5))
    assert all(isinstance(e, NonFiniteReduction) for e in errs)
    _, errs = _run(2, lambda r: sessions[r].all_reduce_sum([1.0] * (1 + r), timeout=5))
    assert all(isinstance(e, BufferLengthMismatch) for e in errs)
    out, errs = _run(2, lambda r: sessions[r].all_reduce_sum([2.0], timeout=5))   # group still usable
    assert out == [[4.0], [4.0]] and not any(errs)
    for s in sessions:
        s.close()


def test_missing_rank_times_out_without_touching_the_buffer_and_group_recovers():
    a = join("g-timeout", 0, 2)
    buf = [1.0, 2.0]
    t0 = time.monotonic()
    with pytest.raises(CollectiveTimeout) as ei:
        a.all_reduce_sum(buf, timeout=0.3)
    assert 0.25 < time.monotonic() - t0 < 5 and ei.value.waited_ms >= 250
    assert buf == [1.0, 2.0]
    b = join("g-timeout", 1, 2)
    sessions = [a, b]
    out, errs = _run(2, lambda r: sessions[r].all_reduce_sum([1.0], timeout=5))
    assert out == [[2.0], [2.0]] and not any(errs)
    a.close()
    b.close()


def test_rank_drop_aborts_the_round_and_rank_can_rejoin():
    a, b = join("g-drop", 0, 2), join("g-drop", 1, 2)
    result = {}

    def waiter():
        try:
            a.all_reduce_sum([1.0], timeout=10)
        except BaseException as exc:  # noqa: BLE001
            result["err"] = exc

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.2)
    b.close()                      # leaves between steps: nothing of its own is in flight
    t.join(10)
    assert isinstance(result["err"], ParticipantLeft) and result["err"].rank == 1
    b2 = join("g-drop", 1, 2)
    sessions = [a, b2]
    out, errs = _run(2, lambda r: sessions[r].all_reduce_sum([3.0], timeout=5))
    assert out == [[6.0], [6.0]] and not any(errs)
    a.close()
    b2.close()


def test_duplicate_contribution_is_rejected_without_aborting_the_round():
    a, b = join("g-dup", 0, 2), join("g-dup", 1, 2)
    got = {}

    def first():
        got["a"] = a.all_reduce_sum([1.0], timeout=10)

    t = threading.Thread(target=first)
    t.start()
    time.sleep(0.2)
    with pytest.raises(DuplicateContribution):
        a.all_reduce_sum([5.0], timeout=1)
    got["b"] = b.all_reduce_sum([2.0], timeout=10)
    t.join(10)
    assert got["a"] == got["b"] == [3.0]
    a.close()
    b.close()


@pytest.mark.parametrize("DistributedDevice", [DistributedDevice, NativeDistributedDevice])
def test_distributed_device_mean_and_two_phase_commit(DistributedDevice):
    devs = [DistributedDevice("g-dev", r, 2).with_collective_timeout(5) for r in range(2)]
    bufs = [torch.tensor([1.0, 3.0]), torch.tensor([3.0, 5.0])]
    _, errs = _run(2, lambda r: devs[r].synchronize_gradients(bufs[r]))
    assert not any(errs) and bufs[0].tolist() == bufs[1].tolist() == [2.0, 4.0]
    m = [torch.tensor([1.0]), torch.tensor([2.0])]
    _run(2, lambda r: devs[r].aggregate_metrics(m[r], MetricReduce.SUM))
    assert m[0].item() == m[1].item() == 3.0
    # a failure on rank 0 after the sum is rejected by every rank and nobody commits
    devs[0].fail_mean_scale = lambda: True
    bufs = [torch.tensor([1.0]), torch.tensor([3.0])]
    _, errs = _run(2, lambda r: devs[r].synchronize_gradients(bufs[r]))
    assert all(isinstance(e, PeerTensorFailure) for e in errs) and errs[1].failed_ranks == 1
    assert bufs[0].tolist() == [1.0] and bufs[1].tolist() == [3.0]
    ck = devs[1].checkpoint()
    assert ck["provider"] == "spiral_selfsup.distributed" and ck["world_size"] == "2"
    assert ck["state"]["strategy"] == "all_reduce_mean" and ck["state"]["collective_timeout_nanos"] == "5000000000"
    for d in devs:
        d.close()
    assert CpuDevice().world_size() == 1


@pytest.mark.parametrize("DistributedDevice", [DistributedDevice, NativeDistributedDevice])
def test_two_rank_trainer_step_equals_local_step_on_averaged_gradient(DistributedDevice):
    """crates/spiral-selfsup/tests/module_trainer_accumulators.rs:83-115."""
    xs = [st.Tensor.randn(4, 3, seed=10 + r) for r in range(2)]
    ys = [st.Tensor.randn(4, 2, seed=20 + r) for r in range(2)]
    loss = st.nn.MeanSquaredError()
    models = [st.nn.Linear("fc", 3, 2) for _ in range(2)]
    devs = [DistributedDevice("g-train", r, 2).with_collective_timeout(10) for r in range(2)]

    def work(r):
        tr = st.nn.ModuleTrainer(fallback_learning_rate=0.1)
        tr.set_training_device(devs[r])
        tr.train_epoch(models[r], loss, [(xs[r], ys[r])])
        return tr.last_accumulator_sync()

    out, errs = _run(2, work)
    assert not any(errs) and out[0]["world_size"] == 2 and out[0]["buffers"] == 2
    local = st.nn.Linear("fc", 3, 2)
    for r in range(2):
        local.backward(xs[r], loss.backward(local.forward(xs[r]), ys[r]))
    for p in local.parameters():
        p.scale_accumulators(0.5)
    local.apply_step(0.1)
    for m in models:
        assert torch.allclose(m.weight.value, local.weight.value, atol=1e-6)
        assert torch.allclose(m.bias.value, local.bias.value, atol=1e-6)
    for d in devs:
        d.close()
