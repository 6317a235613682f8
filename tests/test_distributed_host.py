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


def test_collective_arena_is_transactional_and_reports_digests():
    from spiraltorch_b200.distributed import arena as A
    ar = A.CollectiveArena()
    rows = [[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]]
    rep = ar.all_reduce_sum(rows)
    assert rows == [[9.0, 12.0]] * 3 and rep.participants == 3 and rep.width == 2 and rep.committed
    rep.validate()
    assert len(rep.input_sha256) == 64 and rep.input_sha256 != rep.output_sha256
    again = ar.all_reduce_sum([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert again.input_sha256 == rep.input_sha256 and again.output_sha256 == rep.output_sha256
    bad = [[1.0, 2.0], [float("nan"), 4.0]]
    with pytest.raises(A.CollectiveError) as ei:
        ar.all_reduce_sum(bad)
    assert ei.value.kind == "NonFiniteInput" and ei.value.fields["participant"] == 1 and bad[0] == [1.0, 2.0]
    with pytest.raises(A.CollectiveError) as ei:
        ar.all_reduce_sum([[3e38], [3e38]])
    assert ei.value.kind == "NonFiniteReduction"
    with pytest.raises(A.CollectiveError):
        ar.all_reduce_sum([[1.0], [1.0, 2.0]])
    with pytest.raises(A.CollectiveError):
        ar.all_reduce_sum([])
    targets = [[0.0, 0.0], [1.0, 1.0]]
    ar.broadcast([7.0, 8.0], targets)
    assert targets == [[7.0, 8.0], [7.0, 8.0]]
    # the lease puts the batches back unless committed
    ar.enqueue_gradient([1.0, 2.0])
    ar.enqueue_gradient([3.0, 4.0])
    with ar.lease_gradient_batches() as lease:
        assert len(lease.batches()) == 2 and ar.pending() == 0
    assert ar.pending() == 2
    with ar.lease_gradient_batches() as lease:
        lease.commit()
    assert ar.pending() == 0


def test_distributed_trainer_and_gossip_autograd():
    from spiraltorch_b200.distributed import arena as A
    tr = A.DistributedTrainer(2, 3, 0.1)
    tr.broadcast_parameters([1.0, 1.0, 1.0])
    grads = [[1.0, 2.0, 3.0], [3.0, 2.0, 1.0]]
    tr.apply_step(grads)
    assert grads == [[1.0, 2.0, 3.0], [3.0, 2.0, 1.0]]
    assert all(abs(p - (1.0 - 0.05 * 4.0)) < 1e-6 for p in tr.parameters())
    before = tr.parameters()
    with pytest.raises(A.DistributedTrainerError):
        tr.apply_step([[float("inf"), 0.0, 0.0], [0.0, 0.0, 0.0]])
    assert tr.parameters() == before
    assert tr.merge_async_gradients() is False
    tr.submit_async_gradient([1.0] * 6)
    tr.submit_async_gradient([3.0] * 6)
    assert tr.merge_async_gradients() is True
    assert all(abs(p - (0.8 - 0.1 * 2.0)) < 1e-6 for p in tr.parameters())
    with pytest.raises(A.DistributedTrainerError):
        tr.submit_async_gradient([1.0])

    # line graph 0 - 1 - 2: a gradient seeded at 0 reaches 1 damped once and 2 damped twice
    mesh = A.AmebaAutograd(max_hops=4, tolerance=1e-6)
    mesh.register_agent(A.AgentConfig(0, 2).with_neighbors([1]).with_learning_rate(0.1).with_damping(0.5))
    mesh.register_agent(A.AgentConfig(1, 2).with_neighbors([0, 2]).with_learning_rate(0.1).with_damping(0.5))
    mesh.register_agent(A.AgentConfig(2, 2).with_neighbors([1]).with_learning_rate(0.1).with_damping(0.5))
    mesh.seed_gradient(0, [1.0, -2.0])
    assert mesh.propagate_round() == 1 and mesh.pending_messages() == 1
    assert mesh.drain() == 2 and mesh.pending_messages() == 0
    assert mesh.weights(0) == pytest.approx([-0.1, 0.2])
    assert mesh.weights(1) == pytest.approx([-0.05, 0.1])
    assert mesh.weights(2) == pytest.approx([-0.025, 0.05])
    with pytest.raises(A.AutogradError):
        mesh.register_agent(A.AgentConfig(0, 2))
    with pytest.raises(A.AutogradError):
        mesh.register_agent(A.AgentConfig(5, 2).with_damping(1.5))
    mesh.register_agent(A.AgentConfig(9, 2).with_neighbors([42]))
    mesh.seed_gradient(9, [1.0, 1.0])
    with pytest.raises(A.AutogradError, match="unknown neighbour"):
        mesh.propagate_round()
    assert mesh.weights(9) == [0.0, 0.0] and mesh.pending_messages() == 1


def test_lane_distribution_and_consensus():
    from spiraltorch_b200.distributed import lanes as LN
    assert LN.canonical_lane_draw(0) == pytest.approx(0.8833108082136426, abs=1e-15)   # splitmix64(0) = 0xE220A8397B1DCDAF
    d = LN.LaneDistribution.from_weights([(256, 2.0), (64, 1.0), (1024, 1.0)])
    assert [l for l, _ in d.entries] == [64, 256, 1024]
    assert d.mass() == pytest.approx(1.0) and d.entries[1][1] == pytest.approx(0.5)
    assert d.effective_sample_size() == pytest.approx(1 / (0.25 ** 2 * 2 + 0.25))
    s = d.sample(0)
    assert s["params"]["lane"] == 1024 and s["seed"] == "0" and s["rng_algorithm"] == "splitmix64_u53_v1"
    d.validate_sample(s)
    with pytest.raises(LN.LaneProbabilityError):
        d.validate_sample({**s, "support_index": "0"})
    med = LN.consensus_lane_params(d, "median")
    mean = LN.consensus_lane_params(d, "weighted_mean")
    assert med["params"]["lane"] == 256 and mean["params"]["lane"] == 400        # (16 + 128 + 256)
    assert med["report"]["input_sha256"] == d.sha256() and med["report"]["output_sha256"] != mean["report"]["output_sha256"]
    for bad in ([], [(0, 1.0)], [(8, 1.0), (8, 2.0)], [(8, float("nan"))], [(8, -1.0)]):
        with pytest.raises(LN.LaneProbabilityError):
            LN.LaneDistribution.from_weights(bad)
    with pytest.raises(LN.LaneProbabilityError):
        LN.LaneDistribution.from_probabilities([(8, 0.5), (16, 0.4)])             # mass 0.9 is rejected, not repaired
    with pytest.raises(LN.LaneProbabilityError):
        LN.parse_policy("mode")
    merged = LN.merge_votes([(128, 1.0), (256, 1.0), (128, 2.0)])
    assert merged.entries[0] == (128, pytest.approx(0.75))
    assert LN.distributed_consensus([(512, 1.0)])["params"]["lane"] == 512        # no process group: local votes


def _lane_rank(rank, world, port, q):
    import os
    import torch.distributed as dist
    from spiraltorch_b200.distributed import lanes as LN
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = LN.distributed_consensus([(128, 1.0)] if rank == 0 else [(512, 1.0), (128, 0.5)], policy="median")
    q.put((rank, out["params"]["lane"], out["report"]["output_sha256"]))
    dist.destroy_process_group()


def test_lane_consensus_across_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_lane_rank, args=(r, 2, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert res[0][1] == res[1][1] == 128 and res[0][2] == res[1][2]
