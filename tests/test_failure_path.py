"""Failure detection without a GPU fault.

* On the GPU (world size 1): a fused GEMM -> reduce-scatter launch is given an arrival target one above
  what will ever be delivered (a healthy peer that withholds one signal) and a wait limit of a few
  milliseconds.  The kernel must return by itself, leave ``ERR_FLAG_TIMEOUT`` with the site code of the
  local-tile wait in the error record, ``native.poll()`` must raise ``DeviceWaitTimeout``, and the NEXT
  launch on the same CUDA context (same fused context, correct target) must succeed.  Nothing traps,
  faults or spins without a limit.
* On CPU ranks (gloo): ``agree_on_status`` / ``FusedTPContext.check`` semantics - one rank that saw a
  failure makes every rank report it, so nobody commits a partial result and their collectives stay paired.

Semantics follow the reference's rendezvous rule that a failed participant makes every participant leave
with an error (crates/spiral-selfsup/src/trainer/distributed.rs:407-423).
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spiraltorch_b200.ops import native


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_context_stays_usable():
    from spiraltorch_b200.parallel.symm import FusedTPContext
    torch.manual_seed(0)
    dev = "cuda"
    tp = FusedTPContext(None, device=dev)
    T, K, N = 512, 256, 512
    x = torch.randn(T, K, device=dev).bfloat16()
    w = torch.randn(N, K, device=dev).bfloat16()
    good = tp.gemm_rs(x, w)
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0
    native.set_wait_timeout(5e-3)
    try:
        tp.gemm_rs(x, w, _withhold=1)           # one arrival will never come
        torch.cuda.synchronize()                # returns: the wait is bounded
        code, detail, _block, count = native.read_error_word(clear=False)
        assert code == 2, (code, hex(detail))   # ERR_FLAG_TIMEOUT
        assert detail == 0xA603, hex(detail)    # the local-tile wait of the reduce-scatter epilogue
        assert count >= 1
        with pytest.raises(native.DeviceWaitTimeout):
            native.poll()
        assert native.read_error_word()[0] == 0     # poll() cleared the record
    finally:
        native.set_wait_timeout(None)
    again = tp.gemm_rs(x, w)                    # same context, same CUDA context: must work
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0
    assert torch.equal(again, good)
    ref = x.float() @ w.float().T
    assert ((again.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2


@pytest.mark.gpu
def test_fused_context_check_marks_context_unusable():
    from spiraltorch_b200.parallel.symm import FusedContextBroken, FusedTPContext
    dev = "cuda"
    tp = FusedTPContext(None, device=dev)
    x = torch.randn(256, 128, device=dev).bfloat16()
    w = torch.randn(256, 128, device=dev).bfloat16()
    native.set_wait_timeout(5e-3)
    try:
        tp.gemm_rs(x, w, _withhold=1)
        with pytest.raises(native.DeviceWaitTimeout):
            tp.check(synchronize=True)
    finally:
        native.set_wait_timeout(None)
    assert not tp.usable
    with pytest.raises(FusedContextBroken):
        tp.gemm_rs(x, w)
    fresh = FusedTPContext(None, device=dev)    # a rebuilt context works on the same CUDA context
    fresh.gemm_rs(x, w)
    fresh.check(synchronize=True)


@pytest.mark.gpu
def test_launchers_refuse_host_operands_before_any_launch():
    from spiraltorch_b200.ops import attention as A
    from spiraltorch_b200.ops import gemm as G
    from spiraltorch_b200.parallel.symm import FusedTPContext
    a = torch.randn(128, 64, device="cuda").bfloat16()
    b_host = torch.randn(128, 64).bfloat16()
    with pytest.raises(ValueError):
        G.gemm(a, b_host)
    with pytest.raises(ValueError):
        G.gemm(a, a, bias=torch.zeros(128).bfloat16())
    q = torch.randn(1, 128, 2, 64, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        A.attention_forward(q, q.cpu(), q.cpu())
    with pytest.raises(ValueError):
        A.attention_forward(q, q[:, :, :1], q[:, :, :1])        # K/V with fewer heads than Q
    with pytest.raises(ValueError):
        A.attention_forward(q, q, q[:, :64])                    # K and V of different lengths
    tp = FusedTPContext(None, device="cuda")
    with pytest.raises(ValueError):
        tp.ag_gemm(a, b_host)
    with pytest.raises(ValueError):
        tp.gemm_rs(a, a, residual=torch.zeros(128, 128).bfloat16())
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


# ---- CPU ranks -------------------------------------------------------------------------------
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _agree_worker(rank: int, world: int, port: int, bad_rank: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from spiraltorch_b200.parallel.symm import agree_on_status
        first = agree_on_status(dist.group.WORLD, True)                 # everybody healthy
        second = agree_on_status(dist.group.WORLD, rank != bad_rank)    # one rank saw a timeout
        third = agree_on_status(dist.group.WORLD, True)                 # collectives are still paired
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(f"{int(first)}{int(second)}{int(third)}")
    finally:
        dist.destroy_process_group()


def test_one_failed_rank_makes_every_rank_report_failure(tmp_path):
    world = 3
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_agree_worker, args=(r, world, port, 1, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in range(world):
        assert (tmp_path / f"r{r}.txt").read_text() == "101"


def test_agree_on_status_single_process():
    from spiraltorch_b200.parallel.symm import agree_on_status
    assert agree_on_status(None, True) is True
    assert agree_on_status(None, False) is False
