"""Fused compute+collective kernels on one GPU (world size 1: the peer is the local device) and,
when at least two GPUs are visible, on two ranks launched with torchrun."""
import os
import subprocess
import sys

import pytest
import torch

from spiraltorch_b200.ops import gemm as G
from spiraltorch_b200.ops import native
from spiraltorch_b200.ops import optim as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def test_ag_gemm_and_gemm_rs_world1():
    from spiraltorch_b200.parallel.symm import FusedTPContext
    torch.manual_seed(0)
    tp = FusedTPContext(None, device=DEV)
    T, K, N = 1024, 512, 768
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    for rep in range(3):  # repeated launches exercise the epoch / cumulative-counter logic
        aux = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        y, x_full = tp.ag_gemm(x, w, key="t", act="gelu", aux_out=aux)
        ref_pre = x.float() @ w.float().T
        assert torch.equal(x_full, x)
        assert _rel(aux, ref_pre) < 1e-2
        assert _rel(y, torch.nn.functional.gelu(ref_pre, approximate="tanh")) < 1e-2
        wt = torch.randn(K, N, device=DEV).bfloat16()
        y2, _ = tp.ag_gemm(x, wt, b_mn=True, key="t2")
        assert _rel(y2, x.float() @ wt.float()) < 1e-2
        res = torch.randn(T, N, device=DEV).bfloat16()
        z = tp.gemm_rs(x, w, residual=res)
        assert _rel(z, ref_pre + res.float()) < 1e-2
        z2 = tp.gemm_rs(x, wt, b_mn=True)
        assert _rel(z2, x.float() @ wt.float()) < 1e-2
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


def test_dp_step_world1_matches_adamw_and_sgd():
    from spiraltorch_b200.parallel.symm import FusedDPStep, PeerSignals, SymmetricHeap
    torch.manual_seed(1)
    heap = SymmetricHeap(None, torch.device(DEV))
    sig = PeerSignals(heap)
    n = 8 * 1000
    for kind in ("adamw", "sgd"):
        grad = heap.empty(n, torch.float32)
        w = heap.empty(n, torch.bfloat16)
        grad.tensor.copy_(torch.randn(n, device=DEV))
        w.tensor.copy_(torch.randn(n, device=DEV).bfloat16())
        g0 = grad.tensor.clone()
        master = w.tensor.float().clone()
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        dp = FusedDPStep(heap, sig, grad, w, kind=kind, bucket_elems=4096)
        coef = torch.tensor([0.5], device=DEV)
        dp.step(lr=1e-2, weight_decay=0.1, grad_scale=2.0, scale_tensor=coef, momentum=0.9)
        if kind == "adamw":
            O.adamw_reference(g0, master, m, v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, False)
        else:
            gg = g0 * 1.0 + 0.1 * master
            m.mul_(0.9).add_(gg)
            master.sub_(1e-2 * m)
        assert _rel(w.tensor, master) < 1e-2
        got_master = torch.cat([b[2] for b in dp.buckets])
        assert _rel(got_master, master) < 1e-5
        assert grad.tensor.abs().max().item() == 0
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


def test_gpt_fused_context_matches_plain_world1():
    from spiraltorch_b200.models.gpt import GPTConfig, GPTModel
    from spiraltorch_b200.parallel.symm import FusedTPContext
    cfg = GPTConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=2, ffn=512, seq_len=256, init_std=0.05)
    a = GPTModel(cfg, device=DEV, seed=3)
    b = GPTModel(cfg, device=DEV, seed=3, tp=FusedTPContext(None, device=DEV))
    tokens = torch.randint(0, 512, (2, 256), device=DEV)
    targets = torch.randint(0, 512, (2, 256), device=DEV)
    la = a.forward_backward(tokens, targets)
    lb = b.forward_backward(tokens, targets)
    assert abs(la.item() - lb.item()) < 2e-2
    rel = (a.flat_grad - b.flat_grad).norm() / a.flat_grad.norm()
    assert rel.item() < 2e-2
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_kernels_two_ranks():
    script = os.path.join(os.path.dirname(__file__), "multi_gpu", "run_fused_tp.py")
    import socket
    with socket.socket() as sock:           # a free port: the machine is shared with other jobs
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), script],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "FUSED_TP_OK" in proc.stdout


def test_fused_info_nce_world1_matches_reference():
    from spiraltorch_b200.parallel.contrastive import FusedInfoNCE
    from spiraltorch_b200.parallel.symm import PeerSignals, SymmetricHeap
    from spiraltorch_b200.selfsup import info_nce_torch
    torch.manual_seed(5)
    heap = SymmetricHeap(None, torch.device(DEV))
    op = FusedInfoNCE(heap, PeerSignals(heap), rows=1024, dim=256, temperature=0.1)
    base = torch.randn(1024, 256, device=DEV)
    for rep in range(2):
        a = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
        p = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
        loss = op.apply(a, p)
        loss.backward()
        a2 = a.detach().bfloat16().float().requires_grad_(True)
        p2 = p.detach().bfloat16().float().requires_grad_(True)
        ref, _ = info_nce_torch(a2, p2, 0.1, normalize=False)
        ref.backward()
        assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
        assert _rel(a.grad, a2.grad) < 5e-2 and _rel(p.grad, p2.grad) < 5e-2
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


def test_contrastive_encoder_learns():
    from spiraltorch_b200.models.contrastive import ContrastiveEncoder, contrastive_step
    torch.manual_seed(6)
    enc = ContrastiveEncoder(device=DEV)
    opt = torch.optim.AdamW(enc.parameters(), lr=1e-3)
    base = torch.randn(1024, 512, device=DEV)
    losses = []
    for i in range(20):
        opt.zero_grad(set_to_none=True)
        losses.append(contrastive_step(enc, base, seed=i).item())
        opt.step()
    assert losses[-1] < losses[0] and losses[-1] < 1.0, losses


def test_dp_step_two_phase_clips_by_global_norm_world1():
    """Global-norm clipping inside the fused data-parallel step: reduce + squared norm per bucket, then the clipped
    update; the result must equal clipping the whole gradient first and running the plain fused optimizer."""
    from spiraltorch_b200.parallel.symm import FusedDPStep, PeerSignals, SymmetricHeap
    torch.manual_seed(2)
    heap = SymmetricHeap(None, torch.device(DEV))
    sig = PeerSignals(heap)
    n = 8 * 3000
    for kind, max_norm in (("adamw", 0.5), ("sgd", 1e9)):        # one case that clips, one that does not
        grad, w = heap.empty(n, torch.float32), heap.empty(n, torch.bfloat16)
        grad.tensor.copy_(torch.randn(n, device=DEV) * 0.1)
        w.tensor.copy_(torch.randn(n, device=DEV).bfloat16())
        g0, master = grad.tensor.clone(), w.tensor.float().clone()
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        dp = FusedDPStep(heap, sig, grad, w, kind=kind, bucket_elems=8192, max_grad_norm=max_norm)
        assert len(dp.buckets) > 1
        dp.step(lr=1e-2, weight_decay=0.1, momentum=0.9)
        norm = g0.norm()
        assert abs(dp.grad_norm().item() - norm.item()) < 1e-3 * norm.item()
        gc = g0 * (max_norm / (norm + 1e-6)) if norm > max_norm else g0
        if kind == "adamw":
            O.adamw_reference(gc, master, m, v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, False)
        else:
            m.mul_(0.9).add_(gc + 0.1 * master)
            master.sub_(1e-2 * m)
        assert _rel(w.tensor, master) < 1e-2
        assert _rel(torch.cat([b[2] for b in dp.buckets]), master) < 1e-5
        assert grad.tensor.abs().max().item() == 0
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


@pytest.mark.parametrize("shape", [(64, 256, 128), (50, 70, 11)])
def test_info_nce_grad_kernel_matches_formula_in_both_orientations(shape):
    from spiraltorch_b200.parallel import contrastive as C
    R, cols, off = shape
    torch.manual_seed(R)
    logits = torch.randn(R, cols, device=DEV) * 3
    lse = torch.logsumexp(logits, dim=1)
    coef = torch.tensor([0.37 / R], device=DEV)
    before = C.launch_count
    dl, dl_t = C.info_nce_grad(logits, lse, coef, off)
    assert C.launch_count == before + 1 and dl.dtype == torch.bfloat16 and dl_t.shape == (cols, R)
    want = torch.softmax(logits, dim=1)
    want[torch.arange(R), torch.arange(R) + off] -= 1.0
    want = want * coef
    assert float((dl.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    assert torch.equal(dl_t, dl.t().contiguous())
    cpu = C.info_nce_grad(logits.cpu(), lse.cpu(), coef.cpu(), off)[0]
    assert float((cpu.float() - dl.float().cpu()).abs().max()) <= 1e-2 * float(want.abs().max())
