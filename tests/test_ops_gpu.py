"""Numerics of every sm_100a kernel against a plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from spiraltorch_b200.ops import attention as A
from spiraltorch_b200.ops import elementwise as E
from spiraltorch_b200.ops import gemm as G
from spiraltorch_b200.ops import loss as L
from spiraltorch_b200.ops import native
from spiraltorch_b200.ops import norm as N
from spiraltorch_b200.ops import optim as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def _no_device_error():
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1000, 776, 520), (4096, 128, 1024), (77, 40, 8)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    torch.manual_seed(1)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV).bfloat16()
    c = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = (a.float().T if a_mn else a.float()) @ (b.float() if b_mn else b.float().T)
    assert _rel(c, ref) < 1e-2
    _no_device_error()


def test_gemm_epilogues():
    torch.manual_seed(2)
    M, N, K = 384, 520, 264
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    res = torch.randn(M, N, device=DEV).bfloat16()
    aux = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = G.gemm(a, b, bias=bias, act="gelu", residual=res, alpha=0.5, aux_out=aux)
    pre = 0.5 * (a.float() @ b.float().T) + bias.float()
    ref = torch.nn.functional.gelu(pre, approximate="tanh") + res.float()
    assert _rel(out, ref) < 1e-2 and _rel(aux, pre) < 1e-2
    out = G.gemm(a, b, act="gelu_bwd", aux_in=res)
    assert _rel(out, (a.float() @ b.float().T) * G.gelu_tanh_grad(res.float())) < 1e-2
    out = G.gemm(a, b, bias=bias, act="relu")
    assert _rel(out, torch.relu(a.float() @ b.float().T + bias.float())) < 1e-2
    acc = torch.ones(M, N, device=DEV)
    G.gemm(a, b, out=acc, accumulate=True)
    assert _rel(acc, 1 + a.float() @ b.float().T) < 1e-2
    ab = torch.randn(5, 200, 64, device=DEV).bfloat16()
    bb = torch.randn(5, 136, 64, device=DEV).bfloat16()
    assert _rel(G.gemm(ab, bb), ab.float() @ bb.float().transpose(1, 2)) < 1e-2
    _no_device_error()


def test_linear_autograd():
    torch.manual_seed(3)
    x = torch.randn(256, 128, device=DEV).bfloat16().requires_grad_(True)
    w = torch.randn(192, 128, device=DEV).bfloat16().requires_grad_(True)
    b = torch.randn(192, device=DEV).bfloat16().requires_grad_(True)
    y = G.linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    (xf @ wf.T + bf).backward(dy.float())
    assert _rel(x.grad, xf.grad) < 2e-2 and _rel(w.grad, wf.grad) < 2e-2 and _rel(b.grad, bf.grad) < 2e-2


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,S,H,causal", [(1, 128, 1, True), (2, 512, 3, False), (1, 300, 2, True), (2, 1024, 2, True)])
def test_attention_fwd_bwd(D, B, S, H, causal):
    torch.manual_seed(4)
    qkv = torch.randn(B, S, 3, H, D, device=DEV).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    do = torch.randn(B, S, H, D, device=DEV).bfloat16()
    o, lse = A.attention_forward(q, k, v, causal)
    dq, dk, dv = A.attention_backward(q, k, v, o, lse, do, causal)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ro, rl = A.attention_reference(qf, kf, vf, causal, 1 / math.sqrt(D))
    g = torch.autograd.grad(ro, (qf, kf, vf), do.float())
    assert (o.float() - ro).abs().max().item() < 2e-2
    assert (lse - rl).abs().max().item() < 1e-3
    for mine, ref in zip((dq, dk, dv), g):
        assert _rel(mine, ref) < 2e-2
    _no_device_error()


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("B,Sq,Sk,H,D,causal", [(4, 2048, 2048, 8, 128, True), (1, 200, 333, 2, 128, False),
                                                  (3, 640, 640, 5, 64, True), (1, 129, 129, 1, 64, True),
                                                  (2, 384, 1000, 2, 64, False)])
def test_attention_fwd_pair_and_single_tile_kernels(pair, B, Sq, Sk, H, D, causal):
    """Both forward kernels (two query tiles per CTA with P and O in tensor memory; one tile per CTA) against the fp32
    statement: more work items than SMs, ragged tails in queries and keys, an odd number of query tiles, and logits
    whose running maximum grows by more than the lazy-rescale step."""
    from spiraltorch_b200.ops import attention as A
    torch.manual_seed(7)
    q = torch.randn(B, Sq, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Sk, H, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Sk, H, D, device="cuda", dtype=torch.bfloat16)
    # later keys get larger logits, so the running maximum keeps rising across KV tiles
    ramp = torch.linspace(0.5, 4.0, Sk, device="cuda").view(1, Sk, 1, 1)
    k = (k * ramp).to(torch.bfloat16)
    was = A.pair_kernel_enabled()
    try:
        A.set_pair_kernel(pair)
        o, lse = A.attention_forward(q, k, v, causal=causal)
        torch.cuda.synchronize()
    finally:
        A.set_pair_kernel(was)
    o_ref, lse_ref = A.attention_reference(q.float(), k.float(), v.float(), causal, 1.0 / D ** 0.5)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref).abs().max().item() < 3e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("rms", [True, False])
@pytest.mark.parametrize("rows,d", [(64, 768), (1000, 2048), (33, 8192), (7, 264)])
def test_norm_fwd_bwd(rms, rows, d):
    torch.manual_seed(5)
    x = torch.randn(rows, d, device=DEV).bfloat16()
    res = torch.randn(rows, d, device=DEV).bfloat16()
    gamma = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    beta = None if rms else (0.1 * torch.randn(d, device=DEV)).bfloat16()
    dy = torch.randn(rows, d, device=DEV).bfloat16()
    y, s, mean, rstd = N.norm_forward(x, gamma, beta, 1e-5, rms, residual=res)
    ry, rs, rmean, rrstd = N.norm_reference(x, gamma, beta, 1e-5, rms, residual=res)
    assert _rel(y, ry) < 1e-2 and _rel(s, rs) < 1e-2 and _rel(rstd, rrstd) < 1e-3
    dg = torch.zeros(d, device=DEV)
    db = None if rms else torch.zeros(d, device=DEV)
    dx = N.norm_backward(dy, s, gamma, mean, rstd, rms, dg, db, False, dres=res)
    xs = s.float().requires_grad_(True)
    gf = gamma.float().requires_grad_(True)
    bf = None if rms else beta.float().requires_grad_(True)
    yy = N.norm_reference(xs, gf, bf, 1e-5, rms)[0]
    yy.backward(dy.float())
    assert _rel(dx, xs.grad + res.float()) < 2e-2
    assert _rel(dg, gf.grad) < 2e-2
    if not rms:
        assert _rel(db, bf.grad) < 2e-2


def test_rope_roundtrip_and_reference():
    torch.manual_seed(6)
    T, H, D, S = 512, 6, 128, 128
    x = torch.randn(T, 3 * H * D, device=DEV).bfloat16()
    ref = x.clone()
    cos, sin = E.rope_tables(S, D, 10000.0, DEV)
    view = ref[:, : 2 * H * D].reshape(T, 2 * H, D)
    expect = E.rope_reference(view, cos, sin, S, False)
    y = E.rope_(x.clone(), 2 * H, D, S)
    assert _rel(y[:, : 2 * H * D].reshape(T, 2 * H, D), expect) < 1e-2
    assert torch.equal(y[:, 2 * H * D:], x[:, 2 * H * D:])
    back = E.rope_(y.clone(), 2 * H, D, S, backward=True)
    assert _rel(back, x) < 2e-2


@pytest.mark.parametrize("V", [50304, 256, 1000])
def test_cross_entropy(V):
    torch.manual_seed(7)
    rows = 257
    ld = (V + 7) // 8 * 8
    buf = (3 * torch.randn(rows, ld, device=DEV)).bfloat16()
    logits = buf[:, :V]
    tgt = torch.randint(0, V, (rows,), device=DEV)
    tgt[5] = L.IGNORE_INDEX
    lf = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=L.IGNORE_INDEX)
    ref.backward()
    x = logits.clone() if V % 8 == 0 else logits
    x = x.detach().requires_grad_(True)
    loss = L.cross_entropy(x, tgt)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3
    assert (x.grad.float() - lf.grad).abs().max().item() < 2e-4 + 1e-2 * lf.grad.abs().max().item()


def test_embedding_and_colsum_and_softmax():
    torch.manual_seed(8)
    V, d, T, S = 300, 256, 1024, 128
    w = torch.randn(V, d, device=DEV).bfloat16()
    pos = torch.randn(S, d, device=DEV).bfloat16()
    idx = torch.randint(0, V, (T,), device=DEV)
    out = E.embedding_forward(idx, w, pos, S)
    assert _rel(out, w[idx].float() + pos[torch.arange(T, device=DEV) % S].float()) < 1e-2
    shard = E.embedding_forward(idx, w[100:200].contiguous(), None, 0, vocab_start=100)
    ok = (idx >= 100) & (idx < 200)
    assert torch.equal(shard[~ok], torch.zeros_like(shard[~ok])) and torch.equal(shard[ok], w[idx[ok]])
    dy = torch.randn(T, d, device=DEV).bfloat16()
    dw = torch.zeros(V, d, device=DEV)
    dpos = torch.zeros(S, d, device=DEV)
    E.embedding_backward(idx, dy, dw, dpos, S)
    rw = torch.zeros(V, d, device=DEV).index_add_(0, idx, dy.float())
    assert _rel(dw, rw) < 1e-3
    assert _rel(dpos, dy.float().view(-1, S, d).sum(0)) < 1e-3
    cs = E.colsum(dy)
    assert _rel(cs, dy.float().sum(0)) < 1e-3
    for shape in ((1001, 264), (77, 100), (5, 8)):         # ragged row counts; 100 columns take the scalar kernel
        t = torch.randn(*shape, device=DEV).bfloat16()
        assert _rel(E.colsum(t), t.float().sum(0)) < 1e-3
    x = torch.randn(37, 1000, device=DEV)
    y, h = E.row_softmax(x, hardmax=True)
    assert _rel(y, torch.softmax(x, -1)) < 1e-4
    assert torch.equal(h.argmax(-1), x.argmax(-1)) and h.sum().item() == 37
    for kind in ("gelu", "relu"):
        t = torch.randn(64, 256, device=DEV).bfloat16().requires_grad_(True)
        f = E.gelu if kind == "gelu" else E.relu
        f(t).backward(dy[:64])
        tf = t.detach().float().requires_grad_(True)
        rf = torch.nn.functional.gelu(tf, approximate="tanh") if kind == "gelu" else torch.relu(tf)
        rf.backward(dy[:64].float())
        assert _rel(t.grad, tf.grad) < 2e-2


def test_fused_optimizers():
    torch.manual_seed(9)
    n = 100_003
    g = torch.randn(n, device=DEV)
    master = torch.randn(n, device=DEV)
    m, v = torch.rand(n, device=DEV), torch.rand(n, device=DEV)
    w = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ref = [t.clone() for t in (g, master, m, v)]
    coef = torch.tensor([0.5], device=DEV)
    O.adamw_step(g, master, m, v, w, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3,
                 grad_scale=0.25, scale_tensor=coef, zero_grad=True)
    O.adamw_reference(ref[0], ref[1], ref[2], ref[3], None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, 0.125, False)
    assert _rel(master, ref[1]) < 1e-5 and _rel(m, ref[2]) < 1e-5 and _rel(v, ref[3]) < 1e-5
    assert _rel(w, master) < 1e-2 and g.abs().max().item() == 0
    ss = torch.zeros(1, device=DEV)
    x = torch.randn(50_001, device=DEV)
    O.sumsq(x, ss)
    assert abs(ss.item() - x.pow(2).sum().item()) / x.pow(2).sum().item() < 1e-4
    c, nrm = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    O.clip_coef(ss, 1.0, 1.0, c, nrm)
    assert abs(c.item() - 1.0 / (x.norm().item() + 1e-6)) < 1e-5
    # Amegagrad tapes against the CPU restatement
    wt = torch.randn(33, 70, device=DEV) * 0.3
    gt = torch.zeros_like(wt)
    wave = torch.randn_like(wt)
    wc, gc = wt.cpu().clone(), gt.cpu().clone()
    kw = dict(curvature=-1.0, tol=1e-6, saturation=1e6, porosity=0.2)
    O.hyper_accumulate(gt, wave, **kw)
    O.hyper_accumulate(gc, wave.cpu(), **kw)
    assert _rel(gt.cpu(), gc) < 1e-5
    rt = torch.randn_like(wt)
    rc = rt.cpu().clone()
    O.hyper_apply(wt, gt, rt, curvature=-1.0, lr=0.05, lr_real=0.01, tol=1e-6, saturation=1e6, porosity=0.2)
    O.hyper_apply(wc, gc, rc, curvature=-1.0, lr=0.05, lr_real=0.01, tol=1e-6, saturation=1e6, porosity=0.2)
    assert _rel(wt.cpu(), wc) < 1e-4 and gt.abs().max().item() == 0 and rt.abs().max().item() == 0
    pr = O.project_to_poincare(wave, -0.5)
    assert _rel(pr.cpu(), O.project_to_poincare(wave.cpu(), -0.5)) < 1e-5


def test_gemm_weight_gradient_split_k():
    torch.manual_seed(10)
    T, M, N = 8192, 2048, 512
    dy = torch.randn(T, M, device=DEV).bfloat16()
    x = torch.randn(T, N, device=DEV).bfloat16()
    assert G._split_k(M, N, T) > 1  # this shape takes the split-K path
    acc = torch.full((M, N), 0.5, device=DEV)
    G.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    assert _rel(acc, 0.5 + dy.float().T @ x.float()) < 1e-2
    _no_device_error()


@pytest.mark.gpu
def test_recurrent_gate_kernels_match_reference():
    from spiraltorch_b200.ops import recurrent as R
    torch.manual_seed(0)
    B, H = 37, 96
    z = torch.randn(B, 4 * H, device="cuda")
    c0 = torch.randn(B, H, device="cuda")
    n0 = R.launch_count
    h, c, act = R.lstm_gate_forward(z, c0)
    hr, cr, ar = R.lstm_gate_reference(z, c0)
    assert torch.allclose(h, hr, atol=1e-5) and torch.allclose(c, cr, atol=1e-5) and torch.allclose(act, ar, atol=1e-5)
    # autograd through the kernel pair against autograd through the PyTorch statement
    z1, c1 = z.clone().requires_grad_(True), c0.clone().requires_grad_(True)
    z2, c2 = z.clone().requires_grad_(True), c0.clone().requires_grad_(True)
    h1, cc1 = R.lstm_gate(z1, c1)
    h2, cc2, _ = R.lstm_gate_reference(z2, c2)
    gh, gc = torch.randn_like(h1), torch.randn_like(cc1)
    torch.autograd.backward([h1, cc1], [gh, gc])
    torch.autograd.backward([h2, cc2], [gh, gc])
    assert torch.allclose(z1.grad, z2.grad, atol=1e-5) and torch.allclose(c1.grad, c2.grad, atol=1e-5)
    zw = torch.randn(B, 2 * H, device="cuda", requires_grad=True)
    y = R.wave_gate(zw)
    yr = torch.tanh(zw[:, :H]) * torch.sigmoid(zw[:, H:])
    g = torch.randn_like(y)
    (d1,) = torch.autograd.grad(y, zw, g)
    (d2,) = torch.autograd.grad(yr, zw, g)
    assert torch.allclose(y, yr, atol=1e-6) and torch.allclose(d1, d2, atol=1e-6)
    x = torch.randn(B, 5 * 16, device="cuda")
    assert torch.equal(R.sequence_last_step(x, 5, 16), x.reshape(B, 5, 16)[:, -1])
    assert R.launch_count >= n0 + 6
    native.raise_on_device_error()


@pytest.mark.gpu
def test_module_moved_to_gpu_keeps_tapes_with_weights():
    """A module built on the host with hypergrad tapes and then moved: the tapes must follow the weights
    (a host accumulator handed to the fused step kernel would be a host pointer on the device)."""
    import spiraltorch_b200 as st
    from spiraltorch_b200.nn import gnn
    adj = torch.zeros(6, 6)
    for i in range(6):
        adj[i, (i + 1) % 6] = adj[(i + 1) % 6, i] = 1.0
    net = gnn.ZSpaceGraphNetwork("g", gnn.GraphContext.from_adjacency(adj), [3, 8, 1], learning_rate=0.3)
    model = gnn.ZSpaceGraphRegressor(net, gnn.GraphReadout("mean"))
    model.to("cuda")
    assert all(p.hypergrad.gradient.is_cuda for p in model.parameters())
    loss = st.nn.MeanSquaredError()
    g = torch.Generator().manual_seed(0)
    first = last = None
    for _ in range(40):
        x = torch.randn(6, 3, generator=g)
        xt, yt = st.Tensor._wrap(x.cuda()), st.Tensor._wrap(x[:, 0].mean().reshape(1, 1).cuda())
        pred = model.forward(xt)
        val = float(loss.forward(pred, yt).torch())
        first = val if first is None else first
        last = val
        model.backward(xt, loss.backward(pred, yt))
        model.apply_step(1e-2)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    assert all(torch.isfinite(p.value).all() for p in model.parameters())
    lin = st.nn.Linear(4, 4, name="l")
    lin.attach_hypergrad(-1.0, 1e-2)
    lin.to("cuda")
    lin.backward(st.Tensor._wrap(torch.randn(2, 4).cuda()), st.Tensor._wrap(torch.randn(2, 4).cuda()))
    lin.apply_step(1e-2)
    torch.cuda.synchronize()


def test_deterministic_reduction_gives_bit_identical_gradients(monkeypatch):
    """With SPIRAL_DETERMINISTIC_REDUCTION the split-K weight gradients and the embedding scatter-add take their
    fixed-order forms: two runs of the same step give bit-identical flat gradients (and agree with the default,
    atomics-based path to rounding)."""
    from spiraltorch_b200.models.gpt import GPTConfig, GPTModel
    cfg = GPTConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=2, ffn=1024, seq_len=1024, init_std=0.05)
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (8, 1024), device="cuda")       # few distinct ids: many collisions in the scatter-add
    targets = torch.randint(0, 512, (8, 1024), device="cuda")

    def run():
        m = GPTModel(cfg, device="cuda", seed=9)
        m.forward_backward(tokens, targets)
        torch.cuda.synchronize()
        return m.flat_grad.clone()
    monkeypatch.setenv("SPIRAL_DETERMINISTIC_REDUCTION", "1")
    a, b = run(), run()
    assert torch.equal(a, b)
    monkeypatch.setenv("SPIRAL_DETERMINISTIC_REDUCTION", "0")
    c = run()
    assert ((a - c).norm() / a.norm()).item() < 1e-3


def test_cuda_graph_replay_matches_eager_forward_backward():
    """The captured forward/backward of a small GPT gives the same loss and gradients as the eager call, replay
    after replay, and leaves the gradient buffer untouched by its warm-up and capture passes."""
    from spiraltorch_b200.models.gpt import GPTConfig, GPTModel
    from spiraltorch_b200.training import GraphedForwardBackward
    cfg = GPTConfig(vocab_size=256, d_model=128, n_layers=2, n_heads=2, ffn=256, seq_len=128, init_std=0.05,
                    norm="layer", positional="learned")
    a, b = GPTModel(cfg, device="cuda", seed=4), GPTModel(cfg, device="cuda", seed=4)
    torch.manual_seed(0)
    batches = [(torch.randint(0, 256, (4, 128), device="cuda"), torch.randint(0, 256, (4, 128), device="cuda"))
               for _ in range(3)]
    g = GraphedForwardBackward(b, batches[0])
    assert b.flat_grad.abs().max().item() == 0
    for tok, tgt in batches:
        la = a.forward_backward(tok, tgt)
        lb = g(tok, tgt)
        assert abs(la.item() - lb.item()) < 1e-4
    torch.cuda.synchronize()
    assert g.replays == 3
    assert ((a.flat_grad - b.flat_grad).norm() / a.flat_grad.norm()).item() < 1e-3
