"""The public ``st.nn`` / ``st.Tensor`` API on CUDA must run on the repository's kernels and agree with
the CPU path (fp32 PyTorch) to bf16 tolerance: per-op forward/backward checks of ``nn.functional``,
attention with additive biases and ragged lengths, and two small models trained through
``SpiralSession("cuda").trainer()`` whose per-op launch counters prove the kernel path was taken."""
import math

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200.nn import functional as Fn
from spiraltorch_b200.ops import attention as A
from spiraltorch_b200.ops import conv as C
from spiraltorch_b200.ops import gemm as G
from spiraltorch_b200.ops import native, norm as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def _bf(*ts):
    """Round test inputs to bf16-representable values: the kernels round operands to bf16 at their boundary, and
    comparing like with like keeps ReLU / max-pool decisions identical on both paths."""
    out = tuple(t.bfloat16().float() for t in ts)
    return out if len(out) > 1 else out[0]


def _grads(fn, inputs, dy):
    leaves = [t.detach().clone().requires_grad_(True) if t is not None and t.is_floating_point() else t for t in inputs]
    y = fn(*leaves)
    gs = torch.autograd.grad(y, [t for t in leaves if t is not None and t.requires_grad], dy.to(y.device))
    return y.detach(), gs


@pytest.mark.parametrize("act", [None, "relu", "gelu"])
def test_linear_forward_and_gradients(act):
    torch.manual_seed(0)
    x, w, b, dy = _bf(torch.randn(96, 40), torch.randn(40, 72) * 0.2, torch.randn(1, 72), torch.randn(96, 72))
    before = G.launch_count
    y_g, g_g = _grads(lambda a, ww, bb: Fn.linear(a, ww, bb, act), [x.to(DEV), w.to(DEV), b.to(DEV)], dy)
    assert G.launch_count - before == 3          # forward, data gradient, weight gradient on the tcgen05 GEMM
    y_c, g_c = _grads(lambda a, ww, bb: Fn.linear(a, ww, bb, act), [x, w, b], dy)
    assert _rel(y_g, y_c) < 2e-2
    for a, c in zip(g_g, g_c):
        assert _rel(a, c) < 3e-2


def test_layer_norm_with_residual_forward_and_gradients():
    torch.manual_seed(1)
    x, r, g, b, dy = _bf(torch.randn(200, 64), torch.randn(200, 64), 1 + 0.1 * torch.randn(1, 64),
                         0.1 * torch.randn(1, 64), torch.randn(200, 64))
    before = N.launch_count
    y_g, g_g = _grads(lambda a, gg, bb, rr: Fn.layer_norm(a, gg, bb, 1e-5, rr), [t.to(DEV) for t in (x, g, b, r)], dy)
    assert N.launch_count > before
    y_c, g_c = _grads(lambda a, gg, bb, rr: Fn.layer_norm(a, gg, bb, 1e-5, rr), [x, g, b, r], dy)
    assert _rel(y_g, y_c) < 3e-2
    for a, c in zip(g_g, g_c):
        assert _rel(a, c) < 4e-2


def test_embedding_forward_and_gradient():
    torch.manual_seed(2)
    w, dy = _bf(torch.randn(50, 32), torch.randn(63, 32))
    ids = torch.randint(0, 50, (7, 9))
    y_g, g_g = _grads(lambda ww: Fn.embedding(ids.to(DEV), ww), [w.to(DEV)], dy)
    y_c, g_c = _grads(lambda ww: Fn.embedding(ids, ww), [w], dy)
    assert _rel(y_g, y_c) < 1e-2 and _rel(g_g[0], g_c[0]) < 2e-2


@pytest.mark.parametrize("shape", [
    # (N, C, H, W, OC, kernel, stride, padding)
    (4, 64, 16, 16, 64, (3, 3), (1, 1), (1, 1)),      # implicit GEMM through 4-D TMA boxes
    (2, 8, 12, 12, 16, (3, 3), (1, 1), (1, 1)),       # 3x3 with few channels: im2col kernel + GEMM
    (3, 3, 11, 9, 5, (5, 3), (2, 1), (2, 0)),         # general geometry: unfold + GEMM
])
def test_conv2d_forward_and_gradients(shape):
    n, c, h, w_, oc, k, s, p = shape
    torch.manual_seed(3)
    x, w, b = _bf(torch.randn(n, c, h, w_), torch.randn(oc, c * k[0] * k[1]) / math.sqrt(c * k[0] * k[1]),
                  torch.randn(1, oc))
    f = lambda xx, ww, bb: Fn.conv2d(xx, ww, bb, k, s, p)          # noqa: E731
    y_c = f(x, w, b)
    dy = _bf(torch.randn_like(y_c))
    before = G.launch_count + C.launch_count
    y_g, g_g = _grads(f, [x.to(DEV), w.to(DEV), b.to(DEV)], dy)
    assert G.launch_count + C.launch_count - before >= 3
    _, g_c = _grads(f, [x, w, b], dy)
    assert _rel(y_g, y_c) < 2e-2
    for a, cc in zip(g_g, g_c):
        assert _rel(a, cc) < 3e-2


def test_max_pool_forward_and_gradient():
    torch.manual_seed(4)
    x, dy = _bf(torch.randn(3, 6, 10, 8), torch.randn(3, 6, 5, 4))
    y_g, g_g = _grads(Fn.max_pool2x2, [x.to(DEV)], dy)
    y_c, g_c = _grads(Fn.max_pool2x2, [x], dy)
    assert _rel(y_g, y_c) < 1e-2 and _rel(g_g[0], g_c[0]) < 1e-2


# ---- attention with biases, lengths, non-causal masks -------------------------------------------
@pytest.mark.parametrize("cfg", [
    # (B, S, H, D, causal, key_bias heads?, attn_bias heads?, lengths)
    (2, 256, 2, 64, False, False, False, None),
    (2, 200, 2, 64, False, True, None, [200, 77]),           # S not a multiple of 128, ragged lengths
    (3, 300, 1, 128, True, False, True, [300, 129, 1]),
    (2, 128, 2, 128, False, None, False, [0, 128]),          # an empty context gives zero rows
    (1, 384, 2, 64, True, True, True, None),
])
def test_attention_bias_and_lengths_forward_backward(cfg):
    B, S, H, D, causal, kb_heads, ab_heads, lengths = cfg
    torch.manual_seed(5)
    q, k, v = (torch.randn(B, S, H, D, device=DEV).bfloat16() for _ in range(3))
    kb = None if kb_heads is None else (torch.randn(B, H, S, device=DEV) if kb_heads else torch.randn(B, S, device=DEV))
    ab = None if ab_heads is None else (torch.randn(B, H, S, S, device=DEV) if ab_heads
                                        else torch.randn(B, S, S, device=DEV))
    ln = None if lengths is None else torch.tensor(lengths, device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    o, lse = A.attention_forward(q, k, v, causal, scale, key_bias=kb, attn_bias=ab, lengths=ln)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    o_ref, lse_ref = A.attention_reference(qf, kf, vf, causal, scale, key_bias=kb, attn_bias=ab, lengths=ln)
    assert _rel(o, o_ref) < 2e-2
    live = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), live)
    assert (lse[live] - lse_ref[live]).abs().max().item() < 2e-2
    do = torch.randn(B, S, H, D, device=DEV).bfloat16()
    dq, dk, dv = A.attention_backward(q, k, v, o, lse, do, causal, scale, key_bias=kb, attn_bias=ab, lengths=ln)
    g = torch.autograd.grad(o_ref, (qf, kf, vf), do.float())
    for got, want in zip((dq, dk, dv), g):
        assert torch.isfinite(got.float()).all()
        assert _rel(got, want) < 4e-2
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


def test_tensor_scaled_dot_attention_with_biases_takes_the_kernel():
    torch.manual_seed(6)
    ctxs, seq, d = 3, 160, 64
    q, k, v = (torch.randn(ctxs * seq, d) for _ in range(3))
    zb, ab = torch.randn(ctxs, seq), torch.randn(ctxs * seq, seq)
    cpu = st.Tensor(q).scaled_dot_attention(st.Tensor(k), st.Tensor(v), contexts=ctxs, sequence=seq,
                                            z_bias=st.Tensor(zb), attn_bias=st.Tensor(ab))
    before = A.launch_count
    gpu = st.Tensor(q).cuda().scaled_dot_attention(st.Tensor(k).cuda(), st.Tensor(v).cuda(), contexts=ctxs,
                                                   sequence=seq, z_bias=st.Tensor(zb).cuda(),
                                                   attn_bias=st.Tensor(ab).cuda())
    assert A.launch_count == before + 1
    assert _rel(gpu.torch(), cpu.torch()) < 2e-2
    ln_cpu = st.Tensor(q).layer_norm_affine_add(st.Tensor(k), st.Tensor(torch.ones(1, d)), st.Tensor(torch.zeros(1, d)))
    ln_gpu = st.Tensor(q).cuda().layer_norm_affine_add(st.Tensor(k).cuda(), st.Tensor(torch.ones(1, d)).cuda(),
                                                       st.Tensor(torch.zeros(1, d)).cuda())
    assert _rel(ln_gpu.torch(), ln_cpu.torch()) < 3e-2


def test_functional_attention_is_differentiable_on_the_kernels():
    torch.manual_seed(7)
    q, k, v = (torch.randn(2, 192, 64, device=DEV, requires_grad=True) for _ in range(3))
    zb = torch.randn(2, 192, device=DEV)
    out = Fn.scaled_dot_attention(q, k, v, z_bias=zb, lengths=torch.tensor([192, 100], device=DEV))
    out.square().sum().backward()
    qc, kc, vc = (t.detach().cpu().requires_grad_(True) for t in (q, k, v))
    ref = Fn.scaled_dot_attention(qc, kc, vc, z_bias=zb.cpu(), lengths=torch.tensor([192, 100]))
    ref.square().sum().backward()
    assert _rel(out.detach(), ref.detach()) < 3e-2
    for a, c in zip((q, k, v), (qc, kc, vc)):
        assert _rel(a.grad, torch.nan_to_num(c.grad)) < 6e-2


# ---- models through the public trainer ------------------------------------------------------------
def _train(device: str, build, epochs: int, lr: float = 5e-2):
    model, loss, batches = build()
    sess = st.SpiralSession(device, seed=11)
    if device == "cuda":
        model.to("cuda")
        batches = [(x.cuda(), y.cuda()) for x, y in batches]
    trainer = sess.trainer(fallback_learning_rate=lr)
    losses = [trainer.train_epoch(model, loss, batches).average_loss for _ in range(epochs)]
    return losses, {n: t.torch().cpu() for n, t in model.state_dict()}


def _readme_model():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 8, generator=g)
    wv = torch.randn(8, 1, generator=g) / math.sqrt(8)
    y = torch.sin(x @ wv) + 0.01 * torch.randn(256, 1, generator=g)
    model = st.nn.Sequential()
    fc1 = st.nn.Linear(8, 32, name="fc1").init_normal(0.3, seed=1)
    head = st.nn.Linear(32, 1, name="head").init_normal(0.3, seed=2)
    model.add(fc1); model.add(st.nn.Relu()); model.add(head)
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 256, 32)]
    return model, st.nn.MeanSquaredError(), batches


def test_readme_model_trains_on_the_kernels_and_matches_cpu():
    counts0 = dict(Fn.launch_counts)
    gemm0 = G.launch_count
    gpu_losses, gpu_state = _train("cuda", _readme_model, 6)
    assert Fn.launch_counts["linear"] - counts0["linear"] >= 6 * 8 * 2        # two Linear layers per batch
    assert G.launch_count - gemm0 >= 6 * 8 * 2 * 3                            # fwd + dgrad + wgrad each
    cpu_losses, cpu_state = _train("cpu", _readme_model, 6)
    assert gpu_losses[-1] < gpu_losses[0]
    for a, b in zip(gpu_losses, cpu_losses):
        assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (gpu_losses, cpu_losses)
    for name in cpu_state:
        assert _rel(gpu_state[name], cpu_state[name]) < 5e-2, name


def test_zconv_recipe_trains_on_the_kernels_and_matches_cpu():
    from spiraltorch_b200.models import recipes

    def build():
        model, loss, batches, _ = recipes.zconv_classification(seed=0)
        return model, loss, batches
    counts0 = dict(Fn.launch_counts)
    gpu_losses, gpu_state = _train("cuda", build, 4, lr=0.5)
    for op in ("conv2d", "max_pool2x2", "linear"):
        assert Fn.launch_counts[op] - counts0[op] >= 4 * 4, op
    cpu_losses, cpu_state = _train("cpu", build, 4, lr=0.5)
    assert gpu_losses[-1] < gpu_losses[0]
    for a, b in zip(gpu_losses, cpu_losses):
        assert abs(a - b) < 5e-2 * max(1.0, abs(b)), (gpu_losses, cpu_losses)
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


# ---- whole-sequence recurrent scans ---------------------------------------------------------------------
@pytest.mark.parametrize("cell,hidden,dilation", [("tanh", 32, 1), ("wave", 64, 2), ("wave", 32, 1), ("wave", 16, 3),
                                                  ("lstm", 64, 1), ("lstm", 40, 1)])
def test_rnn_sequence_kernel_matches_step_loop(cell, hidden, dilation):
    from spiraltorch_b200.ops import recurrent as R
    torch.manual_seed(8)
    B, T, I = 9, 7, 24
    G_ = {"tanh": 1, "wave": 2, "lstm": 4}[cell]
    x, w_ih, w_hh, b, dh = _bf(torch.randn(B, T, I), torch.randn(I, G_ * hidden) * 0.3,
                               torch.randn(hidden, G_ * hidden) * 0.3, torch.randn(1, G_ * hidden) * 0.1,
                               torch.randn(B, hidden))
    f = lambda *a: R.rnn_sequence(*a, cell, dilation)       # noqa: E731
    before = R.launch_count
    y_g, g_g = _grads(f, [t.to(DEV) for t in (x, w_ih, w_hh, b)], dh)
    assert R.launch_count - before == 2                     # one forward scan, one backward scan
    y_c, g_c = _grads(f, [x, w_ih, w_hh, b], dh)
    assert _rel(y_g, y_c) < 2e-2
    for a, c in zip(g_g, g_c):
        assert _rel(a, c) < 4e-2
    torch.cuda.synchronize()
    assert native.read_error_word()[0] == 0


def test_wave_rnn_module_training_step_runs_on_the_scan_kernel():
    from spiraltorch_b200.ops import recurrent as R
    torch.manual_seed(9)
    layer = st.nn.WaveRnn("wave", 32, 64, 16, dilation=2)
    cpu_x, cpu_g = torch.randn(32, 16 * 32), torch.randn(32, 64)
    ref_dx = layer.backward(st.Tensor(cpu_x), st.Tensor(cpu_g)).torch()
    ref_acc = {p.name: p.gradient.clone() for p in layer.parameters()}
    layer.zero_accumulators()
    layer.to("cuda")
    before = R.launch_count
    y = layer.forward(st.Tensor(cpu_x).cuda())
    dx = layer.backward(st.Tensor(cpu_x).cuda(), st.Tensor(cpu_g).cuda()).torch()
    assert R.launch_count - before == 3                     # forward scan; forward + backward scan of backward()
    assert y.shape() == (32, 64)
    assert _rel(dx, ref_dx) < 5e-2
    for p in layer.parameters():
        assert _rel(p.gradient, ref_acc[p.name]) < 5e-2, p.name


def _wave_model(seed):
    torch.manual_seed(seed)
    m = st.nn.Sequential()
    m.add(st.nn.WaveRnn("wave", 32, 64, 16))
    m.add(st.nn.Linear(64, 8, name="head"))
    m.to("cuda")
    return m


def test_graphed_train_step_matches_eager_steps_and_reports_non_finite_inputs():
    loss = st.nn.MeanSquaredError()
    torch.manual_seed(11)
    batches = [(torch.randn(32, 16 * 32, device="cuda"), torch.randn(32, 8, device="cuda")) for _ in range(4)]
    eager, graphed = _wave_model(5), _wave_model(5)
    step = st.nn.GraphedTrainStep(graphed, loss, st.Tensor._wrap(batches[0][0]), st.Tensor._wrap(batches[0][1]), learning_rate=1e-2)
    for p, q in zip(eager.parameters(), graphed.parameters()):
        assert torch.equal(p.value, q.value)                      # warm-up and capture left the parameters untouched
    for x, y in batches:
        xe, ye = st.Tensor._wrap(x), st.Tensor._wrap(y)
        pred = eager.forward(xe)
        want = float(loss.forward(pred, ye).torch())
        eager.backward(xe, loss.backward(pred, ye))
        eager.apply_step(1e-2)
        got = float(step(xe, ye))
        assert got == pytest.approx(want, rel=2e-3)
    step.check()
    assert step.replays == 4
    for p, q in zip(eager.parameters(), graphed.parameters()):
        assert _rel(q.value, p.value) < 2e-3, p.name
    # an eager forward after graphed training must see the trained weights, not a stale low-precision copy
    xe = st.Tensor._wrap(batches[0][0])
    assert _rel(graphed.forward(xe).torch(), eager.forward(xe).torch()) < 2e-2
    bad = batches[0][1].clone()
    bad[0, 0] = float("nan")
    step(xe, st.Tensor._wrap(bad))
    with pytest.raises(st.TensorError):
        step.check()
