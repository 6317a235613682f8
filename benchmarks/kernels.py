#!/usr/bin/env python
"""Per-kernel micro-benchmarks against the library op on the same GPU, with roofline fractions.

    python benchmarks/kernels.py gemm attn_fwd attn_bwd conv norm adamw ce transforms layers [--iters 10] [--json out.json]
    python benchmarks/kernels.py gemm --profile      # 2 launches of ours only: the target of an ncu capture

Every timing: 3 warm-up launches, then ``iters`` launches each preceded by a write of a 256 MiB
buffer (L2 flush), timed with CUDA events on the launching stream; the median is reported.
Roofline denominators come from ``MEASURED_PEAKS.json`` at the repository root (written by the
round driver); without it the documented fallbacks 6.65 TB/s and 1.59 PFLOP/s are used and the
output says "of fallback".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from spiraltorch_b200.ops import attention as A  # noqa: E402
from spiraltorch_b200.ops import conv as C  # noqa: E402
from spiraltorch_b200.ops import gemm as G  # noqa: E402
from spiraltorch_b200.ops import loss as L  # noqa: E402
from spiraltorch_b200.ops import norm as N  # noqa: E402
from spiraltorch_b200.ops import optim as O  # noqa: E402

DEV = "cuda"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timed(fn, iters):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def row(name, shape, ours_ms, lib_ms, flops=None, bytes_=None):
    hbm, tf, kind = peaks()
    r = {"kernel": name, "shape": shape, "ours_ms": round(ours_ms, 4), "library_ms": None if lib_ms is None else round(lib_ms, 4)}
    if lib_ms:
        r["speedup_vs_library"] = round(lib_ms / ours_ms, 3)
    if flops:
        r["tflops"] = round(flops / ours_ms / 1e9, 1)
        r[f"frac_of_{kind}_bf16_peak"] = round(flops / ours_ms / 1e9 / tf, 3)
    if bytes_:
        r["gbs"] = round(bytes_ / ours_ms / 1e6, 1)
        r[f"frac_of_{kind}_hbm"] = round(bytes_ / ours_ms / 1e6 / hbm, 3)
    print(json.dumps(r), flush=True)
    return r


def bench_gemm(iters, profile):
    out = []
    shapes = [(16384, 6144, 2048, False, False), (16384, 2048, 8192, False, False), (16384, 8192, 2048, False, True),
              (8192, 2048, 16384, True, True), (16384, 50304, 2048, False, False), (16384, 2304, 768, False, False)]
    if profile:
        shapes = [(16384, 6144, 2048, False, False)]
    for M, Nn, K, a_mn, b_mn in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device=DEV).bfloat16()
        b = torch.randn((K, Nn) if b_mn else (Nn, K), device=DEV).bfloat16()
        c = torch.empty(M, Nn, device=DEV, dtype=torch.bfloat16)
        ours = lambda: G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c)  # noqa: E731
        if profile:
            ours(); ours(); torch.cuda.synchronize()
            return out
        af, bf = (a.t() if a_mn else a), (b if b_mn else b.t())
        t1, t2 = timed(ours, iters), timed(lambda: torch.matmul(af, bf, out=c), iters)
        out.append(row("gemm_bf16" + ("_amn" if a_mn else "") + ("_bmn" if b_mn else ""), [M, Nn, K], t1, t2,
                       flops=2.0 * M * Nn * K))
    return out


def bench_attn(iters, profile, backward):
    out = []
    cfgs = [(8, 2048, 16, 128), (32, 512, 12, 64)] if not profile else [(4, 2048, 16, 128)]
    for B, S, H, D in cfgs:
        qkv = torch.randn(B, S, 3, H, D, device=DEV).bfloat16()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        do = torch.randn(B, S, H, D, device=DEV).bfloat16()
        o, lse = A.attention_forward(q, k, v, True)
        if backward:
            ours = lambda: A.attention_backward(q, k, v, o, lse, do, True)  # noqa: E731
        else:
            ours = lambda: A.attention_forward(q, k, v, True)  # noqa: E731
        if profile:
            ours(); ours(); torch.cuda.synchronize()
            return out
        qt, kt, vt = (t.transpose(1, 2).detach().requires_grad_(backward) for t in (q, k, v))
        if backward:
            oo = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
            lib = lambda: torch.autograd.grad(oo, (qt, kt, vt), do.transpose(1, 2), retain_graph=True)  # noqa: E731
        else:
            lib = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)  # noqa: E731
        fl = (10.0 if backward else 4.0) * B * H * S * S * D / 2
        out.append(row("attn_bwd" if backward else "attn_fwd", [B, S, H, D], timed(ours, iters), timed(lib, iters), flops=fl))
    return out


def bench_conv(iters, profile):
    out = []
    cfgs = [(256, 32, 64, 128), (256, 16, 128, 256), (256, 8, 256, 512), (256, 64, 64, 64)] if not profile else [(64, 32, 64, 128)]
    for Nb, H, Ci, Co in cfgs:
        x = torch.randn(Nb, H, H, Ci, device=DEV).bfloat16()
        w = (torch.randn(Co, 9 * Ci, device=DEV) * 0.05).bfloat16()
        b = torch.randn(Co, device=DEV).bfloat16()
        ours = lambda: C.conv3x3(x, w, b, relu=True)  # noqa: E731
        if profile:
            ours(); ours(); torch.cuda.synchronize()
            return out
        xc = x.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
        wc = w.reshape(Co, 3, 3, Ci).permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
        lib = lambda: torch.relu_(torch.nn.functional.conv2d(xc, wc, b, padding=1))  # noqa: E731
        fl = 2.0 * Nb * H * H * 9 * Ci * Co
        out.append(row("conv3x3_bias_relu_fwd", [Nb, H, H, Ci, Co], timed(ours, iters), timed(lib, iters), flops=fl))
        dy = torch.randn(Nb, H, H, Co, device=DEV).bfloat16()
        dw = torch.zeros(Co, 9 * Ci, device=DEV)
        t = timed(lambda: C.conv3x3_wgrad(dy, x, dw), iters)
        dyc = dy.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
        tl = timed(lambda: torch.ops.aten.convolution_backward(dyc, xc, wc, None, [1, 1], [1, 1], [1, 1], False, [0, 0], 1,
                                                               [False, True, False]), iters)
        out.append(row("conv3x3_wgrad", [Nb, H, H, Ci, Co], t, tl, flops=fl))
    return out


def bench_norm(iters, profile):
    out = []
    rows, d = (16384, 2048) if not profile else (65536, 2048)
    x = torch.randn(rows, d, device=DEV).bfloat16()
    g = torch.ones(d, device=DEV).bfloat16()
    dy = torch.randn(rows, d, device=DEV).bfloat16()
    y, _, mean, rstd = N.norm_forward(x, g, None, 1e-5, True)
    dg = torch.zeros(d, device=DEV)
    fwd = lambda: N.norm_forward(x, g, None, 1e-5, True)  # noqa: E731
    bwd = lambda: N.norm_backward(dy, x, g, mean, rstd, True, dg, None, False)  # noqa: E731
    if profile:
        fwd(); bwd(); fwd(); bwd(); torch.cuda.synchronize()
        return out
    out.append(row("rmsnorm_fwd", [rows, d], timed(fwd, iters), timed(lambda: torch.nn.functional.rms_norm(x, (d,), g, 1e-5), iters),
                   bytes_=rows * d * 4))
    out.append(row("rmsnorm_bwd", [rows, d], timed(bwd, iters), None, bytes_=rows * d * 6))
    return out


def bench_adamw(iters, profile):
    n = 256 * 1024 * 1024 if not profile else 64 * 1024 * 1024
    g, m, v, master = (torch.randn(n, device=DEV) for _ in range(4))
    v.abs_()
    w = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ours = lambda: O.adamw_step(g, master, m, v, w, lr=1e-3, step=2, weight_decay=0.1, zero_grad=False)  # noqa: E731
    if profile:
        ours(); ours(); torch.cuda.synchronize()
        return []
    p = master.clone().requires_grad_(True)
    p.grad = g.clone()
    opt = torch.optim.AdamW([p], lr=1e-3, fused=True)
    return [row("adamw_fused_master_bf16", [n], timed(ours, iters), timed(opt.step, iters), bytes_=n * (4 * 7 + 2))]


def bench_ce(iters, profile):
    T, V = (16384, 50304) if not profile else (8192, 50304)
    logits = torch.randn(T, V, device=DEV).bfloat16()
    tgt = torch.randint(0, V, (T,), device=DEV)
    ours = lambda: L._stats(logits, tgt, 0)  # noqa: E731
    if profile:
        ours(); ours(); torch.cuda.synchronize()
        return []
    lib = lambda: torch.nn.functional.cross_entropy(logits.float(), tgt)  # noqa: E731
    return [row("cross_entropy_stats", [T, V], timed(ours, iters), timed(lib, iters), bytes_=T * V * 2)]


def bench_glue(iters, profile):
    """Bandwidth-bound glue of the training steps: RoPE, GELU backward, bias-gradient column sum, embedding
    gather / scatter-add, 2x2 max-pool.  Fractions are of the measured copy bandwidth."""
    from spiraltorch_b200.ops import elementwise as E
    out = []
    T, H, Dh, S = 16384, 16, 128, 2048
    if profile:
        # two launches of each kernel on inputs larger than L2, nothing timed
        qkv = torch.randn(4 * T, 3 * H * Dh, device=DEV).bfloat16()
        x = torch.randn(T, 8192, device=DEV).bfloat16()
        dy = torch.randn(T, 8192, device=DEV).bfloat16()
        w = torch.randn(50304, 2048, device=DEV).bfloat16()
        idx = torch.randint(0, 50304, (4 * T,), device=DEV)
        dw = torch.zeros(50304, 2048, device=DEV)
        dyt = torch.randn(4 * T, 2048, device=DEV).bfloat16()
        img = torch.randn(256, 64, 64, 64, device=DEV).bfloat16()
        for _ in range(2):
            E.rope_(qkv, 2 * H, Dh, S)
            E.act_backward(x, dy, "gelu")
            E.colsum(dy)
            E.embedding_forward(idx, w)
            E.embedding_backward(idx, dyt, dw)
            C.maxpool2(img)
        torch.cuda.synchronize()
        return out
    qkv = torch.randn(T, 3 * H * Dh, device=DEV).bfloat16()
    def rope_ref():
        cos, sin = E.rope_tables(S, Dh, 10000.0, qkv.device)
        v = qkv[:, : 2 * H * Dh].reshape(T, 2 * H, Dh)
        return E.rope_reference(v, cos, sin, S, False)
    out.append(row("rope_qk_inplace", [T, 2 * H, Dh], timed(lambda: E.rope_(qkv, 2 * H, Dh, S), iters), timed(rope_ref, iters),
                   bytes_=T * 2 * H * Dh * 4))
    x = torch.randn(T, 8192, device=DEV).bfloat16()
    dy = torch.randn(T, 8192, device=DEV).bfloat16()
    out.append(row("gelu_bwd", [T, 8192], timed(lambda: E.act_backward(x, dy, "gelu"), iters),
                   timed(lambda: torch.ops.aten.gelu_backward(dy, x, approximate="tanh"), iters), bytes_=T * 8192 * 6))
    out.append(row("bias_grad_colsum", [T, 8192], timed(lambda: E.colsum(dy), iters),
                   timed(lambda: dy.float().sum(0), iters), bytes_=T * 8192 * 2))
    V, d = 50304, 2048
    w = torch.randn(V, d, device=DEV).bfloat16()
    idx = torch.randint(0, V, (T,), device=DEV)
    out.append(row("embedding_gather", [T, d], timed(lambda: E.embedding_forward(idx, w), iters),
                   timed(lambda: torch.nn.functional.embedding(idx, w), iters), bytes_=T * d * 4))
    dw = torch.zeros(V, d, device=DEV)
    dyt = torch.randn(T, d, device=DEV).bfloat16()
    dw_lib = torch.zeros(V, d, device=DEV)
    out.append(row("embedding_scatter_add", [T, d], timed(lambda: E.embedding_backward(idx, dyt, dw), iters),
                   timed(lambda: dw_lib.index_add_(0, idx, dyt.float()), iters), bytes_=T * d * (2 + 8)))
    img = torch.randn(256, 64, 64, 64, device=DEV).bfloat16()
    nchw = img.permute(0, 3, 1, 2).contiguous()
    out.append(row("maxpool2x2_nhwc", [256, 64, 64, 64], timed(lambda: C.maxpool2(img), iters),
                   timed(lambda: torch.nn.functional.max_pool2d(nchw, 2), iters), bytes_=img.numel() * 2 * 1.25))
    return out


def bench_transforms(iters, profile):
    """The rows of the reference's published transform table (docs/performance/transforms.md:48-64, RTX 4090 + WGPU,
    times that include host<->device transfers): device-only time of the fused kernel, and the time with the upload
    of the source image from pinned memory and the download of the result."""
    from spiraltorch_b200 import vision as V
    cases = [("resize_512_to_224", (3, 512, 512), dict(resize=(224, 224)), 1.7),
             ("resize_1024_to_384", (3, 1024, 1024), dict(resize=(384, 384)), 4.8),
             ("jitter_256_balanced", (3, 256, 256), dict(jitter=V.ColorJitter.balanced()), 0.9),
             ("jitter_512_vivid", (3, 512, 512), dict(jitter=V.ColorJitter.vivid()), 2.3),
             ("center_crop_256_to_224", (3, 256, 256), dict(crop=(224, 224)), 0.3),
             ("hflip_256", (3, 256, 256), dict(flip=True), 0.2),
             ("classification_pipeline_224", (3, 512, 512), dict(resize=(256, 256), crop=(224, 224),
                                                                 jitter=V.ColorJitter.balanced(), flip=True), 3.1)]
    out = []
    for name, shape, kw, ref_ms in cases:
        host = torch.rand(*shape).pin_memory()
        dev = host.to(DEV)
        if kw.get("jitter") is not None and kw["jitter"].means is None:
            # per-channel means for the contrast term are an input of the kernel; computing them is a separate reduction
            kw = dict(kw, jitter=V.ColorJitter(kw["jitter"].brightness, kw["jitter"].contrast, kw["jitter"].saturation,
                                               kw["jitter"].hue, means=tuple((dev * kw["jitter"].brightness).mean(dim=(1, 2)).tolist())))
        ours = lambda: V.preprocess(dev, **kw)  # noqa: E731
        if profile:
            ours(); ours(); torch.cuda.synchronize()
            return out
        res = ours()
        back = torch.empty(res.shape, dtype=res.dtype).pin_memory()

        def e2e():
            d = host.to(DEV, non_blocking=True)
            back.copy_(V.preprocess(d, **kw), non_blocking=True)
        r = {"kernel": "transform_" + name, "shape": list(shape), "ours_ms": round(timed(ours, iters), 4),
             "ours_with_transfers_ms": round(timed(e2e, iters), 4), "reference_published_gpu_ms": ref_ms,
             "reference_hardware": "RTX 4090 (WGPU), includes transfers"}
        print(json.dumps(r), flush=True)
        out.append(r)
    return out


def bench_layers(iters, profile):
    """One training step of the two small layers the reference quotes timings for (docs/learning_backend_audit.md:
    WaveRnn one-batch step 7.1 ms CPU / 125.9 ms WGPU; GNN trainer step 16.5 ms CPU / 362.8 ms WGPU)."""
    import spiraltorch_b200 as st
    from spiraltorch_b200.nn import gnn
    out = []
    steps, dim, hidden, batch = 16, 32, 64, 32
    wave = st.nn.Sequential()
    wave.add(st.nn.WaveRnn("wave", dim, hidden, steps))
    wave.add(st.nn.Linear(hidden, 8, name="head"))
    wave.to(DEV)
    x = st.Tensor._wrap(torch.randn(batch, steps * dim, device=DEV))
    y = st.Tensor._wrap(torch.randn(batch, 8, device=DEV))
    loss = st.nn.MeanSquaredError()

    def wave_step():
        pred = wave.forward(x)
        wave.backward(x, loss.backward(pred, y))
        wave.apply_step(1e-2)
    adj = (torch.rand(64, 64) < 0.1).float()
    adj = ((adj + adj.t()) > 0).float()
    net = gnn.ZSpaceGraphNetwork("g", gnn.GraphContext.from_adjacency(adj.to(DEV)), [16, 32, 4])
    model = gnn.ZSpaceGraphRegressor(net, gnn.GraphReadout("mean"))
    model.to(DEV)
    gx = st.Tensor._wrap(torch.randn(64, 16, device=DEV))
    gy = st.Tensor._wrap(torch.randn(1, 4, device=DEV))

    def gnn_step():
        pred = model.forward(gx)
        model.backward(gx, loss.backward(pred, gy))
        model.apply_step(1e-2)
    if profile:
        wave_step(); gnn_step(); torch.cuda.synchronize()
        return out
    # the same two steps captured once in a CUDA graph and replayed (st.nn.GraphedTrainStep): the launches are issued
    # from the device, so what is left is the kernels' own time
    wave_g = st.nn.GraphedTrainStep(wave, loss, x, y, learning_rate=1e-2)
    gnn_g = st.nn.GraphedTrainStep(model, loss, gx, gy, learning_rate=1e-2)
    wave_g.check(); gnn_g.check()
    for name, fn, cpu_ms, wgpu_ms in (("wave_rnn_train_step", wave_step, 7.132, 125.897), ("gnn_train_step", gnn_step, 16.503, 362.814),
                                      ("wave_rnn_train_step_graphed", lambda: wave_g(x, y), 7.132, 125.897),
                                      ("gnn_train_step_graphed", lambda: gnn_g(gx, gy), 16.503, 362.814)):
        r = {"kernel": name, "ours_ms": round(timed(fn, iters), 4), "reference_published_cpu_ms": cpu_ms,
             "reference_published_wgpu_ms": wgpu_ms}
        print(json.dumps(r), flush=True)
        out.append(r)
    return out


def bench_fused(iters, profile):
    """The fused all-gather->GEMM and GEMM->reduce-scatter kernels in their world-1 form (the peer is this GPU: the
    same code path, rendezvous flags, arrival counters and epilogues, without NVLink), against the plain GEMM."""
    from spiraltorch_b200.ops.gemm import gemm
    from spiraltorch_b200.parallel.symm import FusedTPContext
    tp = FusedTPContext(None, device=DEV)
    T, K, N = 16384, 2048, 3072
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    w2 = torch.randn(K, N, device=DEV).bfloat16()
    a = torch.randn(T, N, device=DEV).bfloat16()
    if profile:
        for _ in range(2):
            tp.ag_gemm(x, w, key="prof")
            tp.gemm_rs(a, w2)
        torch.cuda.synchronize()
        return []
    out = []
    for name, fn, ref, flops in (("ag_gemm_world1", lambda: tp.ag_gemm(x, w, key="bench"), lambda: gemm(x, w), 2.0 * T * N * K),
                                 ("gemm_rs_world1", lambda: tp.gemm_rs(a, w2), lambda: gemm(a, w2), 2.0 * T * N * K)):
        r = row(name, f"{T}x{N}x{K}", timed(fn, iters), timed(ref, iters), flops=flops)
        out.append(r)
    return out


def bench_scan(iters, profile):
    """Whole-sequence recurrent kernels: forward + backward of the LSTM / wave / Elman layers in one launch each,
    against the per-step PyTorch loop on the same device."""
    from spiraltorch_b200.ops import recurrent as R
    out = []
    for cell, B, T_, I, H, dil in (("wave", 32, 16, 32, 64, 2), ("lstm", 64, 32, 64, 64, 1), ("tanh", 64, 32, 64, 128, 1)):
        G_ = {"tanh": 1, "wave": 2, "lstm": 4}[cell]
        xs = torch.randn(B, T_, I, device=DEV, requires_grad=True)
        w_ih = (torch.randn(I, G_ * H, device=DEV) * 0.2).requires_grad_(True)
        w_hh = (torch.randn(H, G_ * H, device=DEV) * 0.2).requires_grad_(True)
        b = torch.zeros(1, G_ * H, device=DEV, requires_grad=True)

        def ours():
            R.rnn_sequence(xs, w_ih, w_hh, b, cell, dil).sum().backward()

        def loop():
            R.rnn_sequence_reference(xs, w_ih, w_hh, b, cell, dil).sum().backward()
        if profile:
            ours(); ours(); torch.cuda.synchronize()
            continue
        r = {"kernel": f"rnn_scan_{cell}_fwd_bwd", "shape": f"B{B} T{T_} in{I} H{H}", "ours_ms": round(timed(ours, iters), 4),
             "torch_step_loop_ms": round(timed(loop, iters), 4)}
        print(json.dumps(r), flush=True)
        out.append(r)
    return out


def bench_spectral(iters, profile):
    """Spectral kernels: batched shared-memory FFT against cuFFT (`torch.fft.fft`), the fractional multiplier against
    its elementwise torch statement, and the temporal volume renderer against an einsum statement."""
    from spiraltorch_b200.ops import spectral as S
    out = []
    rows, n = (8192, 4096) if profile else (16384, 4096)                 # complex64 [rows, n]: 0.5 GiB in + 0.5 GiB out at full size
    x = torch.randn(rows, n, dtype=torch.complex64, device=DEV)
    xr = torch.randn(rows, n, device=DEV)
    V, C, F = 1 << 22, 4, 16                                             # 100 MB in, 268 MB out
    vox, harm, decay = torch.rand(V, device=DEV), torch.rand(V, C, device=DEV) * 0.1, torch.rand(V, device=DEV)
    if profile:
        for _ in range(2):
            S.fft(x)
            S.specmul_frac_derivative(x, 0.5)
            S.temporal_render(vox, harm, decay, F)
        torch.cuda.synchronize()
        return []
    bytes_fft = 2.0 * rows * n * 8
    out.append(row("fft_c2c_4096", f"{rows}x{n}", timed(lambda: S.fft(x), iters), timed(lambda: torch.fft.fft(x), iters), bytes_=bytes_fft))
    out.append(row("fft_r2c_full_4096", f"{rows}x{n}", timed(lambda: S.fft(xr), iters), timed(lambda: torch.fft.fft(xr), iters),
                   bytes_=rows * n * 4.0 + rows * n * 8.0))
    omega = 2 * math.pi * torch.fft.fftfreq(n, device=DEV)
    mult = torch.where(omega == 0, torch.zeros_like(omega, dtype=torch.complex64), (1j * omega.to(torch.complex64)) ** 0.5)
    out.append(row("specmul_frac_derivative", f"{rows}x{n}", timed(lambda: S.specmul_frac_derivative(x, 0.5), iters),
                   timed(lambda: x * mult, iters), bytes_=bytes_fft))
    t = torch.arange(F, device=DEV, dtype=torch.float32) / 24.0
    k = torch.arange(1, C + 1, device=DEV, dtype=torch.float32)

    def torch_render():
        s = torch.sin(2 * math.pi * t[:, None, None] * k[None, None, :])               # [F, 1, C]
        return (vox[None] + (harm[None] * s).sum(-1)) * torch.exp(-decay[None] * t[:, None])
    out.append(row("temporal_render", f"V{V} C{C} F{F}", timed(lambda: S.temporal_render(vox, harm, decay, F), iters), timed(torch_render, iters),
                   bytes_=V * (C + 2) * 4.0 + V * F * 4.0))
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernels", nargs="*", default=["gemm", "attn_fwd", "attn_bwd", "conv", "norm", "adamw", "ce"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true", help="launch ours twice and exit (ncu target)")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    table = {"gemm": lambda: bench_gemm(args.iters, args.profile),
             "attn_fwd": lambda: bench_attn(args.iters, args.profile, False),
             "attn_bwd": lambda: bench_attn(args.iters, args.profile, True),
             "glue": lambda: bench_glue(args.iters, args.profile),
             "conv": lambda: bench_conv(args.iters, args.profile),
             "norm": lambda: bench_norm(args.iters, args.profile),
             "adamw": lambda: bench_adamw(args.iters, args.profile),
             "ce": lambda: bench_ce(args.iters, args.profile),
             "transforms": lambda: bench_transforms(args.iters, args.profile),
             "layers": lambda: bench_layers(args.iters, args.profile),
             "fused": lambda: bench_fused(args.iters, args.profile),
             "scan": lambda: bench_scan(args.iters, args.profile),
             "spectral": lambda: bench_spectral(args.iters, args.profile)}
    rows = []
    for k in args.kernels:
        rows += table[k]()
    from spiraltorch_b200.ops import native
    native.raise_on_device_error()
    if args.json:
        json.dump({"peaks": dict(zip(("hbm_gbs", "bf16_tflops", "source"), peaks())), "rows": rows}, open(args.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
