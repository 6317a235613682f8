"""Two-or-more-rank check of the fused kernels against the NCCL path (launched by torchrun).

Prints FUSED_TP_OK on rank 0 when (a) ag_gemm / gemm_rs match all-gather / reduce-scatter + GEMM,
(b) the data-parallel bucket step matches all-reduce-mean + AdamW, (c) a small GPT step gives the
same loss and gradients under the fused and the NCCL tensor-parallel contexts.  Also prints
device-timed comparisons of the fused kernels and the NCCL+GEMM sequence (max over ranks).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from spiraltorch_b200.models.gpt import GPTConfig, GPTModel  # noqa: E402
from spiraltorch_b200.ops import gemm as G  # noqa: E402
from spiraltorch_b200.ops import native  # noqa: E402
from spiraltorch_b200.ops import optim as O  # noqa: E402
from spiraltorch_b200.parallel.symm import FusedDPStep, FusedTPContext, PeerSignals  # noqa: E402
from spiraltorch_b200.parallel.tp import TPContext  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


class Sections:
    """Runs test sections; after each one all ranks agree on success so that nobody leaves a
    collective (or a peer-memory kernel) half-way when another rank hit an assertion."""

    def __init__(self, dev):
        self.dev, self.ok = dev, True

    def run(self, name, fn):
        if not self.ok:
            return
        good = 1
        try:
            fn()
            torch.cuda.synchronize()
            native.raise_on_device_error()
        except Exception:  # noqa: BLE001
            import traceback
            print(f"[rank {dist.get_rank()}] section {name} FAILED", flush=True)
            traceback.print_exc()
            good = 0
        t = torch.tensor([good], device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        self.ok = bool(t.item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    big = os.environ.get("ST_FUSED_BENCH", "1") == "1"
    nccl = TPContext(dist.group.WORLD)
    fused = FusedTPContext(dist.group.WORLD, device=dev)
    if rank == 0:
        print(f"world={world} multicast={'yes' if fused.signals.buf.mc_ptr else 'no'}", flush=True)
    sec = Sections(dev)

    def sec_tp_kernels():
        torch.manual_seed(100 + rank)
        T, K, N = 2048 * world, 1024, 768
        x = torch.randn(T // world, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        wt = torch.randn(K, N, device=dev).bfloat16()
        a_full = torch.randn(T, K, device=dev).bfloat16()
        checks = []  # every collective first, comparisons afterwards (keeps the ranks in lock-step)
        for rep in range(3):
            y_ref, xf_ref = nccl.ag_gemm(x, w)
            y, xf = fused.ag_gemm(x, w, key="a")
            checks.append(("gathered rows", xf.clone(), xf_ref, 0.0))
            checks.append(("ag_gemm", y, y_ref, 1e-2))
            y2_ref, _ = nccl.ag_gemm(x, wt, b_mn=True)
            y2, _ = fused.ag_gemm(x, wt, b_mn=True, key="b")
            checks.append(("ag_gemm b_mn", y2, y2_ref, 1e-2))
            z_ref = nccl.gemm_rs(a_full, w)
            z = fused.gemm_rs(a_full, w)
            checks.append(("gemm_rs", z, z_ref, 2e-2))
            z2_ref = nccl.gemm_rs(a_full, wt, b_mn=True)
            z2 = fused.gemm_rs(a_full, wt, b_mn=True)
            checks.append(("gemm_rs b_mn", z2, z2_ref, 2e-2))
        torch.cuda.synchronize()
        native.raise_on_device_error()
        for name, got, ref, tol in checks:
            err = rel(got, ref)
            assert err <= tol, (name, err)

    only_bench = os.environ.get("ST_FUSED_ONLY_BENCH", "0") == "1"
    if not only_bench:
        sec.run("tp_kernels", sec_tp_kernels)
    def sec_dp_step():
        # data-parallel bucket step against all-reduce-mean + AdamW
        n = 8 * world * 4096
        grad = fused.heap.empty(n, torch.float32)
        wbuf = fused.heap.empty(n, torch.bfloat16)
        grad.tensor.copy_(torch.randn(n, device=dev))
        torch.manual_seed(7)
        wbuf.tensor.copy_(torch.randn(n, device=dev).bfloat16())
        g_ref = grad.tensor.clone()
        dist.all_reduce(g_ref)
        g_ref /= world
        master = wbuf.tensor.float().clone()
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        dp = FusedDPStep(fused.heap, fused.signals, grad, wbuf, kind="adamw", bucket_elems=n // 2)
        dist.barrier()
        dp.step(lr=1e-2, weight_decay=0.1)
        O.adamw_reference(g_ref, master, m, v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, False)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert rel(wbuf.tensor, master) < 1e-2, rel(wbuf.tensor, master)
        assert grad.tensor.abs().max().item() == 0

    if not only_bench:
        sec.run("dp_step", sec_dp_step)

    def sec_ag_in_place():
        # the shard written straight into this rank's slot of the gather buffer: no local copy, same result
        torch.manual_seed(400 + rank)
        rows, K, N = 1024, 512, 384
        x = torch.randn(rows, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        y_ref, xf_ref = nccl.ag_gemm(x, w)
        outs = []
        for rep in range(2):
            slot = fused.shard_slot("inplace", rows, K)
            slot.copy_(x)
            y, xf = fused.ag_gemm(slot, w, key="inplace")
            outs.append((y, xf.clone()))
        torch.cuda.synchronize()
        native.raise_on_device_error()
        for y, xf in outs:
            assert torch.equal(xf, xf_ref)
            assert rel(y, y_ref) <= 1e-2, rel(y, y_ref)

    def sec_dp_two_phase():
        # global-norm clipping inside the fused step against all-reduce-mean + clip + AdamW
        n = 8 * world * 4096
        grad = fused.heap.empty(n, torch.float32)
        wbuf = fused.heap.empty(n, torch.bfloat16)
        torch.manual_seed(500 + rank)
        grad.tensor.copy_(torch.randn(n, device=dev))
        torch.manual_seed(9)
        wbuf.tensor.copy_(torch.randn(n, device=dev).bfloat16())
        g_ref = grad.tensor.clone()
        dist.all_reduce(g_ref)
        g_ref /= world
        max_norm = 0.25 * g_ref.norm().item()
        master = wbuf.tensor.float().clone()
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        dp = FusedDPStep(fused.heap, fused.signals, grad, wbuf, kind="adamw", bucket_elems=n // 4, max_grad_norm=max_norm)
        dist.barrier()
        dp.step(lr=1e-2, weight_decay=0.1)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        norm = g_ref.norm()
        assert abs(dp.grad_norm().item() - norm.item()) < 1e-3 * norm.item(), (dp.grad_norm().item(), norm.item())
        O.adamw_reference(g_ref * (max_norm / (norm + 1e-6)), master, m, v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, False)
        assert rel(wbuf.tensor, master) < 1e-2, rel(wbuf.tensor, master)
        assert grad.tensor.abs().max().item() == 0

    def sec_distributed_topk():
        # candidates read straight from the peers' memory (st_gather_candidates) against the all-gather path
        from spiraltorch_b200.ops import rank as RK
        torch.manual_seed(600)
        full = torch.randn(6, 512 * world, device=dev)
        full[:, 5] = full[:, 5 + 512 * (world - 1)]            # a tie across shards
        shard = full[:, rank * 512:(rank + 1) * 512].contiguous()
        before = RK.launch_count
        v_p, i_p = RK.distributed_topk(shard, 37, group=dist.group.WORLD, heap=fused.heap)
        assert RK.launch_count > before
        v_a, i_a = RK.distributed_topk(shard, 37, group=dist.group.WORLD)
        v_r, i_r = RK.rank_select(full, 37, "topk")
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert torch.equal(i_p, i_a) and torch.equal(i_p, i_r) and torch.equal(v_p, v_r)

    def sec_info_nce_plain():
        # FusedInfoNCE without a tensor-parallel context (the data-parallel benchmark's configuration)
        from spiraltorch_b200.parallel.contrastive import FusedInfoNCE
        torch.manual_seed(700 + rank)
        op = FusedInfoNCE(fused.heap, fused.signals, rows=1024, dim=256, temperature=0.1)
        base = torch.randn(1024, 256, device=dev)
        a = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
        p_ = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
        loss = op.apply(a, p_)
        loss.backward()
        a2 = a.detach().bfloat16().float().requires_grad_(True)
        parts = [torch.empty_like(a2) for _ in range(world)]
        dist.all_gather(parts, p_.detach().bfloat16().float())
        logits = a2 @ torch.cat(parts, 0).t() / 0.1
        idx = torch.arange(1024, device=dev) + rank * 1024
        ref = (torch.logsumexp(logits, -1) - logits[torch.arange(1024, device=dev), idx]).mean()
        ref.backward()
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
        assert rel(a.grad, a2.grad) < 5e-2, rel(a.grad, a2.grad)

    if not only_bench:
        sec.run("ag_in_place", sec_ag_in_place)
        sec.run("dp_two_phase", sec_dp_two_phase)
        sec.run("distributed_topk", sec_distributed_topk)
        sec.run("info_nce_plain", sec_info_nce_plain)
    def sec_gpt():
        # small GPT step: fused vs NCCL context
        cfg = GPTConfig(vocab_size=1024, d_model=512, n_layers=2, n_heads=8, ffn=1024, seq_len=512, init_std=0.05)
        ma = GPTModel(cfg, device=dev, seed=5, tp=nccl)
        mb = GPTModel(cfg, device=dev, seed=5, tp=fused)
        gen = torch.Generator().manual_seed(11)
        tokens = torch.randint(0, 1024, (2 * world, 512), generator=gen).to(dev)
        targets = torch.randint(0, 1024, (2 * world, 512), generator=gen).to(dev)
        for _ in range(2):
            la = ma.forward_backward(tokens, targets)
            lb = mb.forward_backward(tokens, targets)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert abs(la.item() - lb.item()) < 2e-2, (la.item(), lb.item())
        r = ((ma.flat_grad - mb.flat_grad).norm() / ma.flat_grad.norm()).item()
        assert r < 3e-2, r

    def sec_gpt_wgrad_overlap():
        # the same comparison with the weight gradients on the side stream beside grid-limited fused kernels
        # (forced on: by default only link-bound world sizes use it); four layers exercise both buffer parities
        cfg = GPTConfig(vocab_size=1024, d_model=512, n_layers=4, n_heads=8, ffn=1024, seq_len=512, init_std=0.05)
        ma = GPTModel(cfg, device=dev, seed=7, tp=nccl)
        prev = os.environ.get("ST_TP_WGRAD_OVERLAP")
        os.environ["ST_TP_WGRAD_OVERLAP"] = "1"
        try:
            mb = GPTModel(cfg, device=dev, seed=7, tp=fused)
        finally:
            if prev is None:
                del os.environ["ST_TP_WGRAD_OVERLAP"]
            else:
                os.environ["ST_TP_WGRAD_OVERLAP"] = prev
        assert mb._wgrad_ctas > 0 and ma._wgrad_ctas == 0
        gen = torch.Generator().manual_seed(13)
        tokens = torch.randint(0, 1024, (2 * world, 512), generator=gen).to(dev)
        targets = torch.randint(0, 1024, (2 * world, 512), generator=gen).to(dev)
        for _ in range(3):
            la = ma.forward_backward(tokens, targets)
            lb = mb.forward_backward(tokens, targets)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert fused.max_ctas == 0
        assert abs(la.item() - lb.item()) < 2e-2, (la.item(), lb.item())
        r = ((ma.flat_grad - mb.flat_grad).norm() / ma.flat_grad.norm()).item()
        assert r < 3e-2, r

    if not only_bench:
        sec.run("gpt", sec_gpt)
        sec.run("gpt_wgrad_overlap", sec_gpt_wgrad_overlap)

    def sec_info_nce():
        from spiraltorch_b200.parallel.contrastive import FusedInfoNCE
        torch.manual_seed(300 + rank)
        op = FusedInfoNCE(fused.heap, fused.signals, rows=1024, dim=256, temperature=0.1, tp=fused)
        base = torch.randn(1024, 256, device=dev)
        res = []
        for rep in range(2):
            a = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
            p_ = torch.nn.functional.normalize(base + 0.3 * torch.randn_like(base), dim=-1).requires_grad_(True)
            loss = op.apply(a, p_)
            loss.backward()
            a2 = a.detach().bfloat16().float().requires_grad_(True)
            p2 = p_.detach().bfloat16().float().requires_grad_(True)
            parts = [torch.empty_like(p2) for _ in range(world)]
            dist.all_gather(parts, p2.detach())
            parts[rank] = p2
            logits = a2 @ torch.cat(parts, 0).t() / 0.1
            idx = torch.arange(1024, device=dev) + rank * 1024
            ref = (torch.logsumexp(logits, -1) - logits[torch.arange(1024, device=dev), idx]).mean()
            ref.backward()
            # positives also receive gradient from the other ranks' losses
            full = torch.zeros(world * 1024, 256, device=dev)
            full[rank * 1024:(rank + 1) * 1024] = p2.grad
            others = torch.autograd.grad(ref, a2, retain_graph=False, allow_unused=True) if False else None
            res.append((loss.detach(), ref.detach(), a.grad.clone(), a2.grad.clone()))
        torch.cuda.synchronize()
        native.raise_on_device_error()
        for loss, ref, ga, gr in res:
            assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
            assert rel(ga, gr) < 5e-2, rel(ga, gr)

    if not only_bench:
        sec.run("info_nce", sec_info_nce)
    def sec_bench():
        if not big:
            return
        import json
        peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                  "MEASURED_PEAKS.json")
        tf_peak = json.load(open(peaks_path))["bf16_tflops"] if os.path.exists(peaks_path) else 1590.0
        link_gbs = 770.0                      # measured peer copy bandwidth per direction
        for T in [int(v) for v in os.environ.get("ST_FUSED_BENCH_T", "16384").split(",")]:
            bench_one(T, 0, tf_peak, link_gbs)

    def trace_report(label, fn):
        """One launch with per-CTA phase stamps: prints, for rank 0, when (relative to the first CTA's
        start, in us) the slowest CTA finished each phase."""
        if os.environ.get("ST_FUSED_TRACE", "0") != "1":
            return
        fused.trace = torch.zeros(480, 4, dtype=torch.int64, device=dev)
        dist.barrier()
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        tr = fused.trace.cpu()
        fused.trace = None
        if rank == 0:
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            rows_g, rows_c, rows_r = tr[:sms], tr[sms:2 * sms], tr[2 * sms:3 * sms]
            gem = rows_g[rows_g[:, 0] > 0]
            comm = rows_c[rows_c[:, 0] > 0]
            remote = rows_r[rows_r[:, 0] > 0][:, 0]
            t0 = min(gem[:, 0].min().item(), comm[:, 0].min().item() if len(comm) else 1 << 62)
            msg = f"TRACE {label}: "
            if len(remote):
                msg += f"remote stores done {(remote.min().item() - t0) / 1e3:.1f}..{(remote.max().item() - t0) / 1e3:.1f}; "
            if len(comm) and label.startswith("gemm_rs"):
                msg += (f"first local tile reached {(comm[:, 0].min().item() - t0) / 1e3:.1f}..{(comm[:, 0].max().item() - t0) / 1e3:.1f} "
                        f"peers' partials ready {(comm[:, 1].min().item() - t0) / 1e3:.1f}..{(comm[:, 1].max().item() - t0) / 1e3:.1f}; ")
            elif len(comm):
                msg += (f"comm ctas {len(comm)} entry<= {(comm[:, 1].max().item() - t0) / 1e3:.1f} "
                        f"push done {(comm[:, 2].min().item() - t0) / 1e3:.1f}..{(comm[:, 2].max().item() - t0) / 1e3:.1f}; ")
            msg += (f"gemm ctas {len(gem)} start<= {(gem[:, 0].max().item() - t0) / 1e3:.1f} "
                    f"entry<= {(gem[:, 1].max().item() - t0) / 1e3:.1f} "
                    f"tiles done {(gem[:, 2].min().item() - t0) / 1e3:.1f}..{(gem[:, 2].max().item() - t0) / 1e3:.1f} "
                    f"end {(gem[:, 3].min().item() - t0) / 1e3:.1f}..{(gem[:, 3].max().item() - t0) / 1e3:.1f}")
            print(msg, flush=True)

    def bench_one(T, nvls, tf_peak, link_gbs):
        import json
        d = 2048
        # the four tensor-parallel linears of the 1.3B model at this world size
        ag_shapes = [("qkv", 6144 // world), ("ffn1", 8192 // world), ("probe_push_only", 256)]
        rs_shapes = [("attn_out", 2048 // world), ("ffn2", 8192 // world), ("probe_comm_only", 64)]
        xs = torch.randn(T // world, d, device=dev).bfloat16()
        gathered = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        t_ag = timed(lambda: dist.all_gather_into_tensor(gathered, xs))
        for name, N in ag_shapes:
            w1 = torch.randn(N, d, device=dev).bfloat16()
            t_n = timed(lambda: nccl.ag_gemm(xs, w1))
            t_f = timed(lambda: fused.ag_gemm(xs, w1, key="bench"))
            trace_report("ag_gemm " + name, lambda: fused.ag_gemm(xs, w1, key="bench"))
            t_g = timed(lambda: G.gemm(gathered, w1))
            flops = 2.0 * T * N * d
            nv_bytes = T * d * 2 * (world - 1) / world
            roof = max(flops / tf_peak / 1e9, nv_bytes / link_gbs / 1e6)       # ms
            if rank == 0:
                print(json.dumps({"op": "ag_gemm", "nvls": nvls, "layer": name, "world": world, "T": T, "K": d, "N": N,
                                  "fused_ms": round(t_f, 4), "nccl_plus_gemm_ms": round(t_n, 4),
                                  "gemm_only_ms": round(t_g, 4), "nccl_all_gather_ms": round(t_ag, 4),
                                  "roofline_ms": round(roof, 4), "frac_of_roofline": round(roof / t_f, 3),
                                  "speedup_vs_nccl": round(t_n / t_f, 3)}), flush=True)
        part = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        shard = torch.empty(T // world, d, device=dev, dtype=torch.bfloat16)
        t_rs = timed(lambda: dist.reduce_scatter_tensor(shard, part))
        for name, Kl in rs_shapes:
            af = torch.randn(T, Kl, device=dev).bfloat16()
            w2 = torch.randn(d, Kl, device=dev).bfloat16()
            r_n = timed(lambda: nccl.gemm_rs(af, w2))
            r_f = timed(lambda: fused.gemm_rs(af, w2))
            trace_report("gemm_rs " + name, lambda: fused.gemm_rs(af, w2))
            r_g = timed(lambda: G.gemm(af, w2))
            flops = 2.0 * T * d * Kl
            nv_bytes = T * d * 2 * (world - 1) / world
            roof = max(flops / tf_peak / 1e9, nv_bytes / link_gbs / 1e6)
            if rank == 0:
                print(json.dumps({"op": "gemm_rs", "nvls": nvls, "layer": name, "world": world, "T": T, "K": Kl, "N": d,
                                  "fused_ms": round(r_f, 4), "gemm_plus_nccl_ms": round(r_n, 4),
                                  "gemm_only_ms": round(r_g, 4), "nccl_reduce_scatter_ms": round(t_rs, 4),
                                  "roofline_ms": round(roof, 4), "frac_of_roofline": round(roof / r_f, 3),
                                  "speedup_vs_nccl": round(r_n / r_f, 3)}), flush=True)

    sec.run("bench", sec_bench)
    dist.barrier()
    if rank == 0 and sec.ok:
        print("FUSED_TP_OK", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if sec.ok else 1)


if __name__ == "__main__":
    main()
