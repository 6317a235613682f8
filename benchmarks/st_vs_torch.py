"""`st.Tensor` GEMM and Hadamard against `torch.mm` / `torch.mul` on the same device.

Parity: bench_st_vs_torch.py of the reference (wall-clock of `Tensor.matmul` and `Tensor.hadamard` versus
PyTorch for a list of square sizes).  Here the device path is timed with CUDA events on the launching
stream after warm-up, with a buffer larger than L2 written between timed launches; on a CPU-only host the
same script times the oracle path with `perf_counter`.

    python benchmarks/st_vs_torch.py --sizes 1024 4096 --backend auto --dtype bf16
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import spiraltorch_b200 as st  # noqa: E402


def _timed(fn, iters: int, device: str, flush) -> float:
    for _ in range(3):
        fn()
    if device == "cuda":
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[512, 1024, 2048])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--backend", default="auto", help="auto | cpu | cuda")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    args = ap.parse_args(argv)
    session = st.SpiralSession(args.backend)
    device = "cuda" if session.effective_backend == "cuda" else "cpu"
    dtype = torch.bfloat16 if (args.dtype == "bf16" and device == "cuda") else torch.float32
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if device == "cuda" else None
    for n in args.sizes:
        ta = torch.randn(n, n, device=device).to(dtype)
        tb = torch.randn(n, n, device=device).to(dtype)
        a, b = st.Tensor(ta), st.Tensor(tb)
        row = {"size": n, "device": device, "dtype": str(dtype).replace("torch.", ""),
               "st_matmul_ms": _timed(lambda: a.matmul(b), args.iters, device, flush),
               "torch_mm_ms": _timed(lambda: torch.mm(ta, tb), args.iters, device, flush),
               "st_hadamard_ms": _timed(lambda: a.hadamard(b), args.iters, device, flush),
               "torch_mul_ms": _timed(lambda: torch.mul(ta, tb), args.iters, device, flush)}
        row["matmul_speedup_vs_torch"] = row["torch_mm_ms"] / max(row["st_matmul_ms"], 1e-9)
        row["matmul_tflops"] = 2.0 * n ** 3 / (row["st_matmul_ms"] * 1e-3) / 1e12
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
