"""Times the rank-k kernels' launch choices on the device and writes the generated heuristics table the three-voice
chooser reads (``spiraltorch_b200/data/rank_heuristics_b200.json``).

    python benchmarks/tune_rank.py                 # sweep, print one JSON line per shape, rewrite the table
    python benchmarks/tune_rank.py --dry-run       # sweep and print only

For every (kind, rows, cols, k) of the sweep the direct single-CTA sort and the two-stage path at several chunk widths
are timed with CUDA events (5 warm-up launches, 20 timed, L2 flushed between launches); the fastest becomes the entry.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spiraltorch_b200 import unison                       # noqa: E402
from spiraltorch_b200.device_caps import DeviceCaps       # noqa: E402
from spiraltorch_b200.ops import rank                     # noqa: E402

SHAPES = [(4096, 1024, 8), (4096, 4096, 32), (1024, 8192, 64), (256, 8192, 256), (8192, 2048, 1), (512, 8192, 8)]


def timed(fn, flush, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)                                    # a buffer larger than L2 evicts the previous launch's data
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print("tune_rank needs a CUDA device", file=sys.stderr)
        return 1
    caps = DeviceCaps.probe()
    flush = torch.zeros(64 * 1024 * 1024, device="cuda")
    entries = []
    for kind in ("topk", "bottomk"):
        for rows, cols, k in SHAPES:
            x = torch.randn(rows, cols, device="cuda")
            base = unison.fallback(rows, cols, k, caps, kind)
            cands = [("direct", None)] + [(f"2ce_{t}", unison.RankChoice(True, base.wg, base.kl, t, base.ctile)) for t in (256, 512, 1024, 2048)
                                          if t < cols and -(-cols // t) * min(k, t) < cols]
            results = {name: timed(lambda c=c: rank.rank_select(x, k, kind, choice=c), flush) for name, c in cands}
            best = min(results, key=results.get)
            choice = dict(cands)[best]
            entry = {"kind": kind, "rows": rows, "cols": cols, "k": k, "use_2ce": choice is not None, "wg": base.wg, "kl": base.kl,
                     "tile": choice.tile if choice else base.tile, "ctile": base.ctile, "ms": round(results[best], 5),
                     "direct_ms": round(results["direct"], 5)}
            print(json.dumps({**entry, "all_ms": {n: round(v, 5) for n, v in results.items()}}), flush=True)
            entries.append(entry)
    if not args.dry_run:
        unison.TABLE_PATH.parent.mkdir(parents=True, exist_ok=True)
        unison.TABLE_PATH.write_text(json.dumps({"device": torch.cuda.get_device_name(0), "entries": entries}, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
