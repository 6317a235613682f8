"""Backend capability matrix and its Markdown renderer.

Same role as the reference's matrix (crates/st-bench/src/backend_matrix.rs:20-700 and its
``backend_matrix`` doc-sync binary): one row per capability, one entry per backend with a state
(ready / planned / stub) and a note, plus summaries per backend and per capability.  This build
has two backends: ``cpu`` (PyTorch CPU, used by the small configurations and every oracle) and
``cuda`` (hand-written sm_100a kernels).

    python -m benchmarks.capability_matrix            # Markdown table
    python -m benchmarks.capability_matrix --json
"""
from __future__ import annotations

import json
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional

BACKENDS = ("cpu", "cuda")
READY, PLANNED, STUB = "ready", "planned", "stub"
MARKER = {READY: "✅", PLANNED: "⚠️", STUB: "❌", None: ""}


@dataclass(frozen=True)
class Entry:
    state: Optional[str]
    note: str


@dataclass(frozen=True)
class Row:
    capability: str
    entries: Dict[str, Entry]

    def entry(self, backend: str) -> Entry:
        return self.entries[parse_backend(backend)]

    def summarize(self) -> Dict[str, int]:
        out = {READY: 0, PLANNED: 0, STUB: 0}
        for e in self.entries.values():
            if e.state:
                out[e.state] += 1
        return out


def parse_backend(name: str) -> str:
    label = name.strip().lower()
    aliases = {"cpu": "cpu", "host": "cpu", "cuda": "cuda", "gpu": "cuda", "sm_100a": "cuda", "b200": "cuda", "auto": "cuda"}
    if label not in aliases:
        raise ValueError(f"unknown backend {name!r}; expected one of {sorted(set(aliases))}")
    return aliases[label]


def _row(cap: str, cpu: Entry, cuda: Entry) -> Row:
    return Row(cap, {"cpu": cpu, "cuda": cuda})


MATRIX: List[Row] = [
    _row("Build flag", Entry(None, "always built"), Entry(None, "nvcc -gencode arch=compute_100a,code=sm_100a (in-tree .so)")),
    _row("Min toolchain", Entry(None, "Python 3.12, PyTorch 2.11, g++ 13"), Entry(None, "CUDA 12.9, driver 580")),
    _row("Tensor ops", Entry(READY, "PyTorch CPU ops behind the reference method names"),
         Entry(READY, "tcgen05 GEMM with fused epilogues, fused norm / softmax / CE / elementwise kernels")),
    _row("Attention", Entry(READY, "fp32 reference (online softmax restated)"),
         Entry(READY, "causal forward + backward on tcgen05, head_dim 64 / 128, additive bias")),
    _row("Convolution", Entry(READY, "im2col + GEMM"), Entry(READY, "implicit-GEMM 3x3 forward / dgrad / wgrad through 4-D TMA boxes")),
    _row("Autodiff / hypergrad", Entry(READY, "torch.autograd + Amegagrad tapes"),
         Entry(READY, "hand-scheduled backward for the transformer; fused hypergrad accumulate / apply kernels")),
    _row("Planner & scheduler", Entry(READY, "rank planner facade, SpiralK heuristics interpreter"),
         Entry(READY, "fixed sm_100a launch choices; persistent tile schedulers inside the kernels")),
    _row("Mixed precision training", Entry(PLANNED, "fp32 only; GradScaler / autocast guard are host utilities"),
         Entry(READY, "bf16 compute, fp32 master weights and optimizer state")),
    _row("Distributed collectives", Entry(READY, "thread rendezvous (C++), gloo process groups"),
         Entry(READY, "fused all-gather→GEMM, GEMM→reduce-scatter, DP bucket step, cross-rank InfoNCE over NVLink peer memory; NCCL baseline")),
    _row("Kernel autotuning", Entry(READY, "autotune store + Wilson-bound acceptance"), Entry(PLANNED, "tile shapes are fixed per problem class")),
    _row("Sparse tensor ops", Entry(PLANNED, "problem profile heuristics only"), Entry(STUB, "no sparse kernels")),
    _row("Quantized inference", Entry(READY, "QAT observer, int8 fake-quant, structured pruning reports"), Entry(STUB, "no fp8 / fp4 kernels yet")),
    _row("Graph fusion pipeline", Entry(None, "not applicable"), Entry(READY, "fusion is explicit: epilogues and fused collectives; no tracing compiler")),
    _row("Dynamic shape compilation", Entry(None, "not applicable"), Entry(READY, "ahead-of-time kernels take runtime shapes; nothing recompiles")),
    _row("ONNX export parity", Entry(STUB, "weights export to JSON / bincode / manifest only"), Entry(STUB, "same")),
    _row("Telemetry", Entry(READY, "plugin bus, JSONL recorder, monitoring hub, atlas, chrono timeline, Chrome trace"),
         Entry(READY, "CUDA-event step timer, per-CTA phase stamps in the fused kernels, device error words")),
    _row("Python wheel support", Entry(READY, "pyproject with console scripts"), Entry(READY, "extension built in-tree by the package")),
    _row("CI coverage", Entry(READY, "pytest -m 'not gpu' (oracles, API, host runtime, thread / gloo ranks)"),
         Entry(READY, "pytest -m gpu numerics vs fp32 references; torchrun harness for 2–8 ranks")),
]


def capability_by_name(name: str) -> Optional[Row]:
    key = name.strip().lower()
    return next((r for r in MATRIX if r.capability.lower() == key), None)


def summarize_backend(backend: str) -> Dict[str, object]:
    b = parse_backend(backend)
    counts = {READY: 0, PLANNED: 0, STUB: 0}
    notes = []
    for r in MATRIX:
        e = r.entries[b]
        if e.state:
            counts[e.state] += 1
        else:
            notes.append({"capability": r.capability, "note": e.note})
    tracked = sum(counts.values())
    return {"backend": b, **counts, "tracked": tracked, "pending": counts[PLANNED] + counts[STUB],
            "readiness_ratio": counts[READY] / tracked if tracked else 0.0,
            "fully_ready": counts[PLANNED] + counts[STUB] == 0, "notes": notes}


def backend_summaries() -> List[Dict[str, object]]:
    return [summarize_backend(b) for b in BACKENDS]


def capabilities_with_state(state: str) -> List[Row]:
    return [r for r in MATRIX if any(e.state == state for e in r.entries.values())]


def pending_capabilities_for_backend(backend: str) -> List[Row]:
    b = parse_backend(backend)
    return [r for r in MATRIX if r.entries[b].state in (PLANNED, STUB)]


def capabilities_with_note_containing(query: str) -> List[Row]:
    q = query.strip().lower()
    return [r for r in MATRIX if q and any(q in e.note.lower() for e in r.entries.values())]


def matrix_summary() -> Dict[str, object]:
    per = backend_summaries()
    ready = sum(s[READY] for s in per)
    tracked = sum(s["tracked"] for s in per)
    return {"capabilities": len(MATRIX), "backends": list(BACKENDS), "ready": ready, "tracked": tracked,
            "readiness_ratio": ready / tracked if tracked else 0.0}


def render_markdown() -> str:
    lines = ["| Capability | " + " | ".join(BACKENDS) + " |", "|---|" + "---|" * len(BACKENDS)]
    for r in MATRIX:
        cells = [f"{MARKER[r.entries[b].state]} {r.entries[b].note}".strip() for b in BACKENDS]
        lines.append(f"| {r.capability} | " + " | ".join(cells) + " |")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if "--json" in argv:
        print(json.dumps({"matrix": [{"capability": r.capability,
                                      "entries": {b: vars(e) for b, e in r.entries.items()}} for r in MATRIX],
                          "summary": matrix_summary(), "backends": backend_summaries()}, ensure_ascii=False, indent=1))
    else:
        print(render_markdown())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
