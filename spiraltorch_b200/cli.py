"""Command-line entry points (the console scripts of the reference's ``[project.scripts]``,
bindings/st-py/pyproject.toml): a model-zoo launcher, an HPO driver (``spiral-train``,
bindings/st-py/spiral/cli.py), a weight exporter (``spiral-export``, spiral/export.py), a plugin
event recorder and a runtime pre-flight report.

    python -m spiraltorch_b200.cli model-zoo mlp_regression --run-dir runs/mlp
    python -m spiraltorch_b200.cli model-zoo gpt-1.3b --gpus 8            # prints the torchrun command
    python -m spiraltorch_b200.cli train --trials 8 --strategy bayesian --param lr=float:1e-3:1e-1
    python -m spiraltorch_b200.cli export weights.json weights.bin
    python -m spiraltorch_b200.cli runtime-preflight
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]

ZOO = {
    "mlp_regression": ("cpu", "MLP regression, CPU fp32, SGD (plumbing check)", None),
    "char-lm": ("dp", "byte-level char LM, data-parallel, fused gradient all-reduce + AdamW", "charlm"),
    "conv-classifier": ("dp", "conv-pool classifier, data-parallel, fused conv kernels + SGD momentum", "conv"),
    "contrastive": ("dp", "InfoNCE encoder, fused cross-rank similarity kernel + AdamW", "contrastive"),
    "gpt-1.3b": ("tp", "GPT 1.3B, tensor-parallel with fused all-gather→GEMM / GEMM→reduce-scatter", None),
    "zconv_classification": ("recipe", "ZConv 3x3 → ReLU → max-pool → Linear on synthetic 8x8 images", None),
    "llm_char_coherence_scan": ("recipe", "next-character model: Embedding → ZSpaceCoherenceScan → Linear", None),
    "llm_char_wave_rnn_mixer": ("recipe", "next-character model: Embedding → WaveRnn → ZSpaceMixer → Linear", None),
    "lstm_probe": ("recipe", "LSTM sequence-mean regression", None),
    "gnn_graph_regression": ("recipe", "two graph convolutions + mean read-out on a ring graph", None),
    "zspace_vae_reconstruction": ("recipe", "Z-space VAE on rank-3 data (own Adam optimiser)", None),
    "zspace_text_vae": ("recipe", "Z-space VAE over wave-encoded character windows", None),
}


def _torchrun(script: str, gpus: int, extra: list) -> list:
    cmd = [sys.executable]
    if gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                "--master-port", os.environ.get("MASTER_PORT", "29500")]
    return cmd + [str(REPO / script)] + extra


def cmd_model_zoo(args) -> int:
    if args.list or not args.model:
        for name, (_, desc, _) in ZOO.items():
            print(f"{name:18s} {desc}")
        return 0
    if args.model not in ZOO:
        print(f"unknown model '{args.model}'; try --list", file=sys.stderr)
        return 2
    kind, _, key = ZOO[args.model]
    if kind == "cpu":
        from .models import mlp_regression
        return mlp_regression.main(["--backend", args.backend] + (["--run-dir", args.run_dir] if args.run_dir else []))
    if kind == "recipe":
        from .models import recipes
        return recipes.main([args.model, "--backend", args.backend] + (["--run-dir", args.run_dir] if args.run_dir else []))
    if kind == "dp":
        cmd = _torchrun("benchmarks/dp_models.py", args.gpus, ["--model", key, "--steps", str(args.steps)])
    else:
        cmd = _torchrun("bench.py", args.gpus, ["--gpus", str(args.gpus), "--steps", str(args.steps)])
    print(" ".join(cmd))
    if args.dry_run:
        return 0
    import subprocess
    return subprocess.call(cmd)


def _parse_param(spec: str):
    from . import hpo
    name, rest = spec.split("=", 1)
    kind, *vals = rest.split(":")
    if kind == "float":
        return hpo.ParamSpec.Float(name, float(vals[0]), float(vals[1]))
    if kind == "int":
        return hpo.ParamSpec.Int(name, int(vals[0]), int(vals[1]))
    if kind == "cat":
        return hpo.ParamSpec.Categorical(name, vals)
    raise SystemExit(f"bad --param '{spec}' (use name=float:lo:hi | name=int:lo:hi | name=cat:a:b:c)")


def cmd_train(args) -> int:
    """HPO over the MLP regression recipe: each trial trains with the suggested hyper-parameters."""
    from . import hpo
    from .models import mlp_regression
    space = hpo.SearchSpace([_parse_param(p) for p in (args.param or ["lr=float:1e-3:1e-1"])])
    strategy = {"random": lambda: hpo.RandomStrategy(args.seed), "bayesian": lambda: hpo.BayesianStrategy(args.seed, 0.3),
                "population": lambda: hpo.PopulationStrategy(args.seed)}[args.strategy]()
    state_path = Path(args.state) if args.state else None
    if state_path and state_path.exists():
        loop = hpo.SearchLoop.from_state(space, json.loads(state_path.read_text()))
    else:
        loop = hpo.SearchLoop(space, strategy, hpo.Objective("minimize"))
    while len(loop.completed()) < args.trials:
        t = loop.suggest()
        hp = t.suggestion
        out = mlp_regression.run(None, "cpu", steps=int(hp.get("steps", args.steps)), batch=int(hp.get("batch", 32)),
                                 lr=float(hp.get("lr", 1e-2)), seed=args.seed, quiet=True)
        loop.observe(t.id, out["final_loss"])
        print(json.dumps({"trial": t.id, "params": hp, "final_loss": out["final_loss"]}))
        if state_path:
            from .config import atomic_write
            atomic_write(state_path, json.dumps(loop.checkpoint()))
    best = loop.best_trial()
    print(json.dumps({"best_trial": best.id, "params": best.suggestion, "final_loss": best.metric}))
    return 0


def cmd_export(args) -> int:
    """Convert a weight file between the JSON, bincode and manifest formats (suffix decides)."""
    from .nn import io as nn_io
    state = nn_io.load(args.src)
    nn_io.save(args.dst, state)
    print(f"{args.src} -> {args.dst}: {len(state)} tensors")
    return 0


def cmd_plugin(args) -> int:
    """Record plugin-bus events of a model-zoo run into a JSONL file."""
    from . import plugin
    from .models import mlp_regression
    with plugin.record(args.out, args.events.split(",") if args.events else None):
        mlp_regression.run(None, "cpu", steps=args.steps, quiet=True)
    print(f"events written to {args.out}")
    return 0


def cmd_preflight(args) -> int:
    from . import build_info, describe_device
    report = {"build": build_info(), "device": describe_device(args.backend)}
    try:
        from .utils import build
        report["native"] = {"cuda_library": str(build.LIB_PATH), "cuda_library_present": build.LIB_PATH.exists(),
                            "host_library_present": build.HOST_LIB_PATH.exists(), "nvcc": build.find_nvcc()}
    except Exception as exc:  # noqa: BLE001
        report["native"] = {"error": repr(exc)}
    print(json.dumps(report, indent=2, default=str))
    return 0


def _write_ppm(path: str, rgb) -> None:
    """``rgb``: uint8 tensor ``[H, W, 3]`` → binary PPM (P6)."""
    h, w, _ = rgb.shape
    with open(path, "wb") as fh:
        fh.write(f"P6 {w} {h} 255\n".encode())
        fh.write(bytes(rgb.contiguous().cpu().flatten().tolist()))


def cmd_z_volume(args) -> int:
    """Render a synthetic Z volume (depth slices of a travelling wave) through the temporal volume
    renderer and the canvas palette into a PPM image (the role of the reference's
    ``tools/visualize-z-volume``, headless: the image goes to a file)."""
    import torch
    from . import vision
    dev = "cuda" if (args.backend != "cpu" and torch.cuda.is_available()) else "cpu"
    d, h, w = args.depth, args.size, args.size
    z = torch.linspace(0, 1, d, device=dev)[:, None, None]
    y = torch.linspace(-1, 1, h, device=dev)[None, :, None]
    x = torch.linspace(-1, 1, w, device=dev)[None, None, :]
    radius = (x * x + y * y).sqrt()
    volume = torch.sin(6.0 * radius - 6.0 * z).mul(0.5).add(0.5) * torch.exp(-2.0 * z)
    # temporal playback: two harmonics per voxel and a depth-dependent decay, rendered for `frames` instants by the
    # temporal renderer kernel; the chosen frame is then composited front to back and painted
    harmonics = torch.stack([0.25 * torch.cos(3.0 * radius).expand(d, h, w), 0.1 * torch.sin(5.0 * radius + z).expand(d, h, w)], dim=-1)
    decay = (0.5 + 2.0 * z).expand(d, h, w).contiguous()
    frames = max(int(getattr(args, "frames", 8)), 1)
    played = vision.TemporalRenderer(frames, getattr(args, "rate", 24.0)).render(volume.contiguous(), decay, harmonics.contiguous())
    pick = min(max(int(getattr(args, "frame", frames // 2)), 0), frames - 1)
    frame = played.frame(pick).clamp(min=0.0)
    image = vision.temporal_volume_render(frame, density_scale=args.density)[..., :3].mean(-1)       # composited luminance
    rgba = vision.canvas_paint(image, palette=args.palette)
    _write_ppm(args.out, rgba[..., :3])
    print(json.dumps({"out": args.out, "shape": [h, w], "device": dev, "mean": float(image.mean()), "frames": frames,
                      "frame": pick, "time_s": played.times[pick]}))
    return 0


def cmd_xai(args) -> int:
    """Grad-CAM of a (randomly initialised or loaded) ResNet backbone on one image; writes the heat map
    as a PPM (the role of the reference's ``tools/xai-cli``)."""
    import torch
    from . import vision
    from .models import vision_backbones as V
    dev = "cuda" if (args.backend != "cpu" and torch.cuda.is_available()) else "cpu"
    torch.manual_seed(args.seed)
    dtype = torch.bfloat16 if dev == "cuda" else torch.float32
    model = V.ResNet(num_classes=args.classes, widths=(64, 128), device=dev, dtype=dtype)
    img = torch.randn(1, 3, args.size, args.size, device=dev)
    cam = V.grad_cam(model, img)
    heat = torch.nn.functional.interpolate(cam[:, None], size=(args.size, args.size), mode="bilinear")[0, 0]
    rgba = vision.canvas_paint(heat, palette="diverging" if args.palette is None else args.palette)
    _write_ppm(args.out, rgba[..., :3])
    print(json.dumps({"out": args.out, "cam_shape": list(cam.shape[1:]), "device": dev, "peak": float(cam.max())}))
    return 0


def cmd_compare_runs(args) -> int:
    from .models.zoo import compare_runs
    print(json.dumps(compare_runs(args.run_dirs, args.metric), indent=2))
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="spiraltorch")
    sub = ap.add_subparsers(dest="cmd", required=True)
    z = sub.add_parser("model-zoo", help="run a model-zoo recipe")
    z.add_argument("model", nargs="?")
    z.add_argument("--list", action="store_true")
    z.add_argument("--backend", default="cpu")
    z.add_argument("--run-dir", default=None)
    z.add_argument("--gpus", type=int, default=1)
    z.add_argument("--steps", type=int, default=10)
    z.add_argument("--dry-run", action="store_true", help="print the launch command only")
    z.set_defaults(fn=cmd_model_zoo)
    t = sub.add_parser("train", help="hyper-parameter search over the MLP regression recipe")
    t.add_argument("--trials", type=int, default=4)
    t.add_argument("--steps", type=int, default=100)
    t.add_argument("--seed", type=int, default=0)
    t.add_argument("--strategy", default="bayesian", choices=["random", "bayesian", "population"])
    t.add_argument("--param", action="append")
    t.add_argument("--state", default=None, help="checkpoint file: resumed if present, updated after every trial")
    t.set_defaults(fn=cmd_train)
    e = sub.add_parser("export", help="convert weights between .json / .bin / .manifest.json")
    e.add_argument("src")
    e.add_argument("dst")
    e.set_defaults(fn=cmd_export)
    p = sub.add_parser("plugin", help="record plugin events of a short run")
    p.add_argument("--out", default="events.jsonl")
    p.add_argument("--events", default=None)
    p.add_argument("--steps", type=int, default=16)
    p.set_defaults(fn=cmd_plugin)
    zv = sub.add_parser("z-volume", help="render a synthetic Z volume to a PPM image")
    zv.add_argument("--out", default="z_volume.ppm")
    zv.add_argument("--size", type=int, default=64)
    zv.add_argument("--depth", type=int, default=16)
    zv.add_argument("--density", type=float, default=1.0)
    zv.add_argument("--palette", default="spiral")
    zv.add_argument("--backend", default="auto")
    zv.add_argument("--frames", type=int, default=8, help="instants rendered by the temporal renderer")
    zv.add_argument("--rate", type=float, default=24.0, help="frames per second of the playback")
    zv.add_argument("--frame", type=int, default=4, help="which rendered instant becomes the image")
    zv.set_defaults(fn=cmd_z_volume)
    xa = sub.add_parser("xai", help="Grad-CAM heat map of a ResNet backbone")
    xa.add_argument("--out", default="gradcam.ppm")
    xa.add_argument("--size", type=int, default=32)
    xa.add_argument("--classes", type=int, default=10)
    xa.add_argument("--seed", type=int, default=0)
    xa.add_argument("--palette", default=None)
    xa.add_argument("--backend", default="auto")
    xa.set_defaults(fn=cmd_xai)
    cr = sub.add_parser("compare-runs", help="rank model-zoo run directories by a logged metric")
    cr.add_argument("run_dirs", nargs="+")
    cr.add_argument("--metric", default="average_loss")
    cr.set_defaults(fn=cmd_compare_runs)
    r = sub.add_parser("runtime-preflight", help="report device, build and native-library status")
    r.add_argument("--backend", default="auto")
    r.set_defaults(fn=cmd_preflight)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return args.fn(args)


def model_zoo_main() -> int:
    return main(["model-zoo"] + sys.argv[1:])


def train_main() -> int:
    return main(["train"] + sys.argv[1:])


def export_main() -> int:
    return main(["export"] + sys.argv[1:])


def plugin_main() -> int:
    return main(["plugin"] + sys.argv[1:])


def preflight_main() -> int:
    return main(["runtime-preflight"] + sys.argv[1:])


if __name__ == "__main__":
    sys.exit(main())
