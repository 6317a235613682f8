"""MLP regression on the CPU backend (plumbing check of the public API, no GPU needed).

Data: ``x[256x8] ~ N(0,1)``, ``w[8] ~ N(0, 1/8)`` from the seed, ``y = sin(x·w) + 0.01·N(0,1)``.
Model: ``Sequential(Linear(8,32,name='fc1') → ReLU → Linear(32,1,name='head'))``.
Training: MSE, plain SGD (``apply_step`` with the fallback learning rate 1e-2), batch 32,
200 steps.  Artefacts: a run directory whose ``weights.json`` has the keys ``fc1::weight``
(8x32, stored ``(in, out)``), ``fc1::bias``, ``head::weight``, ``head::bias``.

    python -m spiraltorch_b200.models.mlp_regression --run-dir runs/mlp [--backend cpu|cuda]

Reference: models/python/mlp_regression.py (same API calls, larger data).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

import spiraltorch_b200 as st
from .zoo import RunDir


def make_data(seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(256, 8, generator=g)
    w = torch.randn(8, generator=g) * math.sqrt(1.0 / 8.0)
    y = torch.sin(x @ w) + 0.01 * torch.randn(256, generator=g)
    return x, y.reshape(-1, 1)


def build_model(seed: int = 0) -> "st.nn.Sequential":
    model = st.nn.Sequential()
    model.add(st.nn.Linear(8, 32, name="fc1").init_normal(std=math.sqrt(1.0 / 8.0), seed=seed + 1))
    model.add(st.nn.Relu())
    model.add(st.nn.Linear(32, 1, name="head").init_normal(std=math.sqrt(1.0 / 32.0), seed=seed + 2))
    return model


def run(run_dir=None, backend: str = "cpu", steps: int = 200, batch: int = 32, lr: float = 1e-2, seed: int = 0,
        quiet: bool = False) -> dict:
    x, y = make_data(seed)
    model = build_model(seed)
    trainer = st.nn.ModuleTrainer(backend=backend, fallback_learning_rate=lr)
    trainer.prepare(model)
    loss = st.nn.MeanSquaredError()
    rd = RunDir(run_dir, "mlp_regression", backend=backend,
                hyper_params={"steps": steps, "batch": batch, "lr": lr, "seed": seed}) if run_dir else None
    n_batches = 256 // batch
    batches = [(st.Tensor(x[i * batch:(i + 1) * batch]), st.Tensor(y[i * batch:(i + 1) * batch]))
               for i in range(n_batches)]
    losses, step, epoch = [], 0, 0
    while step < steps:
        take = batches[: min(n_batches, steps - step)]
        stats = trainer.train_epoch(model, loss, take)
        step += stats.batches
        epoch += 1
        losses.append(stats.average_loss)
        if rd:
            rd.log_epoch(epoch, stats.batches, stats.average_loss)
        if not quiet:
            print(f"[epoch={epoch}] steps={step} avg_loss={stats.average_loss:.6f}")
    final = trainer.evaluate_epoch(model, loss, batches).average_loss
    if rd:
        rd.save_weights(model)
        rd.write_summary({"initial_loss": losses[0], "final_loss": final, "steps": step})
    return {"initial_loss": losses[0], "final_loss": final, "model": model, "steps": step}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="cpu")
    ap.add_argument("--run-dir", default=None)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--lr", type=float, default=1e-2)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    out = run(args.run_dir, args.backend, args.steps, args.batch, args.lr, args.seed)
    print(f"initial_loss={out['initial_loss']:.6f} final_loss={out['final_loss']:.6f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
