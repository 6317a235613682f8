"""Small model-zoo recipes on the public ``st.nn`` API (CPU by default, any backend the session resolves).

Each recipe builds synthetic data from a seed, trains with ``ModuleTrainer`` (or the model's own
optimiser for the VAEs) (parameter gradients are means over the batch of a mean loss, as in the reference,
hence the large learning rates) and, given ``run_dir``, writes the run-directory layout of
:mod:`spiraltorch_b200.models.zoo`.  They mirror the reference's scripts in ``models/python``:
``zconv_classification.py``, ``llm_char_coherence_scan.py``, ``llm_char_wave_rnn_mixer.py``,
``zspace_vae_reconstruction.py``, ``zspace_text_vae.py`` and the Rust ``modelzoo_gnn_graph_regression`` /
``modelzoo_lstm_probe`` examples — same layer stacks and artefacts, smaller data — plus
``llm_char_coherence_wave.py``, ``maxwell_simulated_z_classification.py``, ``mellin_log_grid_classification.py``,
``modelzoo_wave_rnn_sequence``, ``modelzoo_zspace_mixer_regression``, the forward-only ``modelzoo_zrba_telemetry``,
``vision_conv_pool_classification.py`` and the two-stage ``llm_char_finetune.py``.

    python -m spiraltorch_b200.models.recipes zconv_classification --run-dir runs/zconv
"""
from __future__ import annotations

import argparse
import sys
from typing import Callable, Dict

import torch

import spiraltorch_b200 as st
from .zoo import RunDir

_TEXT = ("spiral torch keeps its weights on a curved manifold and its rhythm in a wave; "
         "the roundtable listens above, here and beneath before it speaks. ") * 4


def _one_hot(ids: torch.Tensor, classes: int) -> torch.Tensor:
    return torch.nn.functional.one_hot(ids.long(), classes).float()


def _train(model, loss, batches, epochs: int, lr: float, backend: str, rd, quiet: bool):
    if backend == "cuda":
        # parameters and batches live on the device: every layer then runs on the sm_100a kernels
        model.to("cuda")
        batches = [(x.cuda(), y.cuda()) for x, y in batches]
    trainer = st.nn.ModuleTrainer(backend=backend, fallback_learning_rate=lr)
    trainer.prepare(model)
    history = []
    for epoch in range(1, epochs + 1):
        stats = trainer.train_epoch(model, loss, batches)
        history.append(stats.average_loss)
        if rd:
            rd.log_epoch(epoch, stats.batches, stats.average_loss)
        if not quiet:
            print(f"[epoch={epoch}] batches={stats.batches} avg_loss={stats.average_loss:.6f}")
    final = trainer.evaluate_epoch(model, loss, batches).average_loss
    return history, final


def zconv_classification(seed: int = 0):
    """Two classes of 8×8 one-channel images (a bright left or right half + noise): ZConv 3×3 → ReLU →
    max-pool 2×2 → Linear → softmax cross-entropy."""
    g = torch.Generator().manual_seed(seed)
    n = 128
    labels = torch.randint(0, 2, (n,), generator=g)
    imgs = 0.3 * torch.randn(n, 1, 8, 8, generator=g)
    imgs[labels == 0, :, :, :4] += 1.0
    imgs[labels == 1, :, :, 4:] += 1.0
    model = st.nn.Sequential()
    model.add(st.nn.ZConv("conv1", 1, 4, (8, 8), (3, 3), padding=(1, 1)))
    model.add(st.nn.Relu())
    model.add(st.nn.Pool2d("max", 4, 8, 8, (2, 2)))
    model.add(st.nn.Linear(4 * 4 * 4, 2, name="head"))
    x, y = imgs.reshape(n, -1), labels.reshape(-1, 1).float()
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, n, 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 2.0


def vision_conv_pool_classification(seed: int = 0):
    """Four classes of 16x16 one-channel images (a bright quadrant + noise): ZConv 3x3 -> ReLU -> max-pool 2x2 ->
    ZConv 3x3 -> ReLU -> max-pool 2x2 -> Linear -> softmax cross-entropy (the layer stack of the reference's
    ``models/python/vision_conv_pool_classification.py``)."""
    g = torch.Generator().manual_seed(seed)
    n = 192
    labels = torch.randint(0, 4, (n,), generator=g)
    imgs = 0.3 * torch.randn(n, 1, 16, 16, generator=g)
    for c, (ys, xs) in enumerate(((slice(0, 8), slice(0, 8)), (slice(0, 8), slice(8, 16)), (slice(8, 16), slice(0, 8)),
                                  (slice(8, 16), slice(8, 16)))):
        imgs[labels == c, :, ys, xs] += 1.0
    model = st.nn.Sequential()
    model.add(st.nn.ZConv("conv1", 1, 8, (16, 16), (3, 3), padding=(1, 1)))
    model.add(st.nn.Relu())
    model.add(st.nn.Pool2d("max", 8, 16, 16, (2, 2)))
    model.add(st.nn.ZConv("conv2", 8, 16, (8, 8), (3, 3), padding=(1, 1)))
    model.add(st.nn.Relu())
    model.add(st.nn.Pool2d("max", 16, 8, 8, (2, 2)))
    model.add(st.nn.Linear(16 * 4 * 4, 4, name="head"))
    x, y = imgs.reshape(n, -1), labels.reshape(-1, 1).float()
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, n, 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 2.0


def _char_windows(steps: int, seed: int):
    data = torch.tensor(list(_TEXT.encode()), dtype=torch.float32) % 64        # 64-symbol alphabet
    g = torch.Generator().manual_seed(seed)
    starts = torch.randint(0, data.numel() - steps - 1, (192,), generator=g)
    x = torch.stack([data[s:s + steps] for s in starts.tolist()])
    y = torch.stack([data[s + steps] for s in starts.tolist()]).reshape(-1, 1)
    return x, y


def llm_char_coherence_scan(seed: int = 0):
    """Next-character model without attention: Embedding → ZSpaceCoherenceScan → Linear over the flattened window."""
    steps, dim = 12, 16
    x, y = _char_windows(steps, seed)
    model = st.nn.Sequential()
    model.add(st.nn.Embedding(64, dim, name="embed"))
    model.add(st.nn.ZSpaceCoherenceScan(dim, steps, memory=4))
    model.add(st.nn.Linear(steps * dim, 64, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, x.shape[0], 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 16.0


def llm_char_wave_rnn_mixer(seed: int = 0):
    """Embedding → WaveRnn (dilated gated recurrence) → ZSpaceMixer → Linear."""
    steps, dim, hidden = 12, 16, 32
    x, y = _char_windows(steps, seed)
    model = st.nn.Sequential()
    model.add(st.nn.Embedding(64, dim, name="embed"))
    model.add(st.nn.WaveRnn("wave", dim, hidden, steps, dilation=2))
    model.add(st.nn.ZSpaceMixer("mixer", hidden))
    model.add(st.nn.Linear(hidden, 64, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, x.shape[0], 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 8.0


def lstm_probe(seed: int = 0):
    """Sequence-sum regression with an LSTM: the target is the mean of the first feature over the steps."""
    g = torch.Generator().manual_seed(seed)
    steps, dim = 8, 4
    x = torch.randn(160, steps * dim, generator=g)
    y = x.reshape(160, steps, dim)[:, :, 0].mean(dim=1, keepdim=True)
    model = st.nn.Sequential()
    model.add(st.nn.Lstm("lstm", dim, 16, steps))
    model.add(st.nn.Linear(16, 1, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 160, 32)]
    return model, st.nn.MeanSquaredError(), batches, 8.0


def gnn_graph_regression(seed: int = 0):
    """One 6-node ring graph; node features → two graph convolutions → mean read-out → scalar target."""
    from ..nn import gnn
    g = torch.Generator().manual_seed(seed)
    adj = torch.zeros(6, 6)
    for i in range(6):
        adj[i, (i + 1) % 6] = adj[(i + 1) % 6, i] = 1.0
    ctx = gnn.GraphContext.from_adjacency(adj)
    net = gnn.ZSpaceGraphNetwork("gnn", ctx, [3, 8, 1], learning_rate=0.3)     # the layers step on their own hypergrad tapes
    model = gnn.ZSpaceGraphRegressor(net, gnn.GraphReadout("mean"))
    batches = []
    for _ in range(24):
        feats = torch.randn(6, 3, generator=g)
        batches.append((st.Tensor(feats), st.Tensor(feats[:, 0].mean().reshape(1, 1))))
    return model, st.nn.MeanSquaredError(), batches, 0.05


def llm_char_coherence_wave(seed: int = 0):
    """Embedding → ZSpaceCoherenceWaveBlock (coherence scan + dilated wave gates) → Linear."""
    steps, dim = 12, 16
    x, y = _char_windows(steps, seed)
    model = st.nn.Sequential()
    model.add(st.nn.Embedding(64, dim, name="embed"))
    model.add(st.nn.ZSpaceCoherenceWaveBlock(dim, steps, 4, dilations=[1, 2]))
    model.add(st.nn.Linear(steps * dim, 64, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, x.shape[0], 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 16.0


def wave_rnn_sequence(seed: int = 0):
    """Sequence regression with a WaveRnn: the target is the last step's first feature minus the first step's."""
    g = torch.Generator().manual_seed(seed)
    steps, dim = 8, 4
    x = torch.randn(160, steps * dim, generator=g)
    seq = x.reshape(160, steps, dim)
    y = (seq[:, -1, 0] - seq[:, 0, 0]).reshape(-1, 1)
    model = st.nn.Sequential()
    model.add(st.nn.WaveRnn("wave", dim, 16, steps, dilation=2))
    model.add(st.nn.Linear(16, 1, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 160, 32)]
    return model, st.nn.MeanSquaredError(), batches, 4.0


def zspace_mixer_regression(seed: int = 0):
    """Linear → ZSpaceMixer → ReLU → Linear on a smooth scalar target."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(192, 8, generator=g)
    y = torch.tanh(x[:, :2].sum(1, keepdim=True)) + 0.5 * x[:, 2:3]
    model = st.nn.Sequential()
    model.add(st.nn.Linear(8, 16, name="fc1"))
    model.add(st.nn.ZSpaceMixer("mixer", 16))
    model.add(st.nn.Relu())
    model.add(st.nn.Linear(16, 1, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 192, 32)]
    return model, st.nn.MeanSquaredError(), batches, 0.5


def maxwell_simulated_z_classification(seed: int = 0):
    """Is a Maxwell-coded signal present?  Features: the running Z statistic of 32 simulated blocks, with
    (kappa * lambda = 0.6 sigma) or without the coded mean; model: Linear → ReLU → Linear, 2 classes."""
    from ..theory import simulate_z_curve
    rows, labels = [], []
    for i in range(192):
        present = i % 2
        rows.append(simulate_z_curve(32, 1.0, 1.0, 0.6 if present else 0.0, seed=seed * 1000 + i).float() / 4.0)
        labels.append(float(present))
    x, y = torch.stack(rows), torch.tensor(labels).reshape(-1, 1)
    x = (x - x.mean(0)) / x.std(0).clamp(min=1e-6) / 16.0      # the deterministic initial weights grow with the index
    model = st.nn.Sequential()
    model.add(st.nn.Linear(32, 16, name="fc1"))
    model.add(st.nn.Relu())
    model.add(st.nn.Linear(16, 2, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 192, 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 1.0


def mellin_log_grid_classification(seed: int = 0):
    """Power-law versus exponential decays, told apart by the magnitudes of their Mellin transforms at
    eight points of the critical line (samples on a logarithmic grid)."""
    from ..frac import mellin_log_grid
    g = torch.Generator().manual_seed(seed)
    t = torch.logspace(-2, 2, 128)
    rows, labels = [], []
    for i in range(160):
        kind = i % 2
        a = 0.5 + float(torch.rand((), generator=g))
        f = (1 + t) ** (-1 - a) if kind else torch.exp(-a * t)
        f = f * (1 + 0.02 * torch.randn(128, generator=g))
        rows.append(torch.tensor([abs(mellin_log_grid(f, 1e-2, 1e2, complex(0.5, 0.5 * k))) for k in range(8)]))
        labels.append(float(kind))
    x = torch.stack(rows).float()
    x = (x - x.mean(0)) / x.std(0).clamp(min=1e-6)
    y = torch.tensor(labels).reshape(-1, 1)
    model = st.nn.Sequential()
    model.add(st.nn.Linear(8, 16, name="fc1"))
    model.add(st.nn.Relu())
    model.add(st.nn.Linear(16, 2, name="head"))
    batches = [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, 160, 32)]
    return model, st.nn.SoftmaxCrossEntropy(), batches, 8.0


def _char_lm(steps: int = 12, dim: int = 16, hidden: int = 32):
    model = st.nn.Sequential()
    model.add(st.nn.Embedding(64, dim, name="embed"))
    model.add(st.nn.SpiralRnn("rnn", dim, hidden, steps))
    model.add(st.nn.Linear(hidden, 64, name="head"))
    return model


def llm_char_finetune(run_dir=None, backend: str = "cpu", epochs: int = 8, seed: int = 0, quiet: bool = False) -> dict:
    """Character LM (Embedding -> SpiralRnn -> Linear) trained on one text, saved, reloaded into a fresh model and
    fine-tuned on a second text: the two-stage flow of the reference's ``models/python/llm_char_finetune.py``
    (:1193-1210 save / ``--load-weights`` resume).  Returns both stages' losses and the loss of the base model on
    the second text before fine-tuning."""
    import tempfile
    from pathlib import Path
    steps = 12

    def windows(text: str, n: int, s: int):
        data = torch.tensor(list(text.encode()), dtype=torch.float32) % 64
        g = torch.Generator().manual_seed(s)
        starts = torch.randint(0, data.numel() - steps - 1, (n,), generator=g)
        x = torch.stack([data[i:i + steps] for i in starts.tolist()])
        y = torch.stack([data[i + steps] for i in starts.tolist()]).reshape(-1, 1)
        return [(st.Tensor(x[i:i + 32]), st.Tensor(y[i:i + 32])) for i in range(0, n, 32)]
    text_b = ("the trainer hands its gradient to the bandit, the bandit hands a knob back; "
              "every step is measured, every measure is kept. ") * 4
    base_batches, tune_batches = windows(_TEXT, 192, seed), windows(text_b, 128, seed + 1)
    loss = st.nn.SoftmaxCrossEntropy()
    rd = RunDir(run_dir, "llm_char_finetune", backend=backend, hyper_params={"epochs": epochs, "seed": seed}) if run_dir else None
    base = _char_lm(steps)
    base_hist, base_final = _train(base, loss, base_batches, epochs, 8.0, backend, rd, quiet)
    work = Path(run_dir) if run_dir else Path(tempfile.mkdtemp(prefix="st_finetune_"))
    work.mkdir(parents=True, exist_ok=True)
    st.nn.save(str(work / "base_weights.json"), base)
    tuned = _char_lm(steps)
    st.nn.load(str(work / "base_weights.json"), tuned)                  # the second stage starts from the saved weights
    probe = st.nn.ModuleTrainer(backend=backend)
    if backend == "cuda":
        tuned.to("cuda")
    before = probe.evaluate_epoch(tuned, loss, [(x.cuda(), y.cuda()) for x, y in tune_batches] if backend == "cuda"
                                  else tune_batches).average_loss
    tune_hist, tune_final = _train(tuned, loss, tune_batches, max(2, epochs // 2), 4.0, backend, None, quiet)
    out = {"initial_loss": base_hist[0], "final_loss": tune_final, "base_final_loss": base_final,
           "finetune_loss_before": before, "history": base_hist + tune_hist, "model": tuned}
    if rd:
        rd.save_weights(tuned)
        rd.write_summary({k: v for k, v in out.items() if k not in ("model", "history")} | {"epochs": epochs})
    return out


_TRAINER_RECIPES: Dict[str, Callable] = {
    "vision_conv_pool_classification": vision_conv_pool_classification,
    "zconv_classification": zconv_classification,
    "llm_char_coherence_scan": llm_char_coherence_scan,
    "llm_char_wave_rnn_mixer": llm_char_wave_rnn_mixer,
    "lstm_probe": lstm_probe,
    "gnn_graph_regression": gnn_graph_regression,
    "llm_char_coherence_wave": llm_char_coherence_wave,
    "wave_rnn_sequence": wave_rnn_sequence,
    "zspace_mixer_regression": zspace_mixer_regression,
    "maxwell_simulated_z_classification": maxwell_simulated_z_classification,
    "mellin_log_grid_classification": mellin_log_grid_classification,
}


def _run_vae(name: str, epochs: int, seed: int, rd, quiet: bool):
    g = torch.Generator().manual_seed(seed)
    if name == "zspace_vae_reconstruction":
        basis = torch.randn(3, 12, generator=g)
        data = torch.randn(96, 3, generator=g) @ basis * 0.5            # rank-3 data in 12 dimensions
        vae = st.nn.ZSpaceVae(12, 3, seed=seed)
        vae.configure_optimizer_by_name("adam")
        step = lambda: vae.train_batch(data, learning_rate=2e-2, beta=1e-3)  # noqa: E731
        evaluate = lambda: vae.evaluate_batch(data)["recon_loss"]            # noqa: E731
    else:
        texts = [_TEXT[i:i + 16] for i in range(0, 16 * 12, 16)]
        vae = st.nn.ZSpaceTextVae(16, 4, seed=seed)
        vae.configure_optimizer_by_name("adam")
        step = lambda: vae.train_text_batch(texts, learning_rate=2e-2, beta=1e-3)  # noqa: E731
        evaluate = lambda: vae.evaluate_text_batch(texts)["recon_loss"]            # noqa: E731
    initial = evaluate()
    history = []
    for epoch in range(1, epochs + 1):
        losses = [step().recon_loss for _ in range(10)]
        history.append(sum(losses) / len(losses))
        if rd:
            rd.log_epoch(epoch, 10, history[-1])
        if not quiet:
            print(f"[epoch={epoch}] batches=10 avg_loss={history[-1]:.6f}")
    final = evaluate()
    if rd:
        vae.save(rd.path / "weights.json")
    return {"initial_loss": initial, "final_loss": final, "history": history, "model": vae}


RECIPES = tuple(_TRAINER_RECIPES) + ("zspace_vae_reconstruction", "zspace_text_vae", "llm_char_finetune")


def run(name: str, run_dir=None, backend: str = "cpu", epochs: int = 8, seed: int = 0, quiet: bool = False) -> dict:
    if name not in RECIPES:
        raise KeyError(f"unknown recipe {name!r}; available: {', '.join(RECIPES)}")
    if name == "llm_char_finetune":
        return llm_char_finetune(run_dir, backend, epochs, seed, quiet)
    rd = RunDir(run_dir, name, backend=backend, hyper_params={"epochs": epochs, "seed": seed}) if run_dir else None
    if name in _TRAINER_RECIPES:
        model, loss, batches, lr = _TRAINER_RECIPES[name](seed)
        history, final = _train(model, loss, batches, epochs, lr, backend, rd, quiet)
        out = {"initial_loss": history[0], "final_loss": final, "history": history, "model": model}
        if rd:
            rd.save_weights(model)
    else:
        out = _run_vae(name, epochs, seed, rd, quiet)
    if rd:
        rd.write_summary({"initial_loss": out["initial_loss"], "final_loss": out["final_loss"], "epochs": epochs})
    return out


def zrba_telemetry(run_dir=None, seed: int = 0, rows: int = 24, d_model: int = 16) -> dict:
    """Forward-only Z-RBA probe (the reference's `modelzoo_zrba_telemetry` example): run the block on a
    synthetic indexed batch, score its predictive intervals against the noiseless signal and, given
    `run_dir`, write `zrba_telemetry.json`."""
    import json
    from pathlib import Path
    from ..nn import SpectralFeatureSample, ZFrame, ZIndex, ZRBA, ZRBAConfig
    from ..nn.zspace import ZTensor
    g = torch.Generator().manual_seed(seed)
    idx = [ZIndex(i % 3, i % 2, i % 4) for i in range(rows)]
    signal = torch.sin(torch.arange(rows, dtype=torch.float32) / 3.0)
    mu = signal[:, None] + 0.1 * torch.randn(rows, d_model, generator=g)
    sigma = 0.05 + 0.05 * torch.rand(rows, d_model, generator=g)
    block = ZRBA(ZRBAConfig(d_model=d_model, n_heads=4, cov_rank=4, gate_seed=seed))
    out, cov, tel = block.forward(ZTensor(st.Tensor(mu), st.Tensor(sigma), idx), ZFrame(4),
                                  SpectralFeatureSample(1, 0.8, 0.1, 0.05, float(mu.abs().mean())))
    metrics = tel.metrics(out.mu, out.sigma, (signal * cov.gate.applied).tolist(), 0.9, idx)
    bundle = tel.bundle_metrics(metrics).to_json()
    bundle["attention"] = {"entropy": tel.attention.entropy, "dominant_probability": tel.attention.dominant_probability}
    if run_dir:
        Path(run_dir).mkdir(parents=True, exist_ok=True)
        (Path(run_dir) / "zrba_telemetry.json").write_text(json.dumps(bundle, indent=2))
    return bundle


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("recipe", choices=RECIPES)
    ap.add_argument("--backend", default="cpu")
    ap.add_argument("--run-dir", default=None)
    ap.add_argument("--epochs", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    out = run(args.recipe, args.run_dir, args.backend, args.epochs, args.seed)
    print(f"initial_loss={out['initial_loss']:.6f} final_loss={out['final_loss']:.6f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
