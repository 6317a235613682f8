"""Study drivers of the Hugging Face bridge: planned, resumable, auditable LoRA fine-tune comparisons.

The reference drives families of fine-tune runs (seeds x arms) from a persisted plan, records every step of the
study in an append-only event log, reuses completed runs when a study is resumed, quarantines the artifacts of failed
ones and writes a per-arm summary (bindings/st-py/spiraltorch/hf_optimizer_study.py:532-1043 plans, :281-368 event
log, :1404-1453 study lock, :2025-2325 the run loop, :1936-1987 summary; hf_peft.py for the adapter injection;
hf_optimizer_control.py for the loss-feedback gate on the optimizer).  This module is that machinery around an
in-process runner (PyTorch executes the model, as in the reference):

* ``build_study_plan`` / ``persist_plan``: seeds x arms -> runs with content-addressed identities; a plan on disk
  is never silently replaced by a different one.
* ``EventLog``: JSONL, every event carries the id of its predecessor and its own sha256, so edits and gaps are found
  on load.
* ``study_lock``: one driver per study directory; a lock left by a dead process is reclaimed.
* ``run_study``: executes what is missing, verifies and reuses what is complete, moves what failed aside, and writes
  the summary (per-arm loss statistics and paired per-seed differences against the first arm).
* ``inject_lora``: freezes a torch model and wraps the named ``nn.Linear`` / GPT-2 ``Conv1D`` layers with trainable
  rank-r factors; ``lora_state`` extracts them.
* ``LossFeedbackGate`` and the three feedback arms (``observe``, ``raw_unguarded``, ``raw_loss_guard``): the gate turns
  the smoothed relative change of the training loss into a multiplier on the learning rate.
* ``lora_finetune_run``: the default runner — a byte-level causal LM (or any ``model_factory``, e.g. a
  ``transformers`` GPT-2 built from a config) fine-tuned through LoRA on a text corpus.
"""
from __future__ import annotations

import contextlib
import hashlib
import json
import math
import os
import shutil
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence

import torch

PLAN_SCHEMA = "spiraltorch_b200.hf_study_plan.v1"
EVENT_SCHEMA = "spiraltorch_b200.hf_study_event.v1"
SUMMARY_SCHEMA = "spiraltorch_b200.hf_study_summary.v1"
RUN_CARD_SCHEMA = "spiraltorch_b200.hf_run_card.v1"
PLAN_FILENAME, EVENTS_FILENAME, SUMMARY_FILENAME, LOCK_FILENAME = "study-plan.json", "study-events.jsonl", "study-summary.json", "study.lock"
FEEDBACK_ARMS = ("observe", "raw_unguarded", "raw_loss_guard")
_RESERVED = frozenset({"schema", "sequence", "recorded_at", "study_id", "event_type", "previous_event_id", "event_id"})


class StudyError(ValueError):
    pass


def canonical_json(value: object) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=True, allow_nan=False).encode()


def sha256_id(value: object) -> str:
    return hashlib.sha256(canonical_json(value)).hexdigest()


def atomic_write_json(path: Path, payload: Mapping[str, object]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(f".{path.name}.{os.getpid()}.tmp")
    with open(tmp, "w") as fh:
        json.dump(payload, fh, indent=2, sort_keys=True)
        fh.write("\n")
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)


# ---------------------------------------------------------------------------------------------------------------
# plan
def run_label(seed: int, arm: str) -> str:
    return f"seed-{seed:04d}-{arm}"


def build_study_plan(study_dir, *, arms: Sequence[str] = FEEDBACK_ARMS, seeds: Iterable[int] = (0, 1, 2), base_config: Optional[Mapping[str, object]] = None,
                     arm_configs: Optional[Mapping[str, Mapping[str, object]]] = None, label: str = "lora-feedback") -> dict:
    """Seeds x arms -> runs.  The first arm is the reference arm of the paired comparison.  ``base_config`` is what
    every run shares (model, data, steps), ``arm_configs[arm]`` what an arm overrides; ``seed`` and ``output_dir``
    belong to the plan and may not appear in either."""
    arms, seeds = list(arms), sorted({int(s) for s in seeds})
    if not arms or len(set(arms)) != len(arms) or not seeds:
        raise StudyError("a study needs distinct arms and at least one seed")
    base, per_arm = dict(base_config or {}), {a: dict((arm_configs or {}).get(a, {})) for a in arms}
    for cfg in (base, *per_arm.values()):
        if {"seed", "output_dir"} & set(cfg):
            raise StudyError("seed and output_dir are managed by the plan")
    unknown = set(arm_configs or {}) - set(arms)
    if unknown:
        raise StudyError(f"arm_configs for arms outside the plan: {sorted(unknown)}")
    identity = {"schema": PLAN_SCHEMA, "label": label, "arms": arms, "seeds": seeds, "base_config": base, "arm_configs": per_arm}
    study_id = sha256_id(identity)
    runs = []
    for seed in seeds:
        for arm in arms:
            config = {**base, **per_arm[arm], "arm": arm, "seed": seed}
            runs.append({"label": run_label(seed, arm), "seed": seed, "arm": arm, "config": config, "run_id": sha256_id({"study": study_id, "config": config}),
                         "output_dir": f"runs/{run_label(seed, arm)}"})
    return {**identity, "study_id": study_id, "study_dir": str(Path(study_dir)), "runs": runs}


def persist_plan(plan: Mapping[str, object]) -> Path:
    """Write the plan, or confirm that the plan already there is the same study."""
    path = Path(plan["study_dir"]) / PLAN_FILENAME
    if path.exists():
        existing = json.loads(path.read_text())
        if existing.get("study_id") != plan["study_id"]:
            raise StudyError(f"{path} holds a different study ({existing.get('study_id', '?')[:12]} vs {str(plan['study_id'])[:12]})")
        return path
    atomic_write_json(path, plan)
    return path


# ---------------------------------------------------------------------------------------------------------------
# event log
class EventLog:
    """Append-only JSONL; ``event_id`` = sha256 of the event without it, ``previous_event_id`` chains the events."""

    def __init__(self, path: Path, study_id: str):
        self.path, self.study_id = Path(path), study_id
        self.events: List[dict] = self._load()

    def _load(self) -> List[dict]:
        if not self.path.exists():
            return []
        events, previous = [], None
        for n, line in enumerate(self.path.read_text().splitlines()):
            if not line.strip():
                continue
            try:
                event = json.loads(line)
            except json.JSONDecodeError as exc:
                raise StudyError(f"{self.path}:{n + 1}: not JSON") from exc
            body = {k: v for k, v in event.items() if k != "event_id"}
            if event.get("schema") != EVENT_SCHEMA or event.get("study_id") != self.study_id:
                raise StudyError(f"{self.path}:{n + 1}: event of another study or schema")
            if event.get("sequence") != len(events) or event.get("previous_event_id") != previous or event.get("event_id") != sha256_id(body):
                raise StudyError(f"{self.path}:{n + 1}: event chain broken (edited, reordered or missing events)")
            events.append(event)
            previous = event["event_id"]
        return events

    def append(self, event_type: str, **fields) -> dict:
        clash = _RESERVED & set(fields)
        if clash:
            raise StudyError(f"reserved event fields: {sorted(clash)}")
        body = {"schema": EVENT_SCHEMA, "sequence": len(self.events), "recorded_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                "study_id": self.study_id, "event_type": event_type, "previous_event_id": self.events[-1]["event_id"] if self.events else None, **fields}
        event = {**body, "event_id": sha256_id(body)}
        self.path.parent.mkdir(parents=True, exist_ok=True)
        with open(self.path, "a") as fh:
            fh.write(json.dumps(event, sort_keys=True) + "\n")
            fh.flush()
            os.fsync(fh.fileno())
        self.events.append(event)
        return event

    def completed_by_run(self) -> Dict[str, dict]:
        """Latest ``run_completed`` per run that no later ``run_quarantined`` cancelled."""
        done: Dict[str, dict] = {}
        for e in self.events:
            if e["event_type"] == "run_completed":
                done[e["run_label"]] = e
            elif e["event_type"] == "run_quarantined":
                done.pop(e["run_label"], None)
        return done


def _pid_is_running(pid: int) -> bool:
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


@contextlib.contextmanager
def study_lock(study_dir: Path, study_id: str) -> Iterator[None]:
    """Exclusive-create lock file with the owner's pid; the lock of a process that no longer runs is taken over."""
    path = Path(study_dir) / LOCK_FILENAME
    path.parent.mkdir(parents=True, exist_ok=True)
    for attempt in range(2):
        try:
            fd = os.open(path, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
            break
        except FileExistsError:
            try:
                owner = json.loads(path.read_text())
            except (OSError, json.JSONDecodeError):
                owner = {}
            stale = owner.get("pid") is None or not _pid_is_running(int(owner["pid"]))
            if attempt == 0 and stale:
                with contextlib.suppress(FileNotFoundError):
                    path.unlink()
                continue
            raise StudyError(f"study {study_id[:12]} is being driven by pid {owner.get('pid')}")
    with os.fdopen(fd, "w") as fh:
        json.dump({"pid": os.getpid(), "study_id": study_id}, fh)
    try:
        yield
    finally:
        with contextlib.suppress(FileNotFoundError):
            path.unlink()


# ---------------------------------------------------------------------------------------------------------------
# run loop
def _card_digest(card: Mapping[str, object]) -> str:
    return sha256_id({k: v for k, v in card.items() if k != "card_id"})


def _validate_card(card: Mapping[str, object], run: Mapping[str, object]) -> None:
    if card.get("schema") != RUN_CARD_SCHEMA or card.get("run_id") != run["run_id"]:
        raise StudyError(f"{run['label']}: run card belongs to another run")
    for field in ("eval_loss_before", "eval_loss_after"):
        v = card.get(field)
        if not isinstance(v, (int, float)) or not math.isfinite(v):
            raise StudyError(f"{run['label']}: {field} is not a finite number")
    if card.get("card_id") != _card_digest(card):
        raise StudyError(f"{run['label']}: run card was modified after it was written")


def _quarantine(study_dir: Path, run: Mapping[str, object], log: EventLog, reason: str) -> None:
    src = study_dir / run["output_dir"]
    if src.exists():
        dst = study_dir / "quarantine" / f"{run['label']}-{len(log.events):05d}"
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.move(str(src), str(dst))
    log.append("run_quarantined", run_label=run["label"], run_id=run["run_id"], reason=reason)


def summarize(plan: Mapping[str, object], cards: Mapping[str, Mapping[str, object]]) -> dict:
    """Per-arm mean / std of the final eval loss and of the improvement, and per-seed paired differences against the
    first arm (negative = the arm ended lower than the reference arm on that seed)."""
    arms, ref = list(plan["arms"]), plan["arms"][0]
    by_arm: Dict[str, List[dict]] = {a: [] for a in arms}
    for run in plan["runs"]:
        if run["label"] in cards:
            by_arm[run["arm"]].append({"seed": run["seed"], **cards[run["label"]]})

    def stats(xs: List[float]) -> dict:
        if not xs:
            return {"n": 0, "mean": None, "std": None}
        m = sum(xs) / len(xs)
        return {"n": len(xs), "mean": m, "std": math.sqrt(sum((x - m) ** 2 for x in xs) / (len(xs) - 1)) if len(xs) > 1 else 0.0}
    ref_by_seed = {c["seed"]: c["eval_loss_after"] for c in by_arm[ref]}
    out = {}
    for arm in arms:
        paired = [c["eval_loss_after"] - ref_by_seed[c["seed"]] for c in by_arm[arm] if c["seed"] in ref_by_seed]
        out[arm] = {"eval_loss_after": stats([c["eval_loss_after"] for c in by_arm[arm]]),
                    "improvement": stats([c["eval_loss_before"] - c["eval_loss_after"] for c in by_arm[arm]]),
                    "steps_per_second": stats([c["steps_per_second"] for c in by_arm[arm] if c.get("steps_per_second")]),
                    "paired_delta_vs_reference": stats(paired), "wins_vs_reference": sum(1 for d in paired if d < 0) if arm != ref else None}
    return {"schema": SUMMARY_SCHEMA, "study_id": plan["study_id"], "reference_arm": ref, "arms": out,
            "completed_runs": sorted(cards), "pending_runs": sorted(r["label"] for r in plan["runs"] if r["label"] not in cards)}


def run_study(plan: Mapping[str, object], runner: Optional[Callable[[Mapping[str, object], Path], Mapping[str, object]]] = None, *,
              max_runs: Optional[int] = None, stop_on_failure: bool = False) -> dict:
    """Drive the plan to completion (or for ``max_runs`` new runs).  ``runner(config, output_dir)`` returns the
    measured fields of the run card (at least ``eval_loss_before`` / ``eval_loss_after``)."""
    runner = runner or lora_finetune_run
    study_dir = Path(plan["study_dir"])
    persist_plan(plan)
    with study_lock(study_dir, plan["study_id"]):
        log = EventLog(study_dir / EVENTS_FILENAME, plan["study_id"])
        if not log.events:
            log.append("study_started", runs=len(plan["runs"]))
        done, cards, executed = log.completed_by_run(), {}, 0
        for run in plan["runs"]:
            card_path = study_dir / run["output_dir"] / "run-card.json"
            if run["label"] in done:
                try:
                    card = json.loads(card_path.read_text())
                    _validate_card(card, run)
                    if card["card_id"] != done[run["label"]]["card_id"]:
                        raise StudyError(f"{run['label']}: run card differs from the one the log recorded")
                    cards[run["label"]] = card
                    continue
                except (OSError, json.JSONDecodeError, StudyError) as exc:
                    _quarantine(study_dir, run, log, f"unusable completed run: {exc}")
            elif (study_dir / run["output_dir"]).exists():
                _quarantine(study_dir, run, log, "artifacts of an unfinished run")
            if max_runs is not None and executed >= max_runs:
                continue
            executed += 1
            out_dir = study_dir / run["output_dir"]
            out_dir.mkdir(parents=True, exist_ok=True)
            log.append("run_started", run_label=run["label"], run_id=run["run_id"])
            t0 = time.perf_counter()
            try:
                measured = dict(runner(run["config"], out_dir))
                card = {"schema": RUN_CARD_SCHEMA, "run_id": run["run_id"], "label": run["label"], "arm": run["arm"], "seed": run["seed"], **measured}
                card["card_id"] = _card_digest(card)
                _validate_card(card, run)
            except Exception as exc:  # noqa: BLE001 - a failed run is an outcome of the study, not of the driver
                log.append("run_failed", run_label=run["label"], run_id=run["run_id"], error=f"{type(exc).__name__}: {exc}"[:500])
                _quarantine(study_dir, run, log, "run failed")
                if stop_on_failure:
                    break
                continue
            atomic_write_json(card_path, card)
            log.append("run_completed", run_label=run["label"], run_id=run["run_id"], card_id=card["card_id"], seconds=time.perf_counter() - t0,
                       eval_loss_after=card["eval_loss_after"])
            cards[run["label"]] = card
        summary = summarize(plan, cards)
        summary["events"] = len(log.events)
        summary["failed_runs"] = sorted({e["run_label"] for e in log.events if e["event_type"] == "run_failed"} - set(cards))
        atomic_write_json(study_dir / SUMMARY_FILENAME, summary)
        if not summary["pending_runs"] and not any(e["event_type"] == "study_completed" for e in log.events):
            log.append("study_completed", summary_id=sha256_id({k: v for k, v in summary.items() if k != "events"}))
    return summary


# ---------------------------------------------------------------------------------------------------------------
# LoRA on torch modules
class LoraWrapped(torch.nn.Module):
    """``y = base(x) + (alpha / r) · x A B`` over a frozen ``nn.Linear`` or GPT-2 ``Conv1D``; B starts at zero."""

    def __init__(self, base: torch.nn.Module, rank: int, alpha: float, generator: Optional[torch.Generator] = None):
        super().__init__()
        w = base.weight
        conv1d = type(base).__name__ == "Conv1D"               # transformers' GPT-2 layer stores (in, out)
        fan_in, fan_out = (w.shape[0], w.shape[1]) if conv1d else (w.shape[1], w.shape[0])
        if not 1 <= rank <= min(fan_in, fan_out):
            raise StudyError(f"rank {rank} outside [1, {min(fan_in, fan_out)}]")
        self.base, self.scale = base, alpha / rank
        for p in base.parameters():
            p.requires_grad_(False)
        a = torch.empty(fan_in, rank, dtype=w.dtype, device=w.device)
        a.copy_(torch.randn(fan_in, rank, generator=generator) / math.sqrt(fan_in))
        self.lora_a, self.lora_b = torch.nn.Parameter(a), torch.nn.Parameter(torch.zeros(rank, fan_out, dtype=w.dtype, device=w.device))

    def forward(self, x):
        return self.base(x) + self.scale * ((x @ self.lora_a) @ self.lora_b)

    def merged_delta(self) -> torch.Tensor:
        return self.scale * (self.lora_a @ self.lora_b)


def inject_lora(model: torch.nn.Module, targets: Sequence[str], rank: int, alpha: float = 16.0, seed: int = 0) -> List[str]:
    """Freeze ``model`` and wrap every ``nn.Linear`` / ``Conv1D`` whose qualified name ends with one of ``targets``."""
    for p in model.parameters():
        p.requires_grad_(False)
    gen = torch.Generator().manual_seed(seed)
    wrapped = []
    for name, module in list(model.named_modules()):
        if not any(name == t or name.endswith("." + t) for t in targets):
            continue
        if not (isinstance(module, torch.nn.Linear) or type(module).__name__ == "Conv1D"):
            continue
        parent = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
        setattr(parent, name.rpartition(".")[2], LoraWrapped(module, rank, alpha, gen))
        wrapped.append(name)
    if not wrapped:
        raise StudyError(f"no layer matches the LoRA targets {list(targets)}")
    return wrapped


def lora_state(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v.detach().clone() for k, v in model.state_dict().items() if k.endswith("lora_a") or k.endswith("lora_b")}


# ---------------------------------------------------------------------------------------------------------------
# loss-feedback gate
@dataclass
class LossFeedbackGate:
    """Learning-rate multiplier from the training loss.  Each observation updates an EMA of the loss and an EMA of
    its relative change ``(loss - ema) / max(ema, loss_floor)``.  A smoothed change above ``regression_threshold``
    multiplies the gate by ``1 - attenuation_rate``; below ``-recovery_threshold`` the gate grows by
    ``recovery_rate`` of the distance to ``maximum_gate``.  With ``guard`` on, ``halt_regression_streak`` regressions
    in a row beyond ``halt_threshold`` close the gate (0) until ``resume_improvement_streak`` improvements in a row."""
    loss_ema_alpha: float = 0.2
    relative_delta_ema_alpha: float = 0.3
    loss_floor: float = 1e-3
    regression_threshold: float = 0.02
    halt_threshold: float = 0.10
    recovery_threshold: float = 0.0
    attenuation_rate: float = 0.3
    recovery_rate: float = 0.2
    halt_regression_streak: int = 2
    resume_improvement_streak: int = 2
    warmup_observations: int = 3
    maximum_gate: float = 1.0
    guard: bool = False

    def __post_init__(self):
        self.loss_ema: Optional[float] = None
        self.delta_ema, self.gate, self.halted = 0.0, self.maximum_gate, False
        self.observations = self.regressions = self.improvements = self.halts = 0

    def observe(self, loss: float) -> float:
        if not math.isfinite(loss):
            self.gate = 0.0 if self.guard else self.gate * (1.0 - self.attenuation_rate)
            self.halted = self.guard or self.halted
            self.halts += int(self.guard)
            return self.value()
        self.observations += 1
        if self.loss_ema is None:
            self.loss_ema = loss
            return self.value()
        delta = (loss - self.loss_ema) / max(self.loss_ema, self.loss_floor)
        self.loss_ema += self.loss_ema_alpha * (loss - self.loss_ema)
        self.delta_ema += self.relative_delta_ema_alpha * (delta - self.delta_ema)
        if self.observations <= self.warmup_observations:
            return self.value()
        if self.delta_ema > self.regression_threshold:
            self.gate *= 1.0 - self.attenuation_rate
            self.improvements = 0
            self.regressions = self.regressions + 1 if self.delta_ema > self.halt_threshold else 0
        elif self.delta_ema < -self.recovery_threshold:
            self.gate += self.recovery_rate * (self.maximum_gate - self.gate)
            self.regressions, self.improvements = 0, self.improvements + 1
        if self.guard:
            if not self.halted and self.regressions >= self.halt_regression_streak:
                self.halted, self.halts, self.improvements = True, self.halts + 1, 0
            elif self.halted and self.improvements >= self.resume_improvement_streak:
                self.halted, self.regressions = False, 0
        return self.value()

    def value(self) -> float:
        return 0.0 if self.halted else min(max(self.gate, 0.0), self.maximum_gate)


def gate_for_arm(arm: str, feedback: Optional[Mapping[str, object]] = None) -> Optional[LossFeedbackGate]:
    """``observe`` tracks the gate without applying it (returned with ``applied = False``), ``raw_unguarded`` applies
    it, ``raw_loss_guard`` applies it with the halt / resume guard; any other arm trains without a gate."""
    if arm not in FEEDBACK_ARMS:
        return None
    gate = LossFeedbackGate(**dict(feedback or {}), guard=arm == "raw_loss_guard")
    gate.applied = arm != "observe"
    return gate


# ---------------------------------------------------------------------------------------------------------------
# default runner
class ByteCausalLM(torch.nn.Module):
    """Small pre-norm decoder over bytes; the layer names (``attn.qkv``, ``attn.proj``, ``mlp.fc``, ``mlp.out``) are the LoRA targets."""

    def __init__(self, d_model: int = 64, n_layer: int = 2, n_head: int = 4, max_len: int = 128, vocab: int = 256):
        super().__init__()
        self.tok, self.pos = torch.nn.Embedding(vocab, d_model), torch.nn.Embedding(max_len, d_model)
        self.blocks = torch.nn.ModuleList()
        for _ in range(n_layer):
            blk = torch.nn.Module()
            blk.ln1, blk.ln2 = torch.nn.LayerNorm(d_model), torch.nn.LayerNorm(d_model)
            blk.attn, blk.mlp = torch.nn.Module(), torch.nn.Module()
            blk.attn.qkv, blk.attn.proj = torch.nn.Linear(d_model, 3 * d_model), torch.nn.Linear(d_model, d_model)
            blk.mlp.fc, blk.mlp.out = torch.nn.Linear(d_model, 4 * d_model), torch.nn.Linear(4 * d_model, d_model)
            self.blocks.append(blk)
        self.ln_f, self.head, self.n_head = torch.nn.LayerNorm(d_model), torch.nn.Linear(d_model, vocab, bias=False), n_head

    def forward(self, ids):
        b, t = ids.shape
        x = self.tok(ids) + self.pos(torch.arange(t, device=ids.device))
        for blk in self.blocks:
            q, k, v = blk.attn.qkv(blk.ln1(x)).view(b, t, 3, self.n_head, -1).permute(2, 0, 3, 1, 4)
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + blk.attn.proj(a.transpose(1, 2).reshape(b, t, -1))
            x = x + blk.mlp.out(torch.nn.functional.gelu(blk.mlp.fc(blk.ln2(x))))
        return self.head(self.ln_f(x))


def _synthetic_corpus(seed: int, n: int = 1 << 15) -> bytes:
    """Deterministic text with structure to learn: a second-order chain over a small word list."""
    words = ["spiral", "torch", "tensor", "gate", "loss", "phase", "z", "space", "resonance", "wave", "the", "of", "and", "in"]
    g = torch.Generator().manual_seed(seed)
    nxt = torch.randint(0, len(words), (len(words), len(words), 3), generator=g)
    a, b, out, size = 0, 1, [], 0
    while size < n:
        a, b = b, int(nxt[a, b, int(torch.randint(0, 3, (1,), generator=g))])
        out.append(words[b])
        size += len(words[b]) + 1
    return " ".join(out).encode()[:n]


def _logits(model, ids):
    out = model(ids)
    return out.logits if hasattr(out, "logits") else out


def _lm_loss(model, batch):
    logits = _logits(model, batch[:, :-1])
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), batch[:, 1:].reshape(-1))


def lora_finetune_run(config: Mapping[str, object], output_dir: Path, *, model_factory: Optional[Callable[[], torch.nn.Module]] = None) -> dict:
    """One run of a study.  ``config`` keys (all optional): steps, batch_size, seq_len, lr, weight_decay, lora_rank,
    lora_alpha, lora_targets, eval_batches, corpus (path of a text file; a synthetic corpus otherwise), corpus_seed,
    model (kwargs of ``ByteCausalLM``), pretrain_steps (dense steps on the first half of the corpus before adapters go
    in, standing in for a pretrained checkpoint), feedback (``LossFeedbackGate`` fields), device."""
    c = {"steps": 60, "batch_size": 16, "seq_len": 64, "lr": 3e-3, "weight_decay": 0.0, "lora_rank": 4, "lora_alpha": 8.0,
         "lora_targets": ["attn.qkv", "attn.proj", "mlp.fc", "mlp.out"], "eval_batches": 4, "corpus": None, "corpus_seed": 1234, "model": {},
         "pretrain_steps": 0, "feedback": {}, "device": "cpu", "arm": "observe", "seed": 0, **dict(config)}
    device, seed = torch.device(c["device"]), int(c["seed"])
    raw = Path(c["corpus"]).read_bytes() if c["corpus"] else _synthetic_corpus(int(c["corpus_seed"]))
    data = torch.frombuffer(bytearray(raw), dtype=torch.uint8).long()
    width = int(c["seq_len"]) + 1
    if data.numel() < 4 * width:
        raise StudyError("corpus shorter than four training windows")
    split = data.numel() * 9 // 10
    train, held = data[:split], data[split:]
    if held.numel() < width + 1:
        train, held = data, data[-2 * width:]

    def windows(src: torch.Tensor, n: int, g: torch.Generator) -> torch.Tensor:
        starts = torch.randint(0, src.numel() - width, (n,), generator=g)
        return torch.stack([src[s:s + width] for s in starts.tolist()]).to(device)
    torch.manual_seed(int(c["corpus_seed"]))                     # the base model is shared by every arm and seed of a study
    model = (model_factory() if model_factory else ByteCausalLM(**{"max_len": width, **dict(c["model"])})).to(device)
    if int(c["pretrain_steps"]):
        gp, opt0 = torch.Generator().manual_seed(int(c["corpus_seed"])), torch.optim.AdamW(model.parameters(), lr=3e-3)
        for _ in range(int(c["pretrain_steps"])):
            opt0.zero_grad(set_to_none=True)
            _lm_loss(model, windows(train[: train.numel() // 2], int(c["batch_size"]), gp)).backward()
            opt0.step()
    wrapped = inject_lora(model, list(c["lora_targets"]), int(c["lora_rank"]), float(c["lora_alpha"]), seed)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=float(c["lr"]), weight_decay=float(c["weight_decay"]))
    gate = gate_for_arm(str(c["arm"]), c["feedback"])
    g_eval = torch.Generator().manual_seed(int(c["corpus_seed"]) + 1)
    eval_set = [windows(held, int(c["batch_size"]), g_eval) for _ in range(int(c["eval_batches"]))]

    @torch.no_grad()
    def evaluate() -> float:
        model.eval()
        value = sum(float(_lm_loss(model, b)) for b in eval_set) / len(eval_set)
        model.train()
        return value
    before, g_train, trace = evaluate(), torch.Generator().manual_seed(seed), []
    t0 = time.perf_counter()
    for step in range(int(c["steps"])):
        opt.zero_grad(set_to_none=True)
        loss = _lm_loss(model, windows(train, int(c["batch_size"]), g_train))
        loss.backward()
        loss_value = float(loss.detach())
        multiplier = gate.observe(loss_value) if gate is not None else 1.0
        applied = multiplier if gate is not None and gate.applied else 1.0
        for group in opt.param_groups:
            group["lr"] = float(c["lr"]) * applied
        if applied > 0.0:
            opt.step()
        trace.append({"step": step, "loss": loss_value, "gate": multiplier, "applied": applied})
    seconds = time.perf_counter() - t0
    after = evaluate()
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    torch.save(lora_state(model), output_dir / "adapter.pt")
    with open(output_dir / "trainer-trace.jsonl", "w") as fh:
        fh.writelines(json.dumps(r) + "\n" for r in trace)
    return {"eval_loss_before": before, "eval_loss_after": after, "steps": int(c["steps"]), "steps_per_second": int(c["steps"]) / max(seconds, 1e-9),
            "lora_layers": wrapped, "trainable_parameters": sum(p.numel() for p in params), "final_gate": trace[-1]["gate"] if trace else 1.0,
            "gate_halts": gate.halts if gate is not None else 0, "skipped_steps": sum(1 for r in trace if r["applied"] == 0.0),
            "gate": {k: v for k, v in asdict(gate).items()} if gate is not None else None}


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``spiral-hf-study``: plan and drive a LoRA feedback study, print the summary as JSON."""
    import argparse
    ap = argparse.ArgumentParser(prog="spiral-hf-study", description=main.__doc__)
    ap.add_argument("study_dir")
    ap.add_argument("--arms", nargs="+", default=list(FEEDBACK_ARMS))
    ap.add_argument("--seeds", nargs="+", type=int, default=[0, 1, 2])
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--pretrain-steps", type=int, default=40)
    ap.add_argument("--corpus", default=None)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--max-runs", type=int, default=None)
    ap.add_argument("--plan-only", action="store_true")
    a = ap.parse_args(argv)
    plan = build_study_plan(a.study_dir, arms=a.arms, seeds=a.seeds,
                            base_config={"steps": a.steps, "pretrain_steps": a.pretrain_steps, "corpus": a.corpus, "device": a.device})
    persist_plan(plan)
    print(json.dumps({"study_id": plan["study_id"], "runs": [r["label"] for r in plan["runs"]]} if a.plan_only else run_study(plan, max_runs=a.max_runs), indent=2, sort_keys=True))
    return 0
