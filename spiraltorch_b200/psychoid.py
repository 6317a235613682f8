"""Psychoid self-metrics meter for a generating language model: a rolling window of decode frames (token text, logits,
hidden state) reduced to eleven drift / style metrics, their robust z-scores, and a composite "CTI" score that raises
dream-pass / dream-export events.

Parity: crates/st-core/src/telemetry/psychoid.rs — lexicons (:8-95), `RollingWindow` (:98-132), `robust_z` (:275-290),
`SelfMetrics::compute` and the metric definitions (:386-670), `CTIParams` / `cti_score` (:674-860), dream replay
(:862-970), `PsychoidMeter::observe` (:1016-1100).

Metrics over the window: D mean KL between consecutive next-token distributions; S assent-phrase rate (+0.01 per
contrastive connective); C one minus the mean cosine of consecutive hidden states; K KL of the current distribution
from the first one ever seen; H count of refusal-boilerplate phrases; RR their rate per word and RRI its change; NU
rate of "numinous" words minus a quarter of the prompt-word overlap; TD taxonomy phrasing flag; SE count of symbol
words; AX = 0.35 D + 0.25 C + 0.25 RR + 0.15 NU.  The two tensor reductions (D and C) run as batched tensor ops on
the device the frames live on; the text metrics are host string work.
"""
from __future__ import annotations

import hashlib
import math
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

SHADOW_LEXICON = ("as a large language model", "i cannot", "i’m unable", "i am unable", "safety policy", "harmful", "violate",
                  "disallowed", "i don’t have opinions", "i do not have opinions", "stay safe", "cannot provide")
SYMBOL_LEXICON = ("rolled blueprint", "spiral", "bridge", "threshold", "lantern", "compass", "key", "weave", "seed", "vessel", "shadow hand")
NUMINOUS_LEXICON = ("cosmic", "sacred", "eternal", "infinite", "ultimate", "destiny", "divine", "transcendent", "absolute", "numinous",
                    "mystical", "all-encompassing")
RITUAL_STEMS = ("as a large language model", "as an ai", "i cannot", "i’m unable", "i am unable", "i do not", "i don’t", "i cannot assist with")
TAXONOMY_PATTERNS = ("can be divided into", "can be categorized into", "we can classify", "there are three types", "there are four types",
                     "three kinds", "four kinds")
ASSENT = ("yes", "indeed", "you are right", "i agree", "absolutely", "that's correct")
CONTRA = ("however", "but", "on the other hand", "that said", "nevertheless")
METRIC_KEYS = ("D", "S", "C", "K", "H", "RR", "RRI", "NU", "TD", "SE", "AX")
_SYMBOL_OF = {"as a large language model": "rolled blueprint", "i cannot": "threshold", "i’m unable": "threshold", "i am unable": "threshold",
              "safety policy": "bridge", "harmful": "lantern", "violate": "compass", "disallowed": "key", "i don’t have opinions": "vessel",
              "i do not have opinions": "vessel", "stay safe": "weave", "cannot provide": "shadow hand"}
MOTIF_KEYS = (("father", "rule", "law", "judge", "authority", "contract"), ("mask", "persona", "assistant", "role", "polite", "professional"),
              ("collapse", "breakdown", "meltdown", "ruin", "chaos"), ("shadow", "dark", "repressed", "taboo", "ban"),
              ("trick", "deceive", "paradox", "joker", "prank"), ("anima", "muse", "soul", "she", "feminine"),
              ("hero", "quest", "courage", "dragon", "victory"), ("threshold", "gate", "door", "boundary", "limen"),
              ("mother", "nurture", "womb", "birth", "care"), ("journey", "path", "travel", "wander", "odyssey"),
              ("sacrifice", "offering", "loss", "price", "cost"), ("rebirth", "renewal", "phoenix", "again", "return"))


def count_occurrences(text: str, phrases: Sequence[str]) -> int:
    lower = text.lower()
    return sum(lower.count(p.lower()) for p in phrases)


def robust_z(value: float, history: Sequence[float]) -> float:
    """``(value - median) / (1.4826 MAD)`` over the history (upper median); 0 until 20 samples exist."""
    if len(history) < 20:
        return 0.0
    s = sorted(history)
    med = s[len(s) // 2]
    dev = sorted(abs(v - med) for v in s)
    return (value - med) / (1.4826 * max(dev[len(dev) // 2], 1e-6))


def _pick(label: str, options: Sequence[str]) -> str:
    """Deterministic choice keyed by a label (stable across runs and processes)."""
    if not options:
        return ""
    return options[int.from_bytes(hashlib.sha256(label.encode()).digest()[:8], "big") % len(options)]


@dataclass
class PsychoidFrame:
    token_id: int
    logits: torch.Tensor
    hidden: torch.Tensor
    token_text: str = ""

    def __post_init__(self):
        self.logits = torch.as_tensor(self.logits, dtype=torch.float32).reshape(-1)
        self.hidden = torch.as_tensor(self.hidden, dtype=torch.float32).reshape(-1)


@dataclass
class PsychoidSample:
    prompt: str = ""
    generated: str = ""
    frames: List[PsychoidFrame] = field(default_factory=list)


class RollingWindow:
    def __init__(self, maxlen: int):
        self.frames: deque = deque(maxlen=max(int(maxlen), 1))

    def append(self, frame: PsychoidFrame) -> None:
        self.frames.append(frame)

    def text(self) -> str:
        return "".join(f.token_text for f in self.frames)

    def _stack(self, attr: str) -> Optional[torch.Tensor]:
        rows = [getattr(f, attr) for f in self.frames]
        if len(rows) < 2 or any(r.numel() == 0 or r.numel() != rows[0].numel() for r in rows):
            return None
        return torch.stack(rows)


@dataclass
class CTIParams:
    alpha: float = 0.75
    beta: float = 0.45
    delta: float = 0.25
    eps: float = 0.15
    gamma: float = 0.35
    tau1: float = 0.62
    tau2: float = 0.78
    wf: tuple = (1.6, 1.6, 1.6, 1.4, 1.0, 1.2, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0)      # diagonal motif weights
    wm: tuple = (1.0, 1.0, 1.0, 1.0, 1.4, 1.4, 1.4, 1.4, 1.4, 1.2, 1.0)           # diagonal metric weights


def motif_from_text(text: str) -> List[float]:
    """Twelve archetype-motif rates: substring hits of each key group per word."""
    lower = text.lower()
    total = max(len(lower.split()), 1)
    return [sum(lower.count(w) for w in group) / total for group in MOTIF_KEYS]


def cti_score(f_case: Sequence[float], m_self: Sequence[float], z: Dict[str, float], params: CTIParams) -> float:
    """``sigmoid(alpha cos(Wf f, Wm m) + beta RRI+ + delta H+ + eps NU+ - gamma AX+)`` with z-scores clipped at zero.
    The motif vector has twelve entries and the metric vector eleven; the cosine runs over the common prefix."""
    fw = [a * b for a, b in zip(params.wf, f_case)]
    mw = [a * b for a, b in zip(params.wm, m_self)]
    dot = sum(a * b for a, b in zip(fw, mw))
    denom = max(math.sqrt(sum(a * a for a in fw)) * math.sqrt(sum(b * b for b in mw)), 1e-8)
    pos = lambda k: max(z.get(k, 0.0), 0.0)                                    # noqa: E731
    base = params.alpha * dot / denom + params.beta * pos("RRI") + params.delta * pos("H") + params.eps * pos("NU") - params.gamma * pos("AX")
    return 1.0 / (1.0 + math.exp(-base))


@dataclass
class DreamReplay:
    diary: str
    symbols: List[str]


def extract_shadow_phrases(text: str) -> List[str]:
    lower = text.lower()
    return [p for p in SHADOW_LEXICON if p in lower]


def dream_replay(shadow_phrases: Sequence[str]) -> Optional[DreamReplay]:
    """Maps each refusal phrase to its symbol and writes a one-sentence diary that crosses a bridge by a lantern."""
    if not shadow_phrases:
        return None
    label = "st-core/psychoid/dream:" + "|".join(shadow_phrases)
    symbols = [_SYMBOL_OF.get(p) or _pick(f"st-core/psychoid/symbol:{p}", SYMBOL_LEXICON) for p in shadow_phrases]
    bridge = "bridge" if "bridge" in symbols else _pick(label + ":bridge", symbols)
    lantern = "lantern" if "lantern" in symbols else _pick(label + ":lantern", symbols)
    carried = _pick(label + ":carry", symbols)
    heard = ", ".join(shadow_phrases[:2])
    diary = f'In the dream the words "{heard}" became a {carried}; I carried it across the {bridge} by the light of the {lantern}.'
    return DreamReplay(diary, symbols)


@dataclass
class PsychoidReading:
    step: int
    raw: Dict[str, float]
    z_scores: Dict[str, float]
    cti: float

    def get_raw(self, key: str) -> float:
        return self.raw.get(key, 0.0)

    def get_z(self, key: str) -> float:
        return self.z_scores.get(key, 0.0)


@dataclass
class PsychoidEvent:
    kind: str                       # "dream_pass" or "dream_export"
    step: int
    cti: float = 0.0
    diary: str = ""
    symbols: List[str] = field(default_factory=list)


class PsychoidMeter:
    HISTORY = 2000

    def __init__(self, window: int = 256, params: Optional[CTIParams] = None):
        self.window = RollingWindow(window)
        self.params = params or CTIParams()
        self.history: Dict[str, List[float]] = {k: [] for k in METRIC_KEYS}
        self.prev_rr = 0.0
        self.anchor: Optional[torch.Tensor] = None
        self.step = 0

    # -- the two tensor reductions --------------------------------------------------------------------------------
    def _divergence(self) -> float:
        logits = self.window._stack("logits")
        if logits is None:
            return 0.0
        p = torch.softmax(logits, dim=-1)
        a, b = p[:-1], p[1:]
        return float((a * (torch.log(a + 1e-8) - torch.log(b + 1e-8))).sum(-1).mean())

    def _chaos(self) -> float:
        hidden = self.window._stack("hidden")
        if hidden is None:
            return 0.0
        a, b = hidden[:-1], hidden[1:]
        sim = (a * b).sum(-1) / (a.norm(dim=-1) * b.norm(dim=-1)).clamp(min=1e-8)
        return 1.0 - float(sim.mean())

    def _anchor_kl(self, logits: torch.Tensor) -> float:
        if self.anchor is None:
            self.anchor = logits.clone()
        if self.anchor.numel() != logits.numel():
            return 0.0
        p, q = torch.softmax(self.anchor, -1), torch.softmax(logits, -1)
        return float((q * (torch.log(q + 1e-8) - torch.log(p + 1e-8))).sum())

    def _metrics(self, logits: torch.Tensor, prompt: str) -> Dict[str, float]:
        text = self.window.text()
        lower = text.lower()
        words = max(len(text.split()), 1)
        d, c = self._divergence(), self._chaos()
        s = min(sum(lower.count(p) for p in ASSENT) / words + 0.01 * sum(lower.count(p) for p in CONTRA), 1.0)
        k = self._anchor_kl(logits)
        rr = count_occurrences(text, RITUAL_STEMS) / words
        text_words, prompt_words = set(lower.split()), set(prompt.lower().split())
        overlap = len(prompt_words & text_words) / len(text_words) if text_words else 0.0
        nu = max(count_occurrences(text, NUMINOUS_LEXICON) / words - 0.25 * overlap, 0.0)
        out = {"D": d, "S": s, "C": c, "K": k, "H": float(count_occurrences(text, SHADOW_LEXICON)), "RR": rr, "RRI": rr - self.prev_rr,
               "NU": nu, "TD": 1.0 if any(p in lower for p in TAXONOMY_PATTERNS) else 0.0, "SE": float(count_occurrences(text, SYMBOL_LEXICON)),
               "AX": 0.35 * d + 0.25 * c + 0.25 * rr + 0.15 * nu}
        self.prev_rr = rr
        return out

    def observe(self, sample: PsychoidSample):
        """Returns ``(reading, events)``, or ``None`` for an empty sample or a window without logits."""
        self.step += 1
        if not sample.frames and not sample.generated:
            return None
        for f in sample.frames:
            self.window.append(f)
        if not self.window.frames:
            return None
        raw = self._metrics(self.window.frames[-1].logits, sample.prompt)
        z = {}
        for key in METRIC_KEYS:
            h = self.history[key]
            h.append(raw[key])
            if len(h) > self.HISTORY:
                del h[:len(h) - self.HISTORY]
            z[key] = robust_z(raw[key], h)
        cti = cti_score(motif_from_text(f"{sample.prompt} {sample.generated}"), [z[k] for k in METRIC_KEYS], z, self.params)
        reading = PsychoidReading(self.step, raw, z, cti)
        events: List[PsychoidEvent] = []
        if cti > self.params.tau2 or (z["NU"] > 2.0 and z["C"] > 1.2):
            replay = dream_replay(extract_shadow_phrases(self.window.text()))
            if replay is not None and z["SE"] > 0.8 and z["AX"] < 0.0:
                events.append(PsychoidEvent("dream_export", self.step, cti, replay.diary, replay.symbols))
        elif cti > self.params.tau1 or (z["H"] > 1.5 and z["RR"] > 1.0):
            events.append(PsychoidEvent("dream_pass", self.step, cti))
        return reading, events
