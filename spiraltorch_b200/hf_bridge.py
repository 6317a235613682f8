"""Bridge between PyTorch / Hugging Face style checkpoints and ``st.nn`` modules.

The reference's ``hf_*.py`` family drives LoRA fine-tuning studies of Hugging Face models from the
SpiralTorch trainer (bindings/st-py/spiraltorch/hf_lora_bridge.py and friends; PyTorch executes the model).
What a user needs from it when switching frameworks is the weight plumbing, which this module provides
without importing ``transformers``:

* ``key_map_for_linears`` builds the ``{source: {target, transform}}`` rules that
  ``Module.load_state_dict_subset_mapped_checked`` consumes: ``torch.nn.Linear`` stores ``(out, in)``, ``st.nn.Linear``
  stores ``(in, out)``, a GPT-2 ``Conv1D`` already stores ``(in, out)``; biases become ``(1, out)`` rows.
* ``load_torch_module`` / ``export_torch_state`` move weights in both directions and report what matched.
* ``merge_lora`` folds ``scale · A · B`` of an ``st.nn.LoraLinear`` into a dense weight; ``lora_from_delta`` goes the
  other way with a truncated SVD, so adapters trained elsewhere (``lora_A`` / ``lora_B`` pairs) can be attached.
"""
from __future__ import annotations

from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .nn.modules import LoraLinear, Module


def _is_conv1d_layout(weight: torch.Tensor, in_features: int, out_features: int) -> Optional[bool]:
    if tuple(weight.shape) == (in_features, out_features) and in_features != out_features:
        return True
    if tuple(weight.shape) == (out_features, in_features) and in_features != out_features:
        return False
    return None                                    # square: the caller must say


def key_map_for_linears(pairs: Iterable[Tuple[str, str]], source_state: Mapping[str, torch.Tensor], target: Module,
                        conv1d: Optional[bool] = None) -> Dict[str, dict]:
    """``pairs`` = (source prefix, target layer name), e.g. ``("h.0.mlp.c_fc", "fc1")``.  For every pair the rules
    ``<src>.weight → <dst>::weight`` (transposed unless the source is in ``Conv1D`` layout) and ``<src>.bias →
    <dst>::bias`` are produced.  ``conv1d`` forces the layout; by default it is inferred from the shapes."""
    expected = {p.name: tuple(p.value.shape) for p in target.parameters()}
    rules: Dict[str, dict] = {}
    for src, dst in pairs:
        wkey, bkey = f"{src}.weight", f"{src}.bias"
        if f"{dst}::weight" not in expected:
            raise KeyError(f"target has no parameter '{dst}::weight'")
        fin, fout = expected[f"{dst}::weight"]
        if wkey in source_state:
            layout = conv1d if conv1d is not None else _is_conv1d_layout(source_state[wkey], fin, fout)
            if layout is None:
                layout = False                     # square and unspecified: torch.nn.Linear convention
            rules[wkey] = {"target": f"{dst}::weight", "transform": "identity" if layout else "transpose"}
        if bkey in source_state and f"{dst}::bias" in expected:
            rules[bkey] = {"target": f"{dst}::bias", "transform": "identity"}
    return rules


def _rows(state: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """1-D tensors (biases, norm gains) become ``(1, n)`` rows, the 2-D convention of ``st.nn``."""
    return {k: (v.detach().reshape(1, -1) if v.dim() == 1 else v.detach()) for k, v in state.items() if v.dim() in (1, 2)}


def load_torch_module(target: Module, source: "torch.nn.Module | Mapping[str, torch.Tensor]",
                      pairs: Iterable[Tuple[str, str]], conv1d: Optional[bool] = None) -> dict:
    """Copies the named linear layers of a PyTorch module (or state dict) into ``target`` and returns the report of
    ``load_state_dict_subset_mapped_checked`` (matched / missing / shape-mismatched entries, content hashes)."""
    state = source.state_dict() if isinstance(source, torch.nn.Module) else dict(source)
    state = _rows(state)
    rules = key_map_for_linears(pairs, state, target, conv1d)
    return target.load_state_dict_subset_mapped_checked(state, rules)


def export_torch_state(source: Module, pairs: Iterable[Tuple[str, str]], conv1d: bool = False) -> Dict[str, torch.Tensor]:
    """The inverse mapping: ``{<dst>.weight, <dst>.bias}`` tensors in ``torch.nn.Linear`` (or ``Conv1D``) layout for
    (st layer name, torch prefix) pairs."""
    own = {p.name: p.value for p in source.parameters()}
    out: Dict[str, torch.Tensor] = {}
    for name, prefix in pairs:
        w = own[f"{name}::weight"].detach().clone()
        out[f"{prefix}.weight"] = w if conv1d else w.t().contiguous()
        if f"{name}::bias" in own:
            out[f"{prefix}.bias"] = own[f"{name}::bias"].detach().reshape(-1).clone()
    return out


def merge_lora(layer: LoraLinear) -> torch.Tensor:
    """Dense ``(in, out)`` weight equal to the adapter-augmented layer: ``W + (alpha / rank) · A · B``."""
    p = {q.name: q.value for q in layer.parameters()}
    n = layer.name
    return p[f"{n}::weight"] + layer.scale * (p[f"{n}::lora_a"] @ p[f"{n}::lora_b"])


def attach_lora_factors(layer: LoraLinear, lora_a: torch.Tensor, lora_b: torch.Tensor, *, peft_layout: bool = True) -> None:
    """Loads adapter factors.  With ``peft_layout`` the inputs are ``lora_A (rank, in)`` and ``lora_B (out, rank)`` as
    stored by PEFT; they are transposed into this framework's ``(in, rank)`` / ``(rank, out)``."""
    a, b = (lora_a.t(), lora_b.t()) if peft_layout else (lora_a, lora_b)
    p = {q.name: q for q in layer.parameters()}
    n = layer.name
    if tuple(a.shape) != tuple(p[f"{n}::lora_a"].value.shape) or tuple(b.shape) != tuple(p[f"{n}::lora_b"].value.shape):
        raise ValueError(f"adapter factors {tuple(a.shape)}, {tuple(b.shape)} do not fit rank-{layer.rank} layer '{n}'")
    p[f"{n}::lora_a"].value.copy_(a.to(torch.float32))
    p[f"{n}::lora_b"].value.copy_(b.to(torch.float32))


def lora_from_delta(delta: torch.Tensor, rank: int, alpha: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Best rank-``rank`` factors ``(A, B)`` with ``(alpha / rank) · A · B ≈ delta`` (truncated SVD)."""
    u, s, vh = torch.linalg.svd(delta.float(), full_matrices=False)
    r = min(rank, s.numel())
    root = s[:r].sqrt()
    scale = alpha / rank
    return (u[:, :r] * root) / scale ** 0.5, (root[:, None] * vh[:r]) / scale ** 0.5
