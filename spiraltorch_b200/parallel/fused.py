"""Factory for the tensor-parallel context used by the models.

``make_context(group, "nccl")`` returns the NCCL-collective context (the baseline);
``make_context(group, "fused")`` returns the peer-memory context whose all-gather→GEMM and
GEMM→reduce-scatter run inside one kernel launch (``spiraltorch_b200.parallel.symm``).
"""
from __future__ import annotations

from .tp import TPContext


def make_context(group, mode: str = "nccl") -> TPContext:
    if mode == "fused":
        from .symm import FusedTPContext
        return FusedTPContext(group)
    return TPContext(group, mode="nccl")
