"""Row-wise rank selection (top-k / bottom-k / mid-k), row compaction and distributed top-k.

CUDA tensors run ``csrc/rank/rank.cu``; CPU tensors run a PyTorch restatement of the
reference's CPU mirror (crates/st-core/src/backend/rankk_software.rs:38-110): non-finite
entries are ignored, ties go to the lower column index, unused slots are ``NaN`` / ``-1``.

``plan_rank`` returns a small plan object in the spirit of ``plan_rank`` /
``RankPlan`` (crates/st-core/src/ops/rank_entry.rs): on sm_100a the choices are fixed (one CTA
per row, shared-memory bitonic network, block arg-max for k = 1), so the plan only records them.

``distributed_topk`` is the three-stage scheme of crates/st-core/src/distributed/topk3_stage.rs:
local select → all-gather of the ``(value, index)`` candidates → exact merge
(``merge_topk_shards_f32``, crates/st-core/src/distributed/topk_dist.rs:380).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import native

launch_count = 0
MODES = {"topk": 0, "top": 0, "bottomk": 1, "bottom": 1, "midk": 2, "mid": 2}


@dataclass
class RankPlan:
    kind: str
    rows: int
    cols: int
    k: int
    backend: str
    kernel: str
    workgroup: int
    lanes: int = 32
    shared_bytes: int = 0
    accelerator_fallback: str = "allow"

    def describe(self) -> dict:
        return dict(self.__dict__)


def plan_rank(kind: str, rows: int, cols: int, k: int, backend: str = "auto") -> RankPlan:
    if kind not in MODES:
        raise ValueError(f"unknown rank kind '{kind}'")
    if k > cols:
        raise ValueError(f"k={k} exceeds cols={cols}")
    if backend == "auto":
        backend = "cuda" if torch.cuda.is_available() else "cpu"
    padded = 2
    while padded < cols:
        padded <<= 1
    if backend == "cuda" and cols > 8192 and MODES[kind] != 2:
        chunks = -(-cols // 8192)
        return RankPlan(kind, rows, cols, k, "cuda", f"two_stage_smem_bitonic(chunks={chunks})", 1024,
                        shared_bytes=8192 * 8)
    if backend == "cuda" and cols <= 8192:
        if k == 1 and MODES[kind] != 2:
            return RankPlan(kind, rows, cols, k, "cuda", "block_argmax", 256 if cols >= 1024 else 64)
        return RankPlan(kind, rows, cols, k, "cuda", "smem_bitonic", max(32, min(1024, padded // 2)),
                        shared_bytes=padded * 8)
    return RankPlan(kind, rows, cols, k, "cpu", "stable_sort", 1)


def rank_select_reference(x: torch.Tensor, k: int, mode: int):
    rows, cols = x.shape
    xf = x.float()
    finite = torch.isfinite(xf)
    key = torch.where(finite, -xf if mode == 0 else xf, torch.full_like(xf, float("inf")))
    order = torch.sort(key, dim=1, stable=True).indices
    n_fin = finite.sum(1)
    out_v = torch.full((rows, k), float("nan"), dtype=torch.float32, device=x.device)
    out_i = torch.full((rows, k), -1, dtype=torch.int32, device=x.device)
    slots = torch.arange(k, device=x.device)[None, :]
    take = torch.minimum(n_fin, torch.tensor(k, device=x.device))[:, None]
    start = ((n_fin[:, None] - take) // 2) if mode == 2 else torch.zeros_like(take)
    pos = (start + slots).clamp(max=max(cols - 1, 0))
    idx = torch.gather(order, 1, pos) if cols > 0 else torch.zeros((rows, k), dtype=torch.long, device=x.device)
    valid = slots < take
    out_v[valid] = torch.gather(xf, 1, idx)[valid] if cols > 0 else out_v[valid]
    out_i[valid] = idx[valid].to(torch.int32)
    return out_v, out_i


def rank_select(x: torch.Tensor, k: int, kind: str = "topk", choice=None):
    """Returns ``(values [rows,k] fp32, indices [rows,k] int32)``.  ``choice`` (a ``unison.RankChoice``) may ask for the
    two-stage path with its sweep tile as chunk width on rows that one CTA could also sort directly; top / bottom only,
    and only when a chunk pass actually shrinks the row."""
    global launch_count
    mode = MODES[kind]
    rows, cols = x.shape
    if choice is None and mode != 2 and k > 1 and 1024 <= cols <= MAX_KERNEL_COLS and native.use_native(x):
        choice = _tuned_choice(rows, cols, k, kind)
    if choice is not None and choice.use_2ce and mode != 2 and 0 < k and native.use_native(x) and cols <= MAX_KERNEL_COLS \
            and 0 < choice.tile < cols and -(-cols // choice.tile) * min(k, choice.tile) < cols:
        return _rank_select_two_stage(x, k, kind, chunk=choice.tile)
    if k < 0 or k > max(cols, 0) and cols > 0 and k > cols:
        raise ValueError(f"k={k} exceeds cols={cols}")
    if not native.use_native(x):
        return rank_select_reference(x, k, mode)
    if cols > MAX_KERNEL_COLS:
        if mode == 2 or k == 0:
            return rank_select_reference(x, k, mode)     # mid-k needs the global order statistics
        return _rank_select_two_stage(x, k, kind)
    xf = x.float().contiguous()
    out_v = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    out_i = torch.empty((rows, k), dtype=torch.int32, device=x.device)
    st = native.lib().st_rank_select(native.ptr(xf), native.ptr(out_v), native.ptr(out_i), ctypes.c_int(rows),
                                     ctypes.c_int(cols), ctypes.c_int(k), ctypes.c_int(mode),
                                     native.stream_ptr(x.device))
    native.check(st, "st_rank_select")
    launch_count += 1
    return out_v, out_i


_choice_cache: dict = {}


def _tuned_choice(rows: int, cols: int, k: int, kind: str):
    """The three-voice chooser's pick for this shape (cached per power-of-two row bucket): on rows of 1024 to 8192
    columns the tuned table often prefers per-chunk candidates + merge over one full-width sort."""
    key = (1 << max(rows - 1, 0).bit_length(), cols, k, MODES[kind])
    hit = _choice_cache.get(key)
    if hit is None:
        from .. import unison
        from ..device_caps import DeviceCaps
        hit = unison.choose_unified_rank(rows, cols, k, DeviceCaps.cuda(), "topk" if MODES[kind] == 0 else "bottomk").choice
        if len(_choice_cache) > 4096:
            _choice_cache.clear()
        _choice_cache[key] = hit
    return hit


MAX_KERNEL_COLS = 8192      # one CTA sorts a row of at most this many (value, index) keys in shared memory


def _rank_select_two_stage(x: torch.Tensor, k: int, kind: str, chunk: int = 0):
    """Rows wider than one CTA's shared-memory sort: select per column chunk, then select among the candidates
    (the reference's two-stage path: rankk_exact_2ce.wgsl, crates/st-core/src/distributed/topk3_stage.rs:56).
    Exact, including the tie rule: candidates keep chunk order and, inside a chunk, the kernel's own order, so
    equal values still resolve to the lower column."""
    rows, cols = x.shape
    n_chunks = -(-cols // (min(chunk, MAX_KERNEL_COLS) if chunk > 0 else MAX_KERNEL_COLS))
    width = -(-cols // n_chunks)
    pad = n_chunks * width - cols
    xf = x.float()
    if pad:
        xf = torch.cat([xf, torch.full((rows, pad), float("nan"), dtype=torch.float32, device=x.device)], dim=1)
    kc = min(k, width)
    if n_chunks * kc >= cols:      # k is so large that a chunk pass would not shrink the row: sort it once
        return rank_select_reference(x, k, MODES[kind])
    cv, ci = rank_select(xf.reshape(rows * n_chunks, width), kc, kind)            # stage 1: per chunk
    cv = cv.reshape(rows, n_chunks * kc)
    offs = (torch.arange(n_chunks, device=x.device, dtype=torch.int32) * width).repeat_interleave(kc)[None, :]
    ci = ci.reshape(rows, n_chunks * kc)
    gidx = torch.where(ci >= 0, ci + offs, ci)
    v, pos = rank_select(cv, k, kind)                                              # stage 2 (recurses if still too wide)
    out_i = torch.gather(gidx, 1, pos.clamp(min=0).long())
    out_i = torch.where(pos >= 0, out_i, torch.full_like(out_i, -1))
    return v, out_i.to(torch.int32)


def topk(x, k):
    return rank_select(x, k, "topk")


def bottomk(x, k):
    return rank_select(x, k, "bottomk")


def midk(x, k):
    return rank_select(x, k, "midk")


def compact_rows(x: torch.Tensor, low: float, high: float):
    """Per row keep ``low <= v <= high`` in order: ``(values, indices, counts)`` with zero padding."""
    global launch_count
    import math
    if not (math.isfinite(low) and math.isfinite(high) and low <= high):
        raise ValueError(f"compaction bounds must be finite and ordered, got [{low}, {high}]")
    rows, cols = x.shape
    if not native.use_native(x):
        xf = x.float()
        keep = (xf >= low) & (xf <= high)
        counts = keep.sum(1).to(torch.int32)
        order = torch.sort((~keep).to(torch.int8), dim=1, stable=True).indices
        vals = torch.gather(xf, 1, order)
        slot = torch.arange(cols, device=x.device)[None, :] < counts[:, None]
        zero = torch.zeros_like(vals)
        return torch.where(slot, vals, zero), torch.where(slot, order, torch.zeros_like(order)).to(torch.int32), counts
    xf = x.float().contiguous()
    out_v = torch.empty_like(xf)
    out_i = torch.empty((rows, cols), dtype=torch.int32, device=x.device)
    counts = torch.empty(rows, dtype=torch.int32, device=x.device)
    st = native.lib().st_compact_rows(native.ptr(xf), native.ptr(out_v), native.ptr(out_i), native.ptr(counts),
                                      ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_float(low),
                                      ctypes.c_float(high), native.stream_ptr(x.device))
    native.check(st, "st_compact_rows")
    launch_count += 1
    return out_v, out_i, counts


def merge_topk_shards(values: torch.Tensor, indices: torch.Tensor, k: int, kind: str = "topk"):
    """Exact merge of candidate lists ``[rows, shards*k']`` carrying global column indices.
    Ties are resolved by the lower *global* index, as in the single-device selection."""
    rows = values.shape[0]
    v = values.float()
    key_idx = torch.where(indices >= 0, indices, torch.full_like(indices, 2 ** 31 - 1)).long()
    # order candidates by global index first so that the stable value sort breaks ties by index
    by_idx = torch.sort(key_idx, dim=1, stable=True).indices
    v = torch.gather(v, 1, by_idx)
    gi = torch.gather(indices, 1, by_idx)
    sel_v, sel_p = rank_select(v, k, kind)
    out_i = torch.where(sel_p >= 0, torch.gather(gi, 1, sel_p.clamp(min=0).long()), torch.full_like(sel_p, -1))
    return sel_v, out_i.to(torch.int32)


def distributed_topk(x_shard: torch.Tensor, k: int, *, group=None, col_offset: Optional[int] = None,
                     kind: str = "topk", heap=None):
    """Top-k over rows whose columns are sharded across ranks.  Every rank returns the same
    ``(values, global indices)``.  With a :class:`SymmetricHeap` the candidates are read straight
    from the peers' memory over NVLink; otherwise they are all-gathered by ``torch.distributed``."""
    global launch_count
    import torch.distributed as dist
    rows, cols = x_shard.shape
    world = dist.get_world_size(group) if (dist.is_initialized() and group is not False) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    if col_offset is None:
        col_offset = rank * cols
    kk = min(k, cols)
    lv, li = rank_select(x_shard, kk, kind)
    li = torch.where(li >= 0, li + col_offset, li)
    if world == 1:
        return merge_topk_shards(lv, li, k, kind)
    if heap is not None and x_shard.is_cuda:
        cv = heap.empty(rows * kk, torch.float32)
        ci = heap.empty(rows * kk, torch.int32)
        cv.tensor.copy_(lv.reshape(-1))
        ci.tensor.copy_(li.reshape(-1))
        torch.cuda.synchronize(x_shard.device)
        dist.barrier(group=group)                       # candidates are published
        pv = torch.tensor(cv.peer_ptrs, dtype=torch.int64, device=x_shard.device)
        pi = torch.tensor(ci.peer_ptrs, dtype=torch.int64, device=x_shard.device)
        gv = torch.empty((rows, world * kk), dtype=torch.float32, device=x_shard.device)
        gi = torch.empty((rows, world * kk), dtype=torch.int32, device=x_shard.device)
        st = native.lib().st_gather_candidates(native.ptr(pv), native.ptr(pi), native.ptr(gv), native.ptr(gi),
                                               ctypes.c_int(world), ctypes.c_int(rows), ctypes.c_int(kk),
                                               native.stream_ptr(x_shard.device))
        native.check(st, "st_gather_candidates")
        launch_count += 1
        torch.cuda.synchronize(x_shard.device)
        dist.barrier(group=group)                       # peers may now reuse their buffers
    else:
        gv_list = [torch.empty_like(lv) for _ in range(world)]
        gi_list = [torch.empty_like(li) for _ in range(world)]
        dist.all_gather(gv_list, lv.contiguous(), group=group)
        dist.all_gather(gi_list, li.contiguous(), group=group)
        gv, gi = torch.cat(gv_list, 1), torch.cat(gi_list, 1)
    return merge_topk_shards(gv, gi, k, kind)
