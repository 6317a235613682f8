"""Symmetric (peer-mapped) memory, signals and the fused compute+collective launchers.

``SymmetricHeap`` allocates buffers that every rank of a group can address directly: each
rank gets the list of peer device pointers and, when the fabric supports NVLS, a multicast
alias.  Allocation and handle exchange go through ``torch.distributed._symmetric_memory``
(plumbing); every kernel that touches the buffers is ours (``csrc/comm``).

``FusedTPContext`` implements the tensor-parallel interface of :class:`TPContext` with the
fused kernels: ``ag_gemm`` (all-gather → GEMM in one launch) and ``gemm_rs`` (GEMM →
reduce-scatter in one launch).  ``FusedDPStep`` is the data-parallel bucket step
(reduce-scatter + optimizer + all-gather in one launch).

With a world size of 1 the "peer" is the local GPU, so the same kernels run (and are tested)
on a single device.

Reference parity: there is no counterpart in the reference (its collectives are an
in-process thread rendezvous, crates/spiral-selfsup/src/trainer/distributed.rs:299-430, and
an RCCL all-gather of u64, crates/st-backend-hip/src/rccl_comm.rs:33).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops
from ..ops import native
from .tp import TPContext

MAX_RANKS = 8
launch_count = 0


class _PeerGroup(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("signals", ctypes.c_ulonglong * MAX_RANKS), ("signals_mc", ctypes.c_ulonglong)]


class _AgGemmArgs(ctypes.Structure):
    _fields_ = [("g", _PeerGroup), ("x_shard", ctypes.c_ulonglong),
                ("gather_peers", ctypes.c_ulonglong * MAX_RANKS), ("gather_mc", ctypes.c_ulonglong),
                ("B", ctypes.c_ulonglong), ("C", ctypes.c_ulonglong),
                ("bias", ctypes.c_ulonglong), ("aux_out", ctypes.c_ulonglong), ("aux_in", ctypes.c_ulonglong),
                ("ldb", ctypes.c_longlong), ("ldc", ctypes.c_longlong),
                ("ld_aux_out", ctypes.c_longlong), ("ld_aux_in", ctypes.c_longlong),
                ("T", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("b_mn", ctypes.c_int), ("act", ctypes.c_int), ("alpha", ctypes.c_float),
                ("sub_per_chunk", ctypes.c_int), ("comm_ctas", ctypes.c_int),
                ("slot_enter", ctypes.c_int), ("slot_arrive", ctypes.c_int), ("arrive_target", ctypes.c_uint),
                ("trace", ctypes.c_ulonglong), ("stages", ctypes.c_int), ("local_in_place", ctypes.c_int),
                ("max_ctas", ctypes.c_int)]


class _GemmRsArgs(ctypes.Structure):
    _fields_ = [("g", _PeerGroup), ("A", ctypes.c_ulonglong), ("B", ctypes.c_ulonglong),
                ("stage_peers", ctypes.c_ulonglong * MAX_RANKS), ("out", ctypes.c_ulonglong),
                ("residual", ctypes.c_ulonglong), ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong),
                ("T", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("b_mn", ctypes.c_int),
                ("alpha", ctypes.c_float), ("slot_enter", ctypes.c_int), ("slot_done", ctypes.c_int),
                ("done_target", ctypes.c_uint), ("stage_mc", ctypes.c_ulonglong),
                ("trace", ctypes.c_ulonglong), ("groups", ctypes.c_int), ("lag", ctypes.c_int), ("max_ctas", ctypes.c_int)]


class _DpStepArgs(ctypes.Structure):
    _fields_ = [("g", _PeerGroup),
                ("grad_local", ctypes.c_ulonglong), ("grad_mc", ctypes.c_ulonglong),
                ("grad_peers", ctypes.c_ulonglong * MAX_RANKS),
                ("w_local", ctypes.c_ulonglong), ("w_mc", ctypes.c_ulonglong),
                ("w_peers", ctypes.c_ulonglong * MAX_RANKS),
                ("master", ctypes.c_ulonglong), ("m", ctypes.c_ulonglong), ("v", ctypes.c_ulonglong),
                ("n", ctypes.c_longlong),
                ("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float), ("momentum", ctypes.c_float),
                ("step", ctypes.c_int), ("grad_scale", ctypes.c_float), ("scale_ptr", ctypes.c_ulonglong),
                ("kind", ctypes.c_int), ("slot_enter", ctypes.c_int), ("slot_exit", ctypes.c_int),
                ("cta_counter", ctypes.c_ulonglong), ("max_ctas", ctypes.c_int),
                ("phase", ctypes.c_int), ("gred", ctypes.c_ulonglong), ("sumsq_local", ctypes.c_ulonglong),
                ("norm_peers", ctypes.c_ulonglong * MAX_RANKS), ("max_norm", ctypes.c_float)]


def agree_on_status(group: Optional[dist.ProcessGroup], local_ok: bool,
                    device: Optional[torch.device] = None) -> bool:
    """Every rank says whether its own device error record is clean; the answer is True only when all are.

    A bounded wait that ran out on ONE rank (a peer that never signalled) must stop EVERY rank before anybody
    commits a partial result, and every rank has to make the same decision or their next collectives no longer
    pair up.  One MIN all-reduce of a status word does both (on the group's backend: CPU tensor for gloo,
    device tensor for NCCL).  Plays the role of the rendezvous' "a participant failed: everyone leaves with an
    error" rule (crates/spiral-selfsup/src/trainer/distributed.rs:407-423)."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(local_ok)
    on_cpu = dist.get_backend(group) == "gloo"
    dev = torch.device("cpu") if on_cpu else (device or torch.device("cuda", torch.cuda.current_device()))
    flag = torch.tensor([1 if local_ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(int(flag.item()) == 1)


class FusedContextBroken(native.NativeError):
    """A fused launch of this context gave up a bounded wait: its cumulative arrival counters no longer match
    what the peers will send, so every later launch would time out too.  Build a new context."""


class SymmetricBuffer:
    """A tensor plus the addresses under which every rank (and the switch) can reach it."""

    def __init__(self, tensor: torch.Tensor, peer_ptrs: list[int], mc_ptr: int):
        self.tensor = tensor
        self.peer_ptrs = peer_ptrs
        self.mc_ptr = mc_ptr

    def peers_array(self, byte_offset: int = 0):
        arr = (ctypes.c_ulonglong * MAX_RANKS)()
        for i, p in enumerate(self.peer_ptrs):
            arr[i] = p + byte_offset
        return arr

    def mc(self, byte_offset: int = 0) -> int:
        return self.mc_ptr + byte_offset if self.mc_ptr else 0


class SymmetricHeap:
    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, use_multicast: bool = True):
        self.group = group
        self.device = torch.device(device)
        if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
            self.world, self.rank = 1, 0
        else:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= MAX_RANKS
        self.use_multicast = use_multicast and os.environ.get("ST_DISABLE_MULTIMEM", "0") != "1"
        self._keep = []

    def empty(self, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmetricBuffer:
        if self.world == 1:
            t = torch.zeros(numel, dtype=dtype, device=self.device) if zero else \
                torch.empty(numel, dtype=dtype, device=self.device)
            return SymmetricBuffer(t, [t.data_ptr()], 0)
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        hdl = symm_mem.rendezvous(t, self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(hdl.multicast_ptr) if (self.use_multicast and getattr(hdl, "multicast_ptr", 0)) else 0
        self._keep.append(hdl)
        if zero:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        return SymmetricBuffer(t, ptrs, mc)


class PeerSignals:
    """Symmetric array of 32-bit signal words with a monotonically increasing epoch."""

    WORDS = 4096

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.buf = heap.empty(self.WORDS, torch.int32, zero=True)
        self.epoch = 0
        self._next = 0
        self.local_counter = torch.zeros(4, dtype=torch.int32, device=heap.device)

    def alloc(self, words: int) -> int:
        base = self._next
        self._next += (words + 7) // 8 * 8
        assert self._next <= self.WORDS, "signal area exhausted"
        return base

    def next_group(self) -> _PeerGroup:
        self.epoch += 1
        g = _PeerGroup()
        g.world, g.rank, g.epoch = self.heap.world, self.heap.rank, self.epoch & 0xFFFFFFFF
        g.signals = self.buf.peers_array()
        g.signals_mc = self.buf.mc()
        return g


class FusedTPContext(TPContext):
    """Tensor-parallel context whose column-/row-parallel linears run as fused kernels."""

    def __init__(self, group: Optional[dist.ProcessGroup], device=None, comm_ctas: Optional[int] = None,
                 sub_per_chunk: int = 4):
        super().__init__(group, mode="fused")
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = device
        self.heap = SymmetricHeap(group, device)
        self.signals = PeerSignals(self.heap)
        if comm_ctas is None:
            # one CTA sustains about 40 GB/s of peer writes through its shared-memory ring, and the
            # bytes a rank must send grow with (world-1)/world while its GEMM share shrinks
            env = os.environ.get("ST_TP_COMM_CTAS")
            comm_ctas = int(env) if env else {1: 4, 2: 12, 3: 16, 4: 16}.get(self.world, 24)
        self.comm_ctas = comm_ctas
        self.sub_per_chunk = sub_per_chunk
        self.slot_enter = self.signals.alloc(MAX_RANKS)
        # arrival counters of the all-gather: one area (world x 16 words) and one cumulative count per
        # sub-chunk granularity, because a launch only touches the words of its own granularity
        self.slot_arrive = {s: self.signals.alloc(MAX_RANKS * 16) for s in (1, 2, 4, 8, 16)}
        self._ag_arrivals = {s: 0 for s in (1, 2, 4, 8, 16)}
        self.ag_stages = int(os.environ.get("ST_TP_AG_STAGES", "0"))   # 0 = by world size
        self.rs_groups = int(os.environ.get("ST_TP_RS_GROUPS", "0"))   # 0 = chosen by the launcher, 1 = no interleave
        self.rs_lag = int(os.environ.get("ST_TP_RS_LAG", "0"))         # 0 = one group
        self.max_ctas = 0       # grid limit of the next fused launches (0 = one CTA per SM); the same on every rank
        self.trace: Optional[torch.Tensor] = None     # int64 [>= SMs, 4]: per-CTA phase time stamps (debug)
        self._done_slots: dict[int, tuple[int, int]] = {}   # row blocks → (slot, cumulative target)
        self._gather: dict = {}
        self._stage: dict = {}
        self.usable = True

    # -- failure handling ------------------------------------------------------------------
    def _require_usable(self) -> None:
        if not self.usable:
            raise FusedContextBroken("this fused tensor-parallel context reported a device-side timeout; "
                                     "rebuild it (FusedTPContext(group)) before launching again")

    def check(self, synchronize: bool = False) -> None:
        """Step-boundary health check, to be called by every rank at the same point.

        Reads this rank's error record (after an optional device synchronisation), agrees on the outcome with
        the other ranks and, if any rank saw a failure, marks the context unusable and raises
        :class:`native.DeviceWaitTimeout` on every rank, the ones that saw nothing included."""
        if synchronize:
            torch.cuda.synchronize(self.device)
        local: Optional[BaseException] = None
        try:
            native.raise_on_device_error()
        except native.NativeError as exc:
            local = exc
        if agree_on_status(self.group, local is None, self.device):
            return
        self.usable = False
        if local is not None:
            raise local
        raise native.DeviceWaitTimeout("a peer rank reported a device-side wait timeout in a fused kernel")

    # -- buffers ---------------------------------------------------------------------------
    def _gather_buffer(self, key, T: int, K: int) -> SymmetricBuffer:
        k = (key, T, K)
        buf = self._gather.get(k)
        if buf is None:
            buf = self.heap.empty(T * K, torch.bfloat16)
            self._gather[k] = buf
        return buf

    def _stage_buffer(self, T: int, N: int) -> SymmetricBuffer:
        k = (T, N)
        buf = self._stage.get(k)
        if buf is None:
            buf = self.heap.empty(T * N, torch.bfloat16)
            self._stage[k] = buf
        return buf

    def shard_slot(self, key, rows: int, K: int) -> torch.Tensor:
        """This rank's ``[rows, K]`` slot inside its own gather buffer for ``key``.  A producer that writes the
        shard there (instead of into a fresh tensor) saves the all-gather its local copy: ``ag_gemm`` recognises
        the address and pushes to the peers only."""
        gbuf = self._gather_buffer(key, rows * self.world, K)
        return gbuf.tensor.view(self.world, rows, K)[self.rank]

    # -- fused linears ---------------------------------------------------------------------
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, key="shared",
                act=None, aux_out=None, aux_in=None, bias=None, alpha: float = 1.0):
        """``y = epilogue(all_gather_rows(x_shard) @ op(w))``; returns ``(y, x_full)`` where
        ``x_full`` is the gathered activation (a view of the symmetric buffer keyed by ``key``)."""
        global launch_count
        self._require_usable()
        native.require_cuda("ag_gemm", x_shard, w, aux_out, aux_in, bias)
        rows, K = x_shard.shape
        T = rows * self.world
        N = w.shape[1] if b_mn else w.shape[0]
        x_shard = x_shard.contiguous()
        gbuf = self._gather_buffer(key, T, K)
        in_place = x_shard.data_ptr() == gbuf.tensor.data_ptr() + self.rank * rows * K * 2
        y = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device)
        sub = self.sub_per_chunk
        while sub > 1 and rows % (sub * 128) != 0:
            sub //= 2
        assert sub in self.slot_arrive, "sub_per_chunk must be a power of two up to 16"
        a = _AgGemmArgs()
        a.g = self.signals.next_group()
        a.x_shard = x_shard.data_ptr()
        a.gather_peers = gbuf.peers_array()
        a.gather_mc = 0
        a.B, a.C = w.data_ptr(), y.data_ptr()
        a.bias = 0 if bias is None else bias.data_ptr()
        a.aux_out = 0 if aux_out is None else aux_out.data_ptr()
        a.aux_in = 0 if aux_in is None else aux_in.data_ptr()
        a.ldb, a.ldc = w.stride(0), y.stride(0)
        a.ld_aux_out = 0 if aux_out is None else aux_out.stride(0)
        a.ld_aux_in = 0 if aux_in is None else aux_in.stride(0)
        a.T, a.N, a.K = T, N, K
        a.b_mn = int(b_mn)
        a.act = gemm_ops._ACT_NAMES[act]
        a.alpha = alpha
        a.sub_per_chunk, a.comm_ctas = sub, self.comm_ctas
        a.slot_enter = self.slot_enter
        a.trace = 0 if self.trace is None else self.trace.data_ptr()
        a.stages = self.ag_stages
        a.local_in_place = int(in_place)
        a.max_ctas = int(self.max_ctas)
        self._ag_arrivals[sub] += native.lib().st_ag_arrivals_for(ctypes.c_int(a.max_ctas))
        a.slot_arrive, a.arrive_target = self.slot_arrive[sub], self._ag_arrivals[sub] & 0xFFFFFFFF
        native.check(native.lib().st_ag_gemm(ctypes.byref(a), native.stream_ptr(x_shard.device)), "st_ag_gemm")
        launch_count += 1
        self.bytes_gathered += T * K * 2
        return y, gbuf.tensor.view(T, K)

    def gemm_rs(self, a_full: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False,
                residual: Optional[torch.Tensor] = None, alpha: float = 1.0, _withhold: int = 0) -> torch.Tensor:
        """``reduce_scatter_rows(a_full @ op(w)) (+ residual)`` → ``[T/world, N]``.

        ``_withhold`` (tests of the failure path only) raises this one launch's arrival target above what the
        peers will deliver, so that the bounded wait of the local tiles runs out; the context's own counters are
        not changed by it."""
        global launch_count
        self._require_usable()
        native.require_cuda("gemm_rs", a_full, w, residual)
        T, K = a_full.shape
        N = w.shape[1] if b_mn else w.shape[0]
        rows = T // self.world
        blocks = rows // 128
        sbuf = self._stage_buffer(T, N)
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=a_full.device)
        lib = native.lib()
        slot, cum = self._done_slots.get(blocks, (None, 0))
        if slot is None:
            slot = self.signals.alloc(blocks)
        cum += lib.st_gemm_rs_arrivals_per_launch(ctypes.c_int(self.world), ctypes.c_int(N))
        self._done_slots[blocks] = (slot, cum)
        r = _GemmRsArgs()
        r.g = self.signals.next_group()
        r.A, r.B = a_full.data_ptr(), w.data_ptr()
        r.stage_peers = sbuf.peers_array()
        r.out = out.data_ptr()
        r.residual = 0 if residual is None else residual.data_ptr()
        r.lda, r.ldb = a_full.stride(0), w.stride(0)
        r.T, r.N, r.K = T, N, K
        r.b_mn = int(b_mn)
        r.alpha = alpha
        r.slot_enter, r.slot_done = self.slot_enter, slot
        r.done_target = (cum + _withhold) & 0xFFFFFFFF
        r.stage_mc = 0
        r.groups, r.lag = self.rs_groups, self.rs_lag
        r.max_ctas = int(self.max_ctas)
        r.trace = 0 if self.trace is None else self.trace.data_ptr()
        native.check(lib.st_gemm_rs(ctypes.byref(r), native.stream_ptr(a_full.device)), "st_gemm_rs")
        launch_count += 1
        self.bytes_scattered += T * N * 2
        return out


class FusedDPStep:
    """Data-parallel optimizer step over symmetric flat buffers (one launch per bucket)."""

    def __init__(self, heap: SymmetricHeap, signals: PeerSignals, grad: SymmetricBuffer, weight: SymmetricBuffer,
                 kind: str = "adamw", bucket_elems: int = 1 << 24, max_ctas: int = 0, max_grad_norm: float = 0.0):
        """``max_grad_norm > 0`` selects the two-phase form: :meth:`reduce_bucket` for every bucket (these may
        overlap the backward pass), then :meth:`update_bucket` for every bucket once all reductions are queued -
        the update clips by the global norm of the averaged gradient, which the kernels exchange themselves."""
        self.heap, self.signals, self.grad, self.weight = heap, signals, grad, weight
        self.kind = kind
        self.max_grad_norm = float(max_grad_norm)
        n = grad.tensor.numel()
        W = heap.world
        assert n % (8 * W) == 0, "flat length must be a multiple of 8*world"
        assert weight.tensor.numel() == n
        self.n = n
        self.bucket = max(8 * W, bucket_elems // (8 * W) * (8 * W))
        self.max_ctas = max_ctas
        dev = heap.device
        # optimizer state exists only for the shard this rank owns, bucket by bucket
        self.buckets = []
        off = 0
        while off < n:
            ln = min(self.bucket, n - off)
            shard = ln // W
            master = weight.tensor[off + shard * heap.rank: off + shard * (heap.rank + 1)].float().clone()
            m = torch.zeros(shard, dtype=torch.float32, device=dev)
            v = torch.zeros(shard, dtype=torch.float32, device=dev) if kind == "adamw" else None
            self.buckets.append((off, ln, master, m, v))
            off += ln
        self.slot_enter = signals.alloc(MAX_RANKS)
        self.slot_exit = signals.alloc(MAX_RANKS)
        self.step_count = 0
        self.gred, self.sumsq, self.norm_buf = None, None, None
        if self.max_grad_norm > 0:
            self.gred = [torch.empty(ln // W, dtype=torch.float32, device=dev) for (_, ln, *_r) in self.buckets]
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self.norm_buf = heap.empty(MAX_RANKS, torch.float32, zero=True)

    def begin_step(self) -> None:
        self.step_count += 1
        if self.sumsq is not None:
            self.sumsq.zero_()          # stream-ordered before this step's first reduction

    def reduce_bucket(self, index: int, **kw) -> None:
        self.step_bucket(index, _phase=1, **kw)

    def update_bucket(self, index: int, **kw) -> None:
        self.step_bucket(index, _phase=2, **kw)

    def grad_norm(self) -> torch.Tensor:
        """Global norm of the averaged gradient of the last two-phase step (device scalar)."""
        return self.norm_buf.tensor[: self.heap.world].sum().sqrt()

    def step_bucket(self, index: int, *, lr: float, beta1: float = 0.9, beta2: float = 0.95, eps: float = 1e-8,
                    weight_decay: float = 0.0, momentum: float = 0.9, grad_scale: float = 1.0,
                    scale_tensor: Optional[torch.Tensor] = None, _phase: int = 0) -> None:
        global launch_count
        if _phase and self.gred is None:
            raise ValueError("the two-phase step needs max_grad_norm > 0 at construction")
        off, ln, master, m, v = self.buckets[index]
        a = _DpStepArgs()
        a.g = self.signals.next_group()
        a.grad_local = self.grad.tensor.data_ptr() + off * 4
        a.grad_mc = self.grad.mc(off * 4)
        a.grad_peers = self.grad.peers_array(off * 4)
        a.w_local = self.weight.tensor.data_ptr() + off * 2
        a.w_mc = self.weight.mc(off * 2)
        a.w_peers = self.weight.peers_array(off * 2)
        a.master, a.m = master.data_ptr(), m.data_ptr()
        a.v = 0 if v is None else v.data_ptr()
        a.n = ln
        a.lr, a.beta1, a.beta2, a.eps = lr, beta1, beta2, eps
        a.weight_decay, a.momentum = weight_decay, momentum
        a.step = max(1, self.step_count)
        a.grad_scale = grad_scale / self.heap.world
        a.scale_ptr = 0 if scale_tensor is None else scale_tensor.data_ptr()
        a.kind = 0 if self.kind == "adamw" else 1
        a.slot_enter, a.slot_exit = self.slot_enter, self.slot_exit
        a.cta_counter = self.signals.local_counter.data_ptr()
        a.max_ctas = self.max_ctas
        a.phase = _phase
        if _phase:
            a.gred, a.sumsq_local = self.gred[index].data_ptr(), self.sumsq.data_ptr()
            a.norm_peers = self.norm_buf.peers_array()
            a.max_norm = self.max_grad_norm
        native.check(native.lib().st_dp_step(ctypes.byref(a), native.stream_ptr(self.heap.device)), "st_dp_step")
        launch_count += 1

    def step(self, **kw) -> None:
        self.begin_step()
        if self.max_grad_norm > 0:
            for i in range(len(self.buckets)):
                self.reduce_bucket(i, **kw)
            for i in range(len(self.buckets)):
                self.update_bucket(i, **kw)
            return
        for i in range(len(self.buckets)):
            self.step_bucket(i, **kw)
