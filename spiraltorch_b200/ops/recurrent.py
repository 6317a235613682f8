"""Recurrent-cell kernels: LSTM gate step (forward + one BPTT step), wave gate, last-step gather.

CUDA fp32 tensors run ``csrc/recurrent/recurrent.cu``; everything else runs the PyTorch statement
of the same arithmetic (the oracle).  Reference: ``lstm_forward_gate_step``, ``wave_gate_project`` /
``wave_gate_backward``, ``sequence_last_step_gather`` / ``scatter`` in
crates/st-tensor/src/wgpu_shaders/tensor_utils.wgsl and ``lstm_backward_scan.wgsl``.
"""
from __future__ import annotations

import ctypes

import torch

from . import native

launch_count = 0


def _native(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.float32 for t in ts) and native.use_native(ts[0])


def lstm_gate_reference(z, c_prev):
    H = c_prev.shape[1]
    i, f, g, o = torch.sigmoid(z[:, :H]), torch.sigmoid(z[:, H:2 * H]), torch.tanh(z[:, 2 * H:3 * H]), torch.sigmoid(z[:, 3 * H:])
    c = f * c_prev + i * g
    return o * torch.tanh(c), c, torch.cat([i, f, g, o], 1)


def lstm_gate_forward(z: torch.Tensor, c_prev: torch.Tensor):
    """``z`` [B, 4H] pre-activations (i|f|g|o), ``c_prev`` [B, H] → ``(h, c, activated gates)``."""
    global launch_count
    B, H = c_prev.shape
    if z.shape != (B, 4 * H):
        raise ValueError(f"lstm gate: z must be [{B}, {4 * H}], got {tuple(z.shape)}")
    if not _native(z, c_prev):
        return lstm_gate_reference(z.float(), c_prev.float())
    z, c_prev = z.contiguous(), c_prev.contiguous()
    h, c, act = torch.empty_like(c_prev), torch.empty_like(c_prev), torch.empty_like(z)
    native.check(native.lib().st_lstm_gate_fwd(native.ptr(z), native.ptr(c_prev), native.ptr(c), native.ptr(h), native.ptr(act),
                                               ctypes.c_int(B), ctypes.c_int(H), native.stream_ptr(z.device)), "st_lstm_gate_fwd")
    launch_count += 1
    return h, c, act


def lstm_gate_backward(act, c_prev, c, dh, dc_next=None):
    """→ ``(dz [B, 4H], dc_prev [B, H])``."""
    global launch_count
    B, H = c_prev.shape
    if not _native(act, c_prev, c, dh):
        i, f, g, o = act[:, :H], act[:, H:2 * H], act[:, 2 * H:3 * H], act[:, 3 * H:]
        tc = torch.tanh(c)
        dct = dh * o * (1 - tc * tc) + (0 if dc_next is None else dc_next)
        dz = torch.cat([dct * g * i * (1 - i), dct * c_prev * f * (1 - f), dct * i * (1 - g * g), dh * tc * o * (1 - o)], 1)
        return dz, dct * f
    dz, dc_prev = torch.empty_like(act), torch.empty_like(c_prev)
    dcn = None if dc_next is None else dc_next.contiguous()
    native.check(native.lib().st_lstm_gate_bwd(native.ptr(act.contiguous()), native.ptr(c_prev.contiguous()),
                                               native.ptr(c.contiguous()), native.ptr(dh.contiguous()),
                                               native.ptr(dcn), native.ptr(dz),
                                               native.ptr(dc_prev), ctypes.c_int(B), ctypes.c_int(H),
                                               native.stream_ptr(act.device)), "st_lstm_gate_bwd")
    launch_count += 1
    return dz, dc_prev


class _LstmGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, c_prev):
        h, c, act = lstm_gate_forward(z, c_prev)
        ctx.save_for_backward(act, c_prev, c)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        act, c_prev, c = ctx.saved_tensors
        dh = torch.zeros_like(c) if dh is None else dh
        return lstm_gate_backward(act, c_prev, c, dh.contiguous(), dc)


def lstm_gate(z: torch.Tensor, c_prev: torch.Tensor):
    """Differentiable LSTM gate step: ``(h, c)``."""
    return _LstmGateFn.apply(z, c_prev)


def wave_gate_forward(z: torch.Tensor) -> torch.Tensor:
    global launch_count
    B, H2 = z.shape
    H = H2 // 2
    if not _native(z):
        return torch.tanh(z[:, :H]) * torch.sigmoid(z[:, H:])
    z = z.contiguous()
    y = torch.empty((B, H), dtype=torch.float32, device=z.device)
    native.check(native.lib().st_wave_gate_fwd(native.ptr(z), native.ptr(y), ctypes.c_int(B), ctypes.c_int(H),
                                               native.stream_ptr(z.device)), "st_wave_gate_fwd")
    launch_count += 1
    return y


def wave_gate_backward(z: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    global launch_count
    B, H2 = z.shape
    H = H2 // 2
    if not _native(z, dy):
        t, s = torch.tanh(z[:, :H]), torch.sigmoid(z[:, H:])
        return torch.cat([dy * s * (1 - t * t), dy * t * s * (1 - s)], 1)
    dz = torch.empty_like(z)
    native.check(native.lib().st_wave_gate_bwd(native.ptr(z.contiguous()), native.ptr(dy.contiguous()), native.ptr(dz),
                                               ctypes.c_int(B), ctypes.c_int(H), native.stream_ptr(z.device)), "st_wave_gate_bwd")
    launch_count += 1
    return dz


class _WaveGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z):
        ctx.save_for_backward(z)
        return wave_gate_forward(z)

    @staticmethod
    def backward(ctx, dy):
        (z,) = ctx.saved_tensors
        return wave_gate_backward(z, dy.contiguous())


def wave_gate(z: torch.Tensor) -> torch.Tensor:
    """``tanh(z[:, :H]) * sigmoid(z[:, H:])`` (differentiable)."""
    return _WaveGateFn.apply(z)


def sequence_last_step(x: torch.Tensor, steps: int, dim: int) -> torch.Tensor:
    """``x`` [B, steps*dim] → the last step ``[B, dim]``."""
    global launch_count
    B = x.shape[0]
    if not _native(x):
        return x.reshape(B, steps, dim)[:, -1].contiguous()
    y = torch.empty((B, dim), dtype=torch.float32, device=x.device)
    native.check(native.lib().st_sequence_last_step(native.ptr(x.contiguous()), native.ptr(y), ctypes.c_int(B),
                                                    ctypes.c_int(steps), ctypes.c_int(dim), ctypes.c_int(0),
                                                    native.stream_ptr(x.device)), "st_sequence_last_step")
    launch_count += 1
    return y


# ---- whole-sequence scans (csrc/recurrent/scan.cu) -----------------------------------------------------------
CELLS = {"tanh": 0, "wave": 1, "lstm": 2}
_GATES = {"tanh": 1, "wave": 2, "lstm": 4}


class _ScanArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("zx", "w_hh", "h_all", "hin_all", "z_all", "c_all", "dh_last", "dz_all",
                                               "dhin_all")] + \
               [(n, ctypes.c_int) for n in ("B", "T", "H", "cell", "dilation", "backward")]


def scan_supported(hidden: int, cell: str) -> bool:
    return bool(native.lib().st_rnn_scan_supported(ctypes.c_int(hidden), ctypes.c_int(CELLS[cell])))


def rnn_sequence_reference(x, w_ih, w_hh, bias, cell: str, dilation: int = 1):
    """Step-by-step PyTorch statement: ``x`` [B, T, in] → last hidden state [B, H]."""
    B, T, _ = x.shape
    H = w_hh.shape[0]
    h = torch.zeros(B, H, dtype=x.dtype, device=x.device)
    c = torch.zeros_like(h)
    hs = []
    for t in range(T):
        hin = h
        if cell == "wave" and t >= dilation:
            hin = h + hs[t - dilation]
        z = x[:, t] @ w_ih + hin @ w_hh + bias
        if cell == "tanh":
            h = torch.tanh(z)
        elif cell == "wave":
            h = torch.tanh(z[:, :H]) * torch.sigmoid(z[:, H:])
        else:
            i, f, g, o = torch.sigmoid(z[:, :H]), torch.sigmoid(z[:, H:2 * H]), torch.tanh(z[:, 2 * H:3 * H]), \
                torch.sigmoid(z[:, 3 * H:])
            c = f * c + i * g
            h = o * torch.tanh(c)
        hs.append(h)
    return h


class _RnnSequenceFn(torch.autograd.Function):
    """Input projection for all steps as one GEMM, the recurrence over all steps as one kernel launch; the backward
    is one BPTT launch followed by three GEMMs (dW_hh, dW_ih, dx) and a column sum (db)."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, bias, cell, dilation):
        global launch_count
        from . import gemm as G
        B, T, I = x.shape
        H = w_hh.shape[0]
        GH = _GATES[cell] * H
        dev = x.device
        xb = x.detach().reshape(B * T, I).to(torch.bfloat16).contiguous()
        wib = G.cached_bf16(w_ih)
        zx = G.gemm(xb, wib, b_mn=True, bias=G.cached_bf16(bias).reshape(-1), out_dtype=torch.float32)   # [B*T, GH]
        whh = w_hh.detach().float().contiguous()
        h_all = torch.empty((B, T, H), dtype=torch.float32, device=dev)
        hin_all = torch.empty_like(h_all)
        z_all = torch.empty((B, T, GH), dtype=torch.float32, device=dev)
        c_all = torch.empty_like(h_all) if cell == "lstm" else None
        a = _ScanArgs()
        a.zx, a.w_hh, a.h_all, a.hin_all, a.z_all = zx.data_ptr(), whh.data_ptr(), h_all.data_ptr(), \
            hin_all.data_ptr(), z_all.data_ptr()
        a.c_all = None if c_all is None else c_all.data_ptr()
        a.B, a.T, a.H, a.cell, a.dilation, a.backward = B, T, H, CELLS[cell], int(dilation), 0
        native.check(native.lib().st_rnn_scan(ctypes.byref(a), native.stream_ptr(dev)), "st_rnn_scan")
        launch_count += 1
        ctx.save_for_backward(xb, wib, whh, h_all, hin_all, z_all, c_all)
        ctx.meta = (B, T, I, H, GH, cell, int(dilation))
        return h_all[:, -1].clone()

    @staticmethod
    def backward(ctx, dh_last):
        global launch_count
        from . import elementwise as E
        from . import gemm as G
        xb, wib, whh, h_all, hin_all, z_all, c_all = ctx.saved_tensors
        B, T, I, H, GH, cell, dilation = ctx.meta
        dev = xb.device
        dz_all = torch.empty((B, T, GH), dtype=torch.float32, device=dev)
        dhin_all = torch.empty((B, T, H), dtype=torch.float32, device=dev)
        dh = dh_last.detach().float().contiguous()
        a = _ScanArgs()
        a.zx, a.w_hh, a.h_all, a.hin_all, a.z_all = z_all.data_ptr(), whh.data_ptr(), h_all.data_ptr(), \
            hin_all.data_ptr(), z_all.data_ptr()
        a.c_all = None if c_all is None else c_all.data_ptr()
        a.dh_last, a.dz_all, a.dhin_all = dh.data_ptr(), dz_all.data_ptr(), dhin_all.data_ptr()
        a.B, a.T, a.H, a.cell, a.dilation, a.backward = B, T, H, CELLS[cell], dilation, 1
        native.check(native.lib().st_rnn_scan(ctypes.byref(a), native.stream_ptr(dev)), "st_rnn_scan")
        launch_count += 1
        dzb = dz_all.reshape(B * T, GH).to(torch.bfloat16)
        dx = dw_ih = dw_hh = db = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dzb, wib, out_dtype=torch.float32).reshape(B, T, I)                  # dz · W_ihᵀ
        if ctx.needs_input_grad[1]:
            dw_ih = G.gemm(xb, dzb, a_mn=True, b_mn=True, out_dtype=torch.float32)           # xᵀ · dz
        if ctx.needs_input_grad[2]:
            hinb = hin_all.reshape(B * T, H).to(torch.bfloat16)
            dw_hh = G.gemm(hinb, dzb, a_mn=True, b_mn=True, out_dtype=torch.float32)         # hinᵀ · dz
        if ctx.needs_input_grad[3]:
            db = E.colsum(dzb).reshape(1, GH)
        return dx, dw_ih, dw_hh, db, None, None


def rnn_sequence(x: torch.Tensor, w_ih: torch.Tensor, w_hh: torch.Tensor, bias: torch.Tensor, cell: str,
                 dilation: int = 1) -> torch.Tensor:
    """Last hidden state of an Elman (``"tanh"``), wave-gated (``"wave"``, dilated skip) or LSTM (``"lstm"``) layer
    over ``x`` [B, T, in]; ``w_ih`` [in, G·H], ``w_hh`` [H, G·H], ``bias`` [1, G·H].  Differentiable."""
    if cell not in CELLS:
        raise ValueError(f"unknown recurrent cell '{cell}'")
    if x.is_cuda and w_ih.is_cuda and w_hh.is_cuda and bias.is_cuda and scan_supported(w_hh.shape[0], cell):
        return _RnnSequenceFn.apply(x, w_ih, w_hh, bias, cell, dilation)
    return rnn_sequence_reference(x, w_ih, w_hh, bias, cell, dilation)
