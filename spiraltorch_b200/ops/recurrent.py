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
