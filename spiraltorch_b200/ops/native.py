"""Loader for the native sm_100a library and thin ctypes helpers.

The library is built in-tree (``spiraltorch_b200/_native/libst_b200.so``) and exposes a C
ABI.  On a machine with a CUDA device the library is mandatory: if it is missing and cannot
be built, every CUDA op raises instead of silently running a PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from ..utils import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_load_error: Optional[BaseException] = None


class NativeError(RuntimeError):
    """A native launcher returned a non-zero status."""


class DeviceWaitTimeout(NativeError):
    """A bounded device-side wait ran out of time (the kernel returned cleanly)."""


def lib() -> ctypes.CDLL:
    """Return the loaded native library, building it first when it is stale or missing."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if _load_error is not None:
            raise _load_error
        try:
            path = _build.LIB_PATH
            if not _build.is_current():
                if _build.find_nvcc() is not None:
                    path = _build.build_native()
                elif not path.exists():
                    raise NativeError(
                        f"native library {path} is missing and nvcc is not available to build it")
            handle = ctypes.CDLL(str(path))
            handle.st_last_error.restype = ctypes.c_char_p
            handle.st_read_error_word.argtypes = [ctypes.POINTER(ctypes.c_uint), ctypes.c_int]
            _lib = handle
        except BaseException as exc:  # noqa: BLE001 - remembered and re-raised on every call
            _load_error = exc
            raise
    return _lib


def available() -> bool:
    """True when CUDA ops can run: a CUDA device is present and the library loads."""
    if not torch.cuda.is_available():
        return False
    lib()  # raises loudly on a GPU box without a usable library
    return True


def last_error() -> str:
    msg = lib().st_last_error()
    return msg.decode() if msg else ""


def check(status: int, what: str) -> None:
    if status != 0:
        raise NativeError(f"{what} failed with status {status}: {last_error()}")


def read_error_word(clear: bool = True) -> tuple[int, int, int, int]:
    """Return (code, detail, block, count) written by bounded device waits; 0 = no error."""
    buf = (ctypes.c_uint * 4)()
    lib().st_read_error_word(buf, 1 if clear else 0)
    return tuple(int(x) for x in buf)  # type: ignore[return-value]


def error_pending() -> bool:
    """True when a kernel has left an error record (a host read of mapped memory: no synchronisation)."""
    return read_error_word(clear=False)[0] != 0


def raise_on_device_error() -> None:
    code, detail, block, count = read_error_word(clear=True)
    if code == 0:
        return
    if code in (1, 2):
        raise DeviceWaitTimeout(
            f"device-side bounded wait timed out (code={code}, detail=0x{detail:x}, block={block}, "
            f"count={count})")
    raise NativeError(f"device error code={code} detail=0x{detail:x} block={block} count={count}")


def poll() -> None:
    """Step-boundary check: raise if any kernel launched so far left an error record.

    A bounded wait that runs out (or a bounds check that refused an access) makes the kernel return early with
    its outputs unwritten while the launcher still reports success, so trainers and the host-transfer points of
    ``Tensor`` call this.  It is a host read of mapped pinned memory: no device synchronisation, and a no-op
    until the library has been loaded."""
    if _lib is None:
        return
    if error_pending():
        raise_on_device_error()


def set_wait_timeout(seconds: Optional[float]) -> None:
    """Limit of every bounded device-side wait on the current device (``None`` or 0 restores the 2 s default).
    Applies to kernels launched after the call."""
    ns = 0 if not seconds else max(1, int(seconds * 1e9))
    check(lib().st_set_wait_timeout_ns(ctypes.c_ulonglong(ns)), "st_set_wait_timeout_ns")


def stream_ptr(device: Optional[torch.device] = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    """Device pointer of a CUDA tensor for a native launch.  A host tensor here would make the kernel
    dereference a host address and fault the context, so it is refused."""
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ValueError(f"native launch was given a host tensor of shape {tuple(t.shape)}; move it to the GPU first")
    return ctypes.c_void_p(t.data_ptr())


def same_device(op: str, *tensors: Optional[torch.Tensor]) -> None:
    """Every tensor handed to one launch must live on the same CUDA device: a kernel that is given a host
    pointer (or another GPU's) faults the context, so this is checked before the pointers are taken."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"{op}: operands live on different devices ({dev} and {t.device})")


def require_cuda(op: str, *tensors: Optional[torch.Tensor]) -> None:
    """Refuse a launch unless every operand is a CUDA tensor on one device.  Launchers receive raw addresses:
    a host tensor's address would be encoded into a TMA tensor map or dereferenced by the kernel and fault the
    context, so the check comes before any pointer is taken."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError(f"{op}: operand of shape {tuple(t.shape)} is a host tensor; move it to the GPU first")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"{op}: operands live on different devices ({dev} and {t.device})")


def deterministic_reduction() -> bool:
    """``SPIRAL_DETERMINISTIC_REDUCTION`` (or the master switch ``SPIRAL_DETERMINISTIC``): reductions whose order
    would depend on scheduling - split-K weight gradients that meet in fp32 atomics, the embedding scatter-add -
    take their fixed-order form, so two runs give bit-identical gradients."""
    def on(name: str) -> bool:
        return os.environ.get(name, "0").strip().lower() not in ("0", "", "false", "off", "no")
    return on("SPIRAL_DETERMINISTIC_REDUCTION") or on("SPIRAL_DETERMINISTIC")


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors always take the native path; CPU tensors take the PyTorch CPU path."""
    return t.is_cuda


if os.environ.get("SPIRALTORCH_B200_EAGER_LOAD") == "1" and torch.cuda.is_available():
    lib()
