"""ctypes binding of ``libprimus_b200.so`` (the sm_100a kernels under ``primus_b200/csrc``).

The library exports ``extern "C"`` launchers that take raw device pointers and a CUDA stream.
``call(name, *args)`` converts torch tensors to pointers, appends nothing implicitly, and raises
on a non-zero return code.  On a machine with a GPU the library is mandatory: ops never fall back
to PyTorch for CUDA tensors (``require()`` raises if the library is missing).
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libprimus_b200.so"


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return Path(os.environ.get("PRIMUS_B200_LIB", LIB_PATH))


def available() -> bool:
    return lib_path().exists()


def load():
    """Load (once) and return the ctypes handle."""
    global _LIB
    if _LIB is None:
        with _LOCK:
            if _LIB is None:
                p = lib_path()
                if not p.exists():
                    raise NativeLibraryError(
                        f"{p} not found: build it with `python -m primus_b200.build` "
                        "(CUDA tensors are never routed to a PyTorch fallback)"
                    )
                _LIB = ctypes.CDLL(str(p), mode=ctypes.RTLD_GLOBAL)
    return _LIB


def require():
    return load()


_PTR = ctypes.c_void_p


def _conv(a):
    if a is None:
        return _PTR(0)
    if isinstance(a, torch.Tensor):
        return _PTR(a.data_ptr())
    if isinstance(a, bool):
        return ctypes.c_int(int(a))
    if isinstance(a, int):
        return ctypes.c_long(a)
    if isinstance(a, float):
        return ctypes.c_float(a)
    return a


def stream_ptr() -> ctypes.c_void_p:
    return _PTR(torch.cuda.current_stream().cuda_stream)


# Number of device kernels each launcher enqueues (default 1); used for the launch counter below.
_KERNELS_PER_CALL = {"rmsnorm_bwd": 2, "sumsq": 2, "flash_attn_bwd": 3, "quant_fp8_tensorwise": 2, "quant_fp8_delayed": 2}
LAUNCH_COUNT = 0


def call(name: str, *args) -> None:
    """Invoke ``pb_<name>`` with converted arguments; the current CUDA stream is appended."""
    global LAUNCH_COUNT
    fn = getattr(load(), "pb_" + name)
    fn.restype = ctypes.c_int
    LAUNCH_COUNT += _KERNELS_PER_CALL.get(name, 1)
    rc = fn(*[_conv(a) for a in args], stream_ptr())
    if rc != 0:
        raise NativeLibraryError(f"pb_{name} failed with code {rc}")


def call_ret(name: str, *args) -> int:
    """Invoke a host-only helper that returns a value (no stream appended)."""
    fn = getattr(load(), "pb_" + name)
    fn.restype = ctypes.c_int
    return fn(*[_conv(a) for a in args])


class I32(int):
    """Marks a Python int that must be passed as a 32-bit int."""


def i32(x: int):
    return ctypes.c_int(int(x))


# ---------------------------------------------------------------------------------------------
# Device status word: kernels with bounded waits report a timeout here instead of hanging.
_STATUS: dict[int, torch.Tensor] = {}

STATUS_MESSAGES = {
    0: "ok",
    1: "TMA producer timed out waiting for a free shared-memory stage",
    2: "MMA issuer timed out waiting for operands or an accumulator slot",
    3: "epilogue timed out waiting for an accumulator",
    4: "timed out waiting for a peer flag in global memory",
    5: "bad argument detected on the device",
    6: "routed rows exceed the capacity of the expert-parallel buffers (raise moe_fused_capacity_factor)",
}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _STATUS.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        _STATUS[dev] = t
    return t


def check_status(device=None) -> None:
    """Synchronising check of the device status word; raises if a kernel recorded an error."""
    t = status_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise NativeLibraryError(f"device kernel reported status {code}: {STATUS_MESSAGES.get(code, '?')}")
