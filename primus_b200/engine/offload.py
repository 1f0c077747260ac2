"""Activation offload: tensors saved for backward inside the context are copied to pinned host memory on a side
stream and brought back just before the backward needs them.

The copy out waits for the producing work on the compute stream and the compute stream never waits for it (the
device tensor is released when the copy has finished); the copy back is issued when autograd unpacks the tensor and
the compute stream waits on its event.  Small tensors, parameters and tensors that do not own their storage stay
on the device.  Counterpart of the reference's offload buffer for pipeline stages
(primus/backends/megatron/core/pipeline_parallel/handler/offload_handler.py:27-261: pooled pinned buffers, dedicated
stream, events) and of Megatron's ``cpu_offloading`` / ``cpu_offloading_num_layers`` switches.
"""
from __future__ import annotations

import contextlib

import torch

_STREAMS: dict = {}
_POOL: dict = {}          # (numel, dtype) -> [pinned tensors]
STATS = {"offloaded_bytes": 0, "offloaded_tensors": 0, "kept_tensors": 0}


def _stream(device):
    s = _STREAMS.get(device)
    if s is None:
        s = _STREAMS[device] = torch.cuda.Stream(device=device)
    return s


def _pinned(numel: int, dtype) -> torch.Tensor:
    free = _POOL.get((numel, dtype))
    if free:
        return free.pop()
    return torch.empty(numel, dtype=dtype, pin_memory=True)


def _release(t: torch.Tensor):
    _POOL.setdefault((t.numel(), t.dtype), []).append(t)


class _Packed:
    __slots__ = ("host", "shape", "device", "event", "dtype")


@contextlib.contextmanager
def offload_saved_activations(enabled: bool = True, min_bytes: int = 1 << 20):
    """Context manager; inside it, every tensor that autograd saves for backward and that is a contiguous CUDA tensor
    of at least ``min_bytes`` (and not a parameter) lives in pinned host memory until the backward pass asks for it."""
    if not enabled:
        yield
        return

    def pack(t: torch.Tensor):
        if (not t.is_cuda or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < min_bytes
                or not t.is_contiguous() or t._base is not None or getattr(t, "_is_weight", False)):
            STATS["kept_tensors"] += 1
            return t
        p = _Packed()
        p.shape, p.device, p.dtype = t.shape, t.device, t.dtype
        p.host = _pinned(t.numel(), t.dtype)
        side = _stream(t.device)
        side.wait_stream(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(side):
            p.host.copy_(t.reshape(-1), non_blocking=True)
            p.event = torch.cuda.Event()
            p.event.record(side)
        t.record_stream(side)           # the allocator must not reuse the block before the copy out has run
        STATS["offloaded_bytes"] += t.numel() * t.element_size()
        STATS["offloaded_tensors"] += 1
        return p

    def unpack(p):
        if not isinstance(p, _Packed):
            return p
        side = _stream(p.device)
        with torch.cuda.stream(side):
            side.wait_event(p.event)
            out = torch.empty(p.shape, dtype=p.dtype, device=p.device)
            out.reshape(-1).copy_(p.host, non_blocking=True)
            done = torch.cuda.Event()
            done.record(side)
        torch.cuda.current_stream(p.device).wait_event(done)
        out.record_stream(torch.cuda.current_stream(p.device))
        # the pinned buffer returns to the pool once the copy back has been queued behind `done`; reuse by a later
        # pack happens on the same side stream, so stream order protects it
        _release(p.host)
        return out

    with torch.autograd.graph.saved_tensors_hooks(pack, unpack):
        yield
