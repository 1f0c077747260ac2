"""Symmetric memory for fused compute+collective kernels.

A :class:`SymmetricBuffer` is a device allocation that exists with the same size on every rank of a
node-local process group and is mapped into every rank's address space (CUDA IPC), so kernels can
load / store / reduce peers' data directly over NVLink / NVSwitch (``ld.global`` / ``st.global`` to a
peer pointer, non-multicast TMA loads).  Each buffer carries a small flag area for signalling; a flag
protocol is always *epoch based* (monotonically increasing values) and every wait is bounded.

Host side only does the handle exchange (through ``torch.distributed`` object collectives); the
native part is ``csrc/symm_mem.cu``.

Reference counterparts: primus_turbo's symmetric-memory workspace used by the copy-engine parameter
all-gather (primus/backends/megatron/core/distributed/sdma_param_gather.py:126-243) and the ODC
``SymmBufferRegistry`` (primus/core/odc/primitives/utils.py:258-470).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_DTYPE_SIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.uint8: 1, torch.int64: 8,
               torch.float8_e4m3fn: 1}
_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int64: "<i8", torch.float16: "<f2"}


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` holder so torch can wrap a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """uint8 tensor viewing ``nbytes`` at ``ptr`` (no ownership)."""
    with torch.cuda.device(device):
        return torch.as_tensor(_CudaArray(ptr, nbytes), device=device)


def probe_p2p(max_dev: int = 16) -> dict:
    """Peer-access matrix and capability bits; never leaves a sticky CUDA error behind."""
    lib = _lib.require()
    mat = (ctypes.c_int * (max_dev * max_dev))()
    n = ctypes.c_int(0)
    caps = ctypes.c_int(0)
    lib.pb_probe_p2p(mat, ctypes.c_int(max_dev), ctypes.byref(n), ctypes.byref(caps))
    nd = n.value
    return {"num_devices": nd, "matrix": [[mat[i * max_dev + j] for j in range(nd)] for i in range(nd)],
            "all_p2p": bool(caps.value & 1), "multicast": bool(caps.value & 2), "fabric": bool(caps.value & 4)}


def barrier_wait_cycles() -> int:
    """Cycle limit of the device-side barrier between ranks.  Ranks of one step can be skewed by far more than a
    kernel-internal wait ever is (a checkpoint write, a slow data loader, Python garbage collection on one rank), so the
    default is 60 s of SM clocks rather than the 1.5 s the in-kernel waits use; ``PRIMUS_B200_BARRIER_TIMEOUT_S``
    overrides it.  The wait stays bounded: on expiry the kernel records status 4 and returns."""
    sec = float(os.environ.get("PRIMUS_B200_BARRIER_TIMEOUT_S", "60"))
    return int(max(sec, 0.001) * 1.9e9)


class SymmetricBuffer:
    FLAG_BYTES = 4096  # 1024 int32 flags per rank, placed after the payload

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = -(-nbytes // 4096) * 4096
        total = self.nbytes + self.FLAG_BYTES
        lib = _lib.require()
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            rc = lib.pb_symm_alloc(ctypes.byref(p), ctypes.c_long(total))
            if rc != 0:
                raise RuntimeError(f"symmetric allocation of {total} bytes failed with CUDA error {rc}")
            self.local_ptr = p.value
            handle = ctypes.create_string_buffer(64)
            rc = lib.pb_ipc_export(ctypes.c_void_p(self.local_ptr), handle)
            if rc != 0:
                raise RuntimeError(f"cudaIpcGetMemHandle failed with {rc}")
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            else:
                handles[0] = bytes(handle.raw)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                q = ctypes.c_void_p()
                rc = lib.pb_ipc_open(ctypes.c_char_p(h), ctypes.byref(q))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed with {rc}")
                self.peer_ptrs.append(q.value)
        self._bytes = tensor_from_ptr(self.local_ptr, total, self.device)
        # device arrays of peer payload / flag pointers for kernels
        self.peer_ptr_table = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)
        self.peer_flag_table = torch.tensor([p_ + self.nbytes for p_ in self.peer_ptrs], dtype=torch.int64,
                                            device=self.device)
        self.epoch = 0
        if self.world > 1:
            dist.barrier(group=group)

    # ------------------------------------------------------------------ views
    def local(self, dtype=torch.uint8, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        n = (self.nbytes - offset_bytes) // _DTYPE_SIZE[dtype] if numel is None else numel
        return self._bytes[offset_bytes:offset_bytes + n * _DTYPE_SIZE[dtype]].view(dtype)

    @property
    def flags(self) -> torch.Tensor:
        return self._bytes[self.nbytes:].view(torch.int32)

    def peer_ptr(self, rank: int, offset_bytes: int = 0) -> int:
        return self.peer_ptrs[rank] + offset_bytes

    def peer_tensor(self, rank: int, dtype=torch.uint8, numel: Optional[int] = None, offset_bytes: int = 0):
        """A tensor viewing rank ``rank``'s payload (peer memory!). Only for our own kernels and plain copies."""
        n = (self.nbytes - offset_bytes) // _DTYPE_SIZE[dtype] if numel is None else numel
        t = tensor_from_ptr(self.peer_ptrs[rank] + offset_bytes, n * _DTYPE_SIZE[dtype], self.device)
        return t.view(dtype)

    # ------------------------------------------------------------------ sync
    def barrier(self, slot: int = 0):
        """Device-side barrier over the group on the current stream (bounded wait). Uses flag slots
        [slot*world, (slot+1)*world)."""
        if self.world == 1:
            return
        self.epoch += 1
        base = slot * self.world * 4
        tbl = self.peer_flag_table + base
        _lib.call("symm_barrier", tbl, self.flags[slot * self.world:], self.world, self.rank, self.epoch,
                  _lib.status_word(self.device), barrier_wait_cycles())

    def close(self):
        lib = _lib.require()
        for r, p in enumerate(self.peer_ptrs):
            if r != self.rank:
                lib.pb_ipc_close(ctypes.c_void_p(p))
        lib.pb_symm_free(ctypes.c_void_p(self.local_ptr))
        self.peer_ptrs = []


_HEAPS: dict = {}


def get_workspace(name: str, nbytes: int, group=None) -> SymmetricBuffer:
    """Named, grow-only symmetric workspace (all ranks must call with the same arguments)."""
    key = (name, id(group))
    buf = _HEAPS.get(key)
    if buf is None or buf.nbytes < nbytes:
        if buf is not None:
            torch.cuda.synchronize()
            buf.close()
        buf = SymmetricBuffer(nbytes, group)
        _HEAPS[key] = buf
    return buf
