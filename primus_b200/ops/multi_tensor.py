"""Multi-tensor apply helpers: one kernel launch over a list of tensors (``csrc/multi_tensor.cu``).

``l2norm`` / ``scale`` / ``axpby`` over lists of fp32 or bf16 tensors.  The chunk table (pointer triplets +
sizes) is built on the host, cached per tensor-list identity and uploaded once; the launches themselves do
not synchronise.  The engine's own optimizer works on flat buffers and does not need these; they serve code
that holds per-parameter tensors (LoRA adapters, SFT, user extensions) — the role Apex's
``multi_tensor_applier`` plays in the reference
(primus/backends/megatron/patches/torch_fused_adam_patches.py:40-88).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib

CHUNK = 65536
_DT = np.dtype([("a", "<u8"), ("b", "<u8"), ("out", "<u8"), ("n", "<i4"), ("tensor", "<i4")])
_CODE = {torch.float32: 0, torch.bfloat16: 1}
_CACHE: dict = {}


def _table(a: Sequence[torch.Tensor], b: Optional[Sequence[torch.Tensor]], out: Optional[Sequence[torch.Tensor]]):
    # element sizes are part of the key: chunk offsets depend on them, and the allocator hands freed addresses out again
    key = (tuple((t.data_ptr(), t.numel()) for t in a), a[0].element_size(),
           (tuple(t.data_ptr() for t in b), b[0].element_size()) if b else None,
           (tuple(t.data_ptr() for t in out), out[0].element_size()) if out else None)
    hit = _CACHE.get(key)
    if hit is not None:
        return hit
    rows = []
    for ti, t in enumerate(a):
        assert t.is_contiguous(), "multi-tensor ops need contiguous tensors"
        es = t.element_size()
        eb = b[ti].element_size() if b else 0
        eo = out[ti].element_size() if out else 0
        n = t.numel()
        for s in range(0, n, CHUNK):
            rows.append((t.data_ptr() + s * es, (b[ti].data_ptr() + s * eb) if b else 0,
                         (out[ti].data_ptr() + s * eo) if out else 0, min(CHUNK, n - s), ti))
    host = np.array(rows, dtype=_DT) if rows else np.zeros(0, dtype=_DT)
    dev = torch.from_numpy(host.view(np.uint8).copy()).to(a[0].device) if rows else torch.empty(0, dtype=torch.uint8,
                                                                                             device=a[0].device)
    if len(_CACHE) > 64:
        _CACHE.clear()
    _CACHE[key] = (dev, len(rows))
    return dev, len(rows)


def _code(ts: Sequence[torch.Tensor]) -> int:
    dt = ts[0].dtype
    assert all(t.dtype == dt for t in ts), "all tensors of one list must share a dtype"
    return _CODE[dt]


def multi_tensor_l2norm(tensors: List[torch.Tensor], per_tensor: bool = False):
    """Returns the global L2 norm (0-dim fp32 tensor) and, with ``per_tensor``, the per-tensor norms."""
    if not tensors:
        z = torch.zeros((), dtype=torch.float32)
        return (z, torch.zeros(0)) if per_tensor else z
    if not tensors[0].is_cuda:
        per = torch.stack([t.float().pow(2).sum() for t in tensors])
        tot = per.sum().sqrt()
        return (tot, per.sqrt()) if per_tensor else tot
    dev = tensors[0].device
    table, n = _table(tensors, None, None)
    partial = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
    per = torch.empty(len(tensors), dtype=torch.float32, device=dev) if per_tensor else None
    total = torch.empty(1, dtype=torch.float32, device=dev)
    _lib.call("mt_l2norm", table, n, _code(tensors), partial, per, len(tensors), total)
    tot = total[0].sqrt()
    return (tot, per.sqrt()) if per_tensor else tot


def multi_tensor_scale(srcs: List[torch.Tensor], dsts: List[torch.Tensor], scale: float,
                       found_inf: Optional[torch.Tensor] = None) -> None:
    """dst_i = src_i * scale (dtype conversion allowed); ``found_inf`` (int32 [1]) is set when a source element is
    not finite."""
    if not srcs:
        return
    if not srcs[0].is_cuda:
        for s, d in zip(srcs, dsts):
            if found_inf is not None and not torch.isfinite(s).all():
                found_inf.fill_(1)
            d.copy_(s.float() * scale)
        return
    table, n = _table(srcs, None, dsts)
    _lib.call("mt_scale", table, n, _code(srcs), _code(dsts), float(scale), found_inf)


def multi_tensor_axpby(xs: List[torch.Tensor], ys: List[torch.Tensor], outs: List[torch.Tensor], a: float,
                       b: float) -> None:
    """out_i = a * x_i + b * y_i."""
    if not xs:
        return
    if not xs[0].is_cuda:
        for x, y, o in zip(xs, ys, outs):
            o.copy_(a * x.float() + b * y.float())
        return
    assert _code(xs) == _code(ys)
    table, n = _table(xs, ys, outs)
    _lib.call("mt_axpby", table, n, _code(xs), _code(outs), float(a), float(b))
