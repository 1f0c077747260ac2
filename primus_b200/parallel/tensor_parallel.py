"""Tensor-parallel communication primitives with autograd (NCCL / gloo path).

Sequence parallelism shards activations on the token dimension (dim 0) between TP regions:
all-gather before a column-parallel GEMM, reduce-scatter after a row-parallel GEMM — the
collectives and their conjugate backward ops of the reference's local TP layer
(primus/backends/megatron/core/tensor_parallel/layers.py:67-74,150-167).

The fused all-gather->GEMM / GEMM->reduce-scatter kernels in ``primus_b200.parallel.fused_tp``
replace the (collective, GEMM) pairs built from these primitives when symmetric memory is available.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _ws(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def all_gather_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.device.type == "cpu":
        # gloo has no reduce_scatter_tensor: all-reduce then slice (CPU plumbing tests only)
        tmp = x.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
        return out
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_dim0(g, ctx.group), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


class _AllReduce(torch.autograd.Function):
    """Forward all-reduce, backward identity (output of a row-parallel GEMM without SP)."""

    @staticmethod
    def forward(ctx, x, group):
        if _ws(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """Forward identity, backward all-reduce (input of a column-parallel GEMM without SP)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _ws(ctx.group) > 1:
            g = g.contiguous().clone()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ScatterSeq(torch.autograd.Function):
    """Forward: keep this rank's token slice; backward: all-gather (entering an SP region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = _ws(group)
        if n == 1:
            return x
        r = dist.get_rank(group)
        c = x.shape[0] // n
        return x[r * c:(r + 1) * c].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


def gather_seq(x, group): return _GatherSeq.apply(x, group)
def reduce_scatter_seq(x, group): return _ReduceScatterSeq.apply(x, group)
def all_reduce(x, group): return _AllReduce.apply(x, group)
def copy_to_tp(x, group): return _CopyToTP.apply(x, group)
def scatter_seq(x, group): return _ScatterSeq.apply(x, group)
