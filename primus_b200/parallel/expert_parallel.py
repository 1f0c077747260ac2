"""Expert-parallel token dispatch / combine over NCCL all-to-all (the baseline path; the fused
MegaMoE kernels replace it when ``use_turbo_mega_moe`` is on).

Copies of tokens are sorted by global expert id, exchanged with ``all_to_all_single`` using split sizes
derived from the all-gathered per-expert counts, and arrive ordered ``[source rank][local expert]``.  The
split sizes have to be known on the host, which costs one device->host synchronisation per layer — the
same bubble the reference's all-to-all dispatcher has (``_maybe_dtoh_and_synchronize``,
primus/backends/megatron/patches/moe_patches/moe_alltoall_dtoh_patches.py:22-85) and that the fused
path removes.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        x = x.contiguous()
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(out, g, output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits,
                               group=ctx.group)
        return out, None, None, None


def all_to_all(x, in_splits, out_splits, group):
    return _AllToAll.apply(x, in_splits, out_splits, group)


def exchange_counts(counts_global: torch.Tensor, ep: int, ep_rank: int, group):
    """counts_global: int64 [E] copies this rank routes to every global expert.
    Returns (in_splits, out_splits as python lists, recv_counts [ep, E_local] tensor)."""
    E = counts_global.numel()
    e_local = E // ep
    allc = torch.empty(ep, E, dtype=counts_global.dtype, device=counts_global.device)
    dist.all_gather_into_tensor(allc, counts_global.contiguous(), group=group) if counts_global.is_cuda else \
        dist.all_gather(list(allc.unbind(0)), counts_global.contiguous(), group=group)
    recv = allc[:, ep_rank * e_local:(ep_rank + 1) * e_local].contiguous()  # [src rank, local expert]
    send_per_rank = counts_global.view(ep, e_local).sum(1)
    host = torch.cat([send_per_rank, recv.sum(1)]).tolist()  # the one device->host sync of this path
    return host[:ep], host[ep:], recv
