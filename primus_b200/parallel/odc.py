"""On-demand communication (ODC) for the sharded data-parallel step.

With ``enable_odc`` the gradient reduce-scatter and the parameter all-gather of the distributed optimizer stop being
collectives.  Every rank *pushes* its gradients of a bucket into the shard owners' fp32 accumulators as soon as its own
backward pass has produced them (``pb_odc_scatter_accumulate``: ``red.global.add`` on peer memory), and *pulls* the
updated parameter shards from their owners when it needs them (``pb_odc_gather``).  Ranks meet once per mini-batch —
a device-side barrier before the owners read their accumulators — instead of once per bucket collective, so ranks
whose micro-batches differ in number or length (``sft_lb_mini``) no longer wait for each other inside a step.

Accumulators are double buffered by mini-batch parity: after the barrier of mini-batch ``t`` a fast rank may push
mini-batch ``t + 1`` into the other half while a slow owner still reads half ``t``; the owner clears a half right
after reading it, which is ordered before its arrival at the next barrier.

On CPU tensors (gloo) the pushes are emulated with an all-reduce per bucket, which keeps the arithmetic and the
"one meeting per mini-batch" contract testable without GPUs.

Counterpart of primus/core/odc (``ReductionService`` scatter_accumulate.py:36-431, ``GatherService`` gather.py:93-244,
FSDP integration fsdp/fsdp2.py); keys ``enable_odc`` / ``odc_grad_spike_threshold`` of
primus/configs/modules/megatron/trainer_base.yaml:197-214.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


class ODCReducer:
    def __init__(self, buf):
        self.buf = buf
        self.dp, self.rank = buf.dp_size, buf.dp_rank
        self.cuda = buf.device.type == "cuda"
        self.shard_off, off = {}, 0
        for b in buf.buckets:
            self.shard_off[b.index] = off
            off += (b.end - b.start) // self.dp
        self.total = off
        self.parity = 0
        self.pushed: set = set()
        self.meetings = 0            # device barriers / mini-batches so far (tests read it)
        if self.cuda:
            from .symm_mem import SymmetricBuffer

            assert buf.symmetric, "ODC needs the peer-mapped parameter buffer"
            self.acc_sym = SymmetricBuffer(2 * self.total * 4, buf.dp_group, buf.device)
            self.acc = self.acc_sym.local(torch.float32, 2 * self.total)
            self.acc.zero_()
            torch.cuda.synchronize(buf.device)
            dist.barrier(group=buf.dp_group)      # nobody pushes before every accumulator is cleared

    # ------------------------------------------------------------------ gradients: pushes
    def push_bucket(self, b) -> None:
        """This rank's gradients of bucket ``b`` -> the owners' accumulators (scaled by 1 / dp).  No waiting."""
        buf = self.buf
        g = buf.grad_data[b.start:b.end]
        n = (b.end - b.start) // self.dp
        self.pushed.add(b.index)
        if not self.cuda:
            if buf.grad_scale != 1.0:
                g.mul_(buf.grad_scale)
            dist.all_reduce(g, group=buf.dp_group)       # emulation: every rank ends up with all sums
            return
        from ..ops import _lib

        base = (self.parity * self.total + self.shard_off[b.index]) * 4
        tbl = (ctypes.c_long * self.dp)(*[self.acc_sym.peer_ptr(r, base) for r in range(self.dp)])
        _lib.call("odc_scatter_accumulate", tbl, self.dp, self.rank, g, n, float(buf.grad_scale))

    def finish(self) -> None:
        """The one meeting of the mini-batch: after it, every owner's accumulator holds the complete sums; they are
        moved into the owner's gradient shard and cleared."""
        buf = self.buf
        self.meetings += 1
        if self.cuda:
            self.acc_sym.barrier(0)
            half = self.acc[self.parity * self.total:(self.parity + 1) * self.total]
            for b in buf.buckets:
                s, e = buf.shard_range(b)
                o = self.shard_off[b.index]
                buf.grad_data[s:e].copy_(half[o:o + (e - s)])
            half.zero_()
            self.parity ^= 1
        self.pushed.clear()

    # ------------------------------------------------------------------ parameters: pulls
    def gather_params(self) -> None:
        """Pull the other owners' updated parameter shards (after a barrier: every owner has written its own)."""
        buf = self.buf
        if not self.cuda:
            for b in reversed(buf.buckets):
                s, e = buf.shard_range(b)
                parts = [torch.empty(e - s, dtype=buf.param_data.dtype) for _ in range(self.dp)]
                dist.all_gather(parts, buf.param_data[s:e].clone(), group=buf.dp_group)
                buf.param_data[b.start:b.end].copy_(torch.cat(parts))
            return
        from ..ops import _lib

        buf.sym_param.barrier(1)
        tbl = (ctypes.c_long * self.dp)(*[buf.sym_param.peer_ptr(r) for r in range(self.dp)])
        for b in reversed(buf.buckets):
            n = (b.end - b.start) // self.dp
            _lib.call("odc_gather", tbl, self.dp, self.rank, b.start, n, buf.param_data)
