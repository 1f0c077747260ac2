"""Data-parallel parameter/gradient buffers and the ZeRO-1 distributed optimizer.

* :class:`ParamGradBuffer` places every parameter of one (dtype, data-parallel group) class in a flat
  bf16 ``param_data`` buffer and gives each a view into a flat fp32 ``grad_data`` buffer as
  ``param.main_grad`` — the convention the reference relies on
  (primus/backends/megatron/core/distributed/finalize_model_grad.py:35-38,71-74,
  primus/backends/megatron/core/extensions/primus_turbo.py:197-213).  The buffer is cut into buckets;
  when every parameter of a bucket reported its gradient in the last micro-batch the bucket's
  reduce-scatter starts on a side stream (``overlap_grad_reduce``).
* :class:`DistributedOptimizer` keeps fp32 master weights and Adam moments only for this rank's
  1/dp shard of every bucket, updates them with the fused AdamW kernel (clip coefficient and
  non-finite skip flag stay on the device: no host sync in a step), writes bf16 parameters back into
  the shard region and all-gathers the buckets (``overlap_param_gather`` issues them asynchronously
  on the side stream; the first forward waits per bucket).
  Reference semantics: primus/configs/modules/megatron/trainer_base.yaml:161-195 and
  primus/backends/megatron/core/distributed/sdma_param_gather.py:126-243 (param all-gather).

With ``use_distributed_optimizer=False`` gradients are all-reduced and every rank updates all
parameters (plain DDP).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Iterable, Optional

import torch
import torch.distributed as dist

from ..ops import optim as optim_ops


@dataclass
class Bucket:
    index: int
    start: int  # offsets into the flat buffer (elements)
    end: int
    params: list = field(default_factory=list)
    pending: set = field(default_factory=set)
    rs_handle: Optional[object] = None
    ag_handle: Optional[object] = None
    rs_event: Optional[object] = None


class ParamGradBuffer:
    def __init__(self, params: list[torch.nn.Parameter], dp_group, dp_size: int, dp_rank: int,
                 bucket_size: Optional[int] = None, grad_dtype=torch.float32, use_distributed_optimizer=True,
                 overlap_grad_reduce=False, average_in_collective=True, comm_stream=None, symmetric=False,
                 extra_grad_scale: float = 1.0, grad_reduce_in_bf16: bool = False, odc: bool = False):
        """``extra_grad_scale`` multiplies the gradients before the collective.  Expert parameters need it: every
        expert-parallel rank accumulates the contributions of the tokens of all ``ep`` ranks, each normalised for its
        own rank's micro-batches, and the buffer is then only averaged over the (smaller) expert-data-parallel group,
        so the sum is ``dp / edp`` times the data-parallel mean the dense parameters get (Megatron's
        ``expert_gradient_scaling_factor = edp / dp``)."""
        assert params, "empty parameter list"
        self.extra_grad_scale = float(extra_grad_scale)
        # ``grad_reduce_in_bf16``: gradients are accumulated over the micro-batches in fp32 as always, but travel as bf16
        # (half the bytes of the reduce-scatter / all-reduce); the reduced values are widened back into the fp32 buffer
        self.grad_reduce_in_bf16 = bool(grad_reduce_in_bf16) and dp_size > 1
        self._bf16_stage = None
        self.params = params
        self.dp_group, self.dp_size, self.dp_rank = dp_group, dp_size, dp_rank
        self.use_distributed_optimizer = use_distributed_optimizer
        self.overlap_grad_reduce = overlap_grad_reduce and dp_size > 1
        self.comm_stream = comm_stream
        device = params[0].device
        self.device = device
        self.param_dtype = params[0].dtype
        self.grad_dtype = grad_dtype if params[0].dtype != torch.float32 else torch.float32
        align = 128 * dp_size  # every bucket splits into dp equal, 256-byte aligned shards
        if bucket_size is None:
            bucket_size = max(40_000_000, 1_000_000 * dp_size)
        # parameters are laid out in reverse order so that buckets fill in backward order
        offsets = {}
        buckets: list[Bucket] = []
        cur_start, cur = 0, 0
        cur_params = []
        for p in reversed(params):
            n = p.numel()
            offsets[p] = cur
            cur += -(-n // 64) * 64  # keep every parameter 128-byte aligned for TMA
            cur_params.append(p)
            if cur - cur_start >= bucket_size:
                cur = -(-cur // align) * align
                buckets.append(Bucket(len(buckets), cur_start, cur, cur_params))
                cur_start, cur_params = cur, []
        if cur_params:
            cur = -(-cur // align) * align
            buckets.append(Bucket(len(buckets), cur_start, cur, cur_params))
        self.numel = cur
        self.buckets = buckets
        self.symmetric = bool(symmetric and dp_size > 1 and device.type == "cuda" and self.param_dtype == torch.bfloat16)
        # parameter all-gather by copy-engine pulls on a side stream instead of P2P stores from the AdamW kernel
        self.copy_engine_gather = False
        self._ce_stream = None
        if self.symmetric:
            # peer-mapped buffers: the fused optimizer kernels read peers' gradients and write peers' parameters
            from .symm_mem import SymmetricBuffer

            self.sym_param = SymmetricBuffer(self.numel * 2, dp_group, device)
            self.sym_grad = SymmetricBuffer(self.numel * 4, dp_group, device)
            self.param_data = self.sym_param.local(torch.bfloat16, self.numel)
            self.grad_data = self.sym_grad.local(torch.float32, self.numel)
            self.fused_sumsq = torch.zeros(1, dtype=torch.float32, device=device)   # sum of squares of the reduced shards
        else:
            self.param_data = torch.zeros(self.numel, dtype=self.param_dtype, device=device)
            self.grad_data = torch.zeros(self.numel, dtype=self.grad_dtype, device=device)
        # on-demand communication: gradients are pushed into the owners' accumulators, parameters pulled (parallel/odc.py)
        self.odc = None
        if odc and dp_size > 1 and use_distributed_optimizer and (self.symmetric or device.type == "cpu"):
            from .odc import ODCReducer

            self.odc = ODCReducer(self)
        self.param_offsets = offsets
        self.param_to_bucket = {}
        for b in buckets:
            for p in b.params:
                self.param_to_bucket[p] = b
        for p in params:
            o = offsets[p]
            view = self.param_data[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad_data[o:o + p.numel()].view(p.shape)
            p.grad_added_to_main_grad = False
            p._grad_ready_cb = self._on_grad_ready
        self.is_last_microbatch = True
        self.grad_scale = 1.0 / dp_size if average_in_collective else 1.0
        self._rs_out: dict[int, torch.Tensor] = {}

    # ------------------------------------------------------------------ shards
    def shard_range(self, b: Bucket) -> tuple[int, int]:
        n = (b.end - b.start) // self.dp_size
        s = b.start + self.dp_rank * n
        return s, s + n

    def zero_grad(self):
        self.grad_data.zero_()
        if self.symmetric:
            self.fused_sumsq.zero_()
        for b in self.buckets:
            b.pending = set(b.params)
            b.rs_handle = None
            b.rs_event = None

    # ------------------------------------------------------------------ grad sync
    def _on_grad_ready(self, p):
        if not (self.overlap_grad_reduce and self.is_last_microbatch):
            return
        b = self.param_to_bucket[p]
        b.pending.discard(p)
        if not b.pending and b.rs_handle is None:
            self._start_bucket_sync(b, async_op=True)

    def _start_bucket_sync_fused(self, b: Bucket, async_op: bool):
        """Symmetric buffers: this rank's shard of the bucket is summed straight from the peers' gradient buffers
        (``csrc/dp_fused.cu``), in place, after a device-side barrier that tells every rank that all copies of the bucket
        are final.  Under ``overlap_grad_reduce`` barrier and kernel run on the side stream while the backward pass of
        the earlier layers continues; ranks reach the buckets in the same order, so the barrier slots line up."""
        import ctypes

        from ..ops import _lib
        from ..ops.fused import scratch

        stream = self.comm_stream if (async_op and self.comm_stream is not None) else None
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream)
        else:
            import contextlib

            ctx = contextlib.nullcontext()
        with ctx:
            if self.extra_grad_scale != 1.0:
                self.grad_data[b.start:b.end].mul_(self.extra_grad_scale)
            self.sym_grad.barrier(2 + b.index % 96)
            s, e = self.shard_range(b)
            tbl = (ctypes.c_long * self.dp_size)(*[self.sym_grad.peer_ptr(r) for r in range(self.dp_size)])
            P = _lib.call_ret("dp_num_partials")
            _lib.call("dp_reduce_scatter", tbl, self.dp_size, self.dp_rank, s, e - s, self.grad_data[s:e],
                      self.grad_scale, scratch(self.device, "dp_partials", P), self.fused_sumsq, 1)
            b.rs_handle = True
            if stream is not None:
                b.rs_event = torch.cuda.Event()
                b.rs_event.record(stream)

    def _start_bucket_sync_odc(self, b: Bucket, async_op: bool):
        stream = self.comm_stream if (async_op and self.comm_stream is not None) else None
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                if self.extra_grad_scale != 1.0:
                    self.grad_data[b.start:b.end].mul_(self.extra_grad_scale)
                self.odc.push_bucket(b)
                b.rs_event = torch.cuda.Event()
                b.rs_event.record(stream)
        else:
            if self.extra_grad_scale != 1.0:
                self.grad_data[b.start:b.end].mul_(self.extra_grad_scale)
            self.odc.push_bucket(b)
        b.rs_handle = True

    def _start_bucket_sync(self, b: Bucket, async_op: bool):
        if self.odc is not None:
            return self._start_bucket_sync_odc(b, async_op)
        if self.symmetric:
            return self._start_bucket_sync_fused(b, async_op)
        g = self.grad_data[b.start:b.end]
        stream = self.comm_stream if (async_op and self.comm_stream is not None) else None
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream)
        else:
            import contextlib

            ctx = contextlib.nullcontext()
        with ctx:
            if self.extra_grad_scale != 1.0:
                g.mul_(self.extra_grad_scale)
            on_cpu = g.device.type == "cpu"
            # NCCL averages inside the collective; gloo has no AVG, so pre-scale there
            op = dist.ReduceOp.SUM if (on_cpu or self.grad_scale == 1.0) else dist.ReduceOp.AVG
            if on_cpu and self.grad_scale != 1.0:
                g.mul_(self.grad_scale)
            if self.grad_reduce_in_bf16:
                self._reduce_bucket_bf16(b, g, op, on_cpu)
            elif self.use_distributed_optimizer:
                s, e = self.shard_range(b)
                out = self.grad_data[s:e]
                if on_cpu:
                    dist.all_reduce(g, group=self.dp_group)
                    b.rs_handle = True
                else:
                    b.rs_handle = dist.reduce_scatter_tensor(out, g, op=op, group=self.dp_group,
                                                             async_op=async_op) or True
            else:
                b.rs_handle = dist.all_reduce(g, op=op, group=self.dp_group, async_op=async_op) or True
            if stream is not None:
                b.rs_event = torch.cuda.Event()
                b.rs_event.record(stream)

    def _reduce_bucket_bf16(self, b: Bucket, g: torch.Tensor, op, on_cpu: bool):
        """bf16 on the wire: cast the bucket, reduce, widen the result back.  Runs on the stream the caller selected
        (the side stream under ``overlap_grad_reduce``), so the collective itself is issued synchronously there."""
        if self._bf16_stage is None:
            self._bf16_stage = torch.empty(self.numel, dtype=torch.bfloat16, device=self.device)
        lo = self._bf16_stage[b.start:b.end]
        lo.copy_(g)
        if self.use_distributed_optimizer and not on_cpu:
            s, e = self.shard_range(b)
            out = self._bf16_stage[s:e]
            dist.reduce_scatter_tensor(out, lo, op=op, group=self.dp_group)
            self.grad_data[s:e].copy_(out)
        else:
            dist.all_reduce(lo, op=op, group=self.dp_group)
            g.copy_(lo)
        b.rs_handle = True

    def finish_grad_sync(self):
        """Reduce every bucket that has not been started and wait for all of them."""
        if self.dp_size == 1:
            if self.extra_grad_scale != 1.0:
                self.grad_data.mul_(self.extra_grad_scale)
            return
        for b in self.buckets:
            if b.rs_handle is None:
                self._start_bucket_sync(b, async_op=False)
        for b in self.buckets:
            if b.rs_handle is not True and b.rs_handle is not None and hasattr(b.rs_handle, "wait"):
                b.rs_handle.wait()
            if b.rs_event is not None:
                torch.cuda.current_stream().wait_event(b.rs_event)
        if self.odc is not None:
            self.odc.finish()

    # ------------------------------------------------------------------ param sync
    def start_param_sync(self, async_op=False):
        if self.dp_size == 1 or not self.use_distributed_optimizer:
            return
        if self.odc is not None:
            return self.odc.gather_params()
        for b in reversed(self.buckets):  # forward order: the embedding-side buckets are needed first
            s, e = self.shard_range(b)
            full = self.param_data[b.start:b.end]
            if full.device.type == "cpu":
                parts = [torch.empty(e - s, dtype=full.dtype) for _ in range(self.dp_size)]
                dist.all_gather(parts, self.param_data[s:e].clone(), group=self.dp_group)
                full.copy_(torch.cat(parts))
                continue
            b.ag_handle = dist.all_gather_into_tensor(full, self.param_data[s:e], group=self.dp_group,
                                                      async_op=async_op)

    def start_param_sync_copy_engine(self):
        """Parameter all-gather on the copy engines: after a device barrier (every rank has written its updated shard
        into its symmetric parameter buffer) this rank pulls the other ranks' shards of every bucket with one
        ``cudaMemcpyAsync`` each on a side stream -- no SM runs for the transfer -- and records an event per bucket that
        ``wait_bucket_params`` makes the compute stream wait for.  Buckets go in forward order and the source ranks are
        rotated so that the ranks do not all read from the same peer at once.  The next overwrite of a shard happens
        after the following step's gradient reduction, which every rank reaches only after its forward pass has waited
        for these copies.  (The reference's SDMA parameter all-gather:
        primus/backends/megatron/patches/parallelism/sdma_param_all_gather_patches.py:62-124.)"""
        from ..ops import _lib

        assert self.symmetric and self.odc is None
        if self._ce_stream is None:
            self._ce_stream = torch.cuda.Stream(device=self.param_data.device)
        cs = self._ce_stream
        cs.wait_stream(torch.cuda.current_stream())
        esz = self.param_data.element_size()
        with torch.cuda.stream(cs):
            self.sym_param.barrier(1)
            for b in reversed(self.buckets):
                n = (b.end - b.start) // self.dp_size
                for k in range(1, self.dp_size):
                    r = (self.dp_rank + k) % self.dp_size
                    lo = b.start + r * n
                    _lib.call("copy_engine_pull", self.param_data[lo:lo + n], self.sym_param.peer_ptr(r, lo * esz), n * esz)
                ev = torch.cuda.Event()
                ev.record(cs)
                b.ag_handle = _EventHandle(ev)
            # nobody may free or overwrite a shard that a peer is still reading: a second barrier behind the copies.
            # During training the next step's gradient reduction already orders this; at the end of a run (or before
            # the buffers are released) ``finish_param_sync`` waits for it, so no rank leaves while it is being read.
            self.sym_param.barrier(2)
            self._ce_done = torch.cuda.Event()
            self._ce_done.record(cs)

    def wait_bucket_params(self, b: Bucket):
        """Make the current stream wait for the bucket's parameter all-gather (no-op when none is pending)."""
        h = b.ag_handle
        if h is not None:
            if hasattr(h, "wait"):
                h.wait()
            b.ag_handle = None

    def buckets_of(self, params) -> list:
        seen, out = set(), []
        for p in params:
            b = self.param_to_bucket.get(p)
            if b is not None and b.index not in seen:
                seen.add(b.index)
                out.append(b)
        return out

    def finish_param_sync(self):
        for b in self.buckets:
            self.wait_bucket_params(b)
        if getattr(self, "_ce_done", None) is not None:
            torch.cuda.current_stream().wait_event(self._ce_done)
            self._ce_done = None


class _EventHandle:
    """Completion handle of work on a side stream: ``wait()`` makes the current stream wait for the recorded event."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class DistributedOptimizer:
    """AdamW over the local shards of one or more :class:`ParamGradBuffer`."""

    def __init__(self, buffers: list[ParamGradBuffer], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 clip_grad=1.0, no_wd_filter=None, norm_groups: Iterable = (), check_for_nan=True,
                 state_dtype: torch.dtype = torch.float32, tp_size: int = 1, expert_norm_group=None):
        """``state_dtype``: dtype of the two Adam moments (fp32, or bf16 with the precision-aware optimizer; the master
        weights are always fp32 and the arithmetic of a step is fp32).

        Global gradient norm: the squared sums of the local shards are added over the data-parallel group (when the
        shards are disjoint) and over ``norm_groups`` (tensor x pipeline parallel ranks).  Parameters that every
        tensor-parallel rank holds whole (norm weights, routers, biases of row-parallel layers: no
        ``tensor_model_parallel`` attribute) would be counted ``tp_size`` times by the second reduction, so their
        share is scaled by ``1 / tp_size`` first, as Megatron leaves tensor-parallel duplicates out of the norm.
        ``expert_norm_group``: without the distributed optimizer every rank updates whole parameters and the dense
        gradients are identical across data-parallel ranks, but each expert-parallel rank owns different experts:
        their squared sum is reduced over this group."""
        self.tp_size = max(int(tp_size), 1)
        self.expert_norm_group = expert_norm_group
        self.buffers = buffers
        self.state_dtype = state_dtype
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.clip_grad = clip_grad
        self.norm_groups = [g for g in norm_groups if g is not None]
        self.check_for_nan = check_for_nan
        # ``overlap_param_gather``: the bucket all-gathers after a step are issued asynchronously in forward order and
        # the next forward pass waits per bucket, right before the first layer that reads it (the trainer installs
        # those waits), as the reference overlaps its per-bucket parameter gather with the forward
        # (primus/backends/megatron/patches/parallelism/sdma_param_all_gather_patches.py:49-130)
        self.overlap_param_gather = False
        self.sanitize_grads = False          # set by the trainer (sft_grad_sanitize)
        self.sanitized_count = torch.zeros((), dtype=torch.int64, device=buffers[0].grad_data.device)
        self.grad_spike_threshold = 0.0      # ``odc_grad_spike_threshold``: skip the step when the norm exceeds it
        # ``enable_optimizer_post_validation``: update first, validate later (see ``_post_validated_step``)
        self.post_validation = False
        self.post_validation_exact = True
        self.post_validation_redos = 0
        self._group_lr: dict = {}
        # MXFP4 weight de-oscillation (parallel/weight_deosc.py): runs on the master shards after every update
        self.deosc = None
        self.step_count = 0
        self.state = []
        dev = buffers[0].device
        for buf in buffers:
            for b in buf.buckets:
                s, e = (buf.shard_range(b) if buf.use_distributed_optimizer else (b.start, b.end))
                master = buf.param_data[s:e].float().clone()
                # weight decay is skipped for 1-D parameters (norm weights, biases): per-element mask ranges
                wd_ranges = self._wd_ranges(buf, b, s, e, no_wd_filter)
                self.state.append(dict(buf=buf, bucket=b, s=s, e=e, master=master,
                                       m=torch.zeros_like(master, dtype=state_dtype),
                                       v=torch.zeros_like(master, dtype=state_dtype), wd_ranges=wd_ranges,
                                       dup_ranges=self._tp_duplicate_ranges(buf, b, s, e) if self.tp_size > 1 else []))
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.sumsq_part = torch.zeros(1, dtype=torch.float32, device=dev)
        self.coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.skip = torch.zeros(1, dtype=torch.int32, device=dev)

    @staticmethod
    def _wd_ranges(buf, b, s, e, no_wd_filter):
        """Sub-ranges of [s, e) as (lo, hi, weight-decay multiplier, learning-rate group): 1-D params get no weight decay;
        the group is the parameter's ``lr_group`` attribute (0: the run's learning rate; others: see ``step``)."""
        no_wd_filter = no_wd_filter or (lambda p: p.dim() <= 1)
        ranges = []
        items = sorted(((buf.param_offsets[p], p) for p in b.params), key=lambda t: t[0])
        pos = s
        for o, p in items:
            # ends are rounded up to 4 elements (the gap up to the next parameter is zero padding) so that
            # every range can be processed with 16-byte accesses
            lo, hi = max(o, s), min(-(-(o + p.numel()) // 4) * 4, e)
            if lo >= hi:
                continue
            if lo > pos:
                ranges.append((pos, lo, 0.0, 0))  # alignment padding
            ranges.append((lo, hi, 0.0 if no_wd_filter(p) else 1.0, int(getattr(p, "lr_group", 0))))
            pos = hi
        if pos < e:
            ranges.append((pos, e, 0.0, 0))
        # merge neighbours with the same multiplier and group
        merged = []
        for r in ranges:
            if merged and merged[-1][2:] == r[2:] and merged[-1][1] == r[0]:
                merged[-1] = (merged[-1][0], r[1], r[2], r[3])
            else:
                merged.append(r)
        return merged

    @staticmethod
    def _tp_duplicate_ranges(buf, b, s, e):
        """Sub-ranges of [s, e) that belong to parameters replicated over the tensor-parallel ranks."""
        out = []
        for p in b.params:
            if getattr(p, "tensor_model_parallel", False) or getattr(p, "is_expert", False):
                continue
            o = buf.param_offsets[p]
            lo, hi = max(o, s), min(o + p.numel(), e)
            if lo < hi:
                out.append((lo, hi))
        return sorted(out)

    def _discount_tp_duplicates(self):
        """sumsq -= (tp - 1) / tp * (squared sum of the tensor-parallel duplicates in the local shards)."""
        if self.tp_size == 1 or not any(st["dup_ranges"] for st in self.state):
            return
        self.sumsq_part.zero_()
        for st in self.state:
            for lo, hi in st["dup_ranges"]:
                optim_ops.sumsq_(st["buf"].grad_data[lo:hi], self.sumsq_part, accumulate=True)
        self.sumsq.add_(self.sumsq_part, alpha=-(self.tp_size - 1) / self.tp_size)

    def _reduce_sumsq(self):
        """Adds the squared sums over the ranks that hold disjoint parts of the gradients."""
        if self.buffers[0].dp_size > 1 and self.buffers[0].use_distributed_optimizer:
            dist.all_reduce(self.sumsq, group=self.buffers[0].dp_group)
        for g in self.norm_groups:
            dist.all_reduce(self.sumsq, group=g)

    # ------------------------------------------------------------------
    def compute_grad_norm(self):
        """Global L2 norm of the (already reduced) gradients, left on the device."""
        self.sumsq.zero_()
        self.skip.zero_()
        if self.sanitize_grads:
            # non-finite gradient entries become zero before the norm and the non-finite check see them: the affected
            # elements simply get no update this step (the reference's SFT gradient sanitiser,
            # primus/backends/megatron/patches/sft_grad_sanitize_patches.py:40-60)
            for st in self.state:
                g = st["buf"].grad_data[st["s"]:st["e"]]
                self.sanitized_count += (~torch.isfinite(g)).sum()
                torch.nan_to_num_(g, nan=0.0, posinf=0.0, neginf=0.0)
        expert_sep = self.expert_norm_group is not None and any(
            not st["buf"].use_distributed_optimizer and self._is_expert_buffer(st["buf"]) for st in self.state)
        if expert_sep:
            self.sumsq_part.zero_()
        for st in self.state:
            g = st["buf"].grad_data[st["s"]:st["e"]]
            sep = expert_sep and not st["buf"].use_distributed_optimizer and self._is_expert_buffer(st["buf"])
            optim_ops.sumsq_(g, self.sumsq_part if sep else self.sumsq, accumulate=True)
        if expert_sep:
            dist.all_reduce(self.sumsq_part, group=self.expert_norm_group)
            self.sumsq.add_(self.sumsq_part)
        self._discount_tp_duplicates()
        self._reduce_sumsq()
        if self.check_for_nan:
            self.skip.copy_((~torch.isfinite(self.sumsq)).to(torch.int32))
        if self.grad_spike_threshold and self.grad_spike_threshold > 0:
            # a gradient-norm spike is treated like a non-finite step: nothing is updated (device-side, no host sync)
            spike = (self.sumsq > float(self.grad_spike_threshold) ** 2).to(torch.int32)
            self.skip.copy_(torch.maximum(self.skip, spike))
        optim_ops.clip_coef_(self.sumsq, self.clip_grad if self.clip_grad else 0.0, self.coef, self.grad_norm)
        return self.grad_norm

    @staticmethod
    def _is_expert_buffer(buf) -> bool:
        return bool(getattr(buf.params[0], "is_expert", False))

    def _fused_step(self, lr: float, wd: float):
        """Reduce-scatter, clip and AdamW + all-gather through peer memory (``csrc/dp_fused.cu``)."""
        import ctypes

        from ..ops import _lib
        from ..ops.fused import scratch

        # the reduce-scatter of every bucket has been issued by ``finish_grad_sync`` (or, overlapped, by the gradient
        # hooks of the last micro-batch) and left this rank's reduced shards in place
        self.sumsq.zero_()
        self.skip.zero_()
        for st in self.state:
            buf = st["buf"]
            if not buf.symmetric:
                optim_ops.sumsq_(buf.grad_data[st["s"]:st["e"]], self.sumsq, accumulate=True)
        for buf in self.buffers:
            if buf.symmetric:
                self.sumsq.add_(buf.fused_sumsq)
                buf.sym_grad.barrier(1)  # everybody has read this rank's gradients: they may be zeroed again
        self._discount_tp_duplicates()
        self._reduce_sumsq()
        if self.check_for_nan:
            self.skip.copy_((~torch.isfinite(self.sumsq)).to(torch.int32))
        optim_ops.clip_coef_(self.sumsq, self.clip_grad if self.clip_grad else 0.0, self.coef, self.grad_norm)
        bc1 = 1.0 - self.betas[0] ** self.step_count
        bc2 = 1.0 - self.betas[1] ** self.step_count
        base_lr = lr
        for st in self.state:
            buf = st["buf"]
            tbl = (ctypes.c_long * buf.dp_size)(*[buf.sym_param.peer_ptr(r) for r in range(buf.dp_size)]) \
                if buf.symmetric else None
            for lo, hi, mult, grp in st["wd_ranges"]:
                lr = self._group_lr.get(grp, base_lr)
                hi4 = min(-(-hi // 4) * 4, st["e"])  # ranges end on parameter boundaries; padding follows
                a, b_ = lo - st["s"], hi4 - st["s"]
                if buf.symmetric and not buf.copy_engine_gather:
                    _lib.call("dp_adamw_allgather", tbl, buf.dp_size, buf.dp_rank, lo, hi4 - lo, st["master"][a:b_],
                              st["m"][a:b_], st["v"][a:b_], buf.grad_data[lo:hi4], float(lr), float(self.betas[0]),
                              float(self.betas[1]), float(self.eps), float(wd * mult), float(bc1), float(bc2),
                              self.coef, self.skip)
                else:
                    optim_ops.adamw_step_(st["master"][a:b_], st["m"][a:b_], st["v"][a:b_], buf.grad_data[lo:hi4],
                                          buf.param_data[lo:hi4], lr=lr, beta1=self.betas[0], beta2=self.betas[1],
                                          eps=self.eps, weight_decay=wd * mult, step=self.step_count,
                                          grad_scale=self.coef, skip=self.skip)
        # a de-oscillation window that closes here may rewrite elements of the local shards (every rank closes its
        # windows on the same step): pulled shards are read after it anyway, pushed ones are gathered once more
        snapped = self.deosc.run(self) if self.deosc is not None else False
        for buf in self.buffers:
            if buf.symmetric and buf.copy_engine_gather:
                buf.start_param_sync_copy_engine()
                if not self.overlap_param_gather:
                    buf.finish_param_sync()
            elif buf.symmetric:
                buf.sym_param.barrier(0)  # all parameter shards have landed everywhere
                if snapped:
                    buf.start_param_sync(async_op=False)
                    buf.finish_param_sync()
            else:
                buf.start_param_sync(async_op=False)
                buf.finish_param_sync()
        return self.grad_norm

    def step(self, lr: Optional[float] = None, weight_decay: Optional[float] = None, group_lr: Optional[dict] = None):
        """``group_lr``: learning rates of the parameters whose ``lr_group`` attribute is not 0 (``{group: lr}``;
        embeddings / output layer under ``decoupled_lr``, the head under ``head_lr_mult``)."""
        self._group_lr = dict(group_lr or {})
        lr = self.lr if lr is None else lr
        wd = self.weight_decay if weight_decay is None else weight_decay
        self.step_count += 1
        from ..ops import gemm as _gemm

        _gemm.bump_weight_generation()   # parameters change in place below: quantised copies expire
        if any(buf.symmetric and buf.odc is None for buf in self.buffers):
            return self._fused_step(lr, wd)
        if self.post_validation and self.norm_groups:
            return self._post_validated_step(lr, wd)
        self.compute_grad_norm()
        self._apply_adamw(lr, wd)
        if self.deosc is not None:
            self.deosc.run(self)
        for buf in self.buffers:
            buf.start_param_sync(async_op=self.overlap_param_gather)
            if not self.overlap_param_gather:
                buf.finish_param_sync()
        return self.grad_norm

    def _apply_adamw(self, lr: float, wd: float):
        base_lr = lr
        for st in self.state:
            buf = st["buf"]
            for lo, hi, mult, grp in st["wd_ranges"]:
                lr = self._group_lr.get(grp, base_lr)
                a, b_ = lo - st["s"], hi - st["s"]
                out = buf.param_data[lo:hi] if buf.param_dtype == torch.bfloat16 else None
                optim_ops.adamw_step_(st["master"][a:b_], st["m"][a:b_], st["v"][a:b_], buf.grad_data[lo:hi], out,
                                      lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                                      weight_decay=wd * mult, step=self.step_count, grad_scale=self.coef,
                                      skip=self.skip)
                if out is None:
                    buf.param_data[lo:hi].copy_(st["master"][a:b_])

    def _post_validated_step(self, lr: float, wd: float):
        """Optimizer step for pipeline schedules whose stages finish at different times (zero-bubble family).

        The global gradient norm and the non-finite check need a reduction over the tensor x pipeline ranks, in which
        early stages would sit idle until the last stage has finished its backward passes.  Here every rank updates
        right away with its *local* information (no clipping, no skip), starts the reduction asynchronously, and
        validates when it arrives: if the step had to be clipped or skipped after all, the state is restored and the
        update is redone with the global coefficient.  ``post_validation_exact``: restore from a snapshot of the shards
        (bit-identical to the plain step, costs a copy of the optimizer state while the reduction is in flight);
        otherwise the update is inverted algebraically (no extra memory, the restored values differ in the last bits).
        Role of the reference's post-validation optimizer for its zero-bubble schedules
        (primus/backends/megatron/core/optimizer/zbpp_optimizer.py:120-246; keys ``enable_optimizer_post_validation``,
        ``enable_exactly_numeric_match`` of primus/configs/modules/megatron/zero_bubble.yaml)."""
        self.sumsq.zero_()
        self.skip.zero_()
        for st in self.state:
            optim_ops.sumsq_(st["buf"].grad_data[st["s"]:st["e"]], self.sumsq, accumulate=True)
        self._discount_tp_duplicates()
        if self.buffers[0].dp_size > 1 and self.buffers[0].use_distributed_optimizer:
            dist.all_reduce(self.sumsq, group=self.buffers[0].dp_group)
        handles = [dist.all_reduce(self.sumsq, group=g, async_op=True) for g in self.norm_groups[:1]]
        snap = [(st["master"].clone(), st["m"].clone(), st["v"].clone()) for st in self.state] \
            if self.post_validation_exact else None
        self.coef.fill_(1.0)
        self._apply_adamw(lr, wd)                      # optimistic: as if the norm were below the clip threshold
        for h in handles:
            h.wait()
        for g in self.norm_groups[1:]:
            dist.all_reduce(self.sumsq, group=g)
        if self.check_for_nan:
            self.skip.copy_((~torch.isfinite(self.sumsq)).to(torch.int32))
        if self.grad_spike_threshold and self.grad_spike_threshold > 0:
            self.skip.copy_(torch.maximum(self.skip, (self.sumsq > float(self.grad_spike_threshold) ** 2).to(torch.int32)))
        optim_ops.clip_coef_(self.sumsq, self.clip_grad if self.clip_grad else 0.0, self.coef, self.grad_norm)
        redo = bool(self.skip.item()) or float(self.coef.item()) < 1.0      # the validation: one scalar read
        if redo:
            self.post_validation_redos += 1
            if snap is not None:
                for st, (ma, m, v) in zip(self.state, snap):
                    st["master"].copy_(ma)
                    st["m"].copy_(m)
                    st["v"].copy_(v)
            else:
                self._invert_adamw(lr, wd)
            self._apply_adamw(lr, wd)                  # the kernels read the global coefficient / skip flag now
        if self.deosc is not None:
            self.deosc.run(self)
        for buf in self.buffers:
            buf.start_param_sync(async_op=self.overlap_param_gather)
            if not self.overlap_param_gather:
                buf.finish_param_sync()
        return self.grad_norm

    def _invert_adamw(self, lr: float, wd: float):
        """Undo one un-clipped AdamW update of ``_apply_adamw`` from the gradients that produced it."""
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        base_lr = lr
        for st in self.state:
            buf = st["buf"]
            for lo, hi, mult, grp in st["wd_ranges"]:
                lr = self._group_lr.get(grp, base_lr)
                a, b_ = lo - st["s"], hi - st["s"]
                g = buf.grad_data[lo:hi].float()
                m, v, p = st["m"][a:b_].float(), st["v"][a:b_].float(), st["master"][a:b_]
                upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
                p.add_(upd, alpha=lr).div_(1.0 - lr * wd * mult)
                st["m"][a:b_].copy_((m - (1 - b1) * g) / b1)
                st["v"][a:b_].copy_(((v - (1 - b2) * g * g) / b2).clamp_(min=0.0))

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        return {"step": self.step_count,
                "shards": [dict(master=s["master"], exp_avg=s["m"], exp_avg_sq=s["v"], start=s["s"], end=s["e"])
                           for s in self.state]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for s, t in zip(self.state, sd["shards"]):
            s["master"].copy_(t["master"])
            s["m"].copy_(t["exp_avg"])
            s["v"].copy_(t["exp_avg_sq"])
