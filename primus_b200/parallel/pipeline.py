"""Pipeline-parallel runtime: executes a schedule table (``pipeline_schedules``) on this rank.

Every ``F`` node runs one model chunk on one micro-batch, ``B`` / ``BW`` run its backward, ``W`` runs the
weight-gradient GEMMs that a ``B`` node deferred (``ops.gemm.WGRAD_STORE``), and activations / gradients
travel between neighbouring stages with NCCL (gloo on CPU) point-to-point operations: sends are
asynchronous and complete in the background, receives are posted when the consumer node is reached.
Forward-direction and backward-direction traffic use two separate communicators so that a pending
send in one direction can never block the other (the reference orders even / odd ranks instead:
primus/backends/megatron/core/pipeline_parallel/primuspipe/handlers/communication_handler.py:40-133).
Hand-offs between two chunks that live on the same rank (the fold of a V schedule) stay local.

Counterpart of ``PrimusPipelineParallelLauncher.run`` / ``ScheduleRunner``
(primus/backends/megatron/core/pipeline_parallel/primuspipe/pipeline_launcher.py:141-346,
handlers/fwd_handler.py:40-122, handlers/bwd_handler.py:31-128).
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops
from ..ops import layers as layers_ops
from . import pipeline_schedules as sched
from . import state as ps


class PipelineTimeline:
    """Optional per-node wall-clock record (the data the reference dumps for its pipeline visualiser,
    primus/backends/megatron/core/pipeline_parallel/pp_visualizer.py)."""

    def __init__(self):
        self.events = []

    def add(self, node, t0, t1, compute_start=None, mem_delta=None):
        """``compute_start``: when the node's input had arrived (``start`` .. ``compute_start`` is time spent waiting
        for the neighbouring stage); ``mem_delta``: bytes the node left allocated (activations a forward keeps)."""
        ev = {"kind": node.kind, "mb": node.mb, "chunk": node.chunk, "start": t0, "end": t1,
              "compute_start": t0 if compute_start is None else compute_start}
        if mem_delta is not None:
            ev["mem_delta"] = mem_delta
        self.events.append(ev)

    def dump(self, path: str, pp_rank: int, iteration: int, extra: dict | None = None) -> None:
        """One JSON file per (rank, iteration); ``primus_b200.tools.pp_vis`` merges them."""
        import json
        import os

        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump({"pp_rank": pp_rank, "iteration": iteration, "events": self.events, **(extra or {})}, f)


def _p2p_shape(trainer, batch, seq, model=None):
    """Shape of the tensor the stage held by ``model`` receives (models/gpt.py::handoff_shape)."""
    st = trainer.st
    T = batch * seq
    if trainer.mcfg.sequence_parallel and st.tp > 1:
        T //= st.tp
    if model is not None and hasattr(model, "handoff_shape"):
        return model.handoff_shape(T)
    return (T, trainer.mcfg.hidden_size)


def manual_costs(tc, pp: int, chunks: int):
    """``StageCosts`` from the config's ``pp_cost_f`` / ``pp_cost_b`` / ``pp_cost_w`` (a number for every stage or one per
    virtual stage; missing ones default to 1000 like the reference's heuristic) and ``pp_max_mem`` (activation limit per
    rank in chunk-forwards); None when none of them is set.  (primus/configs/modules/megatron/primus_pipeline.yaml:14-17.)"""
    vals = [getattr(tc, k, None) for k in ("pp_cost_f", "pp_cost_b", "pp_cost_w")]
    mem = getattr(tc, "pp_max_mem", None)
    if all(v is None for v in vals) and mem is None:
        return None
    S = pp * chunks

    def per_stage(v):
        if v is None:
            return [1000.0] * S
        if isinstance(v, (int, float)):
            return [float(v)] * S
        assert len(v) == S, f"pipeline costs: {len(v)} values for {S} virtual stages"
        return [float(x) for x in v]

    limit = None if mem is None else ([float(mem)] * pp if isinstance(mem, (int, float)) else [float(x) for x in mem])
    return sched.StageCosts(per_stage(vals[0]), per_stage(vals[1]), per_stage(vals[2]), 0.0, limit)


def _pos_ids(trainer, mb):
    use = getattr(trainer, "use_position_ids", False) or trainer.st.cp > 1 or getattr(trainer, "num_seq_splits", 1) > 1
    return mb.get("position_ids") if use else None


def run_pipeline_schedule(trainer, micro_batches: list[dict], timeline: PipelineTimeline | None = None,
                          forward_only: bool = False):
    """Executes this rank's row of the schedule table.  ``forward_only`` (evaluation): only the forward nodes run, in
    table order — they depend on forward nodes alone, so the sub-sequence is a valid forward schedule on every rank —
    nothing is kept for a backward pass, and the summed loss is valid on the last stage."""
    st = trainer.st
    pp, r = st.pp, st.pp_rank
    m = len(micro_batches)
    nsplit = getattr(trainer, "num_seq_splits", 1)
    key = (trainer.tcfg.pipeline_schedule, pp, m, st.virtual_pp) if nsplit == 1 else \
        (trainer.tcfg.pipeline_schedule, pp, m, st.virtual_pp, nsplit)
    cache = getattr(trainer, "_pp_schedule_cache", {})
    if key not in cache:   # (a cost-driven table from ``replan_from_measurements`` replaces the entry later)
        algo = trainer.tcfg.pipeline_schedule
        if st.virtual_pp and st.virtual_pp > 1 and algo == "1f1b":
            algo = "interleaved"
        cache[key] = sched.build_schedule(algo, pp, m, st.virtual_pp, num_seq_splits=nsplit)
        manual = manual_costs(trainer.tcfg, pp, cache[key]["chunks"])
        if manual is not None and nsplit == 1 and algo.lower().replace("_", "-") in (
                "zerobubble", "zero-bubble", "zb", "zbv", "zbv-greedy", "zbv-formatted", "v-half", "v-min"):
            # costs given in the config (``pp_cost_f / _b / _w``, ``pp_max_mem``): the cost-driven table from the start
            cache[key] = sched.auto_schedule(algo, pp, m, manual)
        if getattr(trainer.tcfg, "debug_scheduler_table", False) and r == 0 and st.dp_rank == 0 and st.tp_rank == 0:
            rows = ["  ".join(f"{n.kind}{n.mb}" + (f".{n.chunk}" if cache[key]["chunks"] > 1 else "") for n in row)
                    for row in cache[key]["table"]]
            trainer.log("[pipeline] schedule table (one row per rank):\n" + "\n".join(rows))
        trainer._pp_schedule_cache = cache
    sch = cache[key]
    chunks, placement = sch["chunks"], sch["placement"]
    assert chunks == len(trainer.model_chunks), \
        f"schedule {sch['algorithm']} needs {chunks} model chunks per rank, trainer built {len(trainer.model_chunks)}"
    S = pp * chunks
    nodes = sch["table"][r]
    dtype = trainer.mcfg.torch_dtype
    dev = trainer.device
    fwd_g, bwd_g = st.pp_fwd_group, st.pp_bwd_group
    inputs, outputs, local_act, local_grad = {}, {}, {}, {}
    sends = []
    total = trainer.loss_accum
    total.zero_()
    split_w = any(n.kind == "W" for n in nodes)
    for buf in trainer.buffers:
        buf.is_last_microbatch = False

    def global_rank(pp_rank):
        return st.pp_ranks[pp_rank]

    for node in nodes:
        if forward_only and node.kind != "F":
            continue
        t0 = time.perf_counter() if timeline is not None else 0.0
        t_in = None
        mem0 = torch.cuda.memory_allocated(dev) if (timeline is not None and trainer.is_cuda) else 0
        s = sched.stage_of(r, node.chunk, pp, placement)
        mb = micro_batches[node.mb]
        if nsplit > 1:     # this node works on one sequence chunk; attention keeps the earlier chunks' keys and values
            mb = trainer._seq_chunk(mb, node.split)
            if node.kind in ("F", "B", "BW"):
                layers_ops.SEQ_SPLIT.begin((node.mb, node.chunk), node.split, nsplit, forward_only)
        batch, seq = mb["tokens"].shape
        model = trainer.model_chunks[node.chunk]
        if trainer.mcfg.num_hash_layers:    # hash-routed MoE layers index their table with the ids of *this* micro-batch
            from ..models import moe as _moe    # (also when a checkpointed layer runs again inside a backward node)

            _moe.TOKEN_IDS.current = mb["tokens"].reshape(-1)
        k = (node.mb, node.chunk) if nsplit == 1 else (node.mb, node.chunk, node.split)
        if node.kind == "F":
            if s == 0:
                hidden_in = None
            else:
                pr, pc = sched.rank_of_stage(s - 1, pp, placement)
                if pr == r:
                    x = local_act.pop((node.mb, pc))
                else:
                    x = torch.empty(_p2p_shape(trainer, batch, seq, model), dtype=dtype, device=dev)
                    dist.recv(x, src=global_rank(pr), group=fwd_g)
                    if timeline is not None:
                        if trainer.is_cuda:
                            torch.cuda.synchronize()
                        t_in = time.perf_counter()
                if not forward_only:
                    x.requires_grad_(True)
                    inputs[k] = x
                hidden_in = (x, None, batch, seq)
            if s == S - 1:
                w = trainer._loss_weights(mb)
                out = model(mb["tokens"], mb["labels"], loss_weights=w, hidden_in=hidden_in,
                            unit_upstream=True, position_ids=_pos_ids(trainer, mb),
                            cu_seqlens=mb.get("host_cu_seqlens"))
                if not forward_only:
                    outputs[k] = out
                total += out.detach()
            else:
                h, res, _, _ = model(mb["tokens"] if s == 0 else None, hidden_in=hidden_in,
                                     position_ids=_pos_ids(trainer, mb), cu_seqlens=mb.get("host_cu_seqlens"))
                # one tensor per stage boundary: the next stage's first layer only needs the residual stream
                # hidden + residual (its fused add + norm starts from the sum), half the bytes of sending both
                y = model.pack_handoff(h, res) if hasattr(model, "pack_handoff") else (h if res is None else h + res)
                if not forward_only:
                    outputs[k] = y
                nr, nc = sched.rank_of_stage(s + 1, pp, placement)
                if nr == r:
                    local_act[(node.mb, node.chunk)] = y.detach().clone()
                else:
                    sends.append((dist.isend(y.detach(), dst=global_rank(nr), group=fwd_g), y))
        elif node.kind in ("B", "BW"):
            out = outputs.pop(k)
            if split_w and node.kind == "B":
                gemm_ops.WGRAD_STORE.begin(k)
            if s == S - 1:
                out.backward()
            else:
                nr, nc = sched.rank_of_stage(s + 1, pp, placement)
                if nr == r:
                    g = local_grad.pop((node.mb, nc))
                else:
                    g = torch.empty_like(out)
                    dist.recv(g, src=global_rank(nr), group=bwd_g)
                    if timeline is not None:
                        if trainer.is_cuda:
                            torch.cuda.synchronize()
                        t_in = time.perf_counter()
                torch.autograd.backward(out, g)
            if split_w and node.kind == "B":
                gemm_ops.WGRAD_STORE.end()
            if s > 0:
                x = inputs.pop(k)
                pr, pc = sched.rank_of_stage(s - 1, pp, placement)
                if pr == r:
                    local_grad[(node.mb, node.chunk)] = x.grad
                else:
                    sends.append((dist.isend(x.grad, dst=global_rank(pr), group=bwd_g), x.grad))
        elif node.kind == "W":
            gemm_ops.WGRAD_STORE.flush(k)
        if nsplit > 1:
            layers_ops.SEQ_SPLIT.end()
            done = (node.kind == "BW" and node.split == 0) or (forward_only and node.split == nsplit - 1)
            if done:
                layers_ops.SEQ_SPLIT.drop((node.mb, node.chunk))
        if timeline is not None:
            if trainer.is_cuda:
                torch.cuda.synchronize()
            mem1 = torch.cuda.memory_allocated(dev) if trainer.is_cuda else 0
            timeline.add(node, t0, time.perf_counter(), t_in, (mem1 - mem0) if trainer.is_cuda else None)
    for h, _keep in sends:
        h.wait()
    if nsplit > 1:
        layers_ops.SEQ_SPLIT.clear()
    gemm_ops.WGRAD_STORE.flush_all()
    for buf in trainer.buffers:
        buf.is_last_microbatch = True
    return total


def replan_from_measurements(trainer, events: list[dict], num_microbatches: int, log=None) -> dict | None:
    """Cost-driven re-planning of a B / W-split schedule: gathers the timeline events every pipeline rank recorded in
    the measurement window, derives per-stage F / B / W times (waiting for the neighbour excluded) and, on GPUs, an
    activation budget from the bytes a forward leaves allocated and the memory still free under
    ``zero_bubble_adaptive_memory_limit_percentile`` of the device, and installs the table ``auto_schedule`` picks for
    the following iterations.  Every rank computes the same table from the same gathered data.  Returns the
    scheduler's report (None when the schedule has no B / W split).  Role of the reference's zero-bubble runtime
    timers + scheduler (primus/backends/megatron/core/pipeline_parallel/zerobubble/runtime.py,
    scheduler/{zb,zbv}.py: ``zero_bubble_pipeline_timers_start_iter / end_iter``,
    ``zero_bubble_adaptive_memory_limit_percentile``, ``zero_bubble_max_pending_backward``)."""
    st = trainer.st
    pp, m = st.pp, num_microbatches
    algo = trainer.tcfg.pipeline_schedule.lower().replace("_", "-")
    if algo not in ("zerobubble", "zero-bubble", "zb", "zbb", "zbv", "zbv-formatted", "zbv-greedy", "v-half", "v-min"):
        return None
    chunks, placement, base = sched.default_budget(algo, pp)
    mine = {"events": events, "limit": None}
    if trainer.is_cuda:
        fwd = [e["mem_delta"] for e in events if e["kind"] == "F" and e.get("mem_delta", 0) > 0]
        if fwd:
            act = sum(fwd) / len(fwd)
            total = torch.cuda.get_device_properties(trainer.device).total_memory
            pct = float(getattr(trainer.tcfg, "zero_bubble_adaptive_memory_limit_percentile", 85)) / 100.0
            peak = torch.cuda.max_memory_allocated(trainer.device)
            # what the measured steps needed beyond their activations stays reserved; the rest may hold activations
            static = max(0.0, peak - base[st.pp_rank] * act)
            mine["limit"] = max(float(chunks) + 1.0, (pct * total - static) / act)
    gathered = [None] * pp
    dist.all_gather_object(gathered, mine, group=st.pp_group)
    costs = sched.costs_from_events([g["events"] for g in gathered], pp, chunks, placement)
    if all(g["limit"] is not None for g in gathered):
        costs.mem_limit = [float(g["limit"]) for g in gathered]
    manual = getattr(trainer.tcfg, "zero_bubble_max_pending_backward", "auto")
    if manual not in (None, "auto"):       # manual activation budget, in forwards per rank
        costs.mem_limit = [float(int(manual))] * pp
    report = sched.auto_schedule(algo, pp, m, costs)
    cache = getattr(trainer, "_pp_schedule_cache", {})
    cache[(trainer.tcfg.pipeline_schedule, pp, m, st.virtual_pp)] = report
    trainer._pp_schedule_cache = cache
    if log is not None:
        log(f"[pipeline] cost-driven schedule: {report['picked']}; simulated step {report['makespan']:.4g} vs "
            f"{report['fixed_makespan']:.4g} for the fixed table (F {[round(x, 4) for x in costs.f]}, "
            f"B {[round(x, 4) for x in costs.b]}, W {[round(x, 4) for x in costs.w]}); peak activations "
            f"{report['peak_activations']}")
    return report


def pipeline_warmup(trainer, micro_batch: dict) -> None:
    """One throw-away forward + backward of every local model chunk on fabricated boundary tensors, all stages at
    the same time (no stage waits for its neighbour), so that the first real iteration does not pay the one-time costs
    (allocator growth, kernel attribute setup, communicator creation by the first tensor-parallel collectives)
    serially along the pipeline.  RNG state is restored and the gradient buffers are zeroed afterwards; no optimizer
    step is taken.  (The reference's pipeline warm-up patch:
    primus/backends/megatron/patches/pp_warmup_patches.py:21-60,286.)"""
    st = trainer.st
    pp = st.pp
    chunks = len(trainer.model_chunks)
    S = pp * chunks
    algo = trainer.tcfg.pipeline_schedule
    if st.virtual_pp and st.virtual_pp > 1 and algo == "1f1b":
        algo = "interleaved"
    placement = sched.build_schedule(algo, pp, max(pp, 2), st.virtual_pp)["placement"]
    dtype, dev = trainer.mcfg.torch_dtype, trainer.device
    cpu_rng = torch.get_rng_state()
    cuda_rng = torch.cuda.get_rng_state(dev) if trainer.is_cuda else None
    from ..ops import gemm as gemm_mod

    gen_before = gemm_mod.weight_generation()
    for buf in trainer.buffers:
        buf.is_last_microbatch = False          # gradients stay local: nothing is reduced or handed to the optimizer
    batch, seq = micro_batch["tokens"].shape
    try:
        for c, model in enumerate(trainer.model_chunks):
            s = sched.stage_of(st.pp_rank, c, pp, placement)
            hidden_in = None
            if s > 0:
                x = torch.randn(_p2p_shape(trainer, batch, seq, model), device=dev).to(dtype) * 0.02
                x.requires_grad_(True)
                hidden_in = (x, None, batch, seq)
            if s == S - 1:
                out = model(micro_batch["tokens"], micro_batch["labels"],
                            loss_weights=trainer._loss_weights(micro_batch), hidden_in=hidden_in, unit_upstream=True,
                            position_ids=_pos_ids(trainer, micro_batch))
                out.backward()
            else:
                h, res, _, _ = model(micro_batch["tokens"] if s == 0 else None, hidden_in=hidden_in,
                                     position_ids=_pos_ids(trainer, micro_batch))
                y = model.pack_handoff(h, res) if hasattr(model, "pack_handoff") else (h if res is None else h + res)
                torch.autograd.backward(y, torch.randn_like(y) * 1e-3)
        gemm_ops.WGRAD_STORE.flush_all()
    finally:
        for buf in trainer.buffers:
            buf.zero_grad()
            buf.is_last_microbatch = True
        for m in trainer.model_chunks:
            for mod in m.modules():
                if hasattr(mod, "last_aux_loss"):
                    mod.last_aux_loss = None
        torch.set_rng_state(cpu_rng)
        if cuda_rng is not None:
            torch.cuda.set_rng_state(cuda_rng, dev)
        assert gemm_mod.weight_generation() == gen_before
