"""Iteration-time projection: per-layer compute (roofline with measured kernel efficiencies) + parallelism
communication (analytic collective model) + pipeline-schedule simulation + optimizer step, for a single
node or projected to ``target_nodes``.

Structure of the reference's performance projection (primus/core/projection/performance_projection/
projection.py, simulator.py:161-352; per-layer comm estimates module_profilers/transformer_layer.py:91-276;
DP / optimizer model module_profilers/optimizer.py:54-126): layer times are either *simulated* from
FLOPs and bytes (default here: efficiencies measured on B200 for this framework's kernels) or *benchmarked*
by timing the real layer on the available GPU (``--benchmark``), then fed to the pipeline simulator over the
same schedule tables the runtime executes.
"""
from __future__ import annotations

from dataclasses import dataclass

from ...engine.schedules import model_flops_per_token
from ...parallel import pipeline_schedules as pps
from .collective_model import CollectiveModel, Hardware
from .memory import ParallelPlan, param_counts

# Throughputs of this package's kernels on B200 *inside a training step* (sustained, power-capped, operands from
# DRAM), as fractions of the measured bf16 burst peak of the hardware profile (1649 TFLOP/s) resp. of the measured
# copy bandwidth (6551 GB/s).  Sources: profiles/gemm_mxfp8_8192x4096x4096.md (sustained, rotating operands),
# profiles/gemm_bf16_8192x4096x4096.md, the per-kernel times of a profiled Llama-3.1-8B step
# (attention 0.575 ms forward / 2.65 ms backward per layer and micro-batch at seq 8192; SwiGLU, norm and quantisation
# kernels at roughly half their isolated speed because the SM clock is capped to ~1.6 GHz by the GEMMs around them).
KERNEL_EFF = {
    "bf16": dict(gemm_fprop=0.76, gemm_dgrad=0.76, gemm_wgrad=0.64, attn_fwd=0.63, attn_bwd=0.342, elementwise_bw=0.466,
                 quant_passes=0.0),
    # MXFP8 linears inside a step: 2.3 PFLOP/s fprop / dgrad, 2.0 wgrad + fp32 accumulate; attention and the LM head
    # stay bf16; every linear input is quantised in a separate pass (bf16 read, two fp8 copies written)
    "mxfp8": dict(gemm_fprop=1.41, gemm_dgrad=1.41, gemm_wgrad=1.21, attn_fwd=0.63, attn_bwd=0.342, elementwise_bw=0.466,
                  quant_passes=1.0),
}
KERNEL_EFF["tensorwise"] = dict(KERNEL_EFF["mxfp8"], quant_passes=1.5)   # + one maximum reduction per quantised tensor
# the LM head (one very large bf16 GEMM per pass: 1.49 / 1.43 / 1.34 PFLOP/s inside a step)
GEMM_EFF, GEMM_DGRAD_EFF, GEMM_WGRAD_EFF = 0.90, 0.87, 0.81
ELEMENTWISE_BW_EFF = KERNEL_EFF["bf16"]["elementwise_bw"]
# whole step over the sum of its kernels (launch gaps, allocator, small optimizer-side kernels): the fit above already
# reproduces the measured Llama-3.1-8B step (5514 ms MXFP8, 7486 ms bf16 on one GPU), so no further factor
STEP_OVERHEAD = 1.0


@dataclass
class LayerTime:
    fwd: float
    bwd_input: float
    bwd_weight: float
    comm_fwd: float = 0.0
    comm_bwd: float = 0.0

    @property
    def total(self):
        return self.fwd + self.bwd_input + self.bwd_weight + self.comm_fwd + self.comm_bwd


def layer_time(cfg, plan: ParallelPlan, hw: Hardware, moe: bool, coll: CollectiveModel, comm_overlap: float = 0.0,
               precision: str = "bf16") -> LayerTime:
    eff = KERNEL_EFF[precision]
    T = plan.micro_batch * plan.seq / plan.cp
    h = cfg.hidden_size
    peak = hw.bf16_tflops * 1e12
    if cfg.multi_latent_attention:
        nh = cfg.num_attention_heads
        qd = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim
        lin = (h * cfg.q_lora_rank + cfg.q_lora_rank * nh * qd) if cfg.q_lora_rank else h * nh * qd
        lin += h * (cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim) + cfg.kv_lora_rank * nh * (cfg.qk_head_dim + cfg.v_head_dim)
        lin += nh * cfg.v_head_dim * h
        attn_fl = 2.0 * T * plan.seq * nh * (qd + cfg.v_head_dim) / 2
    else:
        lin = h * cfg.qkv_width + cfg.num_attention_heads * cfg.kv_channels * h
        attn_fl = 4.0 * T * plan.seq * cfg.num_attention_heads * cfg.kv_channels / 2
    lin /= plan.tp
    attn_fl /= plan.tp
    if moe:
        mlp = cfg.moe_router_topk * 3 * h * cfg.moe_ffn_hidden_size * 1.1 + h * cfg.num_experts
        if cfg.moe_shared_expert_intermediate_size:
            mlp += 3 * h * cfg.moe_shared_expert_intermediate_size
    else:
        mlp = 3 * h * cfg.ffn_hidden_size / plan.tp
    gemm_fl = 2.0 * T * (lin + mlp)
    # memory-bound part: norms, rope, swiglu, residuals ~ 14 passes over T x h plus 6 over T x ffn
    ffn_w = (cfg.moe_ffn_hidden_size * cfg.moe_router_topk) if moe else cfg.ffn_hidden_size / plan.tp
    ew_bytes = (14 * T * h / (plan.tp if plan.sequence_parallel else 1) + 6 * T * ffn_w) * 2.0
    # quantisation passes of the fp8 recipes: forward x (QKV, FC1 inputs) and the attention output, backward the
    # three incoming gradients of width h and the FC1 gradient; 4 bytes per element moved (bf16 in, two fp8 out)
    q_fwd = eff["quant_passes"] * (3 * T * h + 0 * ffn_w) * 4.0
    q_bwd = eff["quant_passes"] * (3 * T * h + cfg.qkv_width / plan.tp * T) * 4.0
    bw = hw.hbm_gbs * 1e9 * eff["elementwise_bw"]
    ew = ew_bytes / bw
    fwd = gemm_fl / (peak * eff["gemm_fprop"]) + attn_fl / (peak * eff["attn_fwd"]) + ew + q_fwd / bw
    bwd_in = gemm_fl / (peak * eff["gemm_dgrad"]) + 2.5 * attn_fl / (peak * eff["attn_bwd"]) + 1.5 * ew + q_bwd / bw
    bwd_w = gemm_fl / (peak * eff["gemm_wgrad"])
    cf = cb = 0.0
    if plan.tp > 1:
        act = T * h * 2.0
        per = (coll.all_gather(act, plan.tp) + coll.reduce_scatter(act, plan.tp)) if plan.sequence_parallel \
            else coll.all_reduce(act, plan.tp)
        cf += 2 * per
        cb += 2 * per + (2 * coll.all_gather(act, plan.tp) if plan.sequence_parallel else 0.0)
    if moe and plan.ep > 1:
        a2a = coll.all_to_all(T * cfg.moe_router_topk * h * 2.0, plan.ep)
        cf += 2 * a2a
        cb += 2 * a2a
    if plan.cp > 1:
        a2a = coll.all_to_all(T * cfg.qkv_width / plan.tp * 2.0, plan.cp)
        cf += 2 * a2a
        cb += 2 * a2a
    keep = 1.0 - comm_overlap
    return LayerTime(fwd, bwd_in, bwd_w, cf * keep, cb * keep)


def project_performance(cfg, plan: ParallelPlan, hw: Hardware, schedule: str = "1f1b", target_nodes: int | None = None,
                        comm_overlap: float = 0.0, layer_times: dict | None = None, precision: str | None = None) -> dict:
    """Returns iteration time, tokens/s/GPU, TFLOP/s/GPU, MFU and the component breakdown.  ``precision``: ``bf16`` |
    ``mxfp8`` | ``tensorwise`` (default: the model configuration's fp8 recipe)."""
    if precision is None:
        precision = (cfg.fp8_recipe if cfg.fp8_recipe in KERNEL_EFF else "mxfp8") if getattr(cfg, "fp8", None) else "bf16"
    world = plan.world if target_nodes is None else target_nodes * hw.gpus_per_node
    plan = ParallelPlan(**{**plan.__dict__, "world": world})
    coll = CollectiveModel(hw)
    lt_dense = layer_time(cfg, plan, hw, False, coll, comm_overlap, precision)
    lt_moe = layer_time(cfg, plan, hw, True, coll, comm_overlap, precision) if cfg.num_experts else lt_dense
    if layer_times:  # benchmark-anchored: replace compute terms
        for lt, key in ((lt_dense, "dense"), (lt_moe, "moe")):
            if key in layer_times:
                lt.fwd, lt.bwd_input, lt.bwd_weight = layer_times[key]
    L = cfg.num_layers
    chunks = 2 if schedule in ("zbv", "v-half", "v-min", "zbv-formatted") else plan.vpp
    stages = plan.pp * chunks
    per_stage = -(-L // stages)         # the slowest stage; a shorter last stage takes the remainder of an uneven depth
    T = plan.micro_batch * plan.seq / plan.cp
    peak = hw.bf16_tflops * 1e12
    head = 2.0 * T * cfg.hidden_size * cfg.padded_vocab_size / plan.tp
    head_fwd = head / (peak * GEMM_EFF) + T * cfg.padded_vocab_size / plan.tp * 2.0 * 3 / (hw.hbm_gbs * 1e9 * ELEMENTWISE_BW_EFF)
    head_bwd = head / (peak * GEMM_DGRAD_EFF) + head / (peak * GEMM_WGRAD_EFF)
    # stage costs (slowest stage drives the pipeline): mix of dense / moe layers in proportion
    n_moe = sum(1 for i in range(L) if cfg.is_moe_layer(i))
    frac_moe = n_moe / L
    def mix(a, b): return a * (1 - frac_moe) + b * frac_moe
    f = per_stage * (mix(lt_dense.fwd, lt_moe.fwd) + mix(lt_dense.comm_fwd, lt_moe.comm_fwd))
    b = per_stage * (mix(lt_dense.bwd_input, lt_moe.bwd_input) + mix(lt_dense.comm_bwd, lt_moe.comm_bwd))
    w = per_stage * mix(lt_dense.bwd_weight, lt_moe.bwd_weight)
    # fully recomputed layers run their forward pass (and its communication) a second time inside backward
    rec = min(plan.recompute_layers, per_stage)
    b += rec * (mix(lt_dense.fwd, lt_moe.fwd) + mix(lt_dense.comm_fwd, lt_moe.comm_fwd))
    f_last, b_last, w_last = f + head_fwd, b + head_bwd * 0.5, w + head_bwd * 0.5
    m = plan.grad_accum
    if plan.pp > 1:
        sch = pps.build_schedule(schedule, plan.pp, m, plan.vpp if plan.vpp > 1 else None)
        p2p = coll.send_recv(T / (plan.tp if plan.sequence_parallel else 1) * cfg.hidden_size * 2.0 * 2,
                             inter_node=(plan.tp * plan.cp * plan.dp >= hw.gpus_per_node))
        sim = pps.simulate(sch["table"], plan.pp, sch["chunks"], sch["placement"], f, b, w, p2p)
        pipe = sim["makespan"] + (head_fwd + head_bwd)  # head runs once per micro-batch on the last stage
        bubble = sim["bubble_fraction"]
    else:
        pipe = m * (f_last + b_last + w_last)
        bubble = 0.0
    pipe *= STEP_OVERHEAD
    # data parallel gradient reduce-scatter + parameter all-gather (distributed optimizer) and the update
    pc = param_counts(cfg)
    dense_params = (sum(l["dense"] for l in pc["layers"]) / plan.pp + pc["embedding"] + pc["output"]) / plan.tp
    expert_params = sum(l["expert"] for l in pc["layers"]) / plan.pp / plan.ep
    dp = plan.dp * plan.cp
    edp = max(1, (plan.tp * plan.cp * plan.dp) // plan.ep)
    if plan.distributed_optimizer:
        dp_comm = coll.reduce_scatter(dense_params * 4.0, dp) + coll.all_gather(dense_params * 2.0, dp)
        dp_comm += coll.reduce_scatter(expert_params * 4.0, edp) + coll.all_gather(expert_params * 2.0, edp)
        opt_elems = dense_params / dp + expert_params / edp
    else:
        dp_comm = coll.all_reduce(dense_params * 4.0, dp) + coll.all_reduce(expert_params * 4.0, edp)
        opt_elems = dense_params + expert_params
    optimizer = opt_elems * 30.0 / (hw.hbm_gbs * 1e9 * ELEMENTWISE_BW_EFF) + (dense_params + expert_params) * 4.0 / (
        hw.hbm_gbs * 1e9)  # update (read p,m,v,g; write p,m,v,bf16) + grad-buffer zeroing
    # The bucket reductions hide in the last micro-batch's backward and the parameter all-gather in the next forward:
    # measured on 8 GPUs, halving the bytes and hiding the gather moved the step by 0.4 %.  What a synchronous step
    # does pay is the spread of sustained clocks between the chips of a node (~2 % at 8 GPUs)
    dp_exposed = dp_comm * (0.05 if plan.pp == 1 else 0.25)
    rank_skew = 0.02 * pipe * (1.0 - 1.0 / max(world, 1)) / (1.0 - 1.0 / 8.0) if world > 1 else 0.0
    it = pipe + dp_exposed + optimizer + rank_skew
    tokens = plan.global_batch * plan.seq
    tps_gpu = tokens / it / world
    fl_tok = model_flops_per_token(cfg, plan.seq)
    tflops = tps_gpu * fl_tok / 1e12
    return {"iteration_ms": it * 1e3, "tokens_per_s_per_gpu": tps_gpu, "tflops_per_gpu": tflops,
            "mfu": tflops / hw.bf16_tflops, "world": world, "dp": plan.dp, "grad_accum": m,
            "breakdown_ms": {"pipeline": pipe * 1e3, "dp_comm_total": dp_comm * 1e3, "dp_comm_exposed": dp_exposed * 1e3,
                             "optimizer": optimizer * 1e3, "rank_skew": rank_skew * 1e3, "precision": precision, "layer_fwd_dense": lt_dense.fwd * 1e3,
                             "layer_bwd_dense": (lt_dense.bwd_input + lt_dense.bwd_weight) * 1e3,
                             "layer_comm_fwd": mix(lt_dense.comm_fwd, lt_moe.comm_fwd) * 1e3,
                             "layer_comm_bwd": mix(lt_dense.comm_bwd, lt_moe.comm_bwd) * 1e3,
                             "head": (head_fwd + head_bwd) * 1e3},
            "bubble_fraction": bubble, "schedule": schedule}
