"""Per-GPU memory projection for a training configuration.

Accounting follows what the engine actually allocates (``primus_b200/parallel/distributed.py``,
``primus_b200/ops/layers.py``), with the structure of the reference's memory projection
(primus/core/projection/module_profilers/language_model.py:268-368,446-486,535-606;
memory_projection/extrapolation.py:368-440; 5 % safety margin, cli/subcommands/projection.py:106-117):

* parameters: bf16 weight (2 B) + fp32 main grad (4 B) per parameter on the rank, plus fp32 master weight and
  two Adam moments (12 B) divided by the data-parallel size when the distributed optimizer is on;
  dense parameters are sharded by TP and PP, expert parameters by EP and PP;
* activations per layer and micro-batch with the engine's saved set — residual stream (2 x T x h), packed QKV,
  attention output (+ log-sum-exp), FC1 output (2 x ffn) — all bf16, T = micro_batch x seq / (tp x cp);
  a recomputed layer keeps only its input; MoE layers add the permuted expert inputs / FC1 outputs for the
  top-k copies;
* pipeline: a rank holds ``min(pp, GA)`` micro-batches in flight (1F1B), times ``1 + (pp-1)/(pp*vpp)`` for the
  interleaved schedule;
* logits: bf16 ``T x vocab/tp`` (the gradient overwrites them in place) on the last stage;
* communication workspaces (symmetric buffers of the fused TP / EP kernels) and a fixed CUDA-context reserve.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class ParallelPlan:
    world: int = 8
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    vpp: int = 1
    micro_batch: int = 1
    global_batch: int = 128
    seq: int = 8192
    distributed_optimizer: bool = True
    recompute_layers: int = 0        # number of fully recomputed layers per stage
    sequence_parallel: bool = True
    fused_tp: bool = False

    @property
    def dp(self) -> int:
        return max(1, self.world // (self.tp * self.pp * self.cp))

    @property
    def grad_accum(self) -> int:
        return max(1, self.global_batch // (self.micro_batch * self.dp))

    def layers_per_stage(self, num_layers: int) -> int:
        """Layers of every stage but the last (the last one is shorter when the depth has no even split:
        ``decoder_last_pipeline_num_layers``)."""
        return -(-num_layers // (self.pp * self.vpp))

    def last_stage_layers(self, num_layers: int) -> int:
        return num_layers - self.layers_per_stage(num_layers) * (self.pp * self.vpp - 1)

    def validate(self, cfg) -> list[str]:
        errs = []
        if self.world % (self.tp * self.pp * self.cp):
            errs.append("world size not divisible by tp*pp*cp")
        if cfg.num_attention_heads % self.tp or cfg.num_query_groups % self.tp:
            errs.append("attention heads not divisible by tp")
        if cfg.num_layers % (self.pp * self.vpp) and (self.vpp > 1 or self.last_stage_layers(cfg.num_layers) < 1):
            errs.append("layers not divisible by pp*vpp")       # vpp = 1: a shorter last stage takes the remainder
        if cfg.num_experts and (cfg.num_experts % self.ep or (self.tp * self.cp * self.dp) % self.ep):
            errs.append("experts / ranks not divisible by ep")
        if self.global_batch % (self.micro_batch * self.dp):
            errs.append("global batch not divisible by micro batch x dp")
        return errs


def param_counts(cfg) -> dict:
    """Parameter counts split into embedding, output layer, dense-per-layer and expert-per-layer parts."""
    h = cfg.hidden_size
    V = cfg.padded_vocab_size
    if cfg.multi_latent_attention:
        qd = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim
        nh = cfg.num_attention_heads
        attn = (h * cfg.q_lora_rank + cfg.q_lora_rank * nh * qd) if cfg.q_lora_rank else h * nh * qd
        attn += h * (cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim) + cfg.kv_lora_rank * nh * (cfg.qk_head_dim + cfg.v_head_dim)
        attn += nh * cfg.v_head_dim * h
    else:
        attn = h * cfg.qkv_width + cfg.num_attention_heads * cfg.kv_channels * h
    dense_mlp = 3 * h * cfg.ffn_hidden_size
    expert = 3 * h * (cfg.moe_ffn_hidden_size or 0)
    shared = 3 * h * (cfg.moe_shared_expert_intermediate_size or 0)
    layers = []
    for i in range(cfg.num_layers):
        if cfg.is_moe_layer(i):
            layers.append({"dense": attn + shared + h * cfg.num_experts + 2 * h, "expert": expert * cfg.num_experts})
        else:
            layers.append({"dense": attn + dense_mlp + 2 * h, "expert": 0})
    return {"embedding": V * h, "output": V * h if cfg.untie_embeddings_and_output_weights else 0, "layers": layers}


def layer_activation_bytes(cfg, plan: ParallelPlan, moe: bool) -> float:
    """Saved activations of one (not recomputed) layer for one micro-batch on one rank, bytes."""
    T = plan.micro_batch * plan.seq / plan.cp
    Tsp = T / plan.tp if (plan.sequence_parallel and plan.tp > 1) else T
    h = cfg.hidden_size
    b = 2.0  # bf16
    act = 2 * Tsp * h * b                                        # residual stream before each norm
    if cfg.multi_latent_attention:
        nh = cfg.num_attention_heads / plan.tp
        act += T * nh * (2 * (cfg.qk_head_dim + cfg.qk_pos_emb_head_dim) + 2 * cfg.v_head_dim) * b   # q, k, v, out
        act += T * (cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim) * b * 2
    else:
        act += T * cfg.qkv_width / plan.tp * b + T * cfg.num_attention_heads * cfg.kv_channels / plan.tp * b
    act += T * cfg.num_attention_heads / plan.tp * 4             # log-sum-exp
    if moe:
        k = cfg.moe_router_topk
        copies = T * k * 1.15                                    # padding of the expert-major layout
        act += copies * (h + 2 * cfg.moe_ffn_hidden_size + cfg.moe_ffn_hidden_size) * b
        act += T * cfg.num_experts * 4 * 3
        if cfg.moe_shared_expert_intermediate_size:
            act += T * (h + 2 * cfg.moe_shared_expert_intermediate_size) * b
    else:
        act += T * 2 * cfg.ffn_hidden_size / plan.tp * b         # FC1 output (SwiGLU recomputed in backward)
    return act


def project_memory(cfg, plan: ParallelPlan, margin: float = 0.05, context_reserve_gb: float = 1.5) -> dict:
    pc = param_counts(cfg)
    L = cfg.num_layers
    stages = plan.pp * plan.vpp
    per_stage = plan.layers_per_stage(L)
    # worst stage: first (embedding) or last (output layer + logits); take both and report the max
    results = {}
    for which in ("first", "last"):
        idx = list(range(0, per_stage)) if which == "first" else list(range(L - plan.last_stage_layers(L), L))
        layer_sets = [idx]
        if plan.vpp > 1:  # a rank owns vpp chunks; approximate with vpp copies of this stage's layer mix
            layer_sets = [idx] * plan.vpp
        dense = sum(pc["layers"][i]["dense"] for s in layer_sets for i in s) / plan.tp
        expert = sum(pc["layers"][i]["expert"] for s in layer_sets for i in s) / plan.ep
        if which == "first":
            dense += pc["embedding"] / plan.tp
        if which == "last" or plan.pp == 1:
            dense += pc["output"] / plan.tp
        edp = max(1, (plan.tp * plan.cp * plan.dp) // plan.ep)
        opt_div_dense = plan.dp * plan.cp if plan.distributed_optimizer else 1
        opt_div_expert = edp if plan.distributed_optimizer else 1
        weights = (dense + expert) * 2.0
        grads = (dense + expert) * 4.0
        optim = dense * 12.0 / opt_div_dense + expert * 12.0 / opt_div_expert
        n_layers_rank = sum(len(s) for s in layer_sets)
        moe_layers = sum(1 for s in layer_sets for i in s if cfg.is_moe_layer(i))
        rec = min(plan.recompute_layers, n_layers_rank)
        T = plan.micro_batch * plan.seq / plan.cp
        Tsp = T / plan.tp if (plan.sequence_parallel and plan.tp > 1) else T
        act_mb = ((n_layers_rank - moe_layers) * layer_activation_bytes(cfg, plan, False)
                  + (moe_layers * layer_activation_bytes(cfg, plan, True) if moe_layers else 0.0))
        if rec:
            act_mb = act_mb * (n_layers_rank - rec) / n_layers_rank + rec * Tsp * cfg.hidden_size * 2.0
        inflight = min(plan.pp, plan.grad_accum)
        if plan.vpp > 1:
            inflight *= 1.0 + (plan.pp - 1) / (plan.pp * plan.vpp)
        if which == "last" and plan.pp > 1:
            inflight = 1
        acts = act_mb * inflight
        logits = T * cfg.padded_vocab_size / plan.tp * 2.0 if (which == "last" or plan.pp == 1) else 0.0
        work = 0.0
        if plan.fused_tp and plan.tp > 1:
            work += T * max(cfg.hidden_size, 2 * cfg.ffn_hidden_size / plan.tp) * 2.0 * 2
        if plan.ep > 1:
            work += 2 * T * cfg.moe_router_topk * cfg.hidden_size * 2.0
        total = (weights + grads + optim + acts + logits + work) * (1.0 + margin) + context_reserve_gb * 2**30
        results[which] = {"weights_gb": weights / 2**30, "grads_gb": grads / 2**30, "optimizer_gb": optim / 2**30,
                          "activations_gb": acts / 2**30, "logits_gb": logits / 2**30, "workspace_gb": work / 2**30,
                          "total_gb": total / 2**30, "params_on_rank": dense + expert}
    worst = max(results.values(), key=lambda r: r["total_gb"])
    return {"per_stage": results, "peak_gb": worst["total_gb"], "breakdown": worst, "dp": plan.dp,
            "grad_accum": plan.grad_accum}
