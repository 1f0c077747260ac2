"""Learning-rate / weight-decay schedules and the micro-batch calculator.

Keys and semantics follow the reference's trainer preset
(primus/configs/modules/megatron/trainer_base.yaml:72-118): ``lr``, ``min_lr``, ``lr_decay_style``
(constant | linear | cosine | inverse-square-root | WSD), ``lr_warmup_iters`` / ``lr_warmup_fraction`` /
``lr_warmup_init``, ``lr_decay_iters``, ``lr_wsd_decay_style`` / ``lr_wsd_decay_iters``,
``start_weight_decay`` / ``end_weight_decay`` / ``weight_decay_incr_style``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass
class LRScheduler:
    max_lr: float = 3e-4
    min_lr: float = 0.0
    warmup_iters: int = 0
    warmup_init: float = 0.0
    decay_iters: Optional[int] = None
    decay_style: str = "cosine"
    wsd_decay_iters: int = 0
    wsd_decay_style: str = "exponential"
    start_wd: float = 0.1
    end_wd: float = 0.1
    wd_incr_style: str = "constant"
    num_iters: int = 0

    def get_lr(self, it: Optional[int] = None) -> float:
        it = self.num_iters if it is None else it
        if self.warmup_iters > 0 and it <= self.warmup_iters:
            return self.warmup_init + (self.max_lr - self.warmup_init) * it / self.warmup_iters
        if self.decay_style == "constant" or not self.decay_iters:
            return self.max_lr
        if it > self.decay_iters:
            return self.min_lr
        if self.decay_style == "inverse-square-root":
            w = max(self.warmup_iters, 1)
            return max(self.min_lr, self.max_lr * math.sqrt(w) / math.sqrt(max(it, 1)))
        span = self.decay_iters - self.warmup_iters
        ratio = (it - self.warmup_iters) / max(span, 1)
        delta = self.max_lr - self.min_lr
        if self.decay_style == "linear":
            coeff = 1.0 - ratio
        elif self.decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        elif self.decay_style == "WSD":
            anneal_start = self.decay_iters - self.wsd_decay_iters
            if it <= anneal_start:
                coeff = 1.0
            else:
                r = (it - anneal_start) / max(self.wsd_decay_iters, 1)
                coeff = {"linear": 1.0 - r, "cosine": 0.5 * (math.cos(math.pi * r) + 1.0),
                         "exponential": 2.0 * 0.5 ** r - 1.0}[self.wsd_decay_style]
        else:
            raise ValueError(f"unknown lr_decay_style {self.decay_style}")
        return self.min_lr + coeff * delta

    def get_wd(self, it: Optional[int] = None, total: Optional[int] = None) -> float:
        it = self.num_iters if it is None else it
        total = total or self.decay_iters or 1
        if self.wd_incr_style == "constant" or it > total:
            return self.end_wd
        r = it / total
        if self.wd_incr_style == "linear":
            c = r
        elif self.wd_incr_style == "cosine":
            c = 0.5 * (math.cos(math.pi * (1 - r)) + 1.0)
        else:
            raise ValueError(self.wd_incr_style)
        return self.start_wd + c * (self.end_wd - self.start_wd)

    def step(self, n: int = 1):
        self.num_iters += n

    HYPER = ("max_lr", "min_lr", "warmup_iters", "warmup_init", "decay_iters", "decay_style", "wsd_decay_iters",
             "wsd_decay_style", "start_wd", "end_wd", "wd_incr_style")

    def state_dict(self):
        return {"num_iters": self.num_iters, **{k: getattr(self, k) for k in self.HYPER}}

    def load_state_dict(self, sd, use_checkpoint_values: bool = False, log=None):
        """The position in the schedule always comes from the checkpoint.  The schedule itself is this run's unless
        ``use_checkpoint_values`` (``use_checkpoint_opt_param_scheduler``); differences are reported either way."""
        self.num_iters = sd["num_iters"]
        diff = {k: (sd[k], getattr(self, k)) for k in self.HYPER if k in sd and sd[k] != getattr(self, k)}
        if use_checkpoint_values:
            for k, (saved, _) in diff.items():
                setattr(self, k, saved)
        if diff and log is not None:
            which = "the checkpoint's" if use_checkpoint_values else "this run's"
            log("[scheduler] the checkpoint was written with another schedule (" +
                ", ".join(f"{k}: {a} -> {b}" for k, (a, b) in diff.items()) + f"): using {which} values")


def num_microbatches(global_batch: int, micro_batch: int, dp: int) -> int:
    """GA = GBS / (MBS * DP) (primus/backends/megatron/data_loader_store.py:17,26)."""
    if global_batch % (micro_batch * dp):
        raise ValueError(f"global batch {global_batch} not divisible by micro batch {micro_batch} x dp {dp}")
    return global_batch // (micro_batch * dp)


def model_flops_per_token(cfg, seq_len: int, causal_half: bool = False) -> float:
    """Model FLOPs per token for one forward+backward pass (3 x forward), Megatron's accounting:
    2*m*n*k per GEMM, attention scores counted over the full (non-causal) square unless
    ``causal_half``.  This is the numerator of the ``TFLOP/s/GPU`` figure in the training log
    (primus/backends/megatron/patches/training_log/print_rank_last_patches.py:435-466)."""
    h, L, V = cfg.hidden_size, cfg.num_layers, cfg.padded_vocab_size
    fwd = 0.0
    kinds = getattr(cfg, "layer_kinds", None) or [("attention", True)] * L
    for i in range(L):
        mixer, has_mlp = kinds[i]
        if mixer == "conv":            # LFM2 short convolution: in_proj (3h), out_proj, the taps
            fwd += 2 * h * 3 * h + 2 * h * h + 2 * h * cfg.conv_L_cache
            attn = 0.0
        elif mixer == "mamba":         # Mamba-2: projections, convolution, chunked scan (the reference's Zebra-Llama
            # FLOPs patch counts the same terms: primus/backends/megatron/patches/zebra_llama_flops_patches.py)
            di = cfg.mamba_expand * h
            nh = cfg.mamba_num_heads or di // cfg.mamba_head_dim
            conv_dim = di + 2 * cfg.mamba_num_groups * cfg.mamba_state_dim
            fwd += 2 * h * (di + conv_dim + nh) + 2 * di * h + 2 * conv_dim * cfg.mamba_d_conv
            c, n = cfg.mamba_chunk_size, cfg.mamba_state_dim
            fwd += 2 * c * nh * n + 2 * c * di + 4 * di * n       # C B^T and (C B^T) x inside a chunk; state in / out
            attn = 0.0
        elif mixer == "gdn":           # gated delta net: projections, convolution, chunked delta rule
            qk = cfg.linear_num_key_heads * cfg.linear_key_head_dim
            vd = cfg.linear_num_value_heads * cfg.linear_value_head_dim
            conv_dim = 2 * qk + vd
            fwd += 2 * h * (conv_dim + vd + 2 * cfg.linear_num_value_heads) + 2 * vd * h + 2 * conv_dim * cfg.linear_conv_kernel_dim
            c, nv, dk, dv = cfg.linear_chunk_size, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            fwd += nv * (4 * c * dk + 2 * c * c + 2 * c * (dv + dk) + 6 * dk * dv)      # scores, solve, deltas, state
            attn = 0.0
        elif mixer == "v4":            # DeepSeek-V4: low-rank q, one shared latent, grouped low-rank output, compressed branches
            nh, hd = cfg.num_attention_heads, cfg.kv_channels
            fwd += (2 * h * cfg.q_lora_rank + 2 * cfg.q_lora_rank * nh * hd) if cfg.q_lora_rank else 2 * h * nh * hd
            fwd += 2 * h * hd
            fwd += (2 * nh * hd * cfg.o_lora_rank + 2 * cfg.o_groups * cfg.o_lora_rank * h) if cfg.o_lora_rank \
                else 2 * nh * hd * h
            ratio = cfg.compress_ratio_list[i]
            keys = min(cfg.attn_sliding_window or seq_len, seq_len)       # local keys per query
            if ratio == 128:
                fwd += 4 * h * hd
                keys += seq_len / ratio * (0.5 if causal_half else 1.0)
            elif ratio == 4:
                fwd += 8 * h * hd + 2 * h * (cfg.index_head_dim + cfg.index_n_heads) \
                    + 2 * cfg.index_n_heads * cfg.index_head_dim ** 2 + 8 * h * cfg.index_head_dim
                fwd += 2 * cfg.index_n_heads * cfg.index_head_dim * seq_len / ratio * (0.5 if causal_half else 1.0)
                keys += min(cfg.index_topk, seq_len // ratio)
            fwd += 4 * nh * hd * keys
            attn = 0.0
        elif mixer == "kda":           # Kimi delta attention: projections, gate bottleneck, convolution, chunked rule
            nh, dk, dv = cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            qk, vd = nh * dk, nh * dv
            conv_dim = 2 * qk + vd
            fwd += 2 * h * (conv_dim + vd + dk + nh) + 2 * dk * qk + 2 * vd * h + 2 * conv_dim * cfg.linear_conv_kernel_dim
            c = cfg.kda_chunk_size
            fwd += nh * (4 * c * dk + 2 * c * c + 2 * c * (dv + dk) + 6 * dk * dv)
            attn = 0.0
        elif mixer is None:
            attn = 0.0
        elif cfg.multi_latent_attention:
            qd = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim
            nh = cfg.num_attention_heads
            if cfg.q_lora_rank:
                fwd += 2 * h * cfg.q_lora_rank + 2 * cfg.q_lora_rank * nh * qd
            else:
                fwd += 2 * h * nh * qd
            fwd += 2 * h * (cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim)
            fwd += 2 * cfg.kv_lora_rank * nh * (cfg.qk_head_dim + cfg.v_head_dim)
            fwd += 2 * nh * cfg.v_head_dim * h
            if getattr(cfg, "mla_use_output_gate", False):
                fwd += 2 * h * nh * cfg.v_head_dim
            attn = 2 * seq_len * nh * (qd + cfg.v_head_dim)
        else:
            fwd += 2 * h * cfg.qkv_width + 2 * cfg.num_attention_heads * cfg.kv_channels * h
            if cfg.attention_output_gate:
                fwd += 2 * h * cfg.num_attention_heads * cfg.kv_channels
            attn = 4 * seq_len * cfg.num_attention_heads * cfg.kv_channels
        fwd += attn * (0.5 if causal_half else 1.0)
        if getattr(cfg, "hc_mult", 1) > 1:          # two hyper-connection mixers: the projection of the flattened streams
            K = cfg.hc_mult
            fwd += 2 * 2 * K * h * (2 + K) * K + 2 * 4 * K * K * h
        if not has_mlp:
            continue
        if cfg.is_moe_layer(i):
            fwd += 2 * h * cfg.num_experts
            lat = getattr(cfg, "routed_expert_hidden_size", None) or h      # latent experts + the two shared projections
            fwd += cfg.moe_router_topk * 6 * lat * cfg.moe_ffn_hidden_size + (4 * h * lat if lat != h else 0)
            if cfg.moe_shared_expert_intermediate_size:
                fwd += 6 * h * cfg.moe_shared_expert_intermediate_size
        else:
            fwd += 6 * h * cfg.ffn_hidden_size
    fwd += 2 * h * V
    if getattr(cfg, "mtp_num_layers", None):
        # every depth: one more layer of the last layer's kind, the 2h -> h projection and the shared output head
        last = L - 1
        layer = 0.0
        if cfg.multi_latent_attention:
            qd = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim
            nh = cfg.num_attention_heads
            layer += (2 * h * cfg.q_lora_rank + 2 * cfg.q_lora_rank * nh * qd) if cfg.q_lora_rank else 2 * h * nh * qd
            layer += 2 * h * (cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim)
            layer += 2 * cfg.kv_lora_rank * nh * (cfg.qk_head_dim + cfg.v_head_dim) + 2 * nh * cfg.v_head_dim * h
            layer += 2 * seq_len * nh * (qd + cfg.v_head_dim) * (0.5 if causal_half else 1.0)
        else:
            layer += 2 * h * cfg.qkv_width + 2 * cfg.num_attention_heads * cfg.kv_channels * h
            layer += 4 * seq_len * cfg.num_attention_heads * cfg.kv_channels * (0.5 if causal_half else 1.0)
        if cfg.is_moe_layer(last):
            layer += 2 * h * cfg.num_experts + cfg.moe_router_topk * 6 * h * cfg.moe_ffn_hidden_size
            if cfg.moe_shared_expert_intermediate_size:
                layer += 6 * h * cfg.moe_shared_expert_intermediate_size
        else:
            layer += 6 * h * cfg.ffn_hidden_size
        fwd += cfg.mtp_num_layers * (layer + 2 * (2 * h) * h + 2 * h * V)
    return 3.0 * fwd
