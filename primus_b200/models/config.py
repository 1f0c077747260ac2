"""Model configuration: one dataclass carrying the Megatron-style field names that the YAML model
presets use (``primus_b200/configs/models/*.yaml``), so a preset maps 1:1 onto it.

Field names follow the reference's model presets (primus/configs/models/megatron/language_model.yaml:1-196,
llama3_8B.yaml:8-12, qwen3_30B_A3B.yaml:7-25, deepseek_v2_lite.yaml:10-33).
"""
from __future__ import annotations

import ast
import dataclasses
from dataclasses import dataclass, field
from typing import Any, List, Optional


@dataclass
class TransformerConfig:
    # architecture
    num_layers: int = 2
    hidden_size: int = 256
    ffn_hidden_size: int = 688
    num_attention_heads: int = 4
    num_query_groups: Optional[int] = None  # None -> MHA
    kv_channels: Optional[int] = None  # head dim; None -> hidden/heads
    vocab_size: int = 32000
    make_vocab_size_divisible_by: int = 128
    max_position_embeddings: int = 4096
    seq_length: int = 512
    rotary_base: float = 10000.0
    rotary_percent: float = 1.0
    rotary_scaling_factor: float = 1.0
    use_rope_scaling: bool = False    # Llama-3.x frequency scaling: long wavelengths divided by rope_scaling_factor
    rope_scaling_factor: float = 8.0
    rope_scaling_low_freq_factor: float = 1.0
    rope_scaling_high_freq_factor: float = 4.0
    rope_scaling_original_max_position: int = 8192
    norm_epsilon: float = 1e-5
    add_qkv_bias: bool = False       # bias on the fused q / k / v projection (Qwen2 / Qwen2.5)
    hidden_dropout: float = 0.0      # on the embedding output and on every sub-layer output before the residual add
    attention_dropout: float = 0.0   # not built (the attention kernels have no dropout path): must stay 0
    qk_layernorm: bool = False
    untie_embeddings_and_output_weights: bool = True
    swiglu: bool = True
    gated_activation: str = "silu"    # gate of the gated linear unit: "silu" (SwiGLU) or "gelu" (GEGLU, tanh form)
    add_bias_linear: bool = False
    activation_func_clamp_value: float = 0.0
    init_method_std: float = 0.02
    attention_softmax_scale: Optional[float] = None
    # multi-latent attention (DeepSeek)
    multi_latent_attention: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    mscale: float = 0.707
    mscale_all_dim: float = 0.707
    original_max_position_embeddings: int = 4096
    # mixture of experts
    num_experts: Optional[int] = None
    moe_router_topk: int = 2
    moe_ffn_hidden_size: Optional[int] = None
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_layer_freq: Any = 1  # int, list, or python-expression string like "([0]*1+[1]*26)"
    moe_aux_loss_coeff: float = 0.0
    moe_router_load_balancing_type: str = "aux_loss"  # aux_loss | seq_aux_loss | none
    moe_router_score_function: str = "softmax"  # softmax | sigmoid
    moe_router_pre_softmax: bool = False
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3      # aux-loss-free balancing: bias += rate * sign(mean load - load)
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_force_load_balancing: bool = False
    moe_token_dispatcher_type: str = "alltoall"  # alltoall | allgather | mega
    moe_grouped_gemm: bool = True
    use_turbo_mega_moe: bool = False
    moe_fused_capacity_factor: Optional[float] = None   # rows per rank = factor x T x k (None: worst case ep x T x k)
    # parallelism (sizes; groups live in primus_b200.parallel.state)
    tensor_model_parallel_size: int = 1
    sequence_parallel: bool = False
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1
    # numerics / memory
    params_dtype: str = "bf16"  # bf16 | fp32
    fp8: Optional[str] = None  # None | "e4m3"
    fp8_recipe: str = "mxfp8"  # mxfp8 | tensorwise | delayed | blockwise
    fp8_amax_history_len: int = 1          # delayed scaling: steps of recorded maxima
    fp8_amax_compute_algo: str = "most_recent"   # delayed scaling: most_recent | max over the history
    fp8_margin: int = 0                    # delayed scaling: extra powers of two of headroom
    first_last_layers_bf16: bool = False            # keep the first / last decoder layers' GEMMs in bf16 under fp8 / fp4
    num_layers_at_start_in_bf16: int = 1
    num_layers_at_end_in_bf16: int = 1
    fp4: Optional[str] = None  # None | "e2m1": MXFP4 numerics for the linear-layer GEMMs (carried in FP8 storage)
    fp4_recipe: str = "mxfp4"
    recompute_granularity: Optional[str] = None  # None | selective | full
    recompute_method: Optional[str] = None       # full: "uniform" (chunks of recompute_num_layers) | "block" (first N layers)
    recompute_num_layers: Optional[int] = None
    recompute_modules: Optional[List[str]] = None  # selective: "core_attn" (default), "mlp"
    recompute_layer_ids: Optional[List[int]] = None
    cpu_offloading: bool = False                   # keep the saved activations of the first layers in pinned host memory
    cpu_offloading_num_layers: int = 0
    cross_entropy_chunk_tokens: int = 0  # >0: chunked linear-cross-entropy
    window_size: object = None                      # sliding-window attention: W, or Megatron's (left, right) = (W - 1, 0)
    window_attn_skip_freq: object = None            # int N: every N-th layer attends fully; list: 1 = windowed, 0 = full
    softmax_type: str = "vanilla"                   # "learnable": per-head sink logit in the softmax denominator
    hierarchical_context_parallel_sizes: Optional[list] = None   # [a2a, p2p] for cp_comm_type "a2a+p2p"
    cp_comm_type: str = "a2a"                      # context parallelism: "a2a" (Ulysses) or "allgather" (zig-zag chunks)
    mtp_num_layers: int | None = None               # multi-token prediction depths (DeepSeek-V3); None / 0: off
    mtp_loss_scaling_factor: float = 0.1
    final_logit_softcapping: float | None = None    # cap * tanh(logits / cap) before the loss (Grok-style)
    router_logit_softcapping: float | None = None   # same on the MoE router logits
    attn_logit_softcapping: float | None = None     # cap * tanh(scores / cap) inside attention (not for MLA / context parallel)
    # sequence mixers other than attention (models/mixers.py)
    model_type: str = "gpt"                         # "mamba": Mamba / hybrid stack, layer kinds from the hybrid pattern
    lfm_layer_types: Optional[List[str]] = None     # LFM2: per layer "conv" (gated short convolution) | "full_attention"
    conv_L_cache: int = 3                           # taps of the LFM2 short convolution
    conv_bias: bool = False
    mamba_state_dim: int = 128
    mamba_head_dim: int = 64
    mamba_num_groups: int = 8
    mamba_num_heads: Optional[int] = None           # None: mamba_expand * hidden_size / mamba_head_dim
    mamba_expand: int = 2
    mamba_d_conv: int = 4
    mamba_chunk_size: int = 128
    is_hybrid_model: bool = False
    hybrid_attention_ratio: float = 0.0             # share of the layers that are attention layers
    hybrid_mlp_ratio: float = 0.0                   # share of the layers that are MLP layers
    hybrid_override_pattern: Optional[str] = None   # one symbol per layer: M (Mamba), * (attention), - (MLP)
    linear_attention_type: Optional[str] = None     # "gdn": the M layers are gated-delta-net mixers instead of Mamba-2
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 64
    linear_value_head_dim: int = 64
    linear_num_key_heads: int = 8
    linear_num_value_heads: int = 16
    linear_chunk_size: int = 64
    # Qwen3.5-style stacks: linear-attention layers between full-attention layers in a GPT-style stack (every layer keeps
    # its MLP / MoE block).  ``linear_attention_freq``: int N -> every N-th layer attends fully, the others are linear;
    # a list (or a list expression such as "([1]*3+[0])*10") marks the linear layers with 1.
    experimental_attention_variant: Optional[str] = None     # "gated_delta_net"
    linear_attention_freq: object = None
    attention_output_gate: bool = False     # softmax attention output multiplied by sigmoid(gate), gate projected like q
    apply_layernorm_1p: bool = False        # norm gains stored as (gain - 1)
    moe_shared_expert_gate: bool = False    # shared-expert output multiplied by sigmoid(hidden . gate_weight)
    # Kimi-K3 (models/kimi_k3.py): ``model_type: kimi_k3`` makes the layers marked 1 in ``linear_attention_freq`` Kimi
    # delta attention and the others multi-latent attention without rotary embedding and with an output gate
    kda_gate_lower_bound: Optional[float] = -5.0    # bounded log-decay lower_bound * sigmoid(.); None: -exp(A) softplus(.)
    kda_chunk_size: int = 64
    kda_use_full_rank_gate: bool = True             # the low-rank output gate of Kimi Linear is not built
    mla_use_nope: bool = False                      # multi-latent attention without rotation (the "rope" dims stay)
    mla_use_output_gate: bool = False               # attention output times sigmoid(linear_o_gate(h)) before the projection
    attn_res_block_size: Optional[int] = None       # attention residuals: every N-th layer sets a checkpoint aside
    routed_expert_hidden_size: Optional[int] = None     # latent MoE: routed experts work in this (smaller) width
    latent_moe_use_norm: bool = True                # RMSNorm on the combined expert output before the up-projection
    activation_situ_beta: float = 4.0               # gated_activation "situ": beta tanh(g / beta) sigmoid(g) ...
    activation_situ_linear_beta: float = 25.0       # ... times linear_beta tanh(u / linear_beta)
    moe_router_bias_update_rule: str = "sign"       # "quantile": Kimi-K3 quantile balancing
    # DeepSeek-V4 (models/deepseek_v4.py): ``model_type: deepseek_v4``
    hc_mult: int = 1                                # hyper-connections: parallel residual streams (1: plain residual)
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    compress_ratios: object = None                  # per layer 0 (local attention only) | 4 (indexed) | 128 (pooled)
    compress_rope_theta: float = 160000.0           # rotary base of the layers with a compressed branch
    index_topk: int = 512
    index_head_dim: int = 128
    index_n_heads: int = 64
    attn_sliding_window: int = 128                  # local branch: the last N keys (0: all earlier keys)
    attn_sink: bool = True                          # learned per-head sink logit
    o_groups: int = 8                               # grouped low-rank output projection
    o_lora_rank: int = 1024                         # 0: one flat output projection
    v4_indexer_distill_loss_coeff: float = 0.0      # > 0: the indexer learns from the attention it feeds (KL on its picks)
    num_hash_layers: int = 0                        # the first N MoE layers pick experts from a token-id table
    hash_router_seed: int = 1234
    quantile_balancing_num_bins: int = 1024
    quantile_balancing_margin_min: float = -1.0
    quantile_balancing_margin_max: float = 1.0
    quantile_balancing_center_bias: bool = True
    quantile_balancing_update_interval: int = 1
    quantile_balancing_ema_decay: Optional[float] = None

    def layer_window(self, layer_idx: int) -> int:
        """Sliding-window width of a layer (0 = full attention)."""
        if not self.window_size:
            return 0
        w = self.window_size
        width = int(w[0]) + 1 if isinstance(w, (tuple, list)) else int(w)
        f = self.window_attn_skip_freq
        if f is None:
            return width
        if isinstance(f, int):
            return 0 if (layer_idx + 1) % f == 0 else width
        return width if f[layer_idx % len(f)] else 0

    def __post_init__(self):
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.moe_ffn_hidden_size is None:
            self.moe_ffn_hidden_size = self.ffn_hidden_size
        self.compress_ratio_list, self.compress_ratio_mtp = None, []
        if self.model_type == "deepseek_v4":
            r = self.compress_ratios
            if isinstance(r, str):
                r = ast.literal_eval(r)
            self.compress_ratio_list = [0] * self.num_layers if r is None else [int(x) for x in r]
            # the published lists carry one more entry per multi-token-prediction depth behind the decoder layers
            if len(self.compress_ratio_list) > self.num_layers:
                self.compress_ratio_mtp = self.compress_ratio_list[self.num_layers:]
                self.compress_ratio_list = self.compress_ratio_list[:self.num_layers]
            if len(self.compress_ratio_list) != self.num_layers:
                raise ValueError(f"compress_ratios has {len(self.compress_ratio_list)} entries for {self.num_layers} layers")
        if self.model_type == "kimi_k3":
            self.multi_latent_attention = True      # the full-attention layers of the stack
            self.mla_use_nope = True
        self.moe_layer_pattern = parse_moe_layer_freq(self.moe_layer_freq, self.num_layers) \
            if self.num_experts else [0] * self.num_layers
        self.layer_kinds = layer_kinds(self)

    # ------------------------------------------------------------------ derived
    @property
    def padded_vocab_size(self) -> int:
        m = self.make_vocab_size_divisible_by * self.tensor_model_parallel_size
        return -(-self.vocab_size // m) * m

    @property
    def head_dim(self) -> int:
        return self.kv_channels

    @property
    def qkv_width(self) -> int:
        return (self.num_attention_heads + 2 * self.num_query_groups) * self.kv_channels

    @property
    def torch_dtype(self):
        import torch

        return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[self.params_dtype]

    def is_moe_layer(self, layer_idx: int) -> bool:
        return bool(self.num_experts) and bool(self.moe_layer_pattern[layer_idx])

    @classmethod
    def from_dict(cls, d: dict) -> "TransformerConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        known = {k: v for k, v in d.items() if k in names}
        # accepted aliases used by the reference presets
        if "group_query_attention" in d and not d.get("group_query_attention"):
            known["num_query_groups"] = None
        if "bf16" in d and d["bf16"]:
            known.setdefault("params_dtype", "bf16")
        if "padded_vocab_size" in d and "vocab_size" not in d:
            known["vocab_size"] = d["padded_vocab_size"]
        return cls(**known)

    def num_parameters(self) -> int:
        """Total parameter count (embedding + output included)."""
        h, L = self.hidden_size, self.num_layers
        V = self.padded_vocab_size
        n = V * h * (2 if self.untie_embeddings_and_output_weights else 1) + h
        if self.attn_res_block_size:
            n += 2 * h                              # the mix after the last layer
        if self.hc_mult > 1:
            n += self.hc_mult * (self.hc_mult * h + 1) + 1      # the collapse after the last layer
        for i in range(L):
            mixer, has_mlp = self.layer_kinds[i]
            n += h * (int(mixer is not None) + int(has_mlp))  # one norm per sub-layer
            if mixer == "conv":
                n += 3 * h * h + h * self.conv_L_cache + h * h + (5 * h if self.conv_bias else 0)
            elif mixer == "mamba":
                di = self.mamba_expand * h
                nh = self.mamba_num_heads or di // self.mamba_head_dim
                conv_dim = di + 2 * self.mamba_num_groups * self.mamba_state_dim
                n += h * (di + conv_dim + nh) + conv_dim * (self.mamba_d_conv + 1) + 3 * nh + di + di * h
            elif mixer == "gdn":
                qk, vd = self.linear_num_key_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
                conv_dim = 2 * qk + vd
                n += h * (conv_dim + vd + 2 * self.linear_num_value_heads) + conv_dim * self.linear_conv_kernel_dim
                n += 2 * self.linear_num_value_heads + self.linear_value_head_dim + vd * h
            elif mixer == "v4":
                nh, hd = self.num_attention_heads, self.kv_channels
                if self.q_lora_rank:
                    n += h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * nh * hd
                else:
                    n += h * nh * hd
                n += h * hd + hd
                n += nh if self.attn_sink else 0
                n += (nh * hd * self.o_lora_rank + h * self.o_groups * self.o_lora_rank) if self.o_lora_rank else nh * hd * h
                ratio = self.compress_ratio_list[i]

                def comp(d):       # a compressor of width d: projection, position term, norm
                    c = 2 if ratio == 4 else 1
                    return 2 * c * d * h + c * ratio * d + d
                if ratio:
                    n += comp(hd)
                if ratio == 4:
                    n += h * (self.index_head_dim + self.index_n_heads) + self.index_n_heads * self.index_head_dim ** 2
                    n += comp(self.index_head_dim)
            elif mixer == "kda":
                qk, vd = self.linear_num_value_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
                conv_dim = 2 * qk + vd
                full = self.kda_use_full_rank_gate
                fa = self.linear_key_head_dim if full else self.linear_value_head_dim
                n += h * (conv_dim + (vd if full else self.linear_value_head_dim) + fa + self.linear_num_value_heads)
                n += conv_dim * self.linear_conv_kernel_dim + qk * fa + (0 if full else vd * self.linear_value_head_dim)
                n += self.linear_num_value_heads + qk + self.linear_value_head_dim + vd * h
            elif mixer is None:
                pass
            elif self.multi_latent_attention:
                qd = self.qk_head_dim + self.qk_pos_emb_head_dim
                if self.q_lora_rank:
                    n += h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * self.num_attention_heads * qd
                else:
                    n += h * self.num_attention_heads * qd
                n += h * (self.kv_lora_rank + self.qk_pos_emb_head_dim) + self.kv_lora_rank
                n += self.kv_lora_rank * self.num_attention_heads * (self.qk_head_dim + self.v_head_dim)
                n += self.num_attention_heads * self.v_head_dim * h
                if self.mla_use_output_gate:
                    n += h * self.num_attention_heads * self.v_head_dim
            else:
                n += h * self.qkv_width + self.num_attention_heads * self.kv_channels * h
                if self.attention_output_gate:
                    n += h * self.num_attention_heads * self.kv_channels
                if self.add_qkv_bias:
                    n += self.qkv_width
                if self.qk_layernorm:
                    n += 2 * self.kv_channels
            if not has_mlp:
                continue
            if self.hc_mult > 1:                    # two hyper-connection mixers: projection, three scales, offsets
                K = self.hc_mult
                n += 2 * ((2 + K) * K * (K * h + 1) + 3)
            if self.attn_res_block_size:
                n += 2 * h * (2 if i else 1)        # rank-1 scorers before the mixer (not in layer 0) and before the MLP
            if self.is_moe_layer(i):
                lat = self.routed_expert_hidden_size or h
                n += h * self.num_experts + self.num_experts * 3 * lat * self.moe_ffn_hidden_size
                if self.routed_expert_hidden_size:
                    n += 2 * h * lat + (lat if self.latent_moe_use_norm else 0)
                if self.moe_shared_expert_intermediate_size:
                    n += 3 * h * self.moe_shared_expert_intermediate_size + (h if self.moe_shared_expert_gate else 0)
            else:
                n += 3 * h * self.ffn_hidden_size
        return n


def hybrid_layer_pattern(num_layers: int, attention_ratio: float, mlp_ratio: float, override: Optional[str] = None,
                         hybrid: bool = True) -> str:
    """One symbol per layer of a Mamba / hybrid stack: ``M`` Mamba, ``*`` attention, ``-`` MLP.

    * An override pattern is used as given (``|`` separators are dropped).
    * A pure Mamba stack (``hybrid`` false) is all ``M``.
    * A hybrid stack alternates mixer and MLP layers, so half of the layers are mixers; ``int(L / 2 x attention_ratio)`` of
      the mixers are attention layers, each followed by an equal share of the Mamba mixers (the leftover Mamba mixers
      close the stack); above a ratio of 0.5 the surplus attention layers come first.  This is the allocation of the
      reference's hybrid stack (primus/backends/megatron/core/models/hybrid/hybrid_block.py:219-244), which ignores
      ``hybrid_mlp_ratio``.
    * With an explicit ``mlp_ratio`` > 0 the layers are instead spread evenly: ``round(L x attention_ratio)`` attention
      layers between sections of Mamba layers, then ``round(L x mlp_ratio)`` of the Mamba layers turned into MLP layers."""
    if override:
        pat = override.replace("|", "")
        assert len(pat) == num_layers and set(pat) <= set("M*-"), f"hybrid_override_pattern {override!r}: need " \
            f"{num_layers} symbols out of M, *, -"
        return pat
    if not hybrid:
        return "M" * num_layers
    if mlp_ratio <= 0.0:
        half = num_layers // 2
        n_attn = int(half * attention_ratio)
        n_mamba = half - n_attn
        if n_attn == 0:
            return "M-" * half
        if attention_ratio <= 0.5:
            return ("*-" + "M-" * (n_mamba // n_attn)) * n_attn + "M-" * (n_mamba % n_attn)
        return "*-" * (n_attn - n_mamba) + "*-M-" * n_mamba
    n_attn = int(round(num_layers * attention_ratio))
    kinds = ["M"] * num_layers
    n_mamba = num_layers - n_attn
    if n_attn:
        section = n_mamba / (n_attn + 1)
        x = section
        for i in range(num_layers):
            if x < 0.5:
                kinds[i] = "*"
                x += section
            else:
                x -= 1
    n_mlp = int(round(num_layers * mlp_ratio))
    if n_mlp:
        ratio = (n_mamba - n_mlp) / n_mlp
        x = ratio
        for i in range(num_layers):
            if kinds[i] == "M":
                if x < 0.5:
                    kinds[i] = "-"
                    x += ratio
                else:
                    x -= 1
    return "".join(kinds)


def layer_kinds(cfg) -> list:
    """Per layer ``(mixer, has_mlp)``: mixer in ``"attention" | "conv" | "mamba" | None``.  A GPT-style layer is a mixer
    followed by an MLP; the layers of a Mamba / hybrid stack hold one sub-layer each."""
    L = cfg.num_layers
    if cfg.model_type == "deepseek_v4":
        return [("v4", True)] * L
    if cfg.model_type == "mamba":
        pat = hybrid_layer_pattern(L, cfg.hybrid_attention_ratio, cfg.hybrid_mlp_ratio, cfg.hybrid_override_pattern,
                                   hybrid=cfg.is_hybrid_model)
        lat = (cfg.linear_attention_type or "").lower()
        m_kind = "gdn" if lat in ("gdn", "gated_delta_net") else ("kda" if lat in ("kda", "kimi_delta_attention") else "mamba")
        return [{"M": (m_kind, False), "*": ("attention", False), "-": (None, True)}[c] for c in pat]
    if cfg.lfm_layer_types:
        assert len(cfg.lfm_layer_types) == L, f"lfm_layer_types has {len(cfg.lfm_layer_types)} entries for {L} layers"
        bad = set(cfg.lfm_layer_types) - {"conv", "full_attention"}
        assert not bad, f"lfm_layer_types: unknown kinds {sorted(bad)}"
        return [("conv" if t == "conv" else "attention", True) for t in cfg.lfm_layer_types]
    variant = (cfg.experimental_attention_variant or "").lower()
    if cfg.model_type == "kimi_k3":
        variant = "kda"
    if variant and cfg.linear_attention_freq:
        kinds = {"gated_delta_net": "gdn", "gdn": "gdn", "kda": "kda", "kimi_delta_attention": "kda"}
        if variant not in kinds:
            raise NotImplementedError(f"experimental_attention_variant {variant!r}: gated_delta_net and kda are built")
        freq = cfg.linear_attention_freq
        if isinstance(freq, int):
            linear = [int((i + 1) % freq != 0) for i in range(L)]
        else:
            linear = parse_moe_layer_freq(freq, L)      # the same restricted list expressions
        return [(kinds[variant] if x else "attention", True) for x in linear]
    return [("attention", True)] * L


def parse_moe_layer_freq(freq, num_layers: int) -> list[int]:
    """int N -> every N-th layer is MoE; list -> as is; string -> a restricted python list expression
    such as ``"([0]*1+[1]*26)"`` (the form used by the DeepSeek presets;
    primus/backends/megatron/patches/args/moe_layer_freq_patches.py:12)."""
    if isinstance(freq, str):
        node = ast.parse(freq.strip(), mode="eval")
        for sub in ast.walk(node):
            if not isinstance(sub, (ast.Expression, ast.BinOp, ast.List, ast.Constant, ast.Add, ast.Mult, ast.Load,
                                    ast.Tuple)):
                raise ValueError(f"unsupported expression in moe_layer_freq: {freq!r}")
        freq = eval(compile(node, "<moe_layer_freq>", "eval"), {"__builtins__": {}})  # noqa: S307 (validated AST)
    if isinstance(freq, int):
        pat = [1 if (i % freq == 0) else 0 for i in range(num_layers)]
    else:
        pat = [int(x) for x in freq]
    if len(pat) != num_layers:
        raise ValueError(f"moe_layer_freq pattern has {len(pat)} entries for {num_layers} layers")
    return pat
