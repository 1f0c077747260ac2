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
        self.moe_layer_pattern = parse_moe_layer_freq(self.moe_layer_freq, self.num_layers) \
            if self.num_experts else [0] * self.num_layers

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
        for i in range(L):
            n += 2 * h  # two norms
            if self.multi_latent_attention:
                qd = self.qk_head_dim + self.qk_pos_emb_head_dim
                if self.q_lora_rank:
                    n += h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * self.num_attention_heads * qd
                else:
                    n += h * self.num_attention_heads * qd
                n += h * (self.kv_lora_rank + self.qk_pos_emb_head_dim) + self.kv_lora_rank
                n += self.kv_lora_rank * self.num_attention_heads * (self.qk_head_dim + self.v_head_dim)
                n += self.num_attention_heads * self.v_head_dim * h
            else:
                n += h * self.qkv_width + self.num_attention_heads * self.kv_channels * h
                if self.add_qkv_bias:
                    n += self.qkv_width
                if self.qk_layernorm:
                    n += 2 * self.kv_channels
            if self.is_moe_layer(i):
                n += h * self.num_experts + self.num_experts * 3 * h * self.moe_ffn_hidden_size
                if self.moe_shared_expert_intermediate_size:
                    n += 3 * h * self.moe_shared_expert_intermediate_size
            else:
                n += 3 * h * self.ffn_hidden_size
        return n


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
