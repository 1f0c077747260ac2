"""Hugging Face <-> engine weight conversion (Llama, Qwen3 dense / MoE, DeepSeek-V2/V3 MLA + MoE), without going
through an intermediate framework.

``config_from_hf(hf_config)``          -> ``TransformerConfig`` fields derived from a HF ``config.json`` dict
``hf_to_internal(hf_state_dict, cfg)`` -> full (un-sharded) state dict with this engine's parameter names / layouts
``internal_to_hf(state_dict, cfg)``    -> the inverse
``load_hf_into_trainer(trainer, dir)`` -> reads ``*.safetensors`` / ``pytorch_model*.bin`` and fills every rank's shard

Layout facts (same as the reference's bridge-free converters,
primus/backends/megatron/checkpoint/native_loader_{llama,qwen3,deepseek}.py and native_convert_common.py:132-334):
Q/K/V projections are concatenated (this engine keeps ``[q | k | v]``; the per-group interleave of Megatron-core
is applied when a checkpoint is written), gate / up projections are stacked ``[gate; up]``, the vocabulary is
zero-padded to the padded size, expert weights are stacked ``[experts, out, in]``; RoPE weights need no
permutation for Llama / Qwen3 (HF already stores the rotate-half order); the rotary rows of MLA are
de-interleaved (see ``engine/checkpoint.py::_mla_rope_rows``).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Optional

import torch


# ----------------------------------------------------------------------------------------------
def config_from_hf(hf: dict) -> dict:
    """TransformerConfig keyword arguments from a Hugging Face config dict."""
    mt = hf.get("model_type", "llama")
    nh = hf["num_attention_heads"]
    rp = hf.get("rope_parameters") or {}          # newer config files keep theta / scaling in one dict
    theta = hf.get("rope_theta") or rp.get("rope_theta") or 10000.0
    out = dict(num_layers=hf["num_hidden_layers"], hidden_size=hf["hidden_size"],
               ffn_hidden_size=hf.get("intermediate_size"), num_attention_heads=nh,
               num_query_groups=hf.get("num_key_value_heads", nh), vocab_size=hf["vocab_size"],
               norm_epsilon=hf.get("rms_norm_eps", 1e-5), rotary_base=float(theta),
               untie_embeddings_and_output_weights=not hf.get("tie_word_embeddings", False),
               kv_channels=hf.get("head_dim") or hf["hidden_size"] // nh)
    if mt in ("qwen3", "qwen3_moe"):
        out["qk_layernorm"] = True
    if mt in ("qwen3_5_moe_text", "qwen3_5_text", "qwen3_5_moe", "qwen3_5", "qwen3_next"):
        # gated-delta-net layers between gated full-attention layers, zero-centred norm gains, partial rotary embedding
        kinds = hf.get("layer_types") or ["full_attention" if (i + 1) % hf.get("full_attention_interval", 4) == 0
                                          else "linear_attention" for i in range(hf["num_hidden_layers"])]
        out.update(qk_layernorm=True, attention_output_gate=True, apply_layernorm_1p=True,
                   experimental_attention_variant="gated_delta_net",
                   linear_attention_freq=[int(k == "linear_attention") for k in kinds],
                   rotary_percent=float(rp.get("partial_rotary_factor", hf.get("partial_rotary_factor", 0.25))),
                   linear_conv_kernel_dim=hf.get("linear_conv_kernel_dim", 4),
                   linear_key_head_dim=hf["linear_key_head_dim"], linear_value_head_dim=hf["linear_value_head_dim"],
                   linear_num_key_heads=hf["linear_num_key_heads"], linear_num_value_heads=hf["linear_num_value_heads"])
        if hf.get("num_experts"):
            out.update(moe_layer_freq=[1] * hf["num_hidden_layers"], moe_router_pre_softmax=False,
                       moe_shared_expert_intermediate_size=hf.get("shared_expert_intermediate_size") or None,
                       moe_shared_expert_gate=bool(hf.get("shared_expert_intermediate_size")))
    if mt in ("lfm2", "lfm2_moe"):   # gated short convolutions + grouped-query attention with per-head q / k norms
        out.update(lfm_layer_types=list(hf["layer_types"]), conv_L_cache=hf.get("conv_L_cache", 3),
                   conv_bias=bool(hf.get("conv_bias", False)), qk_layernorm=True, norm_epsilon=hf.get("norm_eps", 1e-5),
                   ffn_hidden_size=hf.get("block_ff_dim") or hf.get("intermediate_size"))
    if mt == "lfm2_moe":    # dense first layers, then sigmoid-scored experts chosen with a selection-only bias
        k_dense = hf.get("num_dense_layers", 0)
        out.update(moe_layer_freq=[int(i >= k_dense) for i in range(hf["num_hidden_layers"])],
                   ffn_hidden_size=hf["intermediate_size"], moe_router_score_function="sigmoid",
                   moe_router_enable_expert_bias=bool(hf.get("use_expert_bias", True)),
                   moe_router_topk_scaling_factor=hf.get("routed_scaling_factor") or None)
    if mt == "qwen2" or (mt == "llama" and hf.get("attention_bias")):
        out["add_qkv_bias"] = True       # Qwen2 / Qwen2.5: biases on q, k and v (not on the output projection)
    E = hf.get("num_experts") or hf.get("num_local_experts") or hf.get("n_routed_experts")
    if E:
        out.update(num_experts=E, moe_router_topk=hf.get("num_experts_per_tok", 2),
                   moe_ffn_hidden_size=hf.get("moe_intermediate_size") or hf.get("intermediate_size"))
    if mt == "mixtral":     # every layer is sparse; probabilities are the softmax over the selected logits
        out.update(moe_layer_freq=[1] * hf["num_hidden_layers"], moe_router_pre_softmax=False)
    if mt == "qwen3_moe":
        step = hf.get("decoder_sparse_step", 1)
        only = set(hf.get("mlp_only_layers") or [])
        out["moe_layer_freq"] = [int((i + 1) % step == 0 and i not in only) for i in range(hf["num_hidden_layers"])]
        # normalised top-k probabilities = softmax over the selected logits; otherwise plain softmax scores
        out["moe_router_pre_softmax"] = not hf.get("norm_topk_prob", True)
    if mt in ("deepseek_v2", "deepseek_v3"):
        k_dense = hf.get("first_k_dense_replace", 0)
        out.update(multi_latent_attention=True, q_lora_rank=hf.get("q_lora_rank"), kv_lora_rank=hf["kv_lora_rank"],
                   qk_head_dim=hf["qk_nope_head_dim"], qk_pos_emb_head_dim=hf["qk_rope_head_dim"],
                   v_head_dim=hf["v_head_dim"], num_query_groups=nh,
                   moe_layer_freq=[int(i >= k_dense) for i in range(hf["num_hidden_layers"])],
                   moe_shared_expert_intermediate_size=(hf.get("n_shared_experts") or 0) * hf["moe_intermediate_size"] or None,
                   moe_router_topk_scaling_factor=hf.get("routed_scaling_factor"),
                   moe_router_score_function="sigmoid" if mt == "deepseek_v3" else "softmax",
                   moe_router_enable_expert_bias=mt == "deepseek_v3",
                   moe_router_num_groups=hf.get("n_group"), moe_router_group_topk=hf.get("topk_group"),
                   moe_router_pre_softmax=mt == "deepseek_v2")
        rs = hf.get("rope_scaling") or (rp if rp.get("rope_type", "default") != "default" else {})
        if rs.get("type", rs.get("rope_type")) == "yarn":
            out.update(rotary_scaling_factor=float(rs.get("factor", 1.0)), mscale=float(rs.get("mscale", 1.0)),
                       mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)),
                       original_max_position_embeddings=int(rs.get("original_max_position_embeddings", 4096)))
        else:
            out.update(rotary_scaling_factor=1.0)
    return out


def _pad_vocab(w: torch.Tensor, padded: int) -> torch.Tensor:
    if w.shape[0] == padded:
        return w
    out = w.new_zeros(padded, *w.shape[1:])
    out[: w.shape[0]] = w
    return out


def _deinterleave(dr: int) -> torch.Tensor:
    return torch.cat([torch.arange(0, dr, 2), torch.arange(1, dr, 2)])


def _interleave(dr: int) -> torch.Tensor:
    perm = torch.empty(dr, dtype=torch.long)
    perm[0::2] = torch.arange(0, dr // 2)
    perm[1::2] = torch.arange(dr // 2, dr)
    return perm


def _mla_rows(w: torch.Tensor, cfg, kv_down: bool, perm: torch.Tensor) -> torch.Tensor:
    dr = cfg.qk_pos_emb_head_dim
    if kv_down:
        lat = cfg.kv_lora_rank
        return torch.cat([w[:lat], w[lat:][perm]], 0)
    nh, dn = cfg.num_attention_heads, cfg.qk_head_dim
    x = w.reshape(nh, dn + dr, -1)
    return torch.cat([x[:, :dn], x[:, dn:][:, perm]], 1).reshape(w.shape)


# ----------------------------------------------------------------------------------------------
def mamba2_config_from_hf(hf: dict) -> dict:
    """TransformerConfig keyword arguments for a Hugging Face Mamba-2 config (a pure Mamba stack)."""
    return dict(model_type="mamba", num_layers=hf["num_hidden_layers"], hidden_size=hf["hidden_size"],
                num_attention_heads=hf["num_heads"], vocab_size=hf["vocab_size"], mamba_state_dim=hf["state_size"],
                mamba_head_dim=hf["head_dim"], mamba_num_heads=hf["num_heads"], mamba_num_groups=hf["n_groups"],
                mamba_expand=hf["expand"], mamba_d_conv=hf["conv_kernel"], mamba_chunk_size=hf.get("chunk_size", 128),
                norm_epsilon=hf.get("layer_norm_epsilon", 1e-5),
                untie_embeddings_and_output_weights=not hf.get("tie_word_embeddings", True))


def _mamba2_to_internal(hf: Dict[str, torch.Tensor], cfg) -> Dict[str, torch.Tensor]:
    sd: Dict[str, torch.Tensor] = {}
    V = cfg.padded_vocab_size
    sd["embedding.word_embeddings.weight"] = _pad_vocab(hf["backbone.embeddings.weight"], V)
    sd["decoder.final_layernorm.weight"] = hf["backbone.norm_f.weight"]
    if cfg.untie_embeddings_and_output_weights:
        sd["output_layer.weight"] = _pad_vocab(hf.get("lm_head.weight", hf["backbone.embeddings.weight"]), V)
    for L in range(cfg.num_layers):
        p, h = f"decoder.layers.{L}.mixer.", f"backbone.layers.{L}."
        sd[p + "in_proj.layer_norm_weight"] = hf[h + "norm.weight"]
        for k in ("in_proj.weight", "conv1d.weight", "conv1d.bias", "dt_bias", "A_log", "D", "norm.weight", "out_proj.weight"):
            sd[p + k] = hf[h + "mixer." + k]
    return sd


def _lfm2_to_internal(hf: Dict[str, torch.Tensor], cfg) -> Dict[str, torch.Tensor]:
    sd: Dict[str, torch.Tensor] = {}
    V = cfg.padded_vocab_size
    sd["embedding.word_embeddings.weight"] = _pad_vocab(hf["model.embed_tokens.weight"], V)
    sd["decoder.final_layernorm.weight"] = hf["model.embedding_norm.weight"]
    if cfg.untie_embeddings_and_output_weights:
        sd["output_layer.weight"] = _pad_vocab(hf.get("lm_head.weight", hf["model.embed_tokens.weight"]), V)
    for L in range(cfg.num_layers):
        p, h = f"decoder.layers.{L}.", f"model.layers.{L}."
        a = p + "self_attention."
        if cfg.layer_kinds[L][0] == "conv":
            sd[a + "in_proj.layer_norm_weight"] = hf[h + "operator_norm.weight"]
            sd[a + "in_proj.weight"] = hf[h + "conv.in_proj.weight"]
            sd[a + "conv.weight"] = hf[h + "conv.conv.weight"]
            sd[a + "out_proj.weight"] = hf[h + "conv.out_proj.weight"]
            if cfg.conv_bias:
                sd[a + "in_proj.bias"] = hf[h + "conv.in_proj.bias"]
                sd[a + "conv.bias"] = hf[h + "conv.conv.bias"]
                sd[a + "out_proj.bias"] = hf[h + "conv.out_proj.bias"]
        else:
            sd[a + "linear_qkv.layer_norm_weight"] = hf[h + "operator_norm.weight"]
            sd[a + "linear_qkv.weight"] = torch.cat([hf[h + "self_attn.q_proj.weight"], hf[h + "self_attn.k_proj.weight"],
                                                     hf[h + "self_attn.v_proj.weight"]], 0)
            sd[a + "q_layernorm.weight"] = hf[h + "self_attn.q_layernorm.weight"]
            sd[a + "k_layernorm.weight"] = hf[h + "self_attn.k_layernorm.weight"]
            sd[a + "linear_proj.weight"] = hf[h + "self_attn.out_proj.weight"]
        m, f = p + "mlp.", h + "feed_forward."
        if cfg.is_moe_layer(L):     # Lfm2Moe: stacked experts [E, 2 * ffn (gate | up), hidden], bias used for selection only
            sd[p + "pre_mlp_layernorm.weight"] = hf[h + "ffn_norm.weight"]
            sd[m + "router.weight"] = hf[f + "gate.weight"]
            if cfg.moe_router_enable_expert_bias:
                sd[m + "router.expert_bias"] = hf[f + "expert_bias"].float()
            if f + "experts.gate_up_proj" in hf:
                sd[m + "experts.fc1_weight.weight"] = hf[f + "experts.gate_up_proj"]
                sd[m + "experts.fc2_weight.weight"] = hf[f + "experts.down_proj"]
            else:                   # published checkpoints: one w1 (gate) / w3 (up) / w2 (down) per expert
                sd[m + "experts.fc1_weight.weight"] = torch.stack(
                    [torch.cat([hf[f + f"experts.{e}.w1.weight"], hf[f + f"experts.{e}.w3.weight"]], 0)
                     for e in range(cfg.num_experts)])
                sd[m + "experts.fc2_weight.weight"] = torch.stack(
                    [hf[f + f"experts.{e}.w2.weight"] for e in range(cfg.num_experts)])
            continue
        sd[m + "linear_fc1.layer_norm_weight"] = hf[h + "ffn_norm.weight"]
        sd[m + "linear_fc1.weight"] = torch.cat([hf[f + "w1.weight"], hf[f + "w3.weight"]], 0)
        sd[m + "linear_fc2.weight"] = hf[f + "w2.weight"]
    return sd


def _lfm2_from_internal(sd: Dict[str, torch.Tensor], cfg, stacked_experts: bool) -> Dict[str, torch.Tensor]:
    """Inverse of `_lfm2_to_internal` (names of transformers' Lfm2 / Lfm2Moe models)."""
    hf: Dict[str, torch.Tensor] = {}
    V = cfg.vocab_size
    hf["model.embed_tokens.weight"] = sd["embedding.word_embeddings.weight"][:V]
    hf["model.embedding_norm.weight"] = sd["decoder.final_layernorm.weight"]
    if cfg.untie_embeddings_and_output_weights:
        hf["lm_head.weight"] = sd["output_layer.weight"][:V]
    nq, nkv = cfg.num_attention_heads * cfg.kv_channels, cfg.num_query_groups * cfg.kv_channels
    for L in range(cfg.num_layers):
        p, h = f"decoder.layers.{L}.", f"model.layers.{L}."
        a = p + "self_attention."
        if cfg.layer_kinds[L][0] == "conv":
            hf[h + "operator_norm.weight"] = sd[a + "in_proj.layer_norm_weight"]
            for ours, theirs in (("in_proj", "conv.in_proj"), ("conv", "conv.conv"), ("out_proj", "conv.out_proj")):
                hf[h + theirs + ".weight"] = sd[a + ours + ".weight"]
                if cfg.conv_bias:
                    hf[h + theirs + ".bias"] = sd[a + ours + ".bias"]
        else:
            hf[h + "operator_norm.weight"] = sd[a + "linear_qkv.layer_norm_weight"]
            w = sd[a + "linear_qkv.weight"]
            hf[h + "self_attn.q_proj.weight"], hf[h + "self_attn.k_proj.weight"], hf[h + "self_attn.v_proj.weight"] = \
                w[:nq], w[nq:nq + nkv], w[nq + nkv:]
            hf[h + "self_attn.q_layernorm.weight"] = sd[a + "q_layernorm.weight"]
            hf[h + "self_attn.k_layernorm.weight"] = sd[a + "k_layernorm.weight"]
            hf[h + "self_attn.out_proj.weight"] = sd[a + "linear_proj.weight"]
        m, f = p + "mlp.", h + "feed_forward."
        if cfg.is_moe_layer(L):
            hf[h + "ffn_norm.weight"] = sd[p + "pre_mlp_layernorm.weight"]
            hf[f + "gate.weight"] = sd[m + "router.weight"]
            if cfg.moe_router_enable_expert_bias:
                hf[f + "expert_bias"] = sd[m + "router.expert_bias"]
            w1, w2 = sd[m + "experts.fc1_weight.weight"], sd[m + "experts.fc2_weight.weight"]
            I = w1.shape[1] // 2
            if stacked_experts:
                hf[f + "experts.gate_up_proj"], hf[f + "experts.down_proj"] = w1, w2
            for e in range(0 if stacked_experts else cfg.num_experts):
                hf[f + f"experts.{e}.w1.weight"], hf[f + f"experts.{e}.w3.weight"] = w1[e, :I], w1[e, I:]
                hf[f + f"experts.{e}.w2.weight"] = w2[e]
            continue
        hf[h + "ffn_norm.weight"] = sd[m + "linear_fc1.layer_norm_weight"]
        w = sd[m + "linear_fc1.weight"]
        hf[f + "w1.weight"], hf[f + "w3.weight"] = w[: w.shape[0] // 2], w[w.shape[0] // 2:]
        hf[f + "w2.weight"] = sd[m + "linear_fc2.weight"]
    return hf


def hf_to_internal(hf: Dict[str, torch.Tensor], cfg) -> Dict[str, torch.Tensor]:
    if cfg.model_type == "mamba" and "backbone.embeddings.weight" in hf:
        return _mamba2_to_internal(hf, cfg)
    if cfg.lfm_layer_types:
        return _lfm2_to_internal(hf, cfg)
    sd: Dict[str, torch.Tensor] = {}
    V = cfg.padded_vocab_size
    sd["embedding.word_embeddings.weight"] = _pad_vocab(hf["model.embed_tokens.weight"], V)
    sd["decoder.final_layernorm.weight"] = hf["model.norm.weight"]
    if cfg.untie_embeddings_and_output_weights:
        sd["output_layer.weight"] = _pad_vocab(hf.get("lm_head.weight", hf["model.embed_tokens.weight"]), V)
    for L in range(cfg.num_layers):
        p, h = f"decoder.layers.{L}.", f"model.layers.{L}."
        a = p + "self_attention."
        if cfg.multi_latent_attention:
            perm = _deinterleave(cfg.qk_pos_emb_head_dim)
            sd[a + "input_layernorm.weight"] = hf[h + "input_layernorm.weight"]
            if cfg.q_lora_rank:
                sd[a + "linear_q_down_proj.weight"] = hf[h + "self_attn.q_a_proj.weight"]
                sd[a + "linear_q_up_proj.layer_norm_weight"] = hf[h + "self_attn.q_a_layernorm.weight"]
                sd[a + "linear_q_up_proj.weight"] = _mla_rows(hf[h + "self_attn.q_b_proj.weight"], cfg, False, perm)
            else:
                sd[a + "linear_q_proj.weight"] = _mla_rows(hf[h + "self_attn.q_proj.weight"], cfg, False, perm)
            sd[a + "linear_kv_down_proj.weight"] = _mla_rows(hf[h + "self_attn.kv_a_proj_with_mqa.weight"], cfg, True, perm)
            sd[a + "linear_kv_up_proj.layer_norm_weight"] = hf[h + "self_attn.kv_a_layernorm.weight"]
            sd[a + "linear_kv_up_proj.weight"] = hf[h + "self_attn.kv_b_proj.weight"]
        elif cfg.layer_kinds[L][0] == "gdn":
            g, x = h + "linear_attn.", p + "mixer."
            sd[x + "in_proj.layer_norm_weight"] = hf[h + "input_layernorm.weight"]
            sd[x + "in_proj.weight"] = torch.cat([hf[g + "in_proj_qkv.weight"], hf[g + "in_proj_z.weight"],
                                                  hf[g + "in_proj_b.weight"], hf[g + "in_proj_a.weight"]], 0)
            sd[x + "conv1d.weight"] = hf[g + "conv1d.weight"]
            sd[x + "dt_bias"], sd[x + "A_log"] = hf[g + "dt_bias"], hf[g + "A_log"]
            sd[x + "out_norm.weight"] = hf[g + "norm.weight"]
            sd[x + "out_proj.weight"] = hf[g + "out_proj.weight"]
        else:
            sd[a + "linear_qkv.layer_norm_weight"] = hf[h + "input_layernorm.weight"]
            wq = hf[h + "self_attn.q_proj.weight"]
            if cfg.attention_output_gate:       # rows per head: [query (d) | gate (d)]
                wq = wq.reshape(cfg.num_attention_heads, 2, cfg.kv_channels, -1)
                sd[a + "linear_gate.weight"] = wq[:, 1].reshape(-1, wq.shape[-1])
                wq = wq[:, 0].reshape(-1, wq.shape[-1])
            sd[a + "linear_qkv.weight"] = torch.cat([wq, hf[h + "self_attn.k_proj.weight"],
                                                     hf[h + "self_attn.v_proj.weight"]], 0)
            if cfg.add_qkv_bias:
                sd[a + "linear_qkv.bias"] = torch.cat([hf[h + "self_attn.q_proj.bias"], hf[h + "self_attn.k_proj.bias"],
                                                       hf[h + "self_attn.v_proj.bias"]], 0)
            if cfg.qk_layernorm:
                sd[a + "q_layernorm.weight"] = hf[h + "self_attn.q_norm.weight"]
                sd[a + "k_layernorm.weight"] = hf[h + "self_attn.k_norm.weight"]
        if cfg.layer_kinds[L][0] == "attention":
            sd[a + "linear_proj.weight"] = hf[h + "self_attn.o_proj.weight"]
        m = p + "mlp."
        if cfg.is_moe_layer(L):
            sd[p + "pre_mlp_layernorm.weight"] = hf[h + "post_attention_layernorm.weight"]
            if h + "block_sparse_moe.gate.weight" in hf:     # published Mixtral checkpoints: w1 = gate, w3 = up, w2 = down
                b = h + "block_sparse_moe."
                sd[m + "router.weight"] = hf[b + "gate.weight"]
                sd[m + "experts.fc1_weight.weight"] = torch.stack(
                    [torch.cat([hf[b + f"experts.{e}.w1.weight"], hf[b + f"experts.{e}.w3.weight"]], 0)
                     for e in range(cfg.num_experts)])
                sd[m + "experts.fc2_weight.weight"] = torch.stack(
                    [hf[b + f"experts.{e}.w2.weight"] for e in range(cfg.num_experts)])
                continue
            sd[m + "router.weight"] = hf[h + "mlp.gate.weight"]
            if cfg.moe_router_enable_expert_bias:
                sd[m + "router.expert_bias"] = hf[h + "mlp.gate.e_score_correction_bias"].float()
            if h + "mlp.experts.gate_up_proj" in hf:   # stacked format: [experts, 2 * ffn (gate | up), hidden]
                sd[m + "experts.fc1_weight.weight"] = hf[h + "mlp.experts.gate_up_proj"]
                sd[m + "experts.fc2_weight.weight"] = hf[h + "mlp.experts.down_proj"]
            else:                                       # one entry per expert (published checkpoints)
                sd[m + "experts.fc1_weight.weight"] = torch.stack(
                    [torch.cat([hf[h + f"mlp.experts.{e}.gate_proj.weight"], hf[h + f"mlp.experts.{e}.up_proj.weight"]], 0)
                     for e in range(cfg.num_experts)])
                sd[m + "experts.fc2_weight.weight"] = torch.stack(
                    [hf[h + f"mlp.experts.{e}.down_proj.weight"] for e in range(cfg.num_experts)])
            if cfg.moe_shared_expert_intermediate_size:
                se = h + ("mlp.shared_experts." if h + "mlp.shared_experts.gate_proj.weight" in hf else "mlp.shared_expert.")
                sd[m + "shared_experts.linear_fc1.weight"] = torch.cat(
                    [hf[se + "gate_proj.weight"], hf[se + "up_proj.weight"]], 0)
                sd[m + "shared_experts.linear_fc2.weight"] = hf[se + "down_proj.weight"]
                if cfg.moe_shared_expert_gate:
                    sd[m + "shared_experts.gate_weight"] = hf[h + "mlp.shared_expert_gate.weight"]
        else:
            sd[m + "linear_fc1.layer_norm_weight"] = hf[h + "post_attention_layernorm.weight"]
            sd[m + "linear_fc1.weight"] = torch.cat([hf[h + "mlp.gate_proj.weight"], hf[h + "mlp.up_proj.weight"]], 0)
            sd[m + "linear_fc2.weight"] = hf[h + "mlp.down_proj.weight"]
    return sd


def internal_to_hf(sd: Dict[str, torch.Tensor], cfg, stacked_experts: bool = False) -> Dict[str, torch.Tensor]:
    if cfg.lfm_layer_types:
        return _lfm2_from_internal(sd, cfg, stacked_experts)
    hf: Dict[str, torch.Tensor] = {}
    V = cfg.vocab_size
    hf["model.embed_tokens.weight"] = sd["embedding.word_embeddings.weight"][:V]
    hf["model.norm.weight"] = sd["decoder.final_layernorm.weight"]
    if cfg.untie_embeddings_and_output_weights:
        hf["lm_head.weight"] = sd["output_layer.weight"][:V]
    hq, hkv, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
    for L in range(cfg.num_layers):
        p, h = f"decoder.layers.{L}.", f"model.layers.{L}."
        a = p + "self_attention."
        if cfg.multi_latent_attention:
            perm = _interleave(cfg.qk_pos_emb_head_dim)
            hf[h + "input_layernorm.weight"] = sd[a + "input_layernorm.weight"]
            if cfg.q_lora_rank:
                hf[h + "self_attn.q_a_proj.weight"] = sd[a + "linear_q_down_proj.weight"]
                hf[h + "self_attn.q_a_layernorm.weight"] = sd[a + "linear_q_up_proj.layer_norm_weight"]
                hf[h + "self_attn.q_b_proj.weight"] = _mla_rows(sd[a + "linear_q_up_proj.weight"], cfg, False, perm)
            else:
                hf[h + "self_attn.q_proj.weight"] = _mla_rows(sd[a + "linear_q_proj.weight"], cfg, False, perm)
            hf[h + "self_attn.kv_a_proj_with_mqa.weight"] = _mla_rows(sd[a + "linear_kv_down_proj.weight"], cfg, True, perm)
            hf[h + "self_attn.kv_a_layernorm.weight"] = sd[a + "linear_kv_up_proj.layer_norm_weight"]
            hf[h + "self_attn.kv_b_proj.weight"] = sd[a + "linear_kv_up_proj.weight"]
        elif cfg.layer_kinds[L][0] == "gdn":
            g, x = h + "linear_attn.", p + "mixer."
            qk = cfg.linear_num_key_heads * cfg.linear_key_head_dim
            vd = cfg.linear_num_value_heads * cfg.linear_value_head_dim
            w = sd[x + "in_proj.weight"]
            hf[h + "input_layernorm.weight"] = sd[x + "in_proj.layer_norm_weight"]
            hf[g + "in_proj_qkv.weight"], hf[g + "in_proj_z.weight"] = w[: 2 * qk + vd], w[2 * qk + vd: 2 * qk + 2 * vd]
            hf[g + "in_proj_b.weight"] = w[2 * qk + 2 * vd: 2 * qk + 2 * vd + cfg.linear_num_value_heads]
            hf[g + "in_proj_a.weight"] = w[2 * qk + 2 * vd + cfg.linear_num_value_heads:]
            hf[g + "conv1d.weight"] = sd[x + "conv1d.weight"]
            hf[g + "dt_bias"], hf[g + "A_log"] = sd[x + "dt_bias"], sd[x + "A_log"]
            hf[g + "norm.weight"] = sd[x + "out_norm.weight"]
            hf[g + "out_proj.weight"] = sd[x + "out_proj.weight"]
        else:
            w = sd[a + "linear_qkv.weight"]
            hf[h + "input_layernorm.weight"] = sd[a + "linear_qkv.layer_norm_weight"]
            hf[h + "self_attn.q_proj.weight"] = w[: hq * d]
            if cfg.attention_output_gate:
                both = torch.stack([w[: hq * d].reshape(hq, d, -1), sd[a + "linear_gate.weight"].reshape(hq, d, -1)], 1)
                hf[h + "self_attn.q_proj.weight"] = both.reshape(2 * hq * d, -1)
            hf[h + "self_attn.k_proj.weight"] = w[hq * d:(hq + hkv) * d]
            hf[h + "self_attn.v_proj.weight"] = w[(hq + hkv) * d:]
            if cfg.add_qkv_bias:
                b = sd[a + "linear_qkv.bias"]
                hf[h + "self_attn.q_proj.bias"] = b[: hq * d]
                hf[h + "self_attn.k_proj.bias"] = b[hq * d:(hq + hkv) * d]
                hf[h + "self_attn.v_proj.bias"] = b[(hq + hkv) * d:]
            if cfg.qk_layernorm:
                hf[h + "self_attn.q_norm.weight"] = sd[a + "q_layernorm.weight"]
                hf[h + "self_attn.k_norm.weight"] = sd[a + "k_layernorm.weight"]
        if cfg.layer_kinds[L][0] == "attention":
            hf[h + "self_attn.o_proj.weight"] = sd[a + "linear_proj.weight"]
        m = p + "mlp."
        if cfg.is_moe_layer(L):
            hf[h + "post_attention_layernorm.weight"] = sd[p + "pre_mlp_layernorm.weight"]
            hf[h + "mlp.gate.weight"] = sd[m + "router.weight"]
            if cfg.moe_router_enable_expert_bias:
                hf[h + "mlp.gate.e_score_correction_bias"] = sd[m + "router.expert_bias"]
            w1, w2 = sd[m + "experts.fc1_weight.weight"], sd[m + "experts.fc2_weight.weight"]
            I = w1.shape[1] // 2
            if stacked_experts:
                hf[h + "mlp.experts.gate_up_proj"] = w1
                hf[h + "mlp.experts.down_proj"] = w2
            for e in range(0 if stacked_experts else cfg.num_experts):
                hf[h + f"mlp.experts.{e}.gate_proj.weight"] = w1[e, :I]
                hf[h + f"mlp.experts.{e}.up_proj.weight"] = w1[e, I:]
                hf[h + f"mlp.experts.{e}.down_proj.weight"] = w2[e]
            if cfg.moe_shared_expert_intermediate_size:
                ws = sd[m + "shared_experts.linear_fc1.weight"]
                se = h + ("mlp.shared_expert." if cfg.moe_shared_expert_gate else "mlp.shared_experts.")   # Qwen | DeepSeek
                hf[se + "gate_proj.weight"] = ws[: ws.shape[0] // 2]
                hf[se + "up_proj.weight"] = ws[ws.shape[0] // 2:]
                hf[se + "down_proj.weight"] = sd[m + "shared_experts.linear_fc2.weight"]
                if cfg.moe_shared_expert_gate:
                    hf[h + "mlp.shared_expert_gate.weight"] = sd[m + "shared_experts.gate_weight"]
        else:
            w = sd[m + "linear_fc1.weight"]
            hf[h + "post_attention_layernorm.weight"] = sd[m + "linear_fc1.layer_norm_weight"]
            hf[h + "mlp.gate_proj.weight"] = w[: w.shape[0] // 2]
            hf[h + "mlp.up_proj.weight"] = w[w.shape[0] // 2:]
            hf[h + "mlp.down_proj.weight"] = sd[m + "linear_fc2.weight"]
    return hf


# ----------------------------------------------------------------------------------------------
def read_hf_weights(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of a Hugging Face checkpoint directory (``*.safetensors`` preferred, else ``*.bin``)."""
    out: Dict[str, torch.Tensor] = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        from safetensors.torch import load_file

        for f in files:
            out.update(load_file(f))
        return out
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
        out.update(torch.load(f, map_location="cpu", weights_only=True))
    if not out:
        raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {path}")
    return out


def load_full_into_trainer(trainer, full_sd: Dict[str, torch.Tensor]) -> None:
    """Copy this rank's slice of a full (un-sharded, internal-layout) state dict into the model chunks."""
    from . import checkpoint as C

    st, cfg = trainer.st, trainer.mcfg
    hq, hkv, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
    for m in trainer.model_chunks:
        for name, p in m.named_parameters():
            full = full_sd[name]
            spec = C.shard_spec(name, p, cfg, st)
            if spec["kind"] == "qkv":  # [q | k | v]: shard every part
                n, i = spec["count"], spec["index"]
                parts = (full[: hq * d], full[hq * d:(hq + hkv) * d], full[(hq + hkv) * d:])
                part = torch.cat([t.chunk(n, 0)[i] for t in parts], 0)
            else:
                part = C.slice_global(name, full, spec)
            p.data.copy_(part.to(p.dtype))
        for name, b in m.named_buffers():
            if name in full_sd:
                b.data.copy_(full_sd[name].to(b.dtype))
    C._refresh_master_weights(trainer)


def load_hf_into_trainer(trainer, path: str) -> None:
    load_full_into_trainer(trainer, hf_to_internal(read_hf_weights(path), trainer.mcfg))


def gather_full_state(trainer) -> Optional[Dict[str, torch.Tensor]]:
    """The whole model in the internal layout on rank 0 (None elsewhere): every rank contributes the shards it owns
    (tensor-, expert- and pipeline-parallel), data-parallel replicas are taken from the first replica."""
    import torch.distributed as dist

    from . import checkpoint as C

    st, cfg = trainer.st, trainer.mcfg
    mine = []
    for name, p in C.model_named_parameters(trainer):
        if getattr(p, "embedding_replica", False):
            continue
        spec = C.shard_spec(name, p, cfg, st)
        if C._is_writer(spec, C.saved_key(name), st, False):
            mine.append((name, spec, C.to_saved_layout(name, p.detach().cpu(), cfg, st.tp)))
    if not dist.is_initialized() or dist.get_world_size() == 1:
        everything = [mine]
    else:
        everything = [None] * dist.get_world_size() if dist.get_rank() == 0 else None
        dist.gather_object(mine, everything, dst=0)
        if dist.get_rank() != 0:
            return None
    shards: Dict[str, list] = {}
    for part in everything:
        for name, spec, t in part:
            shards.setdefault(name, []).append((spec, t))
    return {name: C.from_saved_layout(name, C.assemble_global(name, sh), cfg, 1) for name, sh in shards.items()}


def export_trainer_to_hf(trainer, path: str) -> None:
    sd = gather_full_state(trainer)
    if sd is not None:
        save_hf(sd, trainer.mcfg, path)
        trainer.log(f"[hf] wrote {len(sd)} tensors in Hugging Face layout to {path}")


def read_engine_checkpoint(root: str, iteration: Optional[int] = None):
    """(full internal state dict, TransformerConfig) of a ``torch_dist`` checkpoint, read in one process without
    building a trainer: the global tensors come straight from the checkpoint's metadata."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    from ..models.config import TransformerConfig
    from . import checkpoint as C

    it = iteration if iteration is not None else C.latest_iteration(root)
    d = C.checkpoint_dir(root, it) if it is not None else os.path.join(root, "release")
    common = torch.load(os.path.join(d, "common.pt"), map_location="cpu", weights_only=False)
    cfg = TransformerConfig.from_dict(common["args"]["model"])
    reader = FileSystemReader(d)
    md = reader.read_metadata().state_dict_metadata
    sd = {k: torch.empty(tuple(m.size), dtype=m.properties.dtype) for k, m in md.items()
          if isinstance(m, TensorStorageMetadata) and not k.startswith(("optimizer", "rng_state/", "weight_deosc/"))}
    dcp.load(sd, storage_reader=reader, no_dist=True)
    back = {b: a for a, b in C._RENAMES}
    out = {}
    for k, t in sd.items():
        name = k
        for saved, internal in back.items():
            name = name.replace(saved, internal)
        out[name] = C.from_saved_layout(name, t, cfg, 1)
    return out, cfg


def save_hf(trainer_or_sd, cfg, path: str) -> None:
    """Write a Hugging Face style ``model.safetensors`` from a full internal state dict (single-rank models)."""
    from safetensors.torch import save_file

    sd = trainer_or_sd if isinstance(trainer_or_sd, dict) else {k: v.detach().cpu() for k, v in
                                                                trainer_or_sd.model.state_dict().items()}
    os.makedirs(path, exist_ok=True)
    save_file({k: v.contiguous() for k, v in internal_to_hf(sd, cfg).items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "primus_b200_config.json"), "w") as f:
        json.dump({k: v for k, v in vars(cfg).items() if isinstance(v, (int, float, str, bool, list, type(None)))}, f, indent=1)
