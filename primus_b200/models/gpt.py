"""Decoder-only GPT family (Llama / Qwen3 / DeepSeek-style) on the primus_b200 ops.

Activations are token-major 2-D tensors ``[tokens, hidden]`` (``tokens = micro_batch * seq`` or its
sequence-parallel shard).  The residual stream travels between layers as a pair
``(delta, residual)`` so that the residual add is fused into the next RMSNorm.

Parameter names follow the Megatron-core checkpoint layout that the reference's converters define
(primus/backends/megatron/checkpoint/native_loader_llama.py:194-239, native_loader_qwen3.py:250-283,
native_loader_deepseek.py:252-302): ``embedding.word_embeddings.weight``,
``decoder.layers.{i}.self_attention.linear_qkv.{layer_norm_weight,weight}``,
``...linear_proj.weight``, ``...mlp.linear_fc1.{layer_norm_weight,weight}``, ``...mlp.linear_fc2.weight``,
``decoder.final_layernorm.weight``, ``output_layer.weight``.  Internally ``linear_qkv.weight`` rows are
ordered ``[all q heads | all k heads | all v heads]``; :mod:`primus_b200.engine.checkpoint` converts to
and from the per-query-group interleaved order of the checkpoint format.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import fused, gemm, layers
from ..parallel import random as prandom
from ..parallel import state as ps
from ..parallel import tensor_parallel as tpc
from .config import TransformerConfig


def _param(shape, std, dtype, device, is_norm=False, seed_offset=0):
    if is_norm:
        p = torch.ones(shape, dtype=dtype, device=device)
    else:
        p = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std).to(dtype)
    return nn.Parameter(p)


def is_norm_gain(name: str) -> bool:
    """Is this parameter the gain of an RMSNorm that ``apply_layernorm_1p`` stores centred on zero?  (Not the gated
    norms inside the Mamba / gated-delta-net mixers, ``norm.weight`` / ``out_norm.weight``.)"""
    return name.endswith("layer_norm_weight") or name.endswith(("layernorm.weight", "enorm.weight", "hnorm.weight",
                                                                "latent_norm.weight"))


class ParamHolder(nn.Module):
    """A module that only owns named parameters (keeps checkpoint key paths identical to mcore)."""

    def __init__(self, **params):
        super().__init__()
        for k, v in params.items():
            self.register_parameter(k, v)


class SelfAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, layer_idx: int, device, tp: int):
        super().__init__()
        self.cfg = cfg
        dt = cfg.torch_dtype
        h, d = cfg.hidden_size, cfg.kv_channels
        assert cfg.num_attention_heads % tp == 0 and cfg.num_query_groups % tp == 0, "heads must divide by TP"
        self.hq = cfg.num_attention_heads // tp
        self.hkv = cfg.num_query_groups // tp
        std = cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        self.linear_qkv = ParamHolder(
            layer_norm_weight=_param((h,), 0, dt, device, is_norm=True),
            weight=_param(((self.hq + 2 * self.hkv) * d, h), std, dt, device),
        )
        if cfg.add_qkv_bias:   # Qwen2 / Qwen2.5: a bias on the fused q / k / v projection (rows ordered like the weight)
            self.linear_qkv.register_parameter(
                "bias", nn.Parameter(torch.zeros((self.hq + 2 * self.hkv) * d, dtype=dt, device=device)))
            self.linear_qkv.bias.tensor_model_parallel = tp > 1
            self.linear_qkv.bias.partition_dim = 0
        self.linear_proj = ParamHolder(weight=_param((h, self.hq * d), out_std, dt, device))
        if cfg.attention_output_gate:
            # Qwen3.5 / Qwen3-Next: a gate projected from the same normalised input as q, one value per output channel;
            # the attention output is multiplied by its sigmoid before the output projection.  Kept as a projection of
            # its own (column-parallel like q), so the [q | k | v] layout of linear_qkv is the same with and without it.
            self.linear_gate = ParamHolder(weight=_param((self.hq * d, h), std, dt, device))
            self.linear_gate.weight.tensor_model_parallel = tp > 1
            self.linear_gate.weight.partition_dim = 0
        if cfg.qk_layernorm:
            self.q_layernorm = ParamHolder(weight=_param((d,), 0, dt, device, is_norm=True))
            self.k_layernorm = ParamHolder(weight=_param((d,), 0, dt, device, is_norm=True))
        self.linear_qkv.weight.tensor_model_parallel = tp > 1
        self.linear_qkv.weight.partition_dim = 0
        self.linear_proj.weight.tensor_model_parallel = tp > 1
        self.linear_proj.weight.partition_dim = 1
        self.linear_qkv.layer_norm_weight.sequence_parallel = cfg.sequence_parallel
        self.window = cfg.layer_window(layer_idx)
        self.has_sinks = cfg.softmax_type == "learnable"
        if self.has_sinks:   # one sink logit per (local) query head, mcore name core_attention.softmax_offset
            self.core_attention = ParamHolder(softmax_offset=nn.Parameter(torch.zeros(self.hq, dtype=dt, device=device)))
            self.core_attention.softmax_offset.tensor_model_parallel = tp > 1
            self.core_attention.softmax_offset.partition_dim = 0

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        tpg = st.tp_group
        sp = cfg.sequence_parallel and st.tp > 1
        qkv, xsum = layers.norm_linear(hidden, residual, self.linear_qkv.layer_norm_weight,
                                       self.linear_qkv.weight, cfg.norm_epsilon, tpg, sp)
        d = cfg.kv_channels
        if cfg.add_qkv_bias:
            qkv = qkv + self.linear_qkv.bias
        if cfg.qk_layernorm:
            qkv = self._qk_norm(qkv, d)
        cos, sin, pos = rope[:3]
        segments = rope[3] if len(rope) > 3 else None
        scale = cfg.attention_softmax_scale
        if st.cp > 1 and (self.window or self.has_sinks or segments or cfg.attn_logit_softcapping):
            raise NotImplementedError("sliding-window / sink / per-document attention is not available under context "
                                      "parallelism")
        if layers.SEQ_SPLIT.active:
            if st.cp > 1 or self.window or self.has_sinks or segments or cfg.attn_logit_softcapping:
                raise NotImplementedError("num_seq_splits > 1 is built for plain causal attention (no context "
                                          "parallelism, sliding window, sinks, packed documents or soft-capping)")
            ctx_out = layers.seq_split_rope_attention(id(self), qkv, cos, sin, pos, batch, self.hq, self.hkv, d,
                                                      rot_dim=int(d * cfg.rotary_percent), scale=scale)
        elif st.cp > 1 and cfg.cp_comm_type == "allgather":
            ctx_out = layers.allgather_cp_rope_attention(qkv, cos, sin, pos, batch, self.hq, self.hkv, d, st.cp_group,
                                                         st.cp, rot_dim=int(d * cfg.rotary_percent), causal=True,
                                                         scale=scale)
        elif st.cp > 1 and cfg.cp_comm_type == "p2p":
            ctx_out = layers.ring_cp_rope_attention(qkv, cos, sin, pos, batch, self.hq, self.hkv, d, st.cp_group, st.cp,
                                                    rot_dim=int(d * cfg.rotary_percent), scale=scale)
        elif st.cp > 1 and cfg.cp_comm_type == "a2a+p2p":
            ctx_out = layers.hierarchical_cp_rope_attention(qkv, cos, sin, pos, batch, self.hq, self.hkv, d,
                                                            st.cp_a2a_group, st.cp_a2a, st.cp_p2p_group, st.cp_p2p,
                                                            rot_dim=int(d * cfg.rotary_percent), scale=scale)
        elif st.cp > 1:
            if cfg.cp_comm_type != "a2a":
                raise NotImplementedError(f"cp_comm_type {cfg.cp_comm_type!r}: a2a (Ulysses), allgather, p2p (ring) "
                                          "and a2a+p2p are built")
            ctx_out = layers.ulysses_rope_attention(qkv, cos, sin, pos, batch, self.hq, self.hkv, d, st.cp_group, st.cp,
                                                    rot_dim=int(d * cfg.rotary_percent), causal=True, scale=scale)
        else:
            sinks = self.core_attention.softmax_offset.float() if self.has_sinks else None
            ctx_out = selective_checkpoint(
                cfg, "core_attn",
                lambda t: layers.rope_attention(t, cos, sin, pos, batch, self.hq, self.hkv, d,
                                                rot_dim=int(d * cfg.rotary_percent), causal=True, scale=scale,
                                                window=self.window, sinks=sinks, segments=segments,
                                                softcap=cfg.attn_logit_softcapping or 0.0), qkv)
        if cfg.attention_output_gate:
            gate, _ = layers.norm_linear(hidden, residual, self.linear_qkv.layer_norm_weight, self.linear_gate.weight,
                                         cfg.norm_epsilon, tpg, sp)
            ctx_out = (ctx_out.reshape(gate.shape) * torch.sigmoid(gate.float()).to(ctx_out.dtype)).contiguous()
        out = layers.row_parallel_linear(ctx_out, self.linear_proj.weight, tpg, sp)
        return out, xsum

    def _qk_norm(self, qkv, d):
        """Per-head RMSNorm of q and k (Qwen3)."""
        T = qkv.shape[0]
        hq, hkv = self.hq, self.hkv
        q = qkv[:, : hq * d].reshape(T * hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].reshape(T * hkv, d)
        v = qkv[:, (hq + hkv) * d:]
        qn = fused.rmsnorm(q, self.q_layernorm.weight, self.cfg.norm_epsilon).reshape(T, hq * d)
        kn = fused.rmsnorm(k, self.k_layernorm.weight, self.cfg.norm_epsilon).reshape(T, hkv * d)
        return torch.cat([qn, kn, v], dim=1)


class MLP(nn.Module):
    """Dense SwiGLU MLP: fc1 = [gate; up] stacked on the output dim, fc2 row-parallel."""

    def __init__(self, cfg: TransformerConfig, device, tp: int, ffn: Optional[int] = None, with_norm: bool = True):
        super().__init__()
        self.cfg = cfg
        dt = cfg.torch_dtype
        h = cfg.hidden_size
        ffn = ffn or cfg.ffn_hidden_size
        assert ffn % tp == 0
        self.ffn_local = ffn // tp
        std = cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        p = dict(weight=_param((2 * self.ffn_local, h), std, dt, device))
        if with_norm:
            p["layer_norm_weight"] = _param((h,), 0, dt, device, is_norm=True)
        self.linear_fc1 = ParamHolder(**p)
        self.linear_fc2 = ParamHolder(weight=_param((h, self.ffn_local), out_std, dt, device))
        self.linear_fc1.weight.tensor_model_parallel = tp > 1
        self.linear_fc1.weight.partition_dim = 0
        self.linear_fc2.weight.tensor_model_parallel = tp > 1
        self.linear_fc2.weight.partition_dim = 1
        if with_norm:
            self.linear_fc1.layer_norm_weight.sequence_parallel = cfg.sequence_parallel

    def forward(self, hidden, residual):
        cfg = self.cfg
        st = ps.get_state()
        tpg = st.tp_group
        sp = cfg.sequence_parallel and st.tp > 1
        h1, xsum = layers.norm_linear(hidden, residual, self.linear_fc1.layer_norm_weight, self.linear_fc1.weight,
                                      cfg.norm_epsilon, tpg, sp)
        out = layers.swiglu_linear(h1, self.linear_fc2.weight, None, cfg.activation_func_clamp_value, tpg, sp,
                                   cfg.gated_activation)
        return out, xsum

    def forward_normed(self, y):
        """MLP on an already-normalised input (shared experts / per-expert use). No TP comm."""
        h1 = gemm.linear(y, self.linear_fc1.weight)
        return layers.swiglu_linear(h1, self.linear_fc2.weight, None, self.cfg.activation_func_clamp_value,
                                    act=self.cfg.gated_activation)


class TransformerLayer(nn.Module):
    """One layer of the stack: a sequence mixer (attention, MLA, LFM2 short convolution or Mamba-2; ``None`` for the MLP
    layers of a hybrid stack) followed by an MLP / MoE block (absent in the single-sub-layer layers of Mamba / hybrid
    stacks).  The kinds come from ``TransformerConfig.layer_kinds``."""

    def __init__(self, cfg: TransformerConfig, layer_idx: int, device, tp: int, mtp_depth: Optional[int] = None):
        """``mtp_depth`` (0-based): the layer is the inner layer of a multi-token-prediction depth, built like decoder
        layer ``layer_idx`` but without attention residuals (there are no checkpoints to mix behind the stack) and, in
        the DeepSeek-V4 family, with the compression ratio the preset lists for that depth."""
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.mixer_kind, self.has_mlp = cfg.layer_kinds[layer_idx]
        if self.mixer_kind == "attention":
            if cfg.multi_latent_attention:
                from .mla import MLASelfAttention

                self.self_attention = MLASelfAttention(cfg, layer_idx, device, tp)
            else:
                self.self_attention = SelfAttention(cfg, layer_idx, device, tp)
        elif self.mixer_kind == "conv":
            from .mixers import ShortConvMixer

            self.self_attention = ShortConvMixer(cfg, layer_idx, device, tp)
        elif self.mixer_kind == "mamba":
            from .mixers import Mamba2Mixer

            self.mixer = Mamba2Mixer(cfg, layer_idx, device, tp)
        elif self.mixer_kind == "gdn":
            from .mixers import GatedDeltaNetMixer

            self.mixer = GatedDeltaNetMixer(cfg, layer_idx, device, tp)
        elif self.mixer_kind == "kda":
            from .kimi_k3 import KimiDeltaAttentionMixer

            self.mixer = KimiDeltaAttentionMixer(cfg, layer_idx, device, tp)
        elif self.mixer_kind == "v4":
            from .deepseek_v4 import V4Attention

            self.self_attention = V4Attention(cfg, layer_idx, device, tp, mtp_depth)
        # hyper-connections (DeepSeek-V4): the residual stream is ``hc_mult`` parallel streams [T, K, H]; every sub-layer
        # reads a learned mixture of them and writes back through learned weights (models/deepseek_v4.py)
        self.hyper = cfg.hc_mult > 1
        if self.hyper:
            from .deepseek_v4 import HyperMixer

            assert self.mixer_kind is not None and self.has_mlp, "hyper-connections: layers of a mixer and an MLP"
            self.attn_hc = HyperMixer(cfg.hidden_size, cfg.hc_mult, cfg.hc_eps, cfg.hc_sinkhorn_iters, device)
            self.ffn_hc = HyperMixer(cfg.hidden_size, cfg.hc_mult, cfg.hc_eps, cfg.hc_sinkhorn_iters, device)
        # attention residuals (Kimi-K3): the sub-layers read a learned mixture of the running stream and the checkpoints
        # that every ``attn_res_block_size``-th layer sets aside; the checkpoints travel in the ``residual`` slot
        self.attn_res = bool(cfg.attn_res_block_size) and mtp_depth is None
        if self.attn_res:
            from .kimi_k3 import AttentionResidualMixer, checkpoints_before

            assert self.mixer_kind is not None and self.has_mlp, "attention residuals: layers of a mixer and an MLP"
            self.appends_checkpoint = layer_idx % cfg.attn_res_block_size == 0
            self.checkpoints_in = checkpoints_before(layer_idx, cfg.attn_res_block_size)
            if self.checkpoints_in:
                self.attn_res_mixer = AttentionResidualMixer(cfg, device)
            self.mlp_res_mixer = AttentionResidualMixer(cfg, device)
        self.is_moe = False
        if not self.has_mlp:
            return
        if cfg.is_moe_layer(layer_idx):
            from .moe import MoELayer

            self.pre_mlp_layernorm = ParamHolder(weight=_param((cfg.hidden_size,), 0, cfg.torch_dtype, device, True))
            self.pre_mlp_layernorm.weight.sequence_parallel = cfg.sequence_parallel
            self.mlp = MoELayer(cfg, layer_idx, device, tp)
            self.is_moe = True
        else:
            self.mlp = MLP(cfg, device, tp)

    def _drop(self, delta):
        """Hidden dropout on a sub-layer's output before it joins the residual stream (the bias-dropout-add of the
        reference's layers); sequence-parallel shards draw from the model-parallel stream."""
        p = self.cfg.hidden_dropout
        if p <= 0.0 or not self.training:
            return delta
        sp = self.cfg.sequence_parallel and ps.get_state().tp > 1
        return prandom.dropout(delta, p, True, sp)

    def _forward_attn_res(self, stream, checkpoints, rope, batch):
        """``stream`` [T, H]: the running residual sum since the last checkpoint; ``checkpoints`` [T, n, H] or None.
        Order of the reference's layer (primus/backends/megatron/core/models/kimi_k3/kimi_k3_block.py:521-552): mix,
        set the stream aside as a checkpoint and restart it (every ``attn_res_block_size``-th layer), mixer, mix, MLP."""
        n_in = 0 if checkpoints is None else checkpoints.shape[1]
        assert n_in == self.checkpoints_in, f"layer {self.layer_idx}: {n_in} checkpoints arrived, {self.checkpoints_in} expected"
        h = self.attn_res_mixer(stream, checkpoints) if self.checkpoints_in else stream
        if self.appends_checkpoint:
            checkpoints = stream[:, None] if checkpoints is None else torch.cat([checkpoints, stream[:, None]], 1)
            stream = None
        mixer = self.mixer if self.mixer_kind in ("mamba", "gdn", "kda") else self.self_attention
        attn_out = self._drop(mixer(h, None, rope, batch)[0])
        stream = attn_out if stream is None else stream + attn_out
        h = self.mlp_res_mixer(stream, checkpoints)
        if self.is_moe:
            mlp_out = self.mlp(fused.rmsnorm(h, self.pre_mlp_layernorm.weight, self.cfg.norm_epsilon))
        else:
            mlp_out = self.mlp(h, None)[0]
        return stream + self._drop(mlp_out), checkpoints

    def _forward_hyper(self, streams, rope, batch):
        """``streams`` [T, K, H].  The sub-layers see one collapsed stream each and carry their own input norms."""
        mixer = self.mixer if self.mixer_kind in ("mamba", "gdn", "kda") else self.self_attention
        streams = self.attn_hc.apply(streams, lambda h: self._drop(mixer(h, None, rope, batch)[0]))
        if self.is_moe:
            def ffn(h):
                return self._drop(self.mlp(fused.rmsnorm(h, self.pre_mlp_layernorm.weight, self.cfg.norm_epsilon)))
        else:
            def ffn(h):
                return self._drop(self.mlp(h, None)[0])
        return self.ffn_hc.apply(streams, ffn), None

    def forward(self, hidden, residual, rope, batch):
        if self.hyper:
            return self._forward_hyper(hidden, rope, batch)
        if self.attn_res:
            return self._forward_attn_res(hidden, residual, rope, batch)
        if self.mixer_kind is None:
            attn_out, res1 = hidden, residual
        else:
            mixer = self.mixer if self.mixer_kind in ("mamba", "gdn", "kda") else self.self_attention
            attn_out, res1 = mixer(hidden, residual, rope, batch)
            attn_out = self._drop(attn_out)
        if not self.has_mlp:
            return attn_out, res1
        if self.is_moe:
            if res1 is None:
                y, res2 = fused.rmsnorm(attn_out, self.pre_mlp_layernorm.weight, self.cfg.norm_epsilon), attn_out
            else:
                y, res2 = fused.rmsnorm(attn_out, self.pre_mlp_layernorm.weight, self.cfg.norm_epsilon, res1)
            mlp_out = self.mlp(y)
        elif res1 is None:
            mlp_out, res2 = selective_checkpoint(self.cfg, "mlp", lambda a: self.mlp(a, None), attn_out)
        else:
            mlp_out, res2 = selective_checkpoint(self.cfg, "mlp", self.mlp, attn_out, res1)
        return self._drop(mlp_out), res2


class LanguageModelEmbedding(nn.Module):
    def __init__(self, cfg: TransformerConfig, device, tp: int):
        super().__init__()
        V = cfg.padded_vocab_size // tp
        self.word_embeddings = ParamHolder(weight=_param((V, cfg.hidden_size), cfg.init_method_std, cfg.torch_dtype, device))
        self.word_embeddings.weight.tensor_model_parallel = tp > 1
        self.word_embeddings.weight.partition_dim = 0
        self.word_embeddings.weight._fp8_exempt = True   # also the LM head when embeddings are tied
        self.word_embeddings.weight._embedding_like = True
        self.vocab_local = V

    def forward(self, tokens_flat):
        st = ps.get_state()
        w = self.word_embeddings.weight
        if st.tp == 1:
            return fused.embedding(tokens_flat, w)
        out = fused.embedding(tokens_flat, w, st.tp_rank * self.vocab_local, partial=True)
        return out  # partial sums; caller reduces (all-reduce or reduce-scatter under SP)


class Decoder(nn.Module):
    def __init__(self, cfg: TransformerConfig, layer_indices, device, tp: int, post_process: bool):
        super().__init__()
        self.layers = nn.ModuleDict({str(i): TransformerLayer(cfg, i, device, tp) for i in layer_indices})
        self.layer_indices = list(layer_indices)
        if post_process:
            self.final_layernorm = ParamHolder(weight=_param((cfg.hidden_size,), 0, cfg.torch_dtype, device, True))
            self.final_layernorm.weight.sequence_parallel = cfg.sequence_parallel
            if cfg.hc_mult > 1:                 # collapse of the hyper-connection streams after the last layer
                from .deepseek_v4 import HyperHead

                self.hc_head = HyperHead(cfg.hidden_size, cfg.hc_mult, cfg.hc_eps, device)
            if cfg.attn_res_block_size:         # one more mix after the last layer collapses stream + checkpoints
                from .kimi_k3 import AttentionResidualMixer

                self.attn_res_head = AttentionResidualMixer(cfg, device)


class MultiTokenPredictionLayer(nn.Module):
    """One depth of multi-token prediction (DeepSeek-V3): the hidden state of the previous depth and the embedding of
    the token one further ahead are normalised, concatenated, projected back to ``hidden_size`` and run through one
    transformer layer; the shared output head then predicts the token after that.  Parameter names follow mcore:
    ``mtp.layers.{k}.{enorm,hnorm,eh_proj,transformer_layer.*,final_layernorm}``."""

    def __init__(self, cfg: TransformerConfig, device, tp: int, depth: int = 0):
        super().__init__()
        h = cfg.hidden_size
        self.enorm = ParamHolder(weight=_param((h,), 0, cfg.torch_dtype, device, True))
        self.hnorm = ParamHolder(weight=_param((h,), 0, cfg.torch_dtype, device, True))
        self.eh_proj = ParamHolder(weight=_param((h, 2 * h), cfg.init_method_std, cfg.torch_dtype, device))
        self.transformer_layer = TransformerLayer(cfg, cfg.num_layers - 1, device, tp, mtp_depth=depth)
        if cfg.hc_mult > 1:
            # hyper-connections: the projected input is copied into the streams, the inner layer mixes them, and every
            # depth collapses them with a head of its own (the reference's per-depth ``hc_head_fn``:
            # primus/backends/megatron/core/models/deepseek_v4/deepseek_v4_mtp_layer.py:10-22)
            from .deepseek_v4 import HyperHead

            self.hc_head = HyperHead(h, cfg.hc_mult, cfg.hc_eps, device)
        self.final_layernorm = ParamHolder(weight=_param((h,), 0, cfg.torch_dtype, device, True))
        # replicated over the tensor-parallel ranks; under sequence parallelism each rank sees its token shard only, so
        # their gradients are summed over the group like those of the other norm weights
        for holder in (self.enorm, self.hnorm, self.eh_proj, self.final_layernorm):
            holder.weight.sequence_parallel = cfg.sequence_parallel


class GPTModel(nn.Module):
    """One pipeline stage (or the whole model when PP=1) of a decoder-only LM.

    ``forward(tokens, labels, loss_weights, hidden_in=None)`` on the last stage returns per-token losses
    ``[batch, seq]``, or the scalar ``sum(loss_weights * loss)`` when weights are given, or logits when
    ``labels`` is None; other stages return the ``(delta, residual, batch, seq)`` hand-off."""

    def __init__(self, cfg: TransformerConfig, device="cpu", pre_process: bool = True, post_process: bool = True,
                 layer_indices: Optional[list[int]] = None):
        super().__init__()
        self.cfg = cfg
        self.pre_process = pre_process
        self.post_process = post_process
        tp = ps.get_state().tp
        if layer_indices is None:
            layer_indices = list(range(cfg.num_layers))
        if pre_process:
            self.embedding = LanguageModelEmbedding(cfg, device, tp)
        self.decoder = Decoder(cfg, layer_indices, device, tp, post_process)
        if post_process and cfg.untie_embeddings_and_output_weights:
            self.output_layer = ParamHolder(
                weight=_param((cfg.padded_vocab_size // tp, cfg.hidden_size), cfg.init_method_std, cfg.torch_dtype, device))
            self.output_layer.weight.tensor_model_parallel = tp > 1
            self.output_layer.weight.partition_dim = 0
            self.output_layer.weight._fp8_exempt = True   # the LM head stays in bf16 under an fp8 recipe
            self.output_layer.weight._embedding_like = True
        # Tied output head or multi-token prediction on a last stage that is not also the first: the stage holds a replica
        # of the word embeddings.  The first stage's copy is the trained one ("primary"); the trainer adds the replica's
        # gradient to it before the data-parallel reduction and re-sends the weights after every optimizer step (the
        # job of Megatron's embedding group; the replica is not an optimizer parameter, so it is counted once in the
        # gradient norm and saved once).
        needs_embedding = (not cfg.untie_embeddings_and_output_weights) or bool(cfg.mtp_num_layers)
        if needs_embedding and post_process and not pre_process:
            self.embedding = LanguageModelEmbedding(cfg, device, tp)
            self.embedding.word_embeddings.weight.embedding_replica = True
        if needs_embedding and pre_process and not post_process:
            self.embedding.word_embeddings.weight.embedding_primary = True
        if post_process and cfg.mtp_num_layers:
            st = ps.get_state()
            if st.cp > 1:
                raise NotImplementedError("multi-token prediction is not built for context parallelism")
            self.mtp = nn.Module()
            self.mtp.layers = nn.ModuleList([MultiTokenPredictionLayer(cfg, device, tp, depth)
                                             for depth in range(cfg.mtp_num_layers)])
        self._rope_cache = {}
        # ``first_last_layers_bf16``: under a low-precision recipe the GEMMs of the first ``num_layers_at_start_in_bf16``
        # and the last ``num_layers_at_end_in_bf16`` decoder layers stay in bf16 (the layers most sensitive to
        # quantisation noise; Transformer Engine's switch of the same name in the reference's argument set)
        if cfg.first_last_layers_bf16:
            keep = set(range(cfg.num_layers_at_start_in_bf16)) | \
                set(range(cfg.num_layers - cfg.num_layers_at_end_in_bf16, cfg.num_layers))
            for i in layer_indices:
                if i in keep:
                    for p_ in self.decoder.layers[str(i)].parameters():
                        if p_.dim() >= 2:
                            p_._fp8_exempt = True
        fused.set_situ_betas(cfg.activation_situ_beta, cfg.activation_situ_linear_beta)
        fused.set_zero_centered_gamma(cfg.apply_layernorm_1p)
        if cfg.apply_layernorm_1p:
            with torch.no_grad():
                for name, p in self.named_parameters():
                    if is_norm_gain(name):
                        p.zero_()

    # ------------------------------------------------------------------ pipeline hand-off
    # One tensor crosses a stage boundary.  Plain stacks send the residual stream ``hidden + residual`` [T, H];
    # hyper-connections send the K streams [T, K, H]; attention residuals send the running stream together with the
    # checkpoints set aside so far [T, 1 + n, H] -- n depends only on the index of the stage's first layer (the
    # reference folds the same extra axes into the sequence axis at stage boundaries:
    # primus/backends/megatron/core/models/deepseek_v4/deepseek_v4_block.py:341-432,
    # models/kimi_k3/kimi_k3_block.py:23-60).
    def handoff_shape(self, tokens: int) -> tuple:
        """Shape of the tensor this stage receives for ``tokens`` local tokens."""
        cfg = self.cfg
        if cfg.hc_mult > 1:
            return (tokens, cfg.hc_mult, cfg.hidden_size)
        if cfg.attn_res_block_size:
            from .kimi_k3 import checkpoints_before

            return (tokens, 1 + checkpoints_before(self.decoder.layer_indices[0], cfg.attn_res_block_size), cfg.hidden_size)
        return (tokens, cfg.hidden_size)

    def pack_handoff(self, hidden, residual):
        if self.cfg.attn_res_block_size:
            return hidden[:, None] if residual is None else torch.cat([hidden[:, None], residual], 1)
        return hidden if residual is None else hidden + residual

    def unpack_handoff(self, x):
        if self.cfg.attn_res_block_size:
            return x[:, 0].contiguous(), (x[:, 1:].contiguous() if x.shape[1] > 1 else None)
        return x, None

    # ------------------------------------------------------------------ helpers
    def rope_tables(self, device, seq: int):
        cfg = self.cfg
        d = cfg.qk_pos_emb_head_dim if cfg.multi_latent_attention else int(cfg.kv_channels * cfg.rotary_percent)
        key = (str(device), seq, d)
        if key not in self._rope_cache:
            l3 = dict(factor=cfg.rope_scaling_factor, low_freq_factor=cfg.rope_scaling_low_freq_factor,
                      high_freq_factor=cfg.rope_scaling_high_freq_factor,
                      original_max_pos=cfg.rope_scaling_original_max_position) if cfg.use_rope_scaling else None
            cos, sin = fused.rope_tables(max(seq, 1), d, cfg.rotary_base, device, cfg.rotary_scaling_factor, l3)
            self._rope_cache[key] = (cos, sin)
        return self._rope_cache[key]

    def output_weight(self):
        if self.cfg.untie_embeddings_and_output_weights:
            return self.output_layer.weight
        return self.embedding.word_embeddings.weight

    # ------------------------------------------------------------------ forward
    def forward(self, tokens=None, labels=None, loss_weights=None, hidden_in=None, position_ids=None,
                unit_upstream=False, cu_seqlens=None):
        """``cu_seqlens`` (host int tensor [batch, L], -1 padded): cumulative token offsets of the documents packed
        into each sequence; attention is then restricted to each document."""
        cfg = self.cfg
        st = ps.get_state()
        sp = cfg.sequence_parallel and st.tp > 1
        waiters = getattr(self, "_param_waiters", None)   # asynchronous parameter all-gathers (engine/trainer.py)
        if waiters is not None:
            waiters["embedding"]()
        if self.pre_process:
            batch, seq = tokens.shape
            x = self.embedding(tokens.reshape(-1))
            if st.tp > 1:
                x = tpc.reduce_scatter_seq(x, st.tp_group) if sp else tpc.all_reduce(x, st.tp_group)
            x = prandom.dropout(x, cfg.hidden_dropout, self.training, sp)     # embedding dropout
            if cfg.hc_mult > 1:
                x = x[:, None, :].expand(-1, cfg.hc_mult, -1).contiguous()    # every stream starts as the embedding
            hidden, residual = x, None
        else:
            hidden, residual, batch, seq = hidden_in
            if residual is None:
                hidden, residual = self.unpack_handoff(hidden)
        if tokens is not None:      # later pipeline stages get the ids from the schedule runner
            from . import moe as _moe

            _moe.TOKEN_IDS.current = tokens.reshape(-1)
        device = hidden.device
        # a context-parallel rank holds seq / cp of every sequence; a sequence chunk inside a pipeline is 1 / num_splits
        splits = layers.SEQ_SPLIT.num_splits if layers.SEQ_SPLIT.active else 1
        cos, sin = self.rope_tables(device, seq * st.cp * splits)
        pos = None
        if batch > 1 or position_ids is not None:
            pos = (position_ids.reshape(-1).to(torch.int32) if position_ids is not None
                   else torch.arange(seq, device=device, dtype=torch.int32).repeat(batch))
        rope = (cos, sin, pos, _segments(cu_seqlens, batch, seq))
        for group, ckpt in recompute_plan(cfg, self.decoder.layer_indices):
            hidden, residual = _run_group([self.decoder.layers[str(i)] for i in group], hidden, residual, rope, batch,
                                          cfg, ckpt)
        if not self.post_process:
            return hidden, residual, batch, seq
        if cfg.attn_res_block_size:
            hidden, residual = self.decoder.attn_res_head(hidden, residual), None
        if cfg.hc_mult > 1:
            hidden = self.decoder.hc_head(hidden)
        if waiters is not None:
            waiters["head"]()
        w = self.output_weight()
        mtp_loss = None
        if cfg.mtp_num_layers and labels is not None and loss_weights is not None:
            mtp_loss = self._mtp_loss(hidden, residual, tokens, labels, loss_weights, rope, batch, seq, w, unit_upstream)
        if labels is None:
            y, _ = fused.rmsnorm(hidden, self.decoder.final_layernorm.weight, cfg.norm_epsilon, residual) \
                if residual is not None else (fused.rmsnorm(hidden, self.decoder.final_layernorm.weight, cfg.norm_epsilon), None)
            if sp:
                y = tpc.gather_seq(y, st.tp_group)
            return fused.softcap(gemm.linear(y, w), cfg.final_logit_softcapping)
        if (cfg.cross_entropy_chunk_tokens > 0 and loss_weights is not None and unit_upstream and st.tp == 1
                and not cfg.final_logit_softcapping):
            # chunked linear + cross entropy: no [tokens, vocab] logits tensor
            y = fused.rmsnorm(hidden, self.decoder.final_layernorm.weight, cfg.norm_epsilon, residual)[0] \
                if residual is not None else fused.rmsnorm(hidden, self.decoder.final_layernorm.weight, cfg.norm_epsilon)
            loss = layers.chunked_linear_cross_entropy(y, w, labels.reshape(-1), loss_weights.reshape(-1), 0,
                                                       cfg.cross_entropy_chunk_tokens)
            return loss if mtp_loss is None else loss + mtp_loss
        logits, _ = layers.norm_linear(hidden, residual, self.decoder.final_layernorm.weight, w, cfg.norm_epsilon,
                                       st.tp_group, sp)
        logits = fused.softcap(logits, cfg.final_logit_softcapping)
        vocab_local = w.shape[0]
        loss = fused.cross_entropy(logits, labels.reshape(-1), st.tp_rank * vocab_local,
                                   st.tp_group if st.tp > 1 else None,
                                   None if loss_weights is None else loss_weights.reshape(-1), unit_upstream)
        if mtp_loss is not None:
            loss = loss + mtp_loss
        return loss if loss_weights is not None else loss.view(batch, seq)

    def _mtp_loss(self, hidden, residual, tokens, labels, loss_weights, rope, batch, seq, w_out, unit_upstream):
        """sum_k scale / D * CE(depth k): depth k (1-based) sees tokens shifted left by k and predicts labels shifted
        left by k; the last k positions of every sequence carry no target and get weight 0."""
        cfg = self.cfg
        st = ps.get_state()
        sp = cfg.sequence_parallel and st.tp > 1
        h = hidden if residual is None else hidden + residual
        tok, lab = tokens.reshape(batch, seq), labels.reshape(batch, seq)
        wts = loss_weights.reshape(batch, seq)
        total = None
        for k, layer in enumerate(self.mtp.layers, start=1):
            tok, lab, wts = torch.roll(tok, -1, 1), torch.roll(lab, -1, 1), torch.roll(wts, -1, 1).clone()
            wts[:, seq - k:] = 0
            e = self.embedding(tok.reshape(-1))
            if st.tp > 1:   # vocab-parallel partial sums -> this rank's tokens (all of them, or its sequence shard)
                e = tpc.reduce_scatter_seq(e, st.tp_group) if sp else tpc.all_reduce(e, st.tp_group)
            x = torch.cat([fused.rmsnorm(e, layer.enorm.weight, cfg.norm_epsilon),
                           fused.rmsnorm(h, layer.hnorm.weight, cfg.norm_epsilon)], -1)
            x = gemm.linear(x, layer.eh_proj.weight)
            if cfg.hc_mult > 1:
                x = x[:, None, :].expand(-1, cfg.hc_mult, -1).contiguous()
            hid, res = layer.transformer_layer(x, None, rope, batch)
            if cfg.hc_mult > 1:
                hid, res = layer.hc_head(hid), None
            logits, _ = layers.norm_linear(hid, res, layer.final_layernorm.weight, w_out, cfg.norm_epsilon,
                                           st.tp_group, sp)
            logits = fused.softcap(logits, cfg.final_logit_softcapping)
            lk = fused.cross_entropy(logits, lab.reshape(-1), st.tp_rank * w_out.shape[0],
                                     st.tp_group if st.tp > 1 else None, wts.reshape(-1), unit_upstream)
            total = lk if total is None else total + lk
            h = hid if res is None else hid + res
        return total * (cfg.mtp_loss_scaling_factor / cfg.mtp_num_layers)


def _segments(cu_seqlens, batch: int, seq: int):
    """[(start, end)] token ranges in the flattened [batch * seq] layout, or None."""
    if cu_seqlens is None:
        return None
    rows = cu_seqlens.reshape(batch, -1).tolist()
    segs = []
    for b, row in enumerate(rows):
        cu = [c for c in row if c >= 0]
        segs += [(b * seq + a, b * seq + e) for a, e in zip(cu[:-1], cu[1:]) if e > a]
    return segs


def recompute_plan(cfg, layer_indices) -> list:
    """Groups of consecutive layers of this model chunk and whether each group is run under activation checkpointing
    (only the group's input is kept; its layers run again in the backward pass).  ``recompute_granularity: full``:

    * ``recompute_layer_ids`` given: exactly those (global) layers, one checkpoint each;
    * ``recompute_method: uniform``: the chunk is cut into groups of ``recompute_num_layers`` layers, every group is one
      checkpoint (larger groups keep fewer inputs and recompute the same amount);
    * ``recompute_method: block``: the first ``recompute_num_layers`` layers of the chunk are checkpointed one by one,
      the rest keep their activations (for when only part of the memory has to be saved);
    * neither: every layer is its own checkpoint.

    Semantics of Megatron's ``recompute_granularity / recompute_method / recompute_num_layers``
    (primus/configs/modules/megatron/trainer_base.yaml:248-254 in the reference) plus the reference's explicit layer list
    (primus/backends/megatron/patches/recompute_layer_patches.py:326)."""
    idx = list(layer_indices)
    if cfg.recompute_granularity != "full":
        return [([i], False) for i in idx]
    if cfg.recompute_layer_ids is not None:
        ids = set(cfg.recompute_layer_ids)
        return [([i], i in ids) for i in idx]
    method = (cfg.recompute_method or "").lower() or None
    n = cfg.recompute_num_layers
    if method == "uniform":
        n = max(int(n or 1), 1)
        return [(idx[a:a + n], True) for a in range(0, len(idx), n)]
    if method == "block":
        n = len(idx) if n is None else max(int(n), 0)
        return [([i], pos < n) for pos, i in enumerate(idx)]
    if method is not None:
        raise ValueError(f"recompute_method {cfg.recompute_method!r}: uniform or block")
    return [([i], True) for i in idx]


def _run_group(layers_, hidden, residual, rope, batch, cfg, checkpointed: bool):
    def run(h, r):
        for layer in layers_:
            h, r = _run_layer(layer, h, r, rope, batch, cfg)
        return h, r

    if checkpointed and torch.is_grad_enabled():
        if residual is None:
            return prandom.checkpoint(lambda h: run(h, None), hidden)
        return prandom.checkpoint(run, hidden, residual)
    return run(hidden, residual)


def _run_layer(layer, hidden, residual, rope, batch, cfg):
    if cfg.cpu_offloading and torch.is_grad_enabled() and hidden.is_cuda and (
            layer.layer_idx < (cfg.cpu_offloading_num_layers or 0)):
        from ..engine.offload import offload_saved_activations

        with offload_saved_activations():
            return layer(hidden, residual, rope, batch)
    return layer(hidden, residual, rope, batch)


def selective_checkpoint(cfg, module: str, fn, *args):
    """``recompute_granularity: selective``: run ``fn(*args)`` under activation checkpointing when ``module`` is in
    ``recompute_modules`` (default: the core attention only, whose saved output and statistics are then rebuilt from
    q / k / v in the backward pass)."""
    if cfg.recompute_granularity == "selective" and torch.is_grad_enabled() and \
            module in (cfg.recompute_modules or ["core_attn"]):
        return prandom.checkpoint(fn, *args)
    return fn(*args)


def build_model(cfg: TransformerConfig, device="cpu", stage_id: int = 0, n_stages: int = 1,
                seed: Optional[int] = None, layout: Optional[str] = None, manual_split=None) -> GPTModel:
    """Build the model chunk that owns global (virtual) pipeline stage ``stage_id`` of ``n_stages``."""
    from ..parallel.pipeline_layout import layers_for_stage

    idx = layers_for_stage(cfg.num_layers, n_stages, stage_id, None, None, layout, manual_split)
    if seed is not None:
        st = ps.get_state()
        torch.manual_seed(seed + 100 * stage_id + 2718 * st.tp_rank)
    return GPTModel(cfg, device, pre_process=(stage_id == 0), post_process=(stage_id == n_stages - 1),
                    layer_indices=idx)
