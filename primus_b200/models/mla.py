"""Multi-latent attention (DeepSeek-V2 / V3).

    q   = W_q y                                   (or  W_uq rmsnorm(W_dq y)  with q-LoRA)
    c   = W_dkv y  -> [latent (kv_lora_rank) | k_pe (rope dim)]
    k,v = W_ukv rmsnorm(latent)  per head: k_nope (qk_head_dim), v (v_head_dim)
    attention over q = [rope(q_pe) | q_nope], k = [rope(k_pe) shared by all heads | k_nope]   (d_qk = 192, d_v = 128)

The rotary part is placed first inside each head (both in q and k, so the dot products are unchanged),
which lets the in-place RoPE kernel work on a prefix of the head.  YaRN frequency scaling and the
``mscale`` softmax-scale correction follow the DeepSeek recipe (rotary_scaling_factor 40, mscale 0.707:
primus/configs/models/megatron/deepseek_v2_base.yaml in the reference).

Parameter names match the reference's converter (primus/backends/megatron/checkpoint/native_loader_deepseek.py:252-302):
``input_layernorm.weight``, ``self_attention.linear_q_proj.weight`` | (``linear_q_down_proj``, ``linear_q_up_proj`` +
``linear_q_up_proj.layer_norm_weight``), ``linear_kv_down_proj.weight``, ``linear_kv_up_proj.weight`` +
``linear_kv_up_proj.layer_norm_weight``, ``linear_proj.weight``.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import attention, fused, gemm, layers
from ..parallel import state as ps
from ..parallel import tensor_parallel as tpc
from .config import TransformerConfig


def yarn_inv_freq(dim: int, base: float, factor: float, original_max_pos: int = 4096, beta_fast: float = 32.0,
                  beta_slow: float = 1.0, device="cpu") -> torch.Tensor:
    """YaRN: blend of interpolated (1/factor) and extrapolated frequencies with a linear ramp between the
    dimensions whose wavelength covers beta_fast .. beta_slow rotations of the original context."""
    exps = torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim
    extra = 1.0 / (base ** exps)
    inter = extra / factor

    def corr_dim(n_rot):
        return dim * math.log(original_max_pos / (n_rot * 2 * math.pi)) / (2 * math.log(base))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    return inter * (1 - mask) + extra * mask


def yarn_mscale(factor: float, mscale: float) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


class MLASelfAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, layer_idx: int, device, tp: int):
        super().__init__()
        from .gpt import ParamHolder, _param

        # Tensor parallelism splits the heads: the up-projections are column-parallel, the output projection is
        # row-parallel; the two down-projections and the norms are replicated and work on this rank's tokens (under
        # sequence parallelism their gradients are partial sums, added over the group like those of the norm weights).
        assert cfg.num_attention_heads % tp == 0, "attention heads must divide by the tensor-parallel size"
        self.cfg = cfg
        self.tp = tp
        dt = cfg.torch_dtype
        h, nh = cfg.hidden_size, cfg.num_attention_heads // tp
        self.nh = nh
        self.dn, self.dr, self.dv = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
        std = cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        qd = self.dn + self.dr
        self.input_layernorm = ParamHolder(weight=_param((h,), 0, dt, device, True))
        if cfg.q_lora_rank:
            self.linear_q_down_proj = ParamHolder(weight=_param((cfg.q_lora_rank, h), std, dt, device))
            self.linear_q_up_proj = ParamHolder(layer_norm_weight=_param((cfg.q_lora_rank,), 0, dt, device, True),
                                                weight=_param((nh * qd, cfg.q_lora_rank), std, dt, device))
        else:
            self.linear_q_proj = ParamHolder(weight=_param((nh * qd, h), std, dt, device))
        self.linear_kv_down_proj = ParamHolder(weight=_param((cfg.kv_lora_rank + self.dr, h), std, dt, device))
        self.linear_kv_up_proj = ParamHolder(layer_norm_weight=_param((cfg.kv_lora_rank,), 0, dt, device, True),
                                             weight=_param((nh * (self.dn + self.dv), cfg.kv_lora_rank), std, dt, device))
        self.linear_proj = ParamHolder(weight=_param((h, nh * self.dv), out_std, dt, device))
        if cfg.mla_use_output_gate:
            # Kimi-K3: attention output times sigmoid(gate), the gate projected from the normalised layer input
            # (primus/backends/megatron/core/transformer/kimi_k3/kimi_k3_mla_attention.py:68-92 in the reference)
            self.linear_o_gate = ParamHolder(weight=_param((nh * self.dv, h), std, dt, device))
        if tp > 1:
            sp = bool(cfg.sequence_parallel)
            split = [(self.linear_kv_up_proj.weight, 0), (self.linear_proj.weight, 1)]
            replicated = [self.input_layernorm.weight, self.linear_kv_down_proj.weight, self.linear_kv_up_proj.layer_norm_weight]
            if cfg.q_lora_rank:
                split.append((self.linear_q_up_proj.weight, 0))
                replicated += [self.linear_q_down_proj.weight, self.linear_q_up_proj.layer_norm_weight]
            else:
                split.append((self.linear_q_proj.weight, 0))
            if cfg.mla_use_output_gate:
                split.append((self.linear_o_gate.weight, 0))
            for w, dim in split:
                w.tensor_model_parallel, w.partition_dim = True, dim
            st = ps.get_state()
            for w in replicated:
                w.sequence_parallel = sp
                if w.dim() == 2 and torch.distributed.is_initialized():     # drawn per rank: make the replicas equal
                    torch.distributed.broadcast(w.data, src=st.tp_ranks[0], group=st.tp_group)
        factor = cfg.rotary_scaling_factor or 1.0
        m = yarn_mscale(factor, cfg.mscale)
        self.softmax_scale = (m * m) / math.sqrt(qd)
        self._tables = {}

    def rope_tables(self, device, seq: int):
        key = (str(device), seq)
        if key not in self._tables:
            cfg = self.cfg
            factor = cfg.rotary_scaling_factor or 1.0
            if factor > 1:
                inv = yarn_inv_freq(self.dr, cfg.rotary_base, factor, device=device)
            else:
                inv = 1.0 / (cfg.rotary_base ** (torch.arange(0, self.dr, 2, dtype=torch.float32, device=device) / self.dr))
            f = torch.outer(torch.arange(seq, dtype=torch.float32, device=device), inv)
            self._tables[key] = (f.cos().contiguous(), f.sin().contiguous())
        return self._tables[key]

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        nh, dn, dr, dv = self.nh, self.dn, self.dr, self.dv
        if residual is not None:
            y, xsum = fused.rmsnorm(hidden, self.input_layernorm.weight, cfg.norm_epsilon, residual)
        else:
            y, xsum = fused.rmsnorm(hidden, self.input_layernorm.weight, cfg.norm_epsilon), hidden
        st = ps.get_state()
        tpg = st.tp_group if self.tp > 1 else None
        sp = bool(cfg.sequence_parallel) and self.tp > 1

        def everywhere(t):
            """Input of a column-parallel projection: all tokens on every rank (gathered under sequence parallelism;
            otherwise already there, and the gradients of the ranks' head slices are added in the backward pass)."""
            if tpg is None:
                return t
            return tpc.gather_seq(t, tpg) if sp else tpc.copy_to_tp(t, tpg)

        T = y.shape[0] * (self.tp if sp else 1)
        seq = T // batch
        cos, sin = self.rope_tables(y.device, seq * st.cp)   # positions are global under context parallelism
        pos = rope[2]
        if cfg.attn_logit_softcapping:
            raise NotImplementedError("attn_logit_softcapping is not built for multi-latent attention")
        if len(rope) > 3 and rope[3]:
            raise NotImplementedError("per-document attention (packed sequences) is not built for multi-latent attention")
        if cfg.q_lora_rank:
            ql = gemm.linear(y, self.linear_q_down_proj.weight)
            ql = fused.rmsnorm(ql, self.linear_q_up_proj.layer_norm_weight, cfg.norm_epsilon)
            q = gemm.linear(everywhere(ql), self.linear_q_up_proj.weight)
        else:
            q = gemm.linear(everywhere(y), self.linear_q_proj.weight)
        q = q.view(T, nh, dn + dr)
        c = gemm.linear(y, self.linear_kv_down_proj.weight)
        latent = fused.rmsnorm(c[:, :cfg.kv_lora_rank].contiguous(), self.linear_kv_up_proj.layer_norm_weight,
                               cfg.norm_epsilon)
        k_pe = everywhere(c[:, cfg.kv_lora_rank:].contiguous()).reshape(T, 1, dr)
        kv = gemm.linear(everywhere(latent), self.linear_kv_up_proj.weight).view(T, nh, dn + dv)
        if cfg.mla_use_nope:
            # no rotation: the dr "rope" dims of q and the shared key dims are ordinary learned features; the head
            # geometry and the softmax scale stay those of the rotary layout (kimi_k3_mla_attention.py:24-60)
            q_pe = q[..., dn:]
        else:
            q_pe = fused.rope(q[..., dn:].contiguous(), cos, sin, pos, dr)
            k_pe = fused.rope(k_pe.contiguous(), cos, sin, pos, dr)
        q_full = torch.cat([q_pe, q[..., :dn]], dim=-1)
        k_full = torch.cat([k_pe.expand(T, nh, dr), kv[..., :dn]], dim=-1)
        v = kv[..., dn:].contiguous()
        if st.cp > 1:
            if cfg.cp_comm_type == "p2p":
                ctx_out = layers.ring_cp_attention(q_full.contiguous(), k_full.contiguous(), v, batch, st.cp_group, st.cp,
                                                   self.softmax_scale)
            elif cfg.cp_comm_type != "allgather":
                raise NotImplementedError("multi-latent attention under context parallelism needs cp_comm_type "
                                          "allgather or p2p")
            else:
                ctx_out = layers.allgather_cp_attention(q_full.contiguous(), k_full.contiguous(), v, batch, st.cp_group,
                                                        st.cp, True, self.softmax_scale)
        else:
            ctx_out = attention.flash_attention(q_full, k_full, v, batch, True, self.softmax_scale)
        ctx_out = ctx_out.reshape(T, nh * dv)
        if cfg.mla_use_output_gate:
            gate = gemm.linear(everywhere(y), self.linear_o_gate.weight)
            ctx_out = (ctx_out * torch.sigmoid(gate.float()).to(ctx_out.dtype)).contiguous()
        out = layers.row_parallel_linear(ctx_out.contiguous(), self.linear_proj.weight, tpg, sp)
        return out, xsum
