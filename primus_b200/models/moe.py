"""Mixture-of-experts layer: router + routed experts (grouped GEMMs) + optional shared experts.

Parameter names: ``router.weight [E, H]`` (+ ``router.expert_bias``), stacked routed experts
``experts.fc1_weight.weight [E_local, 2I, H]`` / ``experts.fc2_weight.weight [E_local, H, I]`` (the EP-sharded
layout of the reference's MegaMoE module, primus/backends/megatron/core/extensions/mega_moe.py:272-305),
``shared_experts.linear_fc{1,2}.weight``.  The checkpoint module splits the stacked tensors into the
per-expert ``linear_fc1.weight{e}`` keys of the grouped-MLP layout on request.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import fused, gemm, layers
from ..ops import moe as moe_ops
from ..parallel import expert_parallel as epc
from ..parallel import state as ps
from .config import TransformerConfig


class AuxLossScaler(torch.autograd.Function):
    """Identity on the activation that injects d(aux_loss) into the backward pass (scaled like the main loss)."""
    scale = 1.0

    @staticmethod
    def forward(ctx, x, aux_loss):
        ctx.save_for_backward(aux_loss)
        return x

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.ones_like(aux) * AuxLossScaler.scale


class _TokenIds:
    """Token ids of the micro-batch in flight ([batch * seq], set by the model's forward pass): hash-routed layers
    index their expert table with them."""
    current = None


TOKEN_IDS = _TokenIds()


class MoELayer(nn.Module):
    def __init__(self, cfg: TransformerConfig, layer_idx: int, device, tp: int):
        super().__init__()
        from .gpt import MLP, ParamHolder, _param

        # Under tensor parallelism the layer works on each rank's sequence shard: the TP ranks are just more ranks with
        # their own tokens (expert tensor parallelism 1), so experts are sharded over the expert-parallel group --
        # which spans the TP ranks -- and router / shared-expert weights are replicated, with their gradients summed
        # over the TP group like those of the norm weights.
        if tp > 1 and not cfg.sequence_parallel:
            raise ValueError("MoE layers under tensor parallelism need sequence_parallel (each rank routes its own tokens)")
        self.cfg = cfg
        self.layer_idx = layer_idx
        st = ps.get_state()
        self.ep, self.ep_rank = st.ep, st.ep_rank
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_ffn_hidden_size
        # latent mixture of experts (Kimi-K3): one down- and one up-projection shared by all experts of the layer put
        # the routed experts in a narrower space; the router and the shared experts read the full-width input, and the
        # combined expert output is normalised before it is lifted back
        # (primus/backends/megatron/core/transformer/kimi_k3/moe/k3_stable_latent_moe.py:14-45 in the reference)
        self.latent = int(cfg.routed_expert_hidden_size or 0)
        Hx = self.latent or H
        assert E % self.ep == 0
        self.e_local = E // self.ep
        dt = cfg.torch_dtype
        std = cfg.init_method_std
        out_std = std / math.sqrt(2.0 * cfg.num_layers)
        self.router = ParamHolder(weight=_param((E, H), std, dt, device))
        if cfg.moe_router_enable_expert_bias:
            self.router.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32, device=device))
            # tokens routed to every expert since the last bias update (this rank's tokens)
            self.router.register_buffer("local_tokens_per_expert", torch.zeros(E, dtype=torch.float32, device=device),
                                        persistent=False)
        # every EP rank draws the full expert set from the same stream and keeps its slice, so that the
        # initial weights do not depend on the EP size
        g = torch.Generator(device="cpu").manual_seed(977 + 31 * layer_idx)
        lo, hi = self.ep_rank * self.e_local, (self.ep_rank + 1) * self.e_local
        w1 = torch.empty(E, 2 * I, Hx).normal_(0.0, std, generator=g)[lo:hi].to(dt).to(device)
        w2 = torch.empty(E, Hx, I).normal_(0.0, out_std, generator=g)[lo:hi].to(dt).to(device)
        self.experts = nn.Module()
        self.experts.fc1_weight = ParamHolder(weight=nn.Parameter(w1.contiguous()))
        self.experts.fc2_weight = ParamHolder(weight=nn.Parameter(w2.contiguous()))
        for p in (self.experts.fc1_weight.weight, self.experts.fc2_weight.weight):
            p.is_expert = self.ep > 1
            p.expert_parallel = self.ep > 1
            # without expert parallelism the experts are replicas that see one sequence shard each
            p.sequence_parallel = tp > 1 and self.ep == 1
        if self.latent:
            self.fc1_latent_proj = ParamHolder(weight=_param((Hx, H), std, dt, device))
            self.fc2_latent_proj = ParamHolder(weight=_param((H, Hx), out_std, dt, device))
            if cfg.latent_moe_use_norm:
                self.latent_norm = ParamHolder(weight=_param((Hx,), 0, dt, device, True))
        if cfg.moe_router_enable_expert_bias and cfg.moe_router_bias_update_rule == "quantile":
            # quantile balancing (models/kimi_k3.py): histograms of this rank's routing margins since the last update
            self.router.register_buffer("local_margin_histogram", torch.zeros(
                E, cfg.quantile_balancing_num_bins, dtype=torch.int64, device=device), persistent=False)
            self._qb_steps = 0
        # DeepSeek-V4: the first ``num_hash_layers`` MoE layers take their experts from a fixed table indexed by the token
        # id (the weights still come from the learned gate); the table travels with the checkpoint
        moe_rank = sum(cfg.moe_layer_pattern[:layer_idx])
        if cfg.num_hash_layers and moe_rank < cfg.num_hash_layers:
            from .deepseek_v4 import hash_table

            self.router.register_buffer("tid2eid", hash_table(
                cfg.padded_vocab_size, E, cfg.moe_router_topk, cfg.hash_router_seed + layer_idx).to(device))
        if cfg.moe_shared_expert_intermediate_size:
            self.shared_experts = MLP(cfg, device, 1, ffn=cfg.moe_shared_expert_intermediate_size, with_norm=False)
            if cfg.moe_shared_expert_gate:      # Qwen MoE: the shared expert's output is scaled by sigmoid(y . gate)
                self.shared_experts.register_parameter("gate_weight", _param((1, H), std, dt, device))
        if tp > 1:
            replicated = [self.router.weight] + ([p for p in self.shared_experts.parameters()]
                                                 if hasattr(self, "shared_experts") else [])
            for name in ("fc1_latent_proj", "fc2_latent_proj", "latent_norm"):
                if hasattr(self, name):
                    replicated.append(getattr(self, name).weight)
            for p in replicated:
                p.sequence_parallel = True
                if torch.distributed.is_initialized():      # drawn from per-rank streams: make the replicas equal
                    torch.distributed.broadcast(p.data, src=st.tp_ranks[0], group=st.tp_group)
        self.last_aux_loss = None
        self.last_tokens_per_expert = None

    # ------------------------------------------------------------------
    def route(self, y):
        cfg = self.cfg
        logits = fused.softcap(gemm.linear(y, self.router.weight), cfg.router_logit_softcapping)
        bias = getattr(self.router, "expert_bias", None)
        fixed = None
        if hasattr(self.router, "tid2eid"):
            ids = TOKEN_IDS.current
            st_ = ps.get_state()
            if ids is not None and st_.tp > 1 and ids.numel() == y.shape[0] * st_.tp:
                ids = ids.reshape(-1)[st_.tp_rank * y.shape[0]:(st_.tp_rank + 1) * y.shape[0]]   # this rank's sequence shard
            if ids is None or ids.numel() != y.shape[0]:
                raise RuntimeError("hash-routed MoE layer: the token ids of the micro-batch are not available")
            fixed = self.router.tid2eid[ids.long()]
        probs, idx, full, counts = moe_ops.router_scores(
            logits, cfg.moe_router_topk, cfg.moe_router_score_function, cfg.moe_router_pre_softmax, bias,
            cfg.moe_router_topk_scaling_factor, cfg.moe_router_num_groups, cfg.moe_router_group_topk,
            return_counts=True, fixed_idx=fixed)
        if cfg.moe_router_force_load_balancing:
            T = y.shape[0]
            k = cfg.moe_router_topk
            idx = (torch.arange(T * k, device=y.device) % cfg.num_experts).view(T, k)
            probs = torch.full_like(probs, 1.0 / k)
            counts = torch.bincount(idx.reshape(-1), minlength=cfg.num_experts).to(torch.int32)
        if bias is not None and torch.is_grad_enabled():
            self.router.local_tokens_per_expert += counts.float()
            if hasattr(self.router, "local_margin_histogram") and self.training:
                from .kimi_k3 import margin_histogram

                self.router.local_margin_histogram += margin_histogram(
                    full.detach(), bias, cfg.moe_router_topk, cfg.quantile_balancing_num_bins,
                    cfg.quantile_balancing_margin_min, cfg.quantile_balancing_margin_max)
        aux = None
        if cfg.moe_aux_loss_coeff and cfg.moe_router_load_balancing_type in ("aux_loss", "seq_aux_loss") \
                and torch.is_grad_enabled():
            seq = cfg.seq_length if cfg.moe_router_load_balancing_type == "seq_aux_loss" and \
                y.shape[0] % cfg.seq_length == 0 else None
            aux = moe_ops.load_balancing_loss(full, idx, cfg.num_experts, cfg.moe_router_topk,
                                              cfg.moe_aux_loss_coeff, seq)
            probs = AuxLossScaler.apply(probs, aux)
            self.last_aux_loss = aux.detach()
        return probs, idx, counts

    @torch.no_grad()
    def update_expert_bias(self, groups=()) -> None:
        """Auxiliary-loss-free load balancing (DeepSeek-V3): after an optimizer step every expert's selection bias moves
        by ``moe_router_bias_update_rate`` towards the mean load, using the token counts of the whole global batch
        (``groups``: the process groups whose ranks saw different tokens).  The reference takes this from Megatron's
        router (``moe_router_enable_expert_bias`` / ``moe_router_bias_update_rate`` in its DeepSeek-V3 presets)."""
        r = self.router
        if hasattr(r, "local_margin_histogram"):
            return self._update_expert_bias_quantile(groups)
        if not hasattr(r, "expert_bias") or not self.cfg.moe_router_bias_update_rate:
            return
        load = r.local_tokens_per_expert.clone()
        for g in groups:
            if g is not None and torch.distributed.get_world_size(g) > 1:
                torch.distributed.all_reduce(load, group=g)
        r.expert_bias += self.cfg.moe_router_bias_update_rate * torch.sign(load.mean() - load)
        r.local_tokens_per_expert.zero_()

    @torch.no_grad()
    def _update_expert_bias_quantile(self, groups=()) -> None:
        """Quantile balancing: the bias is *set* to minus the ``1 - k/E`` quantile of every expert's routing margins over
        the global batch (histograms summed over micro-batches and, by one all-reduce per group, over ranks), mean
        removed; ``quantile_balancing_update_interval`` widens the window and ``quantile_balancing_ema_decay`` blends
        the new value into the old one.  The reference's replacement for the sign rule
        (primus/backends/megatron/core/transformer/kimi_k3/moe/k3_quantile_balancing.py:14-60,232-250)."""
        from .kimi_k3 import quantile_bias

        cfg, r = self.cfg, self.router
        self._qb_steps += 1
        if self._qb_steps % max(int(cfg.quantile_balancing_update_interval), 1):
            return
        hist = r.local_margin_histogram.clone()
        for g in groups:
            if g is not None and torch.distributed.get_world_size(g) > 1:
                torch.distributed.all_reduce(hist, group=g)
        if int(hist.sum()) > 0:
            new = quantile_bias(hist, cfg.moe_router_topk, cfg.quantile_balancing_margin_min,
                                cfg.quantile_balancing_margin_max, cfg.quantile_balancing_center_bias).to(r.expert_bias)
            d = cfg.quantile_balancing_ema_decay
            r.expert_bias.copy_(new if not d else d * r.expert_bias + (1.0 - d) * new)
        r.local_margin_histogram.zero_()
        r.local_tokens_per_expert.zero_()

    def experts_forward(self, x_perm, probs_perm, sched):
        cfg = self.cfg
        h1 = moe_ops.grouped_linear(x_perm, self.experts.fc1_weight.weight, sched)
        act = fused.swiglu(h1, probs_perm, cfg.activation_func_clamp_value, cfg.gated_activation)
        return moe_ops.grouped_linear(act, self.experts.fc2_weight.weight, sched)

    def forward(self, y):
        cfg = self.cfg
        T, H = y.shape
        k = cfg.moe_router_topk
        probs, idx, counts_global = self.route(y)
        flat_e = idx.reshape(-1)
        self.last_tokens_per_expert = counts_global
        x = gemm.linear(y, self.fc1_latent_proj.weight) if self.latent else y
        if cfg.use_turbo_mega_moe and y.is_cuda:
            out = self._forward_fused(x, probs, idx, T, k)
        elif self.ep == 1:
            out = self._forward_local(x, probs, flat_e, counts_global, T, k)
        else:
            out = self._forward_ep(x, probs, flat_e, counts_global, T, k)
        if self.latent:
            if hasattr(self, "latent_norm"):
                out = fused.rmsnorm(out, self.latent_norm.weight, cfg.norm_epsilon)
            out = gemm.linear(out, self.fc2_latent_proj.weight)
        if hasattr(self, "shared_experts"):
            shared = self.shared_experts.forward_normed(y)
            if cfg.moe_shared_expert_gate:
                g = torch.sigmoid(torch.nn.functional.linear(y.float(), self.shared_experts.gate_weight.float()))
                shared = shared * g.to(shared.dtype)
            out = out + shared
        return out

    # ------------------------------------------------------------------ single rank
    def _forward_local(self, y, probs, flat_e, counts, T, k):
        rows_cap = moe_ops.rows_capacity(T * k, self.e_local)
        sched = moe_ops.build_schedule(counts.to(torch.int32), rows_cap)
        src, pos = moe_ops.permutation_maps(flat_e, sched)
        src_token = torch.where(src >= 0, src // k, src)
        inv_pos = pos.view(T, k)
        x_perm = moe_ops.gather_rows(y, src_token, inv_pos)
        pf = torch.cat([probs.reshape(-1).float(), probs.new_zeros(1, dtype=torch.float32)])
        probs_perm = pf[src.long()]  # src = -1 picks the appended zero
        out_perm = self.experts_forward(x_perm, probs_perm, sched)
        return moe_ops.combine_rows(out_perm, inv_pos, src_token)

    # ------------------------------------------------------------------ fused dispatch / combine (symmetric memory)
    def _forward_fused(self, y, probs, idx, T, k):
        """Dispatch and combine fused into the expert GEMMs; no host synchronisation on the routing result."""
        from ..parallel import fused_ep

        cfg = self.cfg
        st = ps.get_state()
        ws = fused_ep.get_workspace(st.ep_group if self.ep > 1 else None, T, k, cfg.num_experts, y.shape[1],
                                    cfg.moe_fused_capacity_factor)
        plan = ws.plan(idx, probs)
        h1, probs_perm = fused_ep.dispatch_gemm1(y, probs, self.experts.fc1_weight.weight, ws, plan)
        act = fused.swiglu(h1, probs_perm, cfg.activation_func_clamp_value, cfg.gated_activation)
        return fused_ep.gemm2_combine(act, self.experts.fc2_weight.weight, ws, plan)

    # ------------------------------------------------------------------ expert parallel (NCCL all-to-all)
    def _forward_ep(self, y, probs, flat_e, counts_global, T, k):
        st = ps.get_state()
        dev = y.device
        in_splits, out_splits, recv_counts = epc.exchange_counts(counts_global, self.ep, self.ep_rank, st.ep_group)
        order = torch.argsort(flat_e, stable=True)              # copies sorted by global expert = by destination
        inv_order = torch.empty_like(order)
        inv_order[order] = torch.arange(order.numel(), device=dev)
        tok_sorted = (order // k).to(torch.int32)
        send = moe_ops.gather_rows(y, tok_sorted, inv_order.view(T, k).to(torch.int32))
        send_probs = probs.reshape(-1).float()[order]
        recv = epc.all_to_all(send, in_splits, out_splits, st.ep_group)
        recv_probs = epc.all_to_all(send_probs, in_splits, out_splits, st.ep_group)
        R = recv.shape[0]
        # arrival order is [source rank][local expert]
        e_ids = torch.arange(self.e_local, device=dev).repeat(self.ep)
        expert_of_row = torch.repeat_interleave(e_ids, recv_counts.reshape(-1), output_size=R)
        counts_local = recv_counts.sum(0).to(torch.int32)
        rows_cap = moe_ops.rows_capacity(R, self.e_local)
        sched = moe_ops.build_schedule(counts_local, rows_cap)
        src, pos = moe_ops.permutation_maps(expert_of_row, sched)
        x_perm = moe_ops.gather_rows(recv, src, pos.view(R, 1))
        pf = torch.cat([recv_probs, recv_probs.new_zeros(1)])
        probs_perm = pf[src.long()]
        out_perm = self.experts_forward(x_perm, probs_perm, sched)
        back = moe_ops.combine_rows(out_perm, pos.view(R, 1), src)       # padded layout -> arrival order
        ret = epc.all_to_all(back, out_splits, in_splits, st.ep_group)   # -> this rank's sorted copies
        return moe_ops.combine_rows(ret, inv_order.view(T, k).to(torch.int32), tok_sorted)
