"""DeepSeek-V4 building blocks: hyper-connections, the single-latent attention with its compressed long-range branches,
the compressor, the sparse-position indexer and the hash router.

Everything here is written as explicit PyTorch formulas (the linear projections go through this package's GEMM); the
score matrices are materialised, so these layers are exact but not memory-lean: head size 512 has no flash-attention
kernel in this package.

* **Hyper-connections** (``HyperMixer`` / ``HyperHead``): the residual stream is ``K = hc_mult`` parallel streams
  ``[T, K, D]``.  Per sub-layer a small fp32 projection of the RMS-normalised, flattened streams gives ``pre`` [K]
  (``sigmoid + eps``: the mixture the sub-layer reads), ``post`` [K] (``2 sigmoid``: how its output is written back) and
  ``comb`` [K, K] (``softmax + eps`` pushed onto the doubly-stochastic matrices by Sinkhorn iterations: how the streams
  mix): ``new[h] = post[h] out + sum_k comb[h, k] x[k]``.  After the last layer ``HyperHead`` collapses the streams with
  sigmoid weights.  (primus/backends/megatron/core/transformer/hyper_connection.py:186-226,229-420 in the reference.)
* **Attention** (``V4Attention``): queries through a low-rank bottleneck, one shared key = value latent of ``kv_channels``
  per token (multi-query), parameter-free RMS per query head, interleaved rotary embedding on the last
  ``qk_pos_emb_head_dim`` channels, a learned sink logit per head, a sliding-window local branch and -- per layer, from
  ``compress_ratios`` -- a compressed branch joined into the same softmax: ratio 128 attends to every pooled entry whose
  window has ended, ratio 4 to the ``index_topk`` entries the indexer picks per query.  Values carry their rotation, so
  the output is rotated back by the query position before the grouped low-rank output projection.
  (transformer/deepseek_v4_attention.py:10-47,1022-1066,1248-1345,1374-1425; v4_attention_kernels/_eager/reference.py.)
* **Compressor**: windows of ``ratio`` tokens are pooled by a per-channel softmax over the window (scores from a second
  projection plus a learned position term); ratio 4 overlaps: every window also sees the previous window through a second
  set of channels.  (transformer/compressor.py:14-24,162-214.)
* **Indexer**: ``I[t, s] = sum_h w[t, h] relu(q[t, h] . k[s])`` over its own small compressed keys, causal on whole
  windows, top-k.  (transformer/indexer.py:12-43,416-548.)  The reference also applies a Hadamard rotation to both
  operands for its low-precision product; it is orthogonal and leaves the scores unchanged, so it is left out here.
* **Hash router**: the first ``num_hash_layers`` MoE layers pick experts from a fixed token-id table and only take the
  weights from the learned gate.  (transformer/moe/v4_hash_router.py:8-40.)
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused, gemm, layers
from ..parallel import state as ps
from .mixers import _param


# ------------------------------------------------------------------------------------------------ hyper-connections
def sinkhorn(m: torch.Tensor, iters: int = 20, eps: float = 1e-6) -> torch.Tensor:
    """Non-negative [..., K, K] -> approximately doubly stochastic: one column normalisation, then ``iters - 1`` rounds
    of rows and columns (so it ends on columns), fp32."""
    m = m.float()
    m = m / (m.sum(-2, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        m = m / (m.sum(-1, keepdim=True) + eps)
        m = m / (m.sum(-2, keepdim=True) + eps)
    return m


def _flat_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    f = x.flatten(-2).float()
    return f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)


def _replicated_over_tp(module) -> None:
    """Parameters every tensor-parallel rank holds whole but that see this rank's token shard only (sequence
    parallelism): equal initial values, gradients added over the group."""
    st = ps.get_state()
    if st.tp > 1:
        for p in module.parameters():
            p.sequence_parallel = True
            if p.dim() >= 2 and torch.distributed.is_initialized():
                torch.distributed.broadcast(p.data, src=st.tp_ranks[0], group=st.tp_group)


class HyperMixer(nn.Module):
    def __init__(self, hidden: int, K: int, eps: float, iters: int, device):
        super().__init__()
        self.K, self.eps, self.iters = K, eps, iters
        out = (2 + K) * K
        self.fn = nn.Module()
        self.fn.register_parameter("weight", nn.Parameter(
            torch.empty(out, K * hidden, dtype=torch.float32, device=device).normal_(0.0, 1.0 / math.sqrt(K * hidden))))
        self.scale = nn.Parameter(torch.ones(3, dtype=torch.float32, device=device))
        self.base = nn.Parameter(torch.zeros(out, dtype=torch.float32, device=device))
        _replicated_over_tp(self)

    def weights(self, x):
        """x [T, K, D] -> pre [T, K], post [T, K], comb [T, K, K] (fp32)."""
        K = self.K
        logits = F.linear(_flat_rms(x, self.eps), self.fn.weight)
        pre = torch.sigmoid(logits[..., :K] * self.scale[0] + self.base[:K]) + self.eps
        post = 2.0 * torch.sigmoid(logits[..., K:2 * K] * self.scale[1] + self.base[K:2 * K])
        comb = logits[..., 2 * K:].reshape(*logits.shape[:-1], K, K) * self.scale[2] + self.base[2 * K:].view(K, K)
        return pre, post, sinkhorn(torch.softmax(comb, -1) + self.eps, self.iters, self.eps)

    def apply(self, x, sub_layer):
        """One sub-layer under hyper-connections: read the ``pre`` mixture, write back with ``post`` and ``comb``."""
        pre, post, comb = self.weights(x)
        read = (pre[..., None] * x.float()).sum(-2).to(x.dtype)
        out = sub_layer(read)
        return (post[..., None] * out.float()[..., None, :] + comb @ x.float()).to(x.dtype)


class HyperHead(nn.Module):
    def __init__(self, hidden: int, K: int, eps: float, device):
        super().__init__()
        self.eps = eps
        self.fn = nn.Module()
        self.fn.register_parameter("weight", nn.Parameter(
            torch.empty(K, K * hidden, dtype=torch.float32, device=device).normal_(0.0, 1.0 / math.sqrt(K * hidden))))
        self.scale = nn.Parameter(torch.ones((), dtype=torch.float32, device=device))
        self.base = nn.Parameter(torch.zeros(K, dtype=torch.float32, device=device))
        _replicated_over_tp(self)

    def forward(self, x):
        w = torch.sigmoid(F.linear(_flat_rms(x, self.eps), self.fn.weight) * self.scale + self.base) + self.eps
        return (w[..., None] * x.float()).sum(-2).to(x.dtype)


# ------------------------------------------------------------------------------------------------ rotary embedding
def yarn_inv_freq(dim: int, theta: float, factor: float = 1.0, beta_fast: float = 32.0, beta_slow: float = 1.0,
                  original_max_pos: int = 0, device=None) -> torch.Tensor:
    """Inverse frequencies of ``dim`` rotary channels; with ``factor`` > 1 the long wavelengths are stretched by it, the
    short ones kept, a linear ramp in wavelength between ``original_max_pos / beta_fast`` and ``/ beta_slow``."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    if factor == 1.0 or original_max_pos <= 0:
        return inv
    wavelen = 2.0 * math.pi / inv
    lo, hi = original_max_pos / beta_fast, original_max_pos / beta_slow
    ramp = ((wavelen - lo) / max(hi - lo, 1e-12)).clamp(0.0, 1.0)
    return inv * (1.0 - ramp) + inv / factor * ramp


def rope_interleaved(x, pos, inv_freq, rot_dim: int, inverse: bool = False):
    """Rotate the channel pairs (2k, 2k+1) of the last ``rot_dim`` channels of ``x`` [..., n, d] by ``pos`` [...] times
    the frequencies (``inverse``: by minus that)."""
    if rot_dim == 0:
        return x
    ang = pos.float()[..., None, None] * inv_freq
    c, s = torch.cos(ang), torch.sin(ang)
    if inverse:
        s = -s
    keep, rot = x[..., :-rot_dim], x[..., -rot_dim:].float()
    a, b = rot[..., 0::2], rot[..., 1::2]
    out = torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)
    return torch.cat([keep, out.to(x.dtype)], -1)


# ------------------------------------------------------------------------------------------------ compressor / indexer
class Compressor(nn.Module):
    """[B, S, D] -> [B, S / ratio, head_dim]: softmax pooling of windows, RMSNorm.  ``ratio`` 4 overlaps windows."""

    def __init__(self, hidden: int, head_dim: int, ratio: int, eps: float, std: float, dtype, device):
        super().__init__()
        self.ratio, self.head_dim, self.eps = ratio, head_dim, eps
        self.overlap = ratio == 4
        self.width = (2 if self.overlap else 1) * head_dim
        self.wkv_gate = nn.Module()
        self.wkv_gate.register_parameter("weight", _param((2 * self.width, hidden), std, dtype, device))
        self.ape = nn.Parameter(torch.empty((2 if self.overlap else 1) * ratio, head_dim, dtype=torch.float32,
                                            device=device).normal_(0.0, 0.02))
        self.kv_norm = nn.Module()
        self.kv_norm.register_parameter("weight", nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device)))

    def _windows(self, t, B, S):
        t = t.reshape(B, S // self.ratio, self.ratio, self.width)
        if not self.overlap:
            return t
        now, nxt = t[..., :self.head_dim], t[..., self.head_dim:]        # second half: seen by the next window
        prev = torch.cat([torch.zeros_like(nxt[:, :1]), nxt[:, :-1]], 1)
        return torch.cat([now, prev], 2)                                 # [B, N, 2 ratio, head_dim]

    def forward(self, hidden, batch: int):
        T = hidden.shape[0]
        S = T // batch
        assert S % self.ratio == 0, f"sequence length {S} is not a multiple of the compression ratio {self.ratio}"
        proj = gemm.linear(hidden, self.wkv_gate.weight)
        kv = self._windows(proj[:, :self.width], batch, S)
        score = self._windows(proj[:, self.width:], batch, S).float() + self.ape
        pooled = (kv.float() * torch.softmax(score, 2)).sum(2)
        pooled = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + self.eps) * self.kv_norm.weight.float()
        return pooled.to(hidden.dtype)


def window_mask(S: int, P: int, ratio: int, device) -> torch.Tensor:
    """[S, P] bool: pooled entry s (tokens [s ratio, (s + 1) ratio)) is visible to query t once its window has ended."""
    t = torch.arange(S, device=device)[:, None]
    return (torch.arange(P, device=device)[None, :] + 1) * ratio - 1 <= t


class Indexer(nn.Module):
    """Per query the ``topk`` compressed positions with the largest ``sum_h w_h relu(q_h . k_s)``; -1 where fewer are
    visible.  Its keys come from a compressor of its own (``index_head_dim`` wide)."""

    def __init__(self, cfg, ratio: int, inv_freq, rot_dim: int, device):
        super().__init__()
        h, dt, std = cfg.hidden_size, cfg.torch_dtype, cfg.init_method_std
        self.nh, self.hd, self.topk, self.ratio = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk, ratio
        self.rot_dim = min(rot_dim, self.hd)
        self.inv_freq = inv_freq if self.rot_dim == rot_dim else inv_freq[: self.rot_dim // 2]
        self.w_dq_w = nn.Module()
        self.w_dq_w.register_parameter("weight", _param((self.hd + self.nh, h), std, dt, device))
        self.w_iuq = nn.Module()
        self.w_iuq.register_parameter("weight", _param((self.nh * self.hd, self.hd), std, dt, device))
        self.indexer_compressor = Compressor(h, self.hd, ratio, cfg.norm_epsilon, std, dt, device)
        self.scale = self.nh ** -0.5 * self.hd ** -0.5

    def forward(self, hidden, pos, batch: int):
        """Returns (idx [B, S, topk] with -1 where nothing is visible, the scores of the picked entries).  The choice
        itself carries no gradient; the scores do when gradients are enabled (they feed the distillation loss)."""
        T = hidden.shape[0]
        S = T // batch
        keys = self.indexer_compressor(hidden, batch)                    # [B, P, hd]
        P = keys.shape[1]
        key_pos = torch.arange(P, device=hidden.device) * self.ratio     # a window sits at its first token
        keys = rope_interleaved(keys[:, :, None], key_pos[None, :].expand(batch, P), self.inv_freq, self.rot_dim)[:, :, 0]
        dqw = gemm.linear(hidden, self.w_dq_w.weight)
        q = gemm.linear(dqw[:, :self.hd].contiguous(), self.w_iuq.weight).view(batch, S, self.nh, self.hd)
        q = rope_interleaved(q, pos.view(batch, S), self.inv_freq, self.rot_dim)
        w = dqw[:, self.hd:].float().view(batch, S, self.nh) * self.scale
        scores = (torch.relu(torch.einsum("bshd,bpd->bshp", q.float(), keys.float())) * w[..., None]).sum(2)
        scores = scores.masked_fill(~window_mask(S, P, self.ratio, hidden.device), float("-inf"))
        k = min(self.topk, P)
        top, idx = scores.topk(k, -1)
        idx = idx.masked_fill(torch.isneginf(top), -1)
        if k < self.topk:
            idx = F.pad(idx, (0, self.topk - k), value=-1)
            top = F.pad(top, (0, self.topk - k), value=float("-inf"))
        return idx, top


def indexer_distill_loss(index_scores, attn_probs, ok):
    """``KL(attention || indexer)`` over the entries the indexer picked, averaged over the queries that see at least one:
    the target is the probability mass the attention heads put on each picked entry (summed over heads, normalised over
    the picked entries, no gradient), the indexer's distribution the softmax of its scores over the same entries.
    ``index_scores`` [B, S, K], ``attn_probs`` [B, H, S, K], ``ok`` [B, S, K].  The reference trains its indexer this
    way (primus/backends/megatron/core/transformer/indexer_distill_loss.py:6-31): the top-k choice passes no gradient."""
    target = attn_probs.detach().sum(1).masked_fill(~ok, 0.0)
    target = target / target.sum(-1, keepdim=True).clamp(min=1e-10)
    logq = torch.log_softmax(index_scores.float().masked_fill(~ok, float("-inf")), -1).masked_fill(~ok, 0.0)
    kl = (target * (torch.log(target.clamp(min=1e-10)) - logq)).sum(-1)
    rows = ok.any(-1)
    return (kl * rows).sum() / rows.sum().clamp(min=1)


# ------------------------------------------------------------------------------------------------ attention
def joint_attention(q, kv, sink, window: int, scale: float, pool=None, pool_mask=None, gathered=None, gathered_ok=None,
                    return_gathered_probs: bool = False):
    """q [B, H, S, D]; kv [B, S, D] (key = value, one head); ``sink`` [H] or None.  Local branch: causal, the last
    ``window`` keys (0: all).  Compressed branch, in the same softmax: ``pool`` [B, P, D] with ``pool_mask`` [S, P]
    (every query sees the same entries), or ``gathered`` [B, S, K, D] with ``gathered_ok`` [B, S, K] (entries picked per
    query).  The sink takes probability mass and contributes nothing.  Returns [B, H, S, D] fp32."""
    B, H, S, D = q.shape
    qf, kvf = q.float(), kv.float()
    i = torch.arange(S, device=q.device)
    allowed = i[None, :] <= i[:, None]
    if window and window > 0:
        allowed &= i[None, :] > i[:, None] - window
    parts = [(torch.einsum("bhsd,btd->bhst", qf, kvf) * scale).masked_fill(~allowed, float("-inf"))]
    if pool is not None:
        parts.append((torch.einsum("bhsd,bpd->bhsp", qf, pool.float()) * scale).masked_fill(~pool_mask, float("-inf")))
    if gathered is not None:
        parts.append((torch.einsum("bhsd,bskd->bhsk", qf, gathered.float()) * scale)
                     .masked_fill(~gathered_ok[:, None], float("-inf")))
    if sink is not None:
        parts.append(sink.float().view(1, H, 1, 1).expand(B, H, S, 1))
    probs = torch.softmax(torch.cat(parts, -1), -1)
    out = torch.einsum("bhst,btd->bhsd", probs[..., :S], kvf)
    if pool is not None:
        out = out + torch.einsum("bhsp,bpd->bhsd", probs[..., S:S + pool.shape[1]], pool.float())
    if gathered is not None:
        pg = probs[..., S:S + gathered.shape[2]]
        out = out + torch.einsum("bhsk,bskd->bhsd", pg, gathered.float())
        if return_gathered_probs:
            return out, pg
    return out


class V4Attention(nn.Module):
    def __init__(self, cfg, layer_idx: int, device, tp: int, mtp_depth=None):
        super().__init__()
        # Tensor parallelism (with sequence parallelism) splits the query heads and, with them, the groups of the output
        # projection; the shared latent, the query bottleneck, the compressor and the indexer are replicated
        assert tp == 1 or cfg.sequence_parallel, "DeepSeek-V4 attention under tensor parallelism needs sequence_parallel"
        assert cfg.num_attention_heads % tp == 0 and (not cfg.o_lora_rank or cfg.o_groups % tp == 0), \
            "heads and output-projection groups must divide by the tensor-parallel size"
        self.cfg, self.tp = cfg, tp
        h, dt, std = cfg.hidden_size, cfg.torch_dtype, cfg.init_method_std
        self.nh, self.hd, self.dr = cfg.num_attention_heads // tp, cfg.kv_channels, cfg.qk_pos_emb_head_dim
        self.ratio = int(cfg.compress_ratio_list[layer_idx])
        if mtp_depth is not None and mtp_depth < len(cfg.compress_ratio_mtp):
            self.ratio = int(cfg.compress_ratio_mtp[mtp_depth])      # the entries behind the decoder layers
        if self.ratio not in (0, 4, 128):
            raise ValueError(f"compress_ratios: 0 (local only), 4 (indexed) or 128 (pooled), got {self.ratio}")
        out_std = std / math.sqrt(2.0 * cfg.num_layers)

        def holder(**params):
            m = nn.Module()
            for k, v in params.items():
                m.register_parameter(k, v)
            return m

        ones = lambda n: nn.Parameter(torch.ones(n, dtype=dt, device=device))      # noqa: E731
        self.input_layernorm = holder(weight=ones(h))
        if cfg.q_lora_rank:
            self.linear_q_down_proj = holder(weight=_param((cfg.q_lora_rank, h), std, dt, device))
            self.linear_q_up_proj = holder(layer_norm_weight=ones(cfg.q_lora_rank),
                                           weight=_param((self.nh * self.hd, cfg.q_lora_rank), std, dt, device))
        else:
            self.linear_q_proj = holder(weight=_param((self.nh * self.hd, h), std, dt, device))
        self.linear_kv = holder(weight=_param((self.hd, h), std, dt, device))
        self.kv_layernorm = holder(weight=ones(self.hd))
        if cfg.attn_sink:
            self.attn_sink = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32, device=device))
        self.G, self.r = cfg.o_groups // tp if cfg.o_lora_rank else cfg.o_groups, cfg.o_lora_rank
        if self.r:
            assert (self.nh * self.hd) % self.G == 0
            self.linear_o_a = holder(weight=_param((self.G * self.r, self.nh * self.hd // self.G), std, dt, device))
            self.linear_o_b = holder(weight=_param((h, self.G * self.r), out_std, dt, device))
        else:
            self.linear_proj = holder(weight=_param((h, self.nh * self.hd), out_std, dt, device))
        # local-only layers rotate with the main base; layers with a compressed branch with the compression base and
        # stretched long wavelengths
        if self.ratio:
            inv = yarn_inv_freq(self.dr, cfg.compress_rope_theta, cfg.rotary_scaling_factor or 1.0, 32.0, 1.0,
                                cfg.original_max_position_embeddings or 0, device)
            self.compressor = Compressor(h, self.hd, self.ratio, cfg.norm_epsilon, std, dt, device)
        else:
            inv = yarn_inv_freq(self.dr, cfg.rotary_base, device=device)
        self.register_buffer("inv_freq", inv, persistent=False)
        if self.ratio == 4:
            self.indexer = Indexer(cfg, self.ratio, inv, self.dr, device)
        self.linear_kv.weight._is_weight = True
        if tp > 1:
            from .mixers import _mark_tp

            _mark_tp(self.linear_q_up_proj.weight if cfg.q_lora_rank else self.linear_q_proj.weight, 0)
            if cfg.attn_sink:
                _mark_tp(self.attn_sink, 0)
            if self.r:
                _mark_tp(self.linear_o_a.weight, 0)
                _mark_tp(self.linear_o_b.weight, 1)
            else:
                _mark_tp(self.linear_proj.weight, 1)
            st = ps.get_state()
            split = {id(p) for p in self.parameters() if getattr(p, "tensor_model_parallel", False)}
            index_only = {id(p) for p in self.indexer.parameters()} if self.ratio == 4 else set()
            for p in self.parameters():
                if id(p) in split:
                    continue
                if torch.distributed.is_initialized():          # drawn per rank: make the replicas equal
                    torch.distributed.broadcast(p.data, src=st.tp_ranks[0], group=st.tp_group)
                # replicated parameters see this rank's tokens or heads only: their gradients are partial sums, added
                # over the group -- except the indexer's, whose loss every rank computes in full
                if id(p) not in index_only:
                    p.sequence_parallel = True

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        assert st.cp == 1, "DeepSeek-V4 attention is not built for context parallelism"
        if residual is not None:
            y, xsum = fused.rmsnorm(hidden, self.input_layernorm.weight, cfg.norm_epsilon, residual)
        else:
            y, xsum = fused.rmsnorm(hidden, self.input_layernorm.weight, cfg.norm_epsilon), hidden
        tpg = st.tp_group if self.tp > 1 else None

        def everywhere(t):          # all tokens on every rank; the backward pass adds the ranks' contributions
            if tpg is None:
                return t
            from ..parallel import tensor_parallel as tpc

            return tpc.gather_seq(t, tpg)

        T = y.shape[0] * self.tp
        S = T // batch
        nh, hd, dr = self.nh, self.hd, self.dr
        pos = rope[2]
        pos = (torch.arange(S, device=y.device).repeat(batch) if pos is None else pos.long()).view(batch, S)
        if cfg.q_lora_rank:
            ql = fused.rmsnorm(gemm.linear(y, self.linear_q_down_proj.weight), self.linear_q_up_proj.layer_norm_weight,
                               cfg.norm_epsilon)
            q = gemm.linear(everywhere(ql), self.linear_q_up_proj.weight)
        else:
            q = gemm.linear(everywhere(y), self.linear_q_proj.weight)
        q = q.view(batch, S, nh, hd).float()
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon)            # per head, no gain
        kv = everywhere(fused.rmsnorm(gemm.linear(y, self.linear_kv.weight), self.kv_layernorm.weight, cfg.norm_epsilon))
        if self.ratio:
            y = everywhere(y)               # the compressor and the indexer pool whole windows of tokens
        q = rope_interleaved(q, pos, self.inv_freq, dr)
        kv = rope_interleaved(kv.view(batch, S, 1, hd), pos, self.inv_freq, dr)[:, :, 0]
        extra = {}
        if self.ratio:
            pool = self.compressor(y, batch)                                                # [B, P, hd]
            P = pool.shape[1]
            ppos = (torch.arange(P, device=y.device) * self.ratio)[None, :].expand(batch, P)
            pool = rope_interleaved(pool[:, :, None], ppos, self.inv_freq, dr)[:, :, 0]
            if self.ratio == 4:
                distill = cfg.v4_indexer_distill_loss_coeff > 0 and self.training and torch.is_grad_enabled()
                with torch.set_grad_enabled(distill):     # the indexer reads a detached input: its loss stays its own
                    idx, index_scores = self.indexer(y.detach(), pos, batch)               # [B, S, K], -1 = none
                ok = idx >= 0
                extra = dict(gathered=pool[torch.arange(batch, device=y.device)[:, None, None], idx.clamp(min=0)],
                             gathered_ok=ok)
            else:
                extra = dict(pool=pool, pool_mask=window_mask(S, P, self.ratio, y.device))
        sink = self.attn_sink if cfg.attn_sink else None
        out = joint_attention(q.permute(0, 2, 1, 3), kv, sink, cfg.attn_sliding_window or 0, hd ** -0.5, **extra,
                              return_gathered_probs=self.ratio == 4)
        if self.ratio == 4:
            out, picked_probs = out
            if distill:
                from .moe import AuxLossScaler

                mass = picked_probs.detach().sum(1, keepdim=True)       # over this rank's heads ...
                if tpg is not None:
                    torch.distributed.all_reduce(mass, group=tpg)       # ... and over all of them
                aux = cfg.v4_indexer_distill_loss_coeff * indexer_distill_loss(index_scores, mass, ok)
                self.last_distill_loss = aux.detach()
                out = AuxLossScaler.apply(out, aux)
        out = out.permute(0, 2, 1, 3)                                                       # [B, S, H, hd]
        # values carry the rotation of their own position: rotating the result back by the query position leaves
        # relative positions only
        out = rope_interleaved(out, pos, self.inv_freq, dr, inverse=True).to(hidden.dtype)
        if self.r:
            g = out.reshape(T, self.G, nh * hd // self.G)
            wa = self.linear_o_a.weight.view(self.G, self.r, nh * hd // self.G)
            low = torch.einsum("tgd,grd->tgr", g, wa).reshape(T, self.G * self.r)
            return layers.row_parallel_linear(low.contiguous(), self.linear_o_b.weight, tpg, tpg is not None), xsum
        return layers.row_parallel_linear(out.reshape(T, nh * hd).contiguous(), self.linear_proj.weight, tpg,
                                          tpg is not None), xsum


# ------------------------------------------------------------------------------------------------ hash router
def hash_table(vocab: int, num_experts: int, topk: int, seed: int) -> torch.Tensor:
    """[vocab, topk] int32: ``topk`` distinct experts per token id, the same on every rank and device."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.rand(vocab, num_experts, generator=g).argsort(-1)[:, :topk].to(torch.int32)
