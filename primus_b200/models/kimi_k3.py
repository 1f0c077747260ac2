"""Building blocks of the Kimi-K3 text backbone that no other family uses.

* **Kimi delta attention** (``KimiDeltaAttentionMixer``): the gated delta rule with a forget gate per *channel* of the
  key dimension instead of one per head.  State ``S`` [dk, dv] per head:

      S_t = (I - beta_t k_t k_t^T) Diag(alpha_t) S_{t-1} + beta_t k_t v_t^T,      o_t = S_t^T (scale q_t)

  with ``alpha_t = exp(g_t)`` and the log-decay ``g = lower_bound * sigmoid(exp(A_log) (z + dt_bias))`` (bounded form) or
  ``-exp(A_log) softplus(z + dt_bias)``.  ``kda_chunked`` evaluates it chunk by chunk: inside a chunk the updates solve a
  unit lower-triangular system, between chunks only the state is carried.  All decay factors are formed as
  ``exp(G_i - G_j)`` with ``i >= j`` (never ``exp(-G_j)`` on its own), so nothing overflows however strong the decay:
  pairs of rows in different 16-row sub-blocks go through the log-decay at the start of the later sub-block, which
  splits the factor into two that are both at most one and keeps the work in matrix products; pairs inside a sub-block
  are summed channel by channel.  (primus/backends/megatron/core/transformer/kimi_k3/kimi_delta_attention.py:198-728,
  kda_kernels/README.md:11-35, kda_kernels/_eager/reference.py:112-151 in the reference.)
* **Attention residuals** (``AttentionResidualMixer``): instead of ``x + sublayer(x)`` a sub-layer reads a softmax
  mixture of the running residual stream and the checkpoints that every ``attn_res_block_size``-th layer sets aside; the
  scores come from the RMS-normalised candidates through a rank-1 scorer, the mixture is taken over the candidates as
  they are, everything in fp32.  (transformer/kimi_k3/attention_residual.py:60-227,
  attn_res_kernels/_eager/reference.py:58-102, layer bookkeeping models/kimi_k3/kimi_k3_block.py:105-127,455-555.)
* **Quantile balancing** (``margin_histogram`` / ``quantile_bias``): the expert bias of the router is *set* from the
  ``1 - k/n`` quantile of every expert's routing margin (raw score minus the token's biased top-(k+1) cut-off), estimated
  from per-expert histograms that are summed over micro-batches and ranks.
  (transformer/kimi_k3/moe/k3_quantile_balancing.py:14-108,165-250, moe/qb_kernels/_eager/reference.py:60-110.)

The NoPE multi-latent attention with an output gate, the SiTU activation and the latent mixture of experts live with
their families (models/mla.py, ops/fused.py, models/moe.py).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm
from ..parallel import state as ps
from .mixers import _norm, _param, causal_depthwise_conv

SUB = 16        # rows of a sub-block inside a chunk


# ------------------------------------------------------------------------------------------------ the recurrence
def kda_gate(z, A_log, dt_bias=None, lower_bound=None):
    """Log-decay per channel.  ``z`` [..., H, dk]; ``A_log`` [H]; ``dt_bias`` [H * dk]."""
    H, dk = z.shape[-2:]
    z = z.float()
    if dt_bias is not None:
        z = z + dt_bias.float().view(H, dk)
    a = torch.exp(A_log.float()).view(H, 1)
    if lower_bound is not None:
        return float(lower_bound) * torch.sigmoid(a * z)
    return -a * F.softplus(z)


def kda_sequential(q, k, v, g, beta, scale=None):
    """The recurrence one token at a time (test oracle).  q, k, g [b, l, h, dk]; v [b, l, h, dv]; beta [b, l, h]."""
    b, l, h, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    S = torch.zeros(b, h, dk, dv, dtype=torch.float32, device=q.device)
    out = []
    for t in range(l):
        S = S * torch.exp(g[:, t].float())[..., None]
        kt = k[:, t].float()
        u = (v[:, t].float() - torch.einsum("bhk,bhkv->bhv", kt, S)) * beta[:, t].float()[..., None]
        S = S + kt[..., :, None] * u[..., None, :]
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].float() * scale, S))
    return torch.stack(out, 1)


def _decayed_products(x, y, G, sub: int):
    """``P[i, j] = sum_d x[i, d] y[j, d] exp(G[i, d] - G[j, d])`` for ``j <= i`` (zero above the diagonal).
    x, y, G: [..., C, dk] with G the inclusive cumulative log-decay of the chunk."""
    C, dk = x.shape[-2:]
    nb = C // sub
    P = x.new_zeros(*x.shape[:-2], C, C)
    tri = torch.ones(sub, sub, dtype=torch.bool, device=x.device).tril()
    for I in range(nb):
        lo, hi = I * sub, (I + 1) * sub
        Gi = G[..., lo:hi, :]
        # inside the sub-block: channel by channel, exponent masked to <= 0 before the exponential
        diff = (Gi[..., :, None, :] - Gi[..., None, :, :]).masked_fill(~tri[..., None], 0.0)
        w = torch.exp(diff) * tri[..., None]
        P[..., lo:hi, lo:hi] = torch.einsum("...id,...jd,...ijd->...ij", x[..., lo:hi, :], y[..., lo:hi, :], w)
        if I:
            ref = G[..., lo - 1:lo, :]                                   # log-decay up to the end of the previous sub-block
            xi = x[..., lo:hi, :] * torch.exp(Gi - ref)                 # G_i - ref <= 0
            yj = y[..., :lo, :] * torch.exp(ref - G[..., :lo, :])       # ref - G_j <= 0 for the earlier rows
            P[..., lo:hi, :lo] = xi @ yj.transpose(-1, -2)
    return P


def kda_chunked(q, k, v, g, beta, chunk: int = 64, scale=None, sub: int = SUB):
    """Chunk-wise evaluation of the recurrence (see the module docstring); fp32 result [b, l, h, dv]."""
    b, l, h, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    chunk = max(sub, chunk // sub * sub)
    pad = (-l) % chunk
    if pad:     # padded steps: no decay (g = 0), no write (beta = 0)
        q, k, v, g = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v, g))
        beta = F.pad(beta, (0, 0, 0, pad))
    L_ = l + pad
    c = L_ // chunk

    def heads_first(t):
        return t.float().permute(0, 2, 1, 3).reshape(b, h, c, chunk, t.shape[-1])

    qf, kf, vf, gf = heads_first(q) * scale, heads_first(k), heads_first(v), heads_first(g)
    bf = beta.float().permute(0, 2, 1).reshape(b, h, c, chunk)
    eye = torch.eye(chunk, device=q.device)
    strict = torch.ones(chunk, chunk, device=q.device).tril(-1)
    S = torch.zeros(b, h, dk, dv, dtype=torch.float32, device=q.device)
    outs = []
    for i in range(c):
        qi, ki, vi, bi = qf[:, :, i], kf[:, :, i], vf[:, :, i], bf[:, :, i]
        G = torch.cumsum(gf[:, :, i], -2)                                # [b, h, chunk, dk], inclusive
        decay_in = torch.exp(G)                                          # from the chunk start to each row (<= 1)
        A = _decayed_products(ki, ki, G, sub)
        rhs = bi[..., None] * (vi - (ki * decay_in) @ S)
        U = torch.linalg.solve_triangular(eye + bi[..., None] * A * strict, rhs, upper=False)
        outs.append((qi * decay_in) @ S + _decayed_products(qi, ki, G, sub) @ U)      # the diagonal counts: o reads S_t
        last = G[..., -1:, :]
        S = S * torch.exp(last).transpose(-1, -2) + (ki * torch.exp(last - G)).transpose(-1, -2) @ U
    o = torch.stack(outs, 2).reshape(b, h, L_, dv).permute(0, 2, 1, 3)
    return o[:, :l]


class KimiDeltaAttentionMixer(nn.Module):
    """``q, k, v = silu(causal_conv(proj(h)))`` (q, k L2-normalised); log-decay from a rank-``dk`` bottleneck
    ``f_b(f_a(h))``; ``beta = sigmoid(b(h))``; the recurrence; per-head RMSNorm gated by ``sigmoid(g(h))``; ``o_proj``.
    The per-head projections that read the layer input are one GEMM (``in_proj``, rows ``[q | k | v | g | b]``), the
    bottlenecks every head shares another (``in_proj_shared``), and the three depthwise convolutions one convolution over
    the concatenated channels.  Tensor parallelism (with sequence parallelism) splits the heads."""

    def __init__(self, cfg, layer_idx: int, device, tp: int):
        super().__init__()
        assert tp == 1 or cfg.sequence_parallel, "Kimi delta attention under tensor parallelism needs sequence_parallel"
        assert cfg.linear_num_key_heads == cfg.linear_num_value_heads, "Kimi delta attention: as many key as value heads"
        assert cfg.linear_num_value_heads % tp == 0, "heads must divide by the tensor-parallel size"
        self.cfg, self.tp = cfg, tp
        h, dt = cfg.hidden_size, cfg.torch_dtype
        self.nh, self.dk, self.dv = cfg.linear_num_value_heads // tp, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.qk_dim, self.v_dim = self.nh * self.dk, self.nh * self.dv
        self.conv_dim = 2 * self.qk_dim + self.v_dim
        std = cfg.init_method_std
        self.in_proj = nn.Module()
        self.in_proj.register_parameter("layer_norm_weight", nn.Parameter(torch.ones(h, dtype=dt, device=device)))
        # the output gate is a full projection (Kimi-K3) or goes through a ``dv``-wide bottleneck ``g_b(g_a(h))`` like the
        # forget gate (Kimi Linear, the delta-attention stacks of the hybrid presets:
        # primus/backends/megatron/core/models/hybrid/kimi_delta_attention.py:278-311,397-410 in the reference)
        self.full_gate = bool(cfg.kda_use_full_rank_gate)
        self.fa = self.dk if self.full_gate else self.dv
        # per-head rows [q | k | v | (g) | b] and, apart from them, the rows every head shares: the bottleneck of the
        # forget gate (and of the output gate); under tensor parallelism the first are split by heads, the second replicated
        self.head_rows = self.conv_dim + (self.v_dim if self.full_gate else 0) + self.nh
        self.shared_rows = self.fa + (0 if self.full_gate else self.dv)
        self.in_proj.register_parameter("weight", _param((self.head_rows, h), std, dt, device))
        self.in_proj_shared = nn.Module()
        self.in_proj_shared.register_parameter("weight", _param((self.shared_rows, h), std, dt, device))
        self.conv1d = nn.Module()
        self.conv1d.register_parameter("weight", _param((self.conv_dim, 1, cfg.linear_conv_kernel_dim), std * 5, dt, device))
        self.f_b_proj = nn.Module()
        self.f_b_proj.register_parameter("weight", _param((self.qk_dim, self.fa), std, dt, device))
        if not self.full_gate:
            self.g_b_proj = nn.Module()
            self.g_b_proj.register_parameter("weight", _param((self.v_dim, self.dv), std, dt, device))
        # exp(A_log) = 1 at the start; the bias puts the initial retention near one (dt ~ logU(1e-3, 1e-1), bias =
        # softplus^-1(dt)), the initialisation the reference settles on (kimi_delta_attention.py:579-602)
        self.A_log = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32, device=device))
        u = torch.rand(self.qk_dim, device=device)
        dt0 = torch.exp(u * (math.log(1e-1) - math.log(1e-3)) + math.log(1e-3))
        self.dt_bias = nn.Parameter((dt0 + torch.log(-torch.expm1(-dt0))).float())
        self.out_norm = nn.Module()
        self.out_norm.register_parameter("weight", nn.Parameter(torch.ones(self.dv, dtype=dt, device=device)))
        self.out_proj = nn.Module()
        self.out_proj.register_parameter("weight", _param((h, self.v_dim), std / math.sqrt(2.0 * cfg.num_layers), dt, device))
        for w in (self.in_proj.weight, self.out_proj.weight, self.f_b_proj.weight):
            w._is_weight = True
        if tp > 1:
            from .mixers import _mark_tp

            QK, V, NH = self.qk_dim * tp, self.v_dim * tp, self.nh * tp
            _mark_tp(self.in_proj.weight, 0, [QK, QK, V] + ([V] if self.full_gate else []) + [NH])
            _mark_tp(self.conv1d.weight, 0, [QK, QK, V])
            _mark_tp(self.f_b_proj.weight, 0)
            if not self.full_gate:
                _mark_tp(self.g_b_proj.weight, 0)
            _mark_tp(self.dt_bias, 0)
            _mark_tp(self.A_log, 0)
            _mark_tp(self.out_proj.weight, 1)
            st = ps.get_state()
            for w in (self.in_proj.layer_norm_weight, self.out_norm.weight, self.in_proj_shared.weight):
                w.sequence_parallel = True          # replicated, gradients are partial sums: added over the group
            if torch.distributed.is_initialized():
                torch.distributed.broadcast(self.in_proj_shared.weight.data, src=st.tp_ranks[0], group=st.tp_group)

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        assert st.cp == 1, "the Kimi-delta-attention mixer is not built for context parallelism"
        y, xsum = _norm(hidden, residual, self.in_proj.layer_norm_weight, cfg.norm_epsilon)
        if self.tp > 1:
            from ..parallel import tensor_parallel as tpc

            y = tpc.gather_seq(y, st.tp_group)
        proj = gemm.linear(y, self.in_proj.weight)
        shared = gemm.linear(y, self.in_proj_shared.weight)
        T = proj.shape[0]
        seq = T // batch
        cd, vd, nh, dk = self.conv_dim, self.v_dim, self.nh, self.dk
        qkv = F.silu(causal_depthwise_conv(proj[:, :cd], self.conv1d.weight[:, 0, :], None, batch))
        f_a = shared[:, :self.fa].contiguous()
        if self.full_gate:
            gate, b_ = proj[:, cd:cd + vd], proj[:, cd + vd:]
        else:
            gate, b_ = gemm.linear(shared[:, self.fa:].contiguous(), self.g_b_proj.weight), proj[:, cd:]
        q = F.normalize(qkv[:, :self.qk_dim].float().view(batch, seq, nh, dk), dim=-1, eps=1e-6)
        k = F.normalize(qkv[:, self.qk_dim:2 * self.qk_dim].float().view(batch, seq, nh, dk), dim=-1, eps=1e-6)
        v = qkv[:, 2 * self.qk_dim:].view(batch, seq, nh, self.dv)
        z = gemm.linear(f_a, self.f_b_proj.weight).view(batch, seq, nh, dk)
        g = kda_gate(z, self.A_log, self.dt_bias, cfg.kda_gate_lower_bound)
        beta = torch.sigmoid(b_.float()).view(batch, seq, nh)
        o = kda_chunked(q, k, v, g, beta, cfg.kda_chunk_size)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * self.out_norm.weight.float()
        o = (o.reshape(T, vd) * torch.sigmoid(gate.float())).to(hidden.dtype)
        if self.tp > 1:
            from ..ops import layers

            return layers.row_parallel_linear(o.contiguous(), self.out_proj.weight, st.tp_group, True), xsum
        return gemm.linear(o.contiguous(), self.out_proj.weight), xsum


# ------------------------------------------------------------------------------------------------ attention residuals
def checkpoints_before(layer_idx: int, block_size) -> int:
    """Checkpoints set aside before (0-based) layer ``layer_idx``: every layer whose index is a multiple of
    ``block_size`` appends one, so the count is ``ceil(layer_idx / block_size)``."""
    return -(-int(layer_idx) // int(block_size)) if block_size else 0


def attn_res_mix(stream, checkpoints, norm_weight, proj_weight, eps: float):
    """``stream`` [T, H], ``checkpoints`` [T, n, H] (or None): softmax over the n + 1 candidates of
    ``rmsnorm(candidate) . (norm_weight * proj_weight)``; returns the mixture of the candidates as they are."""
    cand = stream[:, None] if checkpoints is None else torch.cat([checkpoints, stream[:, None]], 1)
    cf = cand.float()
    normed = cf * torch.rsqrt(cf.pow(2).mean(-1, keepdim=True) + eps)
    scorer = norm_weight.float() * proj_weight.float().reshape(-1)
    probs = torch.softmax((normed * scorer).sum(-1), -1)
    return torch.einsum("tn,tnh->th", probs, cf).to(stream.dtype)


class AttentionResidualMixer(nn.Module):
    """One rank-1 scorer: ``norm_weight`` [H] (ones) and ``proj_weight`` [1, H]."""

    def __init__(self, cfg, device):
        super().__init__()
        self.eps = cfg.norm_epsilon
        dt = cfg.torch_dtype
        self.norm_weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dt, device=device))
        self.proj_weight = _param((1, cfg.hidden_size), cfg.init_method_std, dt, device)
        for p in (self.norm_weight, self.proj_weight):
            p.sequence_parallel = cfg.sequence_parallel

    def forward(self, stream, checkpoints):
        return attn_res_mix(stream, checkpoints, self.norm_weight, self.proj_weight, self.eps)


# ------------------------------------------------------------------------------------------------ quantile balancing
@torch.no_grad()
def margin_histogram(scores, expert_bias, topk: int, num_bins: int, lo: float, hi: float):
    """Per-expert histogram [E, num_bins] (int64) of ``scores[i, j] - tau_i`` over the tokens, ``tau_i`` the
    (k+1)-th largest biased score of token i; margins outside [lo, hi] land in the end bins."""
    T, E = scores.shape
    if T == 0:
        return torch.zeros(E, num_bins, dtype=torch.int64, device=scores.device)
    s = scores.float()
    kth = min(topk + 1, E)
    tau = torch.topk(s + expert_bias.float(), kth, dim=-1).values[:, -1:]
    width = (hi - lo) / num_bins
    idx = ((s - tau - lo) / width).floor().clamp_(0, num_bins - 1).to(torch.int64)
    flat = idx + torch.arange(E, device=scores.device, dtype=torch.int64) * num_bins
    return torch.bincount(flat.reshape(-1), minlength=E * num_bins).view(E, num_bins)


def histogram_quantile(hist, q: float, lo: float, hi: float):
    """The ``q``-quantile of every row's distribution [..., bins] -> [...], interpolated linearly inside the bin that
    holds the target rank (fp64).  A row without counts reports the middle of the range."""
    bins = hist.shape[-1]
    h = hist.to(torch.float64)
    cum = h.cumsum(-1)
    total = cum[..., -1:]
    target = total * float(q)
    idx = torch.searchsorted(cum.contiguous(), target.contiguous()).clamp_(max=bins - 1)
    before = torch.where(idx == 0, torch.zeros_like(target), torch.gather(cum, -1, (idx - 1).clamp_(min=0)))
    frac = ((target - before) / torch.gather(h, -1, idx).clamp_(min=1.0)).clamp_(0.0, 1.0)
    value = lo + (hi - lo) / bins * (idx.to(torch.float64) + frac)
    return torch.where(total > 0, value, torch.full_like(value, 0.5 * (lo + hi))).squeeze(-1)


def quantile_bias(hist, topk: int, lo: float, hi: float, center: bool = True):
    """Next expert bias from the pooled histograms [E, bins]: minus the ``1 - k/E`` quantile of every expert's margins
    (the bias at which the expert would receive its fair share of the tokens), mean removed."""
    E = hist.shape[-2]
    bias = -histogram_quantile(hist, 1.0 - float(topk) / float(E), lo, hi)
    return bias - bias.mean(-1, keepdim=True) if center else bias
