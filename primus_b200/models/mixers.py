"""Sequence mixers other than softmax attention: the LFM2 gated short convolution and the Mamba-2 state-space mixer.

Both take the already-normalised hidden states of a layer ``[T, H]`` (T = batch x sequence, sequence fastest) and return
the sub-layer output that joins the residual stream, like ``SelfAttention`` does; the linear projections run on this
package's GEMM (bf16 or the active FP8 recipe), the sequence operations are written below in plain PyTorch with
explicit formulas (they are also the CPU path and the test oracle).

* ``ShortConvMixer`` — LFM2: ``B, C, x = in_proj(h)``; ``y = out_proj(C * causal_conv(B * x))`` with a depthwise causal
  convolution of ``conv_L_cache`` taps.  Counterpart of ``Lfm2ShortConv`` in the reference
  (primus/backends/megatron/core/transformer/attention.py:91-230; layer choice per
  ``lfm_layer_types``: primus/backends/megatron/core/models/gpt/gpt_layer_specs.py:41-157).
* ``Mamba2Mixer`` — Mamba-2 (state-space duality): ``z, xBC, dt = in_proj(h)``; causal depthwise convolution + SiLU on
  ``xBC``; the selective state-space recurrence ``s_t = exp(dt_t A) s_{t-1} + dt_t B_t x_t``, ``y_t = C_t s_t + D x_t`` evaluated
  chunk-wise as matrix products (``ssd_chunked``); gated RMSNorm ``norm(y * silu(z))`` per group; ``out_proj``.  The mixer of
  the reference's Mamba and hybrid stacks (primus/backends/megatron/core/models/mamba/mamba_layer_specs.py,
  primus/backends/megatron/core/models/hybrid/hybrid_block.py, presets ``mamba_370M`` and ``zebra_llama_*``).

Tensor parallelism splits the heads of the Mamba-2 and gated-delta-net mixers (together with sequence parallelism: the
mixer gathers the normalised tokens, works on its own heads and reduce-scatters its output projection; fused projections
are marked with the sizes of their blocks so that checkpoints re-tile them); the short convolution and context
parallelism are not built (``tp == 1`` / ``cp == 1`` asserted); pipeline, data and expert parallelism work as for any
layer.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused, gemm, layers
from ..parallel import state as ps
from ..parallel import tensor_parallel as tpc


def _param(shape, std, dtype, device):
    p = nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))
    if std > 0:
        nn.init.normal_(p, mean=0.0, std=std)
    else:
        nn.init.zeros_(p)
    return p


def _mark_tp(p, dim: int, parts=None):
    """Head-split parameter: ``parts`` lists the global sizes of the blocks stacked on dim 0 when there are several
    (every rank holds its heads' slice of each block; the checkpoint code re-tiles them)."""
    p.tensor_model_parallel, p.partition_dim = True, dim
    if parts:
        p.tp_parts = list(parts)


def _norm(hidden, residual, weight, eps):
    """Fused residual add + RMSNorm of a sub-layer input: (normalised, summed residual stream)."""
    if residual is None:
        return fused.rmsnorm(hidden, weight, eps), hidden
    return fused.rmsnorm(hidden, weight, eps, residual)


def causal_depthwise_conv(x: torch.Tensor, weight: torch.Tensor, bias, batch: int) -> torch.Tensor:
    """``x`` [batch * seq, C] (sequence fastest), ``weight`` [C, taps]: out[t, c] = sum_k weight[c, k] x[t - (taps-1) + k, c]
    with zeros before the start of every sequence (the semantics of ``nn.Conv1d(groups=C, padding=taps-1)[..., :seq]``)."""
    T, C = x.shape
    taps = weight.shape[1]
    xs = x.view(batch, T // batch, C)
    out = None
    for k in range(taps):
        shift = taps - 1 - k
        term = xs if shift == 0 else F.pad(xs, (0, 0, shift, 0))[:, : T // batch]
        term = term * weight[:, k]
        out = term if out is None else out + term
    if bias is not None:
        out = out + bias
    return out.reshape(T, C)


class ShortConvMixer(nn.Module):
    """LFM2 double-gated short convolution (parameter names follow the reference: ``in_proj``, ``conv``, ``out_proj``).

    Tensor parallelism splits the channels: every rank holds its slice of the three ``in_proj`` blocks (B, C, x), of the
    depthwise filter and of the columns of ``out_proj``; with sequence parallelism the normalised tokens are gathered
    before ``in_proj`` and the output projection is reduce-scattered."""

    def __init__(self, cfg, layer_idx: int, device, tp: int):
        super().__init__()
        assert tp == 1 or cfg.sequence_parallel, "the short-convolution mixer under tensor parallelism needs sequence_parallel"
        assert cfg.hidden_size % tp == 0, "hidden_size must divide by the tensor-parallel size"
        self.cfg, self.tp = cfg, tp
        h, dt = cfg.hidden_size, cfg.torch_dtype
        self.hl = hl = h // tp                     # this rank's channels
        std = cfg.init_method_std
        self.in_proj = nn.Module()
        self.in_proj.register_parameter("layer_norm_weight", nn.Parameter(torch.ones(h, dtype=dt, device=device)))
        self.in_proj.register_parameter("weight", _param((3 * hl, h), std, dt, device))
        self.conv = nn.Module()
        self.conv.register_parameter("weight", _param((hl, 1, cfg.conv_L_cache), std, dt, device))
        self.out_proj = nn.Module()
        self.out_proj.register_parameter("weight", _param((h, hl), std / math.sqrt(2.0 * cfg.num_layers), dt, device))
        if cfg.conv_bias:
            for m, n in ((self.in_proj, 3 * hl), (self.conv, hl), (self.out_proj, h)):
                m.register_parameter("bias", nn.Parameter(torch.zeros(n, dtype=dt, device=device)))
        for w in (self.in_proj.weight, self.out_proj.weight):
            w._is_weight = True
        if tp > 1:
            _mark_tp(self.in_proj.weight, 0, [h, h, h])
            _mark_tp(self.conv.weight, 0)
            _mark_tp(self.out_proj.weight, 1)
            # replicated, each rank sees its tokens only: gradients are summed over the group
            self.in_proj.layer_norm_weight.sequence_parallel = True
            if cfg.conv_bias:
                _mark_tp(self.in_proj.bias, 0, [h, h, h])
                _mark_tp(self.conv.bias, 0)
                self.out_proj.bias.sequence_parallel = True

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        assert st.cp == 1, "the short-convolution mixer is not built for context parallelism"
        y, xsum = _norm(hidden, residual, self.in_proj.layer_norm_weight, cfg.norm_epsilon)
        if self.tp > 1:
            y = tpc.gather_seq(y, st.tp_group)
        bcx = gemm.linear(y, self.in_proj.weight)
        if cfg.conv_bias:
            bcx = bcx + self.in_proj.bias
        h = self.hl
        B, C, x = bcx[:, :h], bcx[:, h:2 * h], bcx[:, 2 * h:]
        conv = causal_depthwise_conv(B * x, self.conv.weight[:, 0, :], self.conv.bias if cfg.conv_bias else None, batch)
        if self.tp > 1:
            out = layers.row_parallel_linear((C * conv).contiguous(), self.out_proj.weight, st.tp_group, True)
        else:
            out = gemm.linear((C * conv).contiguous(), self.out_proj.weight)
        if cfg.conv_bias:
            out = out + self.out_proj.bias
        return out, xsum


# ------------------------------------------------------------------------------------------------ Mamba-2
def _segsum(a: torch.Tensor) -> torch.Tensor:
    """a [..., L] -> S [..., L, L] with S[i, j] = sum_{j < k <= i} a[k] for i >= j and -inf above the diagonal."""
    L = a.shape[-1]
    c = torch.cumsum(a, -1)
    s = c[..., :, None] - c[..., None, :]
    mask = torch.ones(L, L, dtype=torch.bool, device=a.device).tril()
    return s.masked_fill(~mask, float("-inf"))


def ssd_chunked(x, dt, A, B, C, chunk: int):
    """Selective state-space model, chunk-wise (state-space duality).

    x [b, l, h, p], dt [b, l, h] (already positive), A [h] (negative), B and C [b, l, g, n] with h % g == 0.
    Returns y [b, l, h, p] with ``s_t = exp(dt_t A) s_{t-1} + dt_t x_t B_t^T`` (state [p, n] per head) and ``y_t = s_t C_t``.
    Inside a chunk the recurrence is a masked matrix product; between chunks only the [p, n] states are carried."""
    b, l, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    pad = (-l) % chunk
    if pad:
        x, dt, B, C = (F.pad(t, (0, 0) * (t.dim() - 2) + (0, pad)) for t in (x, dt, B, C))
    L = l + pad
    c = L // chunk
    rep = h // g
    xf = (x.float() * dt.float()[..., None]).view(b, c, chunk, h, p)
    a = (dt.float() * A.float()).view(b, c, chunk, h).permute(0, 3, 1, 2)            # [b, h, c, chunk] log-decays
    Bf = B.float().repeat_interleave(rep, 2).view(b, c, chunk, h, n)
    Cf = C.float().repeat_interleave(rep, 2).view(b, c, chunk, h, n)
    a_cum = torch.cumsum(a, -1)
    # within-chunk (diagonal blocks)
    decay = torch.exp(_segsum(a))                                                     # [b, h, c, chunk, chunk]
    y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", Cf, Bf, decay, xf)
    # state each chunk hands on, then the recurrence over chunks
    decay_states = torch.exp(a_cum[..., -1:] - a_cum)                                 # [b, h, c, chunk]
    states = torch.einsum("bclhn,bhcl,bclhp->bchpn", Bf, decay_states, xf)
    states = torch.cat([torch.zeros_like(states[:, :1]), states], 1)
    decay_chunk = torch.exp(_segsum(F.pad(a_cum[..., -1], (1, 0))))                   # [b, h, c + 1, c + 1]
    states = torch.einsum("bhzc,bchpn->bzhpn", decay_chunk, states)[:, :-1]
    y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", Cf, states, torch.exp(a_cum))
    y = (y_diag + y_off).reshape(b, L, h, p)
    return y[:, :l]


def ssd_sequential(x, dt, A, B, C):
    """The recurrence of ``ssd_chunked`` one step at a time (test oracle)."""
    b, l, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep = h // g
    Bf, Cf = B.float().repeat_interleave(rep, 2), C.float().repeat_interleave(rep, 2)
    s = torch.zeros(b, h, p, n, dtype=torch.float32, device=x.device)
    ys = []
    for t in range(l):
        da = torch.exp(dt[:, t].float() * A.float())                                  # [b, h]
        s = s * da[..., None, None] + (dt[:, t].float()[..., None] * x[:, t].float())[..., None] * Bf[:, t][:, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", s, Cf[:, t]))
    return torch.stack(ys, 1)


class Mamba2Mixer(nn.Module):
    """Mamba-2 mixer; parameter names follow Megatron's ``MambaMixer`` (``in_proj``, ``conv1d``, ``dt_bias``, ``A_log``, ``D``,
    ``norm``, ``out_proj``)."""

    def __init__(self, cfg, layer_idx: int, device, tp: int):
        super().__init__()
        # Tensor parallelism splits the heads and the B / C groups (needs sequence parallelism, like the other mixers)
        assert tp == 1 or cfg.sequence_parallel, "the Mamba mixer under tensor parallelism needs sequence_parallel"
        self.cfg, self.tp = cfg, tp
        h, dt = cfg.hidden_size, cfg.torch_dtype
        d_inner = cfg.mamba_expand * h
        self.headdim = cfg.mamba_head_dim
        nheads = cfg.mamba_num_heads or d_inner // self.headdim
        assert nheads * self.headdim == d_inner, "mamba_expand * hidden_size must equal heads * head_dim"
        assert nheads % cfg.mamba_num_groups == 0
        assert nheads % tp == 0 and cfg.mamba_num_groups % tp == 0, "heads and groups must divide by tp"
        self.d_inner, self.nheads = d_inner // tp, nheads // tp                 # this rank's share
        self.ngroups, self.d_state = cfg.mamba_num_groups // tp, cfg.mamba_state_dim
        self.conv_dim = self.d_inner + 2 * self.ngroups * self.d_state
        std = cfg.init_method_std
        self.in_proj = nn.Module()
        self.in_proj.register_parameter("layer_norm_weight", nn.Parameter(torch.ones(h, dtype=dt, device=device)))
        self.in_proj.register_parameter("weight", _param((2 * self.d_inner + 2 * self.ngroups * self.d_state + self.nheads, h),
                                                         std, dt, device))
        self.conv1d = nn.Module()
        self.conv1d.register_parameter("weight", _param((self.conv_dim, 1, cfg.mamba_d_conv), std * 5, dt, device))
        self.conv1d.register_parameter("bias", nn.Parameter(torch.zeros(self.conv_dim, dtype=dt, device=device)))
        # dt bias such that softplus(bias) is log-uniform in [1e-3, 1e-1]; A in [1, 16]: the published initialisation
        u = torch.rand(self.nheads, device=device)
        dt0 = torch.exp(u * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter((dt0 + torch.log(-torch.expm1(-dt0))).float())
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nheads, device=device).uniform_(1, 16)).float())
        self.D = nn.Parameter(torch.ones(self.nheads, dtype=torch.float32, device=device))
        self.norm = nn.Module()
        self.norm.register_parameter("weight", nn.Parameter(torch.ones(self.d_inner, dtype=dt, device=device)))
        self.out_proj = nn.Module()
        self.out_proj.register_parameter("weight", _param((h, self.d_inner), std / math.sqrt(2.0 * cfg.num_layers), dt, device))
        for w in (self.in_proj.weight, self.out_proj.weight):
            w._is_weight = True
        for p in (self.dt_bias, self.A_log, self.D):
            p._no_weight_decay = True
        if tp > 1:
            DI, GN, NH = self.d_inner * tp, self.ngroups * self.d_state * tp, self.nheads * tp
            _mark_tp(self.in_proj.weight, 0, [DI, DI, GN, GN, NH])
            _mark_tp(self.conv1d.weight, 0, [DI, GN, GN])
            _mark_tp(self.conv1d.bias, 0, [DI, GN, GN])
            for p in (self.dt_bias, self.A_log, self.D, self.norm.weight):
                _mark_tp(p, 0)
            _mark_tp(self.out_proj.weight, 1)
            self.in_proj.layer_norm_weight.sequence_parallel = True

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        assert st.cp == 1, "the Mamba mixer is not built for context parallelism"
        y, xsum = _norm(hidden, residual, self.in_proj.layer_norm_weight, cfg.norm_epsilon)
        if self.tp > 1:
            y = tpc.gather_seq(y, st.tp_group)
        zxbcdt = gemm.linear(y, self.in_proj.weight)
        T = zxbcdt.shape[0]
        seq = T // batch
        di, gn = self.d_inner, self.ngroups * self.d_state
        z, xBC, dt = zxbcdt[:, :di], zxbcdt[:, di:di + self.conv_dim], zxbcdt[:, di + self.conv_dim:]
        xBC = F.silu(causal_depthwise_conv(xBC, self.conv1d.weight[:, 0, :], self.conv1d.bias, batch))
        x = xBC[:, :di].view(batch, seq, self.nheads, self.headdim)
        B = xBC[:, di:di + gn].view(batch, seq, self.ngroups, self.d_state)
        C = xBC[:, di + gn:].view(batch, seq, self.ngroups, self.d_state)
        dtp = F.softplus(dt.float() + self.dt_bias).view(batch, seq, self.nheads)
        A = -torch.exp(self.A_log.float())
        yss = ssd_chunked(x, dtp, A, B, C, cfg.mamba_chunk_size)
        yss = yss + x.float() * self.D[None, None, :, None]
        yss = yss.reshape(T, di)
        # gated RMSNorm over each group's share of the inner dimension: norm(y * silu(z)) * weight
        gated = (yss * F.silu(z.float())).view(T, self.ngroups, di // self.ngroups)
        gated = gated * torch.rsqrt(gated.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon)
        out = (gated.view(T, di) * self.norm.weight.float()).to(hidden.dtype)
        if self.tp > 1:
            return layers.row_parallel_linear(out.contiguous(), self.out_proj.weight, st.tp_group, True), xsum
        return gemm.linear(out.contiguous(), self.out_proj.weight), xsum


# ------------------------------------------------------------------------------------------------ gated delta net
def gated_delta_rule_sequential(q, k, v, g, beta, scale=None):
    """The gated delta rule one token at a time (test oracle).  q, k [b, l, h, dk], v [b, l, h, dv], g [b, l, h]
    (log-decay, <= 0), beta [b, l, h].  State S [dk, dv] per head:
    ``S <- exp(g_t) S``; ``S <- S + k_t (beta_t (v_t - k_t^T S))^T``; ``o_t = (scale q_t)^T S``."""
    b, l, h, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    S = torch.zeros(b, h, dk, dv, dtype=torch.float32, device=q.device)
    out = []
    for t in range(l):
        S = S * torch.exp(g[:, t].float())[..., None, None]
        kt, vt = k[:, t].float(), v[:, t].float()
        mem = torch.einsum("bhk,bhkv->bhv", kt, S)
        delta = (vt - mem) * beta[:, t].float()[..., None]
        S = S + kt[..., :, None] * delta[..., None, :]
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].float() * scale, S))
    return torch.stack(out, 1)


def gated_delta_rule_chunked(q, k, v, g, beta, chunk: int = 64, scale=None):
    """The same recurrence chunk-wise.  Inside a chunk the deltas solve a unit lower-triangular system
    ``(I + L) U = beta (V - decayed K S_in)`` with ``L = strict_lower(beta K K^T * decay)``, so one triangular solve
    per chunk replaces the token loop; between chunks only the [dk, dv] state is carried."""
    b, l, h, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    pad = (-l) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
    L_ = l + pad
    c = L_ // chunk
    # [b, h, c, chunk, d]
    qf = (q.float() * scale).permute(0, 2, 1, 3).reshape(b, h, c, chunk, dk)
    kf = k.float().permute(0, 2, 1, 3).reshape(b, h, c, chunk, dk)
    vf = v.float().permute(0, 2, 1, 3).reshape(b, h, c, chunk, dv)
    gf = g.float().permute(0, 2, 1).reshape(b, h, c, chunk)
    bf = beta.float().permute(0, 2, 1).reshape(b, h, c, chunk)
    gc = torch.cumsum(gf, -1)                                           # log-decay from the chunk start to each token
    lower = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    diff = (gc[..., :, None] - gc[..., None, :]).masked_fill(~lower, 0.0)
    decay = torch.exp(diff).masked_fill(~lower, 0.0)                    # [.., i, j] = exp(gc_i - gc_j), j <= i
    kb = kf * bf[..., None]
    strict = decay * torch.ones(chunk, chunk, device=q.device).tril(-1)
    A = torch.eye(chunk, device=q.device) + (kb @ kf.transpose(-1, -2)) * strict
    # T = (I + L)^-1 applied to [beta V | beta K exp(gc)]
    rhs = torch.cat([vf * bf[..., None], kb * torch.exp(gc)[..., None]], -1)
    sol = torch.linalg.solve_triangular(A, rhs, upper=False)
    u_v, u_k = sol[..., :dv], sol[..., dv:]                             # deltas without / per unit of the carried state
    attn_in = (qf @ kf.transpose(-1, -2)) * decay                       # within-chunk scores (j <= i)
    S = torch.zeros(b, h, dk, dv, dtype=torch.float32, device=q.device)
    outs = []
    for i in range(c):
        delta = u_v[:, :, i] - u_k[:, :, i] @ S                          # [chunk, dv]
        inter = (qf[:, :, i] * torch.exp(gc[:, :, i])[..., None]) @ S
        outs.append(inter + attn_in[:, :, i] @ delta)
        last = gc[:, :, i, -1]
        S = S * torch.exp(last)[..., None, None] + \
            (kf[:, :, i] * torch.exp(last[..., None] - gc[:, :, i])[..., None]).transpose(-1, -2) @ delta
    o = torch.stack(outs, 2).reshape(b, h, L_, dv).permute(0, 2, 1, 3)
    return o[:, :l]


class GatedDeltaNetMixer(nn.Module):
    """Gated delta net (linear attention with a decaying, delta-rule-corrected state): ``q, k, v, z, b, a = in_proj(h)``;
    causal depthwise convolution + SiLU on ``[q | k | v]``; L2-normalised q / k; ``beta = sigmoid(b)``,
    ``g = -exp(A_log) softplus(a + dt_bias)``; the gated delta rule; per-head RMSNorm gated by ``silu(z)``; ``out_proj``.
    The 'M' layers of the reference's GDN hybrid stacks (primus/backends/megatron/core/models/hybrid/gated_delta_net.py,
    ``gdn_hybrid_stack_spec`` in hybrid_mamba_mla_layer_specs.py:189-262; presets ``zebra_llama_*_gdn*``); parameter
    names follow it (``in_proj``, ``conv1d``, ``A_log``, ``dt_bias``, ``out_norm``, ``out_proj``)."""

    def __init__(self, cfg, layer_idx: int, device, tp: int):
        super().__init__()
        # Tensor parallelism splits the heads (needs sequence parallelism: the mixer gathers the normalised tokens,
        # works on its own heads and reduce-scatters the output projection)
        assert tp == 1 or cfg.sequence_parallel, "the gated-delta-net mixer under tensor parallelism needs sequence_parallel"
        assert cfg.linear_num_key_heads % tp == 0 and cfg.linear_num_value_heads % tp == 0, "heads must divide by tp"
        self.cfg, self.tp = cfg, tp
        h, dt = cfg.hidden_size, cfg.torch_dtype
        self.nk, self.nv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp      # this rank's heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        assert self.nv % self.nk == 0
        self.qk_dim, self.v_dim = self.nk * self.dk, self.nv * self.dv
        self.conv_dim = 2 * self.qk_dim + self.v_dim
        std = cfg.init_method_std
        self.in_proj = nn.Module()
        self.in_proj.register_parameter("layer_norm_weight", nn.Parameter(torch.ones(h, dtype=dt, device=device)))
        self.in_proj.register_parameter("weight", _param((self.conv_dim + self.v_dim + 2 * self.nv, h), std, dt, device))
        self.conv1d = nn.Module()
        self.conv1d.register_parameter("weight", _param((self.conv_dim, 1, cfg.linear_conv_kernel_dim), std * 5, dt, device))
        u = torch.rand(self.nv, device=device)
        dt0 = torch.exp(u * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter((dt0 + torch.log(-torch.expm1(-dt0))).float())
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nv, device=device).uniform_(1e-3, 16)).float())
        self.out_norm = nn.Module()
        self.out_norm.register_parameter("weight", nn.Parameter(torch.ones(self.dv, dtype=dt, device=device)))
        self.out_proj = nn.Module()
        self.out_proj.register_parameter("weight", _param((h, self.v_dim), std / math.sqrt(2.0 * cfg.num_layers), dt, device))
        for w in (self.in_proj.weight, self.out_proj.weight):
            w._is_weight = True
        if tp > 1:
            QK, V, NV = self.qk_dim * tp, self.v_dim * tp, self.nv * tp
            _mark_tp(self.in_proj.weight, 0, [QK, QK, V, V, NV, NV])
            _mark_tp(self.conv1d.weight, 0, [QK, QK, V])
            _mark_tp(self.dt_bias, 0)
            _mark_tp(self.A_log, 0)
            _mark_tp(self.out_proj.weight, 1)
            # replicated; their gradients are partial sums (over this rank's tokens / heads): added over the group
            self.in_proj.layer_norm_weight.sequence_parallel = True
            self.out_norm.weight.sequence_parallel = True

    def forward(self, hidden, residual, rope, batch):
        cfg = self.cfg
        st = ps.get_state()
        assert st.cp == 1, "the gated-delta-net mixer is not built for context parallelism"
        y, xsum = _norm(hidden, residual, self.in_proj.layer_norm_weight, cfg.norm_epsilon)
        if self.tp > 1:
            y = tpc.gather_seq(y, st.tp_group)
        proj = gemm.linear(y, self.in_proj.weight)
        T = proj.shape[0]
        seq = T // batch
        cd, vd, nv = self.conv_dim, self.v_dim, self.nv
        qkv, z, b_, a_ = proj[:, :cd], proj[:, cd:cd + vd], proj[:, cd + vd:cd + vd + nv], proj[:, cd + vd + nv:]
        qkv = F.silu(causal_depthwise_conv(qkv, self.conv1d.weight[:, 0, :], None, batch))
        q = qkv[:, :self.qk_dim].view(batch, seq, self.nk, self.dk)
        k = qkv[:, self.qk_dim:2 * self.qk_dim].view(batch, seq, self.nk, self.dk)
        v = qkv[:, 2 * self.qk_dim:].view(batch, seq, nv, self.dv)
        rep = nv // self.nk
        if rep > 1:
            q, k = q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2)
        q = F.normalize(q.float(), dim=-1, eps=1e-6)
        k = F.normalize(k.float(), dim=-1, eps=1e-6)
        beta = torch.sigmoid(b_.float()).view(batch, seq, nv)
        g = (-torch.exp(self.A_log.float()) * F.softplus(a_.float() + self.dt_bias)).view(batch, seq, nv)
        o = gated_delta_rule_chunked(q, k, v, g, beta, cfg.linear_chunk_size)            # [b, l, nv, dv] fp32
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * self.out_norm.weight.float()
        o = (o.reshape(T, vd) * F.silu(z.float())).to(hidden.dtype)
        if self.tp > 1:
            return layers.row_parallel_linear(o.contiguous(), self.out_proj.weight, st.tp_group, True), xsum
        return gemm.linear(o.contiguous(), self.out_proj.weight), xsum
