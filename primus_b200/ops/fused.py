"""Autograd wrappers of the memory-bound sm_100a kernels in ``csrc/elementwise.cu``:
RMSNorm (optionally fused with the residual add), RoPE, SwiGLU (plain / probs-weighted / clamped),
cross-entropy (fused forward+gradient, vocab-parallel) and the embedding gradient.

Each op has a ``*_ref`` plain-PyTorch fp32 implementation which (a) is the CPU execution path and
(b) is the oracle of the GPU numerics tests.  CUDA tensors always take the native kernel.

Parity: rmsnorm / fused residual norm (primus/backends/megatron/core/extensions/primus_turbo.py:1697-1700,
fused_residual_rmsnorm.py:327-453), swiglu_with_probs (primus_turbo.py:1954-1980), clamped SwiGLU
(primus/backends/megatron/core/fusions/fused_bias_swiglu.py:25-100), cross-entropy fusion
(examples/megatron/configs/MI355X/llama3.1_8B-BF16-pretrain.yaml:69-71).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from . import _lib

# ----------------------------------------------------------------------------------------------
# scratch buffers (per device, grown on demand, reused across calls on the same stream)
_SCRATCH: dict[tuple[int, str], torch.Tensor] = {}


def scratch(device: torch.device, name: str, numel: int) -> torch.Tensor:
    key = (device.index or 0, name)
    t = _SCRATCH.get(key)
    if t is None or t.numel() < numel:
        t = torch.empty(max(numel, 1), dtype=torch.float32, device=device)
        _SCRATCH[key] = t
    return t


# ----------------------------------------------------------------------------------------------
# RMSNorm
def rmsnorm_ref(x, w, eps, residual=None):
    xs = x.float() if residual is None else (x.float() + residual.float()).to(x.dtype).float()
    rstd = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
    y = (xs * rstd * w.float()).to(x.dtype)
    return (y, xs.to(x.dtype)) if residual is not None else y


class RMSNormFn(torch.autograd.Function):
    """y = rmsnorm(x [+ residual]) * w.  With a residual the summed stream is the second output."""

    @staticmethod
    def forward(ctx, x, w, eps, residual):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        xsum = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            xsum = torch.empty_like(x2)
            _lib.call("rmsnorm_fwd", x2, r2, w, y, xsum, rstd, rows, H, x2.stride(0), y.stride(0), float(eps))
            ctx.save_for_backward(xsum, w, rstd)
        else:
            _lib.call("rmsnorm_fwd", x2, None, w, y, None, rstd, rows, H, x2.stride(0), y.stride(0), float(eps))
            ctx.save_for_backward(x2, w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        ctx.w_ref = w
        if residual is not None:
            return y.view(x.shape), xsum.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dxsum=None):
        xin, w, rstd = ctx.saved_tensors
        H = xin.shape[-1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dxsum is not None:
            dres = dxsum.reshape(-1, H)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(xin)
        P = _lib.call_ret("rmsnorm_bwd_num_partials", rows)
        sc = scratch(xin.device, "rmsnorm_dw", P * H)
        main_grad = getattr(ctx.w_ref, "main_grad", None)
        if main_grad is not None:
            _lib.call("rmsnorm_bwd", dy2, xin, w, rstd, dres, dx, main_grad, sc, rows, H, xin.stride(0),
                      dy2.stride(0), 1)
            dw = None
        else:
            dwf = torch.empty(H, dtype=torch.float32, device=xin.device)
            _lib.call("rmsnorm_bwd", dy2, xin, w, rstd, dres, dx, dwf, sc, rows, H, xin.stride(0),
                      dy2.stride(0), 0)
            dw = dwf.to(w.dtype)
        dx = dx.view(ctx.shape)
        if ctx.has_res:
            return dx, dw, None, dx
        return dx, dw, None, None


# ``apply_layernorm_1p``: the norm weights are stored centred on zero and the norm multiplies by ``1 + weight`` (weight
# decay then pulls the gain towards 1 instead of 0).  Set by the model from its configuration; the gated norms inside the
# Mamba / gated-delta-net mixers keep plain weights.
ZERO_CENTERED_GAMMA = False


def set_zero_centered_gamma(flag: bool) -> None:
    global ZERO_CENTERED_GAMMA
    ZERO_CENTERED_GAMMA = bool(flag)


def gamma(w):
    """The gain a norm applies for the stored weight ``w``."""
    return w + 1.0 if ZERO_CENTERED_GAMMA else w


def rmsnorm(x, w, eps=1e-5, residual=None):
    """RMSNorm over the last dim. ``residual`` given -> returns (y, x + residual)."""
    w = gamma(w)
    if not x.is_cuda:
        return rmsnorm_ref(x, w, eps, residual)
    return RMSNormFn.apply(x, w, eps, residual)


# ----------------------------------------------------------------------------------------------
# RoPE (rotate-half convention, first ``rot_dim`` channels of each head)
def llama3_scale_frequencies(inv, factor: float, low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                             original_max_pos: int = 8192):
    """Llama-3.x long-context frequency scaling: wavelengths above ``original_max_pos / low_freq_factor`` are stretched by
    ``factor``, those below ``original_max_pos / high_freq_factor`` stay, the band between is interpolated (the
    ``use_rope_scaling`` / ``rope_scaling_factor`` switches of the reference's model presets,
    primus/configs/models/megatron/language_model.yaml:46-47)."""
    wavelen = 2.0 * math.pi / inv
    low_wl = original_max_pos / low_freq_factor
    high_wl = original_max_pos / high_freq_factor
    smooth = ((original_max_pos / wavelen) - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = (1.0 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen > low_wl, inv / factor, torch.where(wavelen < high_wl, inv, mid))


def rope_tables(max_pos: int, rot_dim: int, theta: float, device, scaling_factor: float = 1.0, llama3_scaling=None):
    """cos / sin tables [max_pos, rot_dim / 2] in fp32.  ``llama3_scaling``: None or the keyword arguments of
    :func:`llama3_scale_frequencies`."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    if llama3_scaling:
        inv = llama3_scale_frequencies(inv, **llama3_scaling)
    t = torch.arange(max_pos, dtype=torch.float32, device=device) / scaling_factor
    f = torch.outer(t, inv)
    return f.cos().contiguous(), f.sin().contiguous()


def rope_ref(x, cos, sin, pos=None, rot_dim=None):
    """x: [T, heads, d]."""
    T, h, d = x.shape
    rot = rot_dim or d
    half = rot // 2
    idx = torch.arange(T, device=x.device) if pos is None else pos.long()
    c = cos[idx][:, None, :].float()
    s = sin[idx][:, None, :].float()
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rot] = b * c + a * s
    return out.to(x.dtype)


class RoPEFn(torch.autograd.Function):
    """Applies RoPE to a [T, heads, d] view (arbitrary row pitch) and returns a new tensor."""

    @staticmethod
    def forward(ctx, x, cos, sin, pos, rot_dim):
        T, h, d = x.shape
        out = x.contiguous().clone() if not x.is_contiguous() else x.clone()
        _lib.call("rope", out, pos, cos, sin, T, h, d, rot_dim, out.stride(0), 0)
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        ctx.rot_dim = rot_dim
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        T, h, d = dy.shape
        g = dy.contiguous().clone()
        _lib.call("rope", g, pos if ctx.has_pos else None, cos, sin, T, h, d, ctx.rot_dim, g.stride(0), 1)
        return g, None, None, None, None


def rope_inplace_(x, cos, sin, pos=None, rot_dim=None, backward=False):
    """In-place RoPE on a [T, heads, d] strided view (no autograd); used inside fused attention."""
    T, h, d = x.shape
    assert x.stride(2) == 1 and x.stride(1) == d
    if not x.is_cuda:
        if backward:
            x.copy_(rope_ref(x, cos, -sin, pos, rot_dim))
        else:
            x.copy_(rope_ref(x, cos, sin, pos, rot_dim))
        return x
    _lib.call("rope", x, pos, cos, sin, T, h, d, rot_dim or d, x.stride(0), int(backward))
    return x


def rope(x, cos, sin, pos=None, rot_dim=None):
    if not x.is_cuda:
        return rope_ref(x, cos, sin, pos, rot_dim)
    return RoPEFn.apply(x, cos, sin, pos, rot_dim or x.shape[-1])


# ----------------------------------------------------------------------------------------------
# SwiGLU: in [T, 2I] = [gate | up]
GATE_KINDS = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "situ": 2}
# "situ" (Kimi-K3): SiLU whose linear factor is soft-clamped, times a soft-clamped up branch,
# ``beta tanh(g / beta) sigmoid(g) * linear_beta tanh(u / linear_beta)``; runs as composed fp32 operations on every
# device (primus/backends/megatron/core/transformer/kimi_k3/situ_activation.py:8-24 in the reference).
SITU_BETAS = [4.0, 25.0]


def set_situ_betas(beta: float, linear_beta) -> None:
    SITU_BETAS[0], SITU_BETAS[1] = float(beta), (float(linear_beta) if linear_beta else 0.0)


def swiglu_ref(x, probs=None, clamp=0.0, act="silu"):
    I = x.shape[-1] // 2
    g, u = x[..., :I].float(), x[..., I:].float()
    if GATE_KINDS[act] == 2:
        b, lb = SITU_BETAS
        y = b * torch.tanh(g / b) * torch.sigmoid(g) * (lb * torch.tanh(u / lb) if lb else u)
        if probs is not None:
            y = y * probs.float().reshape(*y.shape[:-1], 1)
        return y.to(x.dtype)
    if clamp and clamp > 0:
        g = g.clamp(max=clamp)
        u = u.clamp(-clamp, clamp)
    y = (torch.nn.functional.silu(g) if GATE_KINDS[act] == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
    if probs is not None:
        y = y * probs.float().reshape(*y.shape[:-1], 1)
    return y.to(x.dtype)


class SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, clamp, act="silu"):
        I = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * I)
        T = x2.shape[0]
        out = torch.empty(T, I, dtype=x.dtype, device=x.device)
        p = probs.reshape(-1).float().contiguous() if probs is not None else None
        ctx.kind = GATE_KINDS[act]
        _lib.call("swiglu_fwd", x2, p, out, T, I, float(clamp), ctx.kind)
        ctx.save_for_backward(x2, p if p is not None else torch.empty(0))
        ctx.has_probs = probs is not None
        ctx.clamp = clamp
        ctx.shape = x.shape
        ctx.probs_shape = probs.shape if probs is not None else None
        ctx.probs_dtype = probs.dtype if probs is not None else None
        return out.view(*x.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        x2, p = ctx.saved_tensors
        T, I2 = x2.shape
        I = I2 // 2
        dy2 = dy.reshape(T, I)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        din = torch.empty_like(x2)
        dprobs = torch.empty(T, dtype=torch.float32, device=x2.device) if ctx.has_probs else None
        _lib.call("swiglu_bwd", dy2, x2, p if ctx.has_probs else None, din, dprobs, T, I, float(ctx.clamp), ctx.kind)
        dp = dprobs.view(ctx.probs_shape).to(ctx.probs_dtype) if ctx.has_probs else None
        return din.view(ctx.shape), dp, None, None


def swiglu(x, probs=None, clamp=0.0, act="silu"):
    """Gated linear unit ``act(gate) * up [* probs]`` for x = [gate | up]; ``act``: "silu" (SwiGLU) or "gelu" (GEGLU,
    tanh approximation) -- the reference's swiglu_with_probs / geglu_with_probs
    (primus/backends/megatron/core/extensions/primus_turbo.py:1954-1980)."""
    if not x.is_cuda or GATE_KINDS[act] == 2:
        return swiglu_ref(x, probs, clamp, act)
    return SwiGLUFn.apply(x, probs, clamp, act)


# ----------------------------------------------------------------------------------------------
# Logit soft-capping: cap * tanh(x / cap)
def softcap_ref(x, cap: float):
    return (torch.tanh(x.float() / cap) * cap).to(x.dtype)


class SoftcapFn(torch.autograd.Function):
    """In-place soft-capping of (final / router) logits; the backward uses the saved output.
    (Role of the reference's `fused_softcap`, primus/backends/megatron/core/extensions/logits_processor.py:41-50.)"""

    @staticmethod
    def forward(ctx, x, cap):
        x = x.contiguous()
        _lib.call("softcap_fwd", x, x, x.numel(), float(cap))
        ctx.mark_dirty(x)
        ctx.save_for_backward(x)
        ctx.cap = cap
        return x

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        _lib.call("softcap_bwd", dy, y, dx, dy.numel(), float(ctx.cap))
        return dx, None


def softcap(x, cap: float | None):
    """cap * tanh(x / cap); ``cap`` None or 0 is the identity.  On CUDA the bf16 input is overwritten."""
    if not cap:
        return x
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.numel() % 8:
        return softcap_ref(x, cap)
    if x.requires_grad and x.is_leaf:
        x = x.clone()
    return SoftcapFn.apply(x, cap)


# ----------------------------------------------------------------------------------------------
# Cross entropy (optionally vocab-parallel over a TP group)
class _VocabParallelCERef(torch.autograd.Function):
    """Plain-PyTorch vocab-parallel cross entropy with an explicit backward (collectives are not
    differentiable, so the gradient (softmax - onehot) is formed by hand from the reduced statistics)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        lf = logits.detach().float()
        V = lf.shape[-1]
        m = lf.max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        ex = (lf - m[..., None]).exp()
        se = ex.sum(-1)
        lab = labels - vocab_start
        inr = (lab >= 0) & (lab < V)
        tgt = torch.where(inr, lf.gather(-1, lab.clamp(0, V - 1)[..., None]).squeeze(-1), torch.zeros_like(m))
        dist.all_reduce(se, group=group)
        dist.all_reduce(tgt, group=group)
        p = ex / se[..., None]
        onehot = torch.zeros_like(p)
        onehot.scatter_(-1, lab.clamp(0, V - 1)[..., None], inr[..., None].to(p.dtype))
        ctx.save_for_backward(p - onehot)
        ctx.dtype = logits.dtype
        return m + se.log() - tgt

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return (g * dloss[..., None]).to(ctx.dtype), None, None, None


def cross_entropy_ref(logits, labels, vocab_start=0, group=None):
    """Per-token loss, fp32. Vocab-parallel when ``group`` is given (logits hold a vocab slice)."""
    if group is not None:
        return _VocabParallelCERef.apply(logits, labels, vocab_start, group)
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    tgt = lf.gather(-1, labels[..., None]).squeeze(-1)
    return lse - tgt


class CrossEntropyFn(torch.autograd.Function):
    """loss[t] = logsumexp(logits[t]) - logits[t, label[t]].  The gradient w.r.t. the logits is
    computed in the forward pass and stored *in place of the logits* (which are dead afterwards),
    so no [T, V] buffer outlives the call besides the bf16 logits themselves.

    With ``weights`` the result is the scalar ``sum_t weights[t] * loss[t]`` and the stored gradient is
    already multiplied by ``weights[t]``; ``unit_upstream`` promises that the caller back-propagates a
    gradient of exactly 1 into that scalar, which removes the only remaining pass over the logits."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group, weights, unit_upstream):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        rows = l2.shape[0]
        lab = labels.reshape(-1).contiguous()
        gsc = (weights.reshape(-1).float().contiguous() if weights is not None
               else torch.ones(rows, dtype=torch.float32, device=logits.device))
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        if group is None or dist.get_world_size(group) == 1:
            _lib.call("ce_fused", l2, lab, gsc, loss, rows, V, l2.stride(0))
        else:
            st = torch.empty(3, rows, dtype=torch.float32, device=logits.device)
            _lib.call("ce_stats", l2, lab, st[0], st[1], st[2], rows, V, l2.stride(0), int(vocab_start))
            gmax = st[0].clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            st[1].mul_((st[0] - gmax).exp())
            dist.all_reduce(st[1:], group=group)
            lse = gmax + st[1].log()
            loss = lse - st[2]
            _lib.call("ce_grad", l2, lab, lse.contiguous(), gsc, rows, V, l2.stride(0), int(vocab_start))
        ctx.save_for_backward(l2)
        ctx.shape = logits.shape
        ctx.unit = bool(unit_upstream and weights is not None)
        ctx.weighted = weights is not None
        ctx.mark_non_differentiable(labels)
        if weights is not None:
            return (loss * gsc).sum()
        return loss.view(labels.shape)

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        if not ctx.unit:
            if ctx.weighted:
                g.mul_(dloss.to(g.dtype))
            else:
                g.mul_(dloss.reshape(-1, 1).to(g.dtype))
        return g.view(ctx.shape), None, None, None, None, None


def cross_entropy(logits, labels, vocab_start=0, group=None, weights=None, unit_upstream=False):
    """Per-token loss (fp32, shape of ``labels``), or ``sum(weights * loss)`` when ``weights`` is given.
    Consumes (overwrites) ``logits`` on CUDA."""
    if not logits.is_cuda:
        loss = cross_entropy_ref(logits, labels, vocab_start, group if _dist_group_active(group) else None)
        return (loss * weights.reshape(loss.shape).float()).sum() if weights is not None else loss
    return CrossEntropyFn.apply(logits, labels, vocab_start, group, weights, unit_upstream)


def _dist_group_active(group) -> bool:
    return group is not None and dist.is_initialized() and dist.get_world_size(group) > 1


# ----------------------------------------------------------------------------------------------
class EmbeddingFn(torch.autograd.Function):
    """Row gather whose backward scatter-adds in fp32 into ``weight.main_grad`` when present."""

    @staticmethod
    def forward(ctx, tokens, weight, vocab_start, partial):
        ctx.save_for_backward(tokens)
        ctx.w_ref = weight
        ctx.vocab_start = vocab_start
        V = weight.shape[0]
        if not partial:
            return torch.nn.functional.embedding(tokens, weight)
        loc = tokens - vocab_start
        mask = (loc < 0) | (loc >= V)
        out = torch.nn.functional.embedding(loc.clamp(0, V - 1), weight)
        return out.masked_fill(mask[..., None], 0)

    @staticmethod
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        w = ctx.w_ref
        V, H = w.shape
        main_grad = getattr(w, "main_grad", None)
        dy2 = dy.reshape(-1, H).contiguous()
        tok = tokens.reshape(-1).contiguous()
        if dy.is_cuda:
            tgt = main_grad if main_grad is not None else torch.zeros(V, H, dtype=torch.float32, device=dy.device)
            _lib.call("embedding_bwd", dy2, tok, tgt, tok.numel(), H, int(ctx.vocab_start), V)
            return None, (None if main_grad is not None else tgt.to(w.dtype)), None, None
        loc = tok - ctx.vocab_start
        ok = (loc >= 0) & (loc < V)
        g = torch.zeros(V, H, dtype=torch.float32)
        g.index_add_(0, loc[ok], dy2[ok].float())
        if main_grad is not None:
            main_grad.add_(g)
            return None, None, None, None
        return None, g.to(w.dtype), None, None


def embedding(tokens, weight, vocab_start=0, partial=False):
    """``partial``: the weight holds the vocabulary slice starting at ``vocab_start`` (vocab-parallel);
    tokens outside the slice produce zero rows (summed across the TP group by the caller)."""
    return EmbeddingFn.apply(tokens, weight, vocab_start, partial)
