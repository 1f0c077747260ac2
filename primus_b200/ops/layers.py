"""Fused layer-level autograd functions that keep the saved-activation set minimal.

* :func:`norm_linear`  — (residual add +) RMSNorm + GEMM.  Saves only the residual stream and
  the per-row rstd; the normalised activations are recomputed in backward (one cheap
  memory-bound pass) instead of being stored.  Mirrors the role of
  ``TELayerNormColumnParallelLinear`` / ``PrimusTurboLayerNormColumnParallelLinear``
  (primus/backends/megatron/core/extensions/primus_turbo.py:1689-1830) and of the fused
  residual+norm forward (fused_residual_rmsnorm.py:327-453).
* :func:`swiglu_linear` — SwiGLU (optionally weighted by routing probs) + GEMM; saves the FC1
  output only and recomputes the activation in backward.
* :func:`rope_attention` — RoPE applied in place on the packed QKV projection followed by flash
  attention; backward applies the inverse rotation in place on the packed dQKV.

Each function has a CPU composition of the reference ops with ordinary autograd.
"""
from __future__ import annotations

import math

import torch

from ..parallel import fused_tp
from ..parallel import tensor_parallel as tp_comm
from . import _lib, attention, fused, gemm


# ----------------------------------------------------------------------------------------------
class NormLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, residual, norm_w, weight, eps, tp_group, sp):
        H = hidden.shape[-1]
        x2 = hidden.reshape(-1, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        if residual is not None:
            r2 = residual.reshape(-1, H)
            xsum = torch.empty_like(x2)
            _lib.call("rmsnorm_fwd", x2, r2, norm_w, y, xsum, rstd, rows, H, x2.stride(0), y.stride(0), float(eps))
        else:
            xsum = x2
            _lib.call("rmsnorm_fwd", x2, None, norm_w, y, None, rstd, rows, H, x2.stride(0), y.stride(0), float(eps))
        if sp:
            out, _ = fused_tp.ag_gemm(y, weight, tp_group, fused=fused_tp.ENABLED)
        else:
            out = gemm.gemm(y, weight)
        ctx.save_for_backward(xsum, norm_w, weight, rstd)
        ctx.eps = eps
        ctx.tp = (tp_group, sp)
        ctx.set_materialize_grads(False)
        ctx.has_res = residual is not None
        ctx.shape = hidden.shape
        ctx.refs = (norm_w, weight)
        if residual is not None:
            return out, xsum.view(hidden.shape)
        return out, hidden

    @staticmethod
    def backward(ctx, dout, dxsum):
        xsum, norm_w, weight, rstd = ctx.saved_tensors
        norm_w_ref, weight_ref = ctx.refs
        if dout is None:
            dout = torch.zeros(xsum.shape[0] * (torch.distributed.get_world_size(ctx.tp[0]) if ctx.tp[1] else 1),
                               weight.shape[0], dtype=xsum.dtype, device=xsum.device)
        rows, H = xsum.shape
        tp_group, sp = ctx.tp
        dout2 = dout.reshape(-1, dout.shape[-1])
        if not dout2.is_contiguous():
            dout2 = dout2.contiguous()
        # recompute the normalised activations (not stored in forward)
        y = torch.empty_like(xsum)
        _lib.call("rmsnorm_fwd", xsum, None, norm_w, y, None, None, rows, H, xsum.stride(0), y.stride(0),
                  float(ctx.eps))
        if sp:
            if fused_tp._quantized_gather_ok(y, weight, False) and dout2.shape[1] % 128 == 0:
                y = fused_tp.all_gather_quantized(y, tp_group, row=False, col=True)   # MXFP8: gather the quantised copy
            else:
                y = tp_comm.all_gather_dim0(y, tp_group)
        dw = gemm.wgrad(dout2, y, weight_ref)
        del y
        if sp:
            dy = fused_tp.gemm_rs(dout2, weight, tp_group, b_mn=True, fused=fused_tp.ENABLED_RS)
        else:
            dy = gemm.gemm(dout2, weight, b_mn=True)
            if tp_group is not None:
                torch.distributed.all_reduce(dy, group=tp_group)
        dres = None
        if dxsum is not None:
            dres = dxsum.reshape(rows, H)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(xsum)
        P = _lib.call_ret("rmsnorm_bwd_num_partials", rows)
        sc = fused.scratch(xsum.device, "rmsnorm_dw", P * H)
        main_grad = getattr(norm_w_ref, "main_grad", None)
        if main_grad is not None:
            _lib.call("rmsnorm_bwd", dy, xsum, norm_w, rstd, dres, dx, main_grad, sc, rows, H, xsum.stride(0),
                      dy.stride(0), 1)
            dnw = None
        else:
            dwf = torch.empty(H, dtype=torch.float32, device=xsum.device)
            _lib.call("rmsnorm_bwd", dy, xsum, norm_w, rstd, dres, dx, dwf, sc, rows, H, xsum.stride(0),
                      dy.stride(0), 0)
            dnw = dwf.to(norm_w.dtype)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), dnw, dw, None, None, None


def norm_linear(hidden, residual, norm_w, weight, eps, tp_group=None, sequence_parallel=False):
    """Returns (linear(rmsnorm(hidden + residual)), hidden + residual).

    ``weight`` may be a column-parallel shard: with ``sequence_parallel`` the normalised local token
    shard is all-gathered over ``tp_group`` before the GEMM (reduce-scatter of the input gradient in
    backward); without it the input gradient is all-reduced."""
    sp = bool(sequence_parallel and tp_group is not None)
    norm_w = fused.gamma(norm_w)
    if not hidden.is_cuda:
        if residual is not None:
            y, xsum = fused.rmsnorm_ref(hidden, norm_w, eps, residual)
        else:
            y, xsum = fused.rmsnorm_ref(hidden, norm_w, eps, None), hidden
        if sp:
            y = tp_comm.gather_seq(y, tp_group)
        elif tp_group is not None:
            y = tp_comm.copy_to_tp(y, tp_group)
        return gemm.linear(y, weight), xsum
    return NormLinearFn.apply(hidden, residual, norm_w, weight, eps, tp_group, sp)


# ----------------------------------------------------------------------------------------------
def _swiglu_fp8_fusable(h1, weight, probs, tp_group, act="silu") -> bool:
    """MXFP8 recipe on, plain (no routing probabilities, no tensor parallelism) and every dimension a multiple of 128:
    the SwiGLU kernels then emit MXFP8 directly for the GEMMs around them."""
    # the fused SwiGLU + quantisation kernels scale per block: only under the MXFP8 recipe
    if gemm.fp8_recipe() != "mxfp8" or not gemm.FUSE_SWIGLU_QUANT or probs is not None or tp_group is not None:
        return False
    if fused.GATE_KINDS[act] != 0:      # the fused quantising kernels implement the SiLU gate only
        return False
    if getattr(weight, "_fp8_exempt", False) or h1.dtype != torch.bfloat16:
        return False
    T = h1.numel() // h1.shape[-1]
    I = h1.shape[-1] // 2
    return T % 128 == 0 and I % 128 == 0 and weight.shape[0] % 128 == 0 and weight.is_contiguous()


class SwiGLULinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h1, weight, probs, clamp, tp_group, sp, act="silu"):
        ctx.kind = fused.GATE_KINDS[act]
        I2 = h1.shape[-1]
        I = I2 // 2
        x2 = h1.reshape(-1, I2)
        T = x2.shape[0]
        ctx.fp8_fused = _swiglu_fp8_fusable(h1, weight, probs, tp_group, act) and x2.is_contiguous()
        if ctx.fp8_fused:
            from . import fp8

            # the producer of h1 must consume its gradient only through GEMMs (see backward)
            ctx.grad_via_cache = type(h1.grad_fn).__name__ in ("NormLinearFnBackward", "LinearFnBackward")
            aq = fp8.swiglu_quantize_mxfp8(x2, clamp, True, False)
            wq, wsf = gemm._quantized(weight, "row")
            N = weight.shape[0]
            out = torch.empty(T, N, dtype=torch.bfloat16, device=h1.device)
            fp8.launch_gemm(aq.q_row, aq.sf_row, wq, wsf, out, T, N, I, False, False, 0)
            ctx.tp = (tp_group, sp)
            ctx.save_for_backward(x2, weight, torch.empty(0))
            ctx.has_probs = False
            ctx.probs_meta = None
            ctx.clamp = clamp
            ctx.shape = h1.shape
            ctx.weight_ref = weight
            return out
        act_buf = torch.empty(T, I, dtype=h1.dtype, device=h1.device)
        p = probs.reshape(-1).float().contiguous() if probs is not None else None
        _lib.call("swiglu_fwd", x2, p, act_buf, T, I, float(clamp), ctx.kind)
        if sp:
            out = fused_tp.gemm_rs(act_buf, weight, tp_group, fused=fused_tp.ENABLED_RS)
        else:
            out = gemm.gemm(act_buf, weight)
            if tp_group is not None:
                torch.distributed.all_reduce(out, group=tp_group)
        ctx.tp = (tp_group, sp)
        ctx.save_for_backward(x2, weight, p if p is not None else torch.empty(0))
        ctx.has_probs = probs is not None
        ctx.probs_meta = (probs.shape, probs.dtype) if probs is not None else None
        ctx.clamp = clamp
        ctx.shape = h1.shape
        ctx.weight_ref = weight
        return out

    @staticmethod
    def backward(ctx, dout):
        x2, weight, p = ctx.saved_tensors
        tp_group, sp = ctx.tp
        T, I2 = x2.shape
        I = I2 // 2
        pp = p if ctx.has_probs else None
        dout2 = dout.reshape(-1, dout.shape[-1])
        if not dout2.is_contiguous():
            dout2 = dout2.contiguous()
        if ctx.fp8_fused:
            from . import fp8

            N = weight.shape[0]
            dyq_row = gemm._quantized(dout2, "row")           # quantises both directions once (backward pass)
            dyq_col = gemm._quantized(dout2, "col")
            w_ref = ctx.weight_ref
            dw = None
            if ctx.needs_input_grad[1]:
                aq = fp8.swiglu_quantize_mxfp8(x2, ctx.clamp, False, True)    # recomputed activation, col-wise
                mg = getattr(w_ref, "main_grad", None)
                tgt = mg if mg is not None else torch.empty(N, I, dtype=torch.float32, device=x2.device)
                fp8.launch_gemm(dyq_col[0], dyq_col[1], aq.q_col, aq.sf_col, tgt, N, I, T, True, True,
                                2 if mg is not None else 1)
                if mg is None:
                    dw = tgt.to(weight.dtype)
                else:
                    w_ref.grad_added_to_main_grad = True
                    cb = getattr(w_ref, "_grad_ready_cb", None)
                    if cb is not None:
                        cb(w_ref)
            wq, wsf = gemm._quantized(weight, "col")
            dact = torch.empty(T, I, dtype=torch.bfloat16, device=x2.device)
            fp8.launch_gemm(dyq_row[0], dyq_row[1], wq, wsf, dact, T, I, N, False, True, 0)
            if ctx.grad_via_cache and gemm.WGRAD_STORE.current is None:   # (a deferred dW GEMM would outlive the cache entry)
                # the gradient of h1 leaves as MXFP8 only: the bf16 tensor handed to autograd is a placeholder whose
                # quantised copy is registered for the two GEMMs of the producing linear layer
                din = torch.empty_like(x2)
                gemm.register_quantized(din, fp8.swiglu_bwd_quantize_mxfp8(x2, dact, ctx.clamp))
            else:
                din = torch.empty_like(x2)
                _lib.call("swiglu_bwd", dact, x2, None, din, None, T, I, float(ctx.clamp), 0)
            return din.view(ctx.shape), dw, None, None, None, None, None
        act = torch.empty(T, I, dtype=x2.dtype, device=x2.device)
        _lib.call("swiglu_fwd", x2, pp, act, T, I, float(ctx.clamp), ctx.kind)
        if sp:
            dact, dout2 = fused_tp.ag_gemm(dout2, weight, tp_group, b_mn=True, fused=fused_tp.ENABLED, gather_col=True)
            dw = gemm.wgrad(dout2, act, ctx.weight_ref)
        else:
            dw = gemm.wgrad(dout2, act, ctx.weight_ref)
            dact = gemm.gemm(dout2, weight, b_mn=True, out=act)  # reuse the activation buffer
        din = torch.empty_like(x2)
        dprobs = torch.empty(T, dtype=torch.float32, device=x2.device) if ctx.has_probs else None
        _lib.call("swiglu_bwd", dact, x2, pp, din, dprobs, T, I, float(ctx.clamp), ctx.kind)
        dp = None
        if ctx.has_probs:
            shape, dt = ctx.probs_meta
            dp = dprobs.view(shape).to(dt)
        return din.view(ctx.shape), dw, dp, None, None, None, None


def swiglu_linear(h1, weight, probs=None, clamp=0.0, tp_group=None, sequence_parallel=False, act="silu"):
    """linear(swiglu(h1) * probs) with the activation recomputed in backward.  ``weight`` may be a
    row-parallel shard: the partial outputs are reduce-scattered over tokens (sequence parallel) or
    all-reduced over ``tp_group``."""
    sp = bool(sequence_parallel and tp_group is not None)
    if h1.is_cuda and fused.GATE_KINDS[act] == 2:      # no fused kernel for this gate: composed activation, then the GEMM
        return row_parallel_linear(fused.swiglu_ref(h1, probs, clamp, act), weight, tp_group, sp)
    if not h1.is_cuda:
        out = gemm.linear(fused.swiglu_ref(h1, probs, clamp, act), weight)
        if sp:
            return tp_comm.reduce_scatter_seq(out, tp_group)
        return tp_comm.all_reduce(out, tp_group) if tp_group is not None else out
    return SwiGLULinearFn.apply(h1, weight, probs, clamp, tp_group, sp, act)


class RowParallelLinearFn(torch.autograd.Function):
    """reduce_scatter(x @ W^T) over tokens with a row-parallel weight shard (attention output projection)."""

    @staticmethod
    def forward(ctx, x, weight, tp_group):
        out = fused_tp.gemm_rs(x, weight, tp_group, fused=fused_tp.ENABLED_RS)
        ctx.save_for_backward(x, weight)
        ctx.group = tp_group
        ctx.weight_ref = weight
        return out

    @staticmethod
    def backward(ctx, dout):
        x, weight = ctx.saved_tensors
        dout = dout.contiguous()
        dx, dout_full = fused_tp.ag_gemm(dout, weight, ctx.group, b_mn=True, fused=fused_tp.ENABLED, gather_col=True)
        dw = gemm.wgrad(dout_full, x, ctx.weight_ref)
        return dx, dw, None


def row_parallel_linear(x, weight, tp_group=None, sequence_parallel=False):
    if tp_group is None:
        return gemm.linear(x, weight)
    if sequence_parallel and x.is_cuda:
        return RowParallelLinearFn.apply(x, weight, tp_group)
    out = gemm.linear(x, weight)
    return tp_comm.reduce_scatter_seq(out, tp_group) if sequence_parallel else tp_comm.all_reduce(out, tp_group)


# ----------------------------------------------------------------------------------------------
class RopeAttentionFn(torch.autograd.Function):
    """qkv: packed projection output [T, (Hq + 2 Hkv) * D] laid out [q heads | k heads | v heads].
    RoPE is applied in place to the q and k slices (the projection output has no other consumer)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, pos, batch, hq, hkv, d, rot_dim, causal, scale, window=0, sinks=None,
                segments=None, softcap=0.0):
        T = qkv.shape[0]
        q = qkv[:, : hq * d].view(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        if cos is not None:
            # q and k heads are adjacent in the packed layout: one launch covers both
            qk = qkv[:, : (hq + hkv) * d].view(T, hq + hkv, d)
            fused.rope_inplace_(qk, cos, sin, pos, rot_dim)
        if segments:
            # packed sequences: one attention problem per document (row ranges of the flattened token dimension)
            o = torch.empty(T, hq, d, dtype=qkv.dtype, device=qkv.device)
            lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
            for a, b in segments:
                ob, lb = attention.flash_attn_fwd(q[a:b], k[a:b], v[a:b], 1, causal, scale, 0, window, sinks, softcap)
                o[a:b] = ob
                lse[:, a:b] = lb[0]
        else:
            o, lse = attention.flash_attn_fwd(q, k, v, batch, causal, scale, 0, window, sinks, softcap)
        ctx.save_for_backward(qkv, o, lse, cos if cos is not None else torch.empty(0),
                              sin if sin is not None else torch.empty(0), pos if pos is not None else torch.empty(0),
                              sinks if sinks is not None else torch.empty(0))
        ctx.meta = (batch, hq, hkv, d, rot_dim, causal, scale, cos is not None, pos is not None, window,
                    sinks is not None, segments, softcap)
        return o.view(T, hq * d)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin, pos, sinks = ctx.saved_tensors
        batch, hq, hkv, d, rot_dim, causal, scale, has_rope, has_pos, window, has_sinks, segments, softcap = ctx.meta
        T = qkv.shape[0]
        q = qkv[:, : hq * d].view(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, : hq * d].view(T, hq, d)
        dk = dqkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        dv = dqkv[:, (hq + hkv) * d:].view(T, hkv, d)
        do3 = do.reshape(T, hq, d)
        if segments:
            ds = torch.zeros_like(sinks) if has_sinks else None
            for a, b in segments:
                lb = lse[:, a:b].unsqueeze(0).contiguous()
                attention.flash_attn_bwd(do3[a:b], q[a:b], k[a:b], v[a:b], o[a:b], lb, 1, causal, scale, dq=dq[a:b],
                                         dk=dk[a:b], dv=dv[a:b], window=window, softcap=softcap)
                if has_sinks:
                    ds += attention.sink_grad(do3[a:b], o[a:b], lb, sinks, 1)
        else:
            attention.flash_attn_bwd(do3, q, k, v, o, lse, batch, causal, scale, dq=dq, dk=dk, dv=dv, window=window,
                                     softcap=softcap)
            ds = attention.sink_grad(do3, o, lse, sinks, batch) if has_sinks else None
        if has_rope:
            dqk = dqkv[:, : (hq + hkv) * d].view(T, hq + hkv, d)
            fused.rope_inplace_(dqk, cos, sin, pos if has_pos else None, rot_dim, backward=True)
        return dqkv, None, None, None, None, None, None, None, None, None, None, None, ds, None, None


def rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, rot_dim=None, causal=True, scale=None, window=0, sinks=None,
                   segments=None, softcap=0.0):
    """Self-attention on a packed QKV tensor; returns [T, Hq*D].  ``window`` > 0: sliding-window attention; ``sinks``
    (fp32 [Hq]): learned per-head sink logits; ``segments``: [(start, end)] row ranges of the documents packed into
    the token dimension (attention stays inside each; on CUDA every range must be a multiple of 128 rows)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    rot_dim = rot_dim or d
    composed = qkv.is_cuda and not attention.kernel_supports(d, d)
    if composed:
        attention.warn_composed(d, d)
    if not qkv.is_cuda or composed:
        T = qkv.shape[0]
        q = qkv[:, : hq * d].reshape(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].reshape(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(T, hkv, d)
        if cos is not None:
            q = fused.rope_ref(q, cos, sin, pos, rot_dim)
            k = fused.rope_ref(k, cos, sin, pos, rot_dim)
        if segments:
            o = torch.cat([attention.attention_ref(q[a:b], k[a:b], v[a:b], 1, causal, scale, 0, window, sinks, softcap)[0]
                           for a, b in segments], 0)
        else:
            o = attention.attention_ref(q, k, v, batch, causal, scale, 0, window, sinks, softcap)[0]
        return o.reshape(T, hq * d)
    return RopeAttentionFn.apply(qkv, cos, sin, pos, batch, hq, hkv, d, rot_dim, causal, scale, window, sinks, segments,
                                 softcap or 0.0)


# ----------------------------------------------------------------------------------------------
# Chunked linear + cross entropy: the [T, V] logits are never materialised
class ChunkedLinearCEFn(torch.autograd.Function):
    """``sum_t weights[t] * CE(y[t] W^T, labels[t])`` computed ``chunk`` tokens at a time.

    The cross-entropy kernel leaves the (already weighted) gradient in place of a chunk's logits, so the same
    pass also produces ``dy`` for the chunk and accumulates ``dW``; only ``dy`` ([T, h]) is kept for backward.
    This relies on the caller back-propagating a gradient of exactly 1 into the returned scalar (the trainer's
    ``unit_upstream`` promise).  Same idea as the reference's fused linear cross entropy
    (primus/backends/megatron/patches/fused_linear_ce_patches.py:48-100,171: chunks of 4096 tokens)."""

    @staticmethod
    def forward(ctx, y, w, labels, weights, vocab_start, chunk):
        T = y.shape[0]
        lab = labels.reshape(-1)
        wts = weights.reshape(-1)
        total = torch.zeros((), dtype=torch.float32, device=y.device)
        dy = torch.empty_like(y)
        dw_local = None
        has_main = getattr(w, "main_grad", None) is not None
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            yc = y[s:e]
            logits = gemm.gemm(yc, w)
            total += fused.cross_entropy(logits, lab[s:e], vocab_start, None, wts[s:e], True)
            if y.is_cuda:
                dlogits = logits                       # overwritten with the weighted gradient
            else:
                p = torch.softmax(logits.float(), -1)
                p[torch.arange(e - s), lab[s:e]] -= 1.0
                dlogits = (p * wts[s:e, None].float()).to(y.dtype)
            dy[s:e] = gemm.gemm(dlogits, w, b_mn=True)
            if has_main:
                gemm.wgrad(dlogits, yc, w)
            else:
                g = gemm.gemm(dlogits, yc, a_mn=True, b_mn=True, out_dtype=torch.float32)
                dw_local = g if dw_local is None else dw_local + g
        ctx.save_for_backward(dy)
        ctx.dw_local = dw_local
        ctx.w_dtype = w.dtype
        return total

    @staticmethod
    def backward(ctx, g):
        (dy,) = ctx.saved_tensors
        dw = ctx.dw_local.to(ctx.w_dtype) if ctx.dw_local is not None else None
        return dy, dw, None, None, None, None   # upstream gradient is 1 by contract


def chunked_linear_cross_entropy(y, w, labels, weights, vocab_start=0, chunk=4096):
    return ChunkedLinearCEFn.apply(y, w, labels, weights, vocab_start, chunk)


# ----------------------------------------------------------------------------------------------
# Context parallelism (Ulysses): sequence-sharded activations, head-sharded attention
class _SeqHeadAllToAll(torch.autograd.Function):
    """Equal-split all-to-all over the context-parallel group; the backward pass is the same exchange."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        g = g.contiguous()   # (empty_like of a permuted gradient would inherit its strides)
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def ulysses_rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, cp_group, cp, rot_dim=None, causal=True, scale=None):
    """Self-attention when every rank of the context-parallel group holds ``seq / cp`` tokens of each sequence.

    RoPE is applied to the local tokens with their global positions, one all-to-all turns the sequence
    sharding into a head sharding ([T/cp, all heads] -> [T, heads/cp]), attention runs over the full
    sequence on ``hq/cp`` query and ``hkv/cp`` key/value heads, and the inverse all-to-all restores the
    sequence sharding.  Same scheme as the reference's Ulysses attention
    (primus/backends/megatron/core/extensions/primus_turbo.py: PrimusTurboAttention with cp_comm_type "a2a").
    Returns [T/cp, hq * d]."""
    assert hq % cp == 0 and hkv % cp == 0, "context parallelism (all-to-all) needs heads divisible by cp"
    Tl = qkv.shape[0]
    Sl = Tl // batch
    hq_l, hkv_l = hq // cp, hkv // cp
    q = qkv[:, : hq * d].reshape(Tl, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(Tl, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(Tl, hkv, d)
    if cos is not None:
        q = fused.rope(q, cos, sin, pos, rot_dim or d)
        k = fused.rope(k, cos, sin, pos, rot_dim or d)
    # [cp (destination), Tl, (hq_l + 2 hkv_l) * d]
    send = torch.cat([q.reshape(Tl, cp, hq_l * d), k.reshape(Tl, cp, hkv_l * d), v.reshape(Tl, cp, hkv_l * d)], dim=2)
    send = send.permute(1, 0, 2).contiguous()
    recv = _SeqHeadAllToAll.apply(send, cp_group)                     # [cp (source), batch * Sl, chunk]
    chunk = recv.shape[2]
    full = recv.view(cp, batch, Sl, chunk).permute(1, 0, 2, 3).reshape(batch * cp * Sl, chunk)
    out = rope_attention(full.contiguous(), None, None, None, batch, hq_l, hkv_l, d, rot_dim=rot_dim, causal=causal,
                         scale=scale)                                  # [batch * S, hq_l * d]
    back = out.view(batch, cp, Sl, hq_l * d).permute(1, 0, 2, 3).reshape(cp, Tl, hq_l * d).contiguous()
    got = _SeqHeadAllToAll.apply(back, cp_group)                      # [cp (head group), Tl, hq_l * d]
    return got.permute(1, 0, 2).reshape(Tl, hq * d)


# ----------------------------------------------------------------------------------------------
# Context parallelism (all-gather): zig-zag sequence sharding, K / V gathered, chunk-vs-prefix attention
def zigzag_chunk_ids(cp: int, rank: int) -> tuple[int, int]:
    """The two sequence chunks (of ``2 * cp``) a context-parallel rank holds: ``rank`` and ``2 cp - 1 - rank``, which
    gives every rank the same amount of causal-attention work."""
    return rank, 2 * cp - 1 - rank


def _zigzag_to_natural_index(cp: int, batch: int, c: int, device) -> torch.Tensor:
    """Row permutation that turns the all-gathered tensor ``[cp (owner), batch, 2 (slot), c]`` into natural order
    ``[batch, 2 cp (chunk), c]``."""
    owner = torch.tensor([j if j < cp else 2 * cp - 1 - j for j in range(2 * cp)], device=device)
    slot = torch.tensor([0 if j < cp else 1 for j in range(2 * cp)], device=device)
    b = torch.arange(batch, device=device).view(batch, 1, 1)
    t = torch.arange(c, device=device).view(1, 1, c)
    src = ((owner.view(1, -1, 1) * batch + b) * 2 + slot.view(1, -1, 1)) * c + t     # [batch, 2cp, c]
    return src.reshape(-1)


class AllGatherCPAttentionFn(torch.autograd.Function):
    """Causal self-attention under all-gather context parallelism (the reference's ``cp_comm_type: allgather``, which
    it takes from Transformer-Engine; primus/configs/models/megatron/language_model.yaml:151-153).

    Every rank holds two zig-zag chunks of each sequence.  K and V (after RoPE) are all-gathered once, put back into
    natural order, and each local query chunk at key position ``q_off`` attends to the key prefix ``[0, q_off + c)``
    with the offset form of the flash-attention kernels; the backward reduce-scatters dK / dV to their owners.  No
    constraint on the number of heads (works for MLA head shapes and for fewer KV heads than ranks)."""

    @staticmethod
    def forward(ctx, q, k, v, batch, group, cp, rank, causal, scale):
        Tl, hq, dqk = q.shape
        hkv, dv = k.shape[1], v.shape[2]
        c = Tl // batch // 2
        S = 2 * cp * c
        W = hkv * (dqk + dv)
        kv = torch.cat([k.reshape(Tl, hkv * dqk), v.reshape(Tl, hkv * dv)], dim=1).contiguous()
        gathered = torch.empty(cp * Tl, W, dtype=kv.dtype, device=kv.device)
        torch.distributed.all_gather_into_tensor(gathered, kv, group=group)
        idx = _zigzag_to_natural_index(cp, batch, c, kv.device)
        full = gathered.index_select(0, idx)                                     # [batch * S, W], natural order
        kf = full[:, : hkv * dqk].unflatten(1, (hkv, dqk))
        vf = full[:, hkv * dqk:].unflatten(1, (hkv, dv))
        o = torch.empty(Tl, hq, dv, dtype=q.dtype, device=q.device)
        lses = []
        chunks = zigzag_chunk_ids(cp, rank)
        for b in range(batch):
            for slot, j in enumerate(chunks):
                r0 = (b * 2 + slot) * c
                q_off = j * c
                kp, vp = kf[b * S: b * S + q_off + c], vf[b * S: b * S + q_off + c]
                if q.is_cuda:
                    ob, lse = attention.flash_attn_fwd(q[r0:r0 + c], kp, vp, 1, causal, scale, q_off if causal else 0)
                else:
                    ob, lse = attention.attention_ref(q[r0:r0 + c], kp, vp, 1, causal, scale, q_off if causal else 0)
                o[r0:r0 + c] = ob
                lses.append(lse)
        ctx.save_for_backward(q, full, o, idx, *lses)
        ctx.meta = (batch, group, cp, rank, causal, scale, hkv, dqk, dv, c)
        return o

    @staticmethod
    def backward(ctx, do):
        q, full, o, idx, *lses = ctx.saved_tensors
        batch, group, cp, rank, causal, scale, hkv, dqk, dv, c = ctx.meta
        Tl, hq, _ = q.shape
        S = 2 * cp * c
        W = hkv * (dqk + dv)
        kf = full[:, : hkv * dqk].unflatten(1, (hkv, dqk))
        vf = full[:, hkv * dqk:].unflatten(1, (hkv, dv))
        do = do.contiguous()
        dq = torch.empty_like(q)
        dfull = torch.zeros(batch * S, W, dtype=torch.float32, device=q.device)
        chunks = zigzag_chunk_ids(cp, rank)
        n = 0
        for b in range(batch):
            for slot, j in enumerate(chunks):
                r0 = (b * 2 + slot) * c
                q_off = j * c
                L = q_off + c
                kp, vp = kf[b * S: b * S + L], vf[b * S: b * S + L]
                if q.is_cuda:
                    dqb, dkb, dvb = attention.flash_attn_bwd(do[r0:r0 + c], q[r0:r0 + c], kp, vp, o[r0:r0 + c], lses[n],
                                                             1, causal, scale, q_off=q_off if causal else 0)
                else:
                    with torch.enable_grad():
                        qr, kr, vr = (t.detach().float().requires_grad_() for t in (q[r0:r0 + c], kp, vp))
                        orf, _ = attention.attention_ref(qr, kr, vr, 1, causal, scale, q_off if causal else 0)
                        orf.backward(do[r0:r0 + c].float())
                    dqb, dkb, dvb = qr.grad.to(q.dtype), kr.grad, vr.grad
                dq[r0:r0 + c] = dqb
                dfull[b * S: b * S + L, : hkv * dqk] += dkb.reshape(L, hkv * dqk).float()
                dfull[b * S: b * S + L, hkv * dqk:] += dvb.reshape(L, hkv * dv).float()
                n += 1
        # natural order -> owner order, then every owner receives the sum of the cp contributions
        dgath = torch.empty(cp * Tl, W, dtype=torch.float32, device=q.device)
        dgath.index_copy_(0, idx, dfull)
        from ..parallel import tensor_parallel as tp_comm_mod

        dkv = tp_comm_mod.reduce_scatter_dim0(dgath.to(q.dtype), group)           # [Tl, W]
        dk = dkv[:, : hkv * dqk].reshape(Tl, hkv, dqk)
        dv_ = dkv[:, hkv * dqk:].reshape(Tl, hkv, dv)
        return dq, dk, dv_, None, None, None, None, None, None


def allgather_cp_attention(q, k, v, batch, cp_group, cp, causal=True, scale=None):
    """q [Tl, hq, dqk], k [Tl, hkv, dqk], v [Tl, hkv, dv] of this rank's two zig-zag chunks per sequence (RoPE already
    applied with global positions) -> attention output [Tl, hq, dv]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    rank = torch.distributed.get_rank(cp_group)
    return AllGatherCPAttentionFn.apply(q, k, v, batch, cp_group, cp, rank, causal, scale)


def allgather_cp_rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, cp_group, cp, rot_dim=None, causal=True,
                                scale=None):
    """Packed-QKV form of :func:`allgather_cp_attention` (RoPE with the global positions of the local tokens)."""
    Tl = qkv.shape[0]
    q = qkv[:, : hq * d].reshape(Tl, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(Tl, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(Tl, hkv, d)
    if cos is not None:
        rope_fn = fused.rope if qkv.is_cuda else fused.rope_ref
        q = rope_fn(q, cos, sin, pos, rot_dim or d)
        k = rope_fn(k, cos, sin, pos, rot_dim or d)
    out = allgather_cp_attention(q.contiguous(), k.contiguous(), v.contiguous(), batch, cp_group, cp, causal, scale)
    return out.reshape(Tl, hq * d)


# ----------------------------------------------------------------------------------------------
# Context parallelism (ring / p2p): K / V blocks travel around the ring, partial results are merged by log-sum-exp
def _block_fwd(q, k, v, causal, scale):
    """(o, lse [Hq, c]) of one query chunk against one key chunk (same length), fp32 merge inputs."""
    if q.is_cuda:
        o, lse = attention.flash_attn_fwd(q, k, v, 1, causal, scale)
    else:
        o, lse = attention.attention_ref(q, k, v, 1, causal, scale)
    return o.float(), lse[0].float()


def _block_bwd(do, q, k, v, o, lse, causal, scale):
    """Gradients of one (query chunk, key chunk) block given the *final* output and log-sum-exp of the query rows
    (p = exp(s - lse) is then the block's share of the full softmax)."""
    if q.is_cuda:
        return attention.flash_attn_bwd(do, q, k, v, o, lse.unsqueeze(0).contiguous(), 1, causal, scale)
    c, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    qf, dof, of = q.float().permute(1, 0, 2), do.float().permute(1, 0, 2), o.float().permute(1, 0, 2)   # [Hq, c, d]
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, 0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, 0)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(c, k.shape[0], dtype=torch.bool, device=q.device).tril(), float("-inf"))
    p = torch.exp(s - lse.float().unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(hkv, g, -1, d).sum(1)
    dv = dv.view(hkv, g, -1, v.shape[2]).sum(1)
    return dq.permute(1, 0, 2).to(q.dtype), dk.permute(1, 0, 2).to(k.dtype), dv.permute(1, 0, 2).to(v.dtype)


def _ring_exchange(send: torch.Tensor, group, cp: int, rank: int):
    """Starts sending ``send`` to the next rank of the ring and receiving the previous rank's buffer; returns
    (recv tensor, requests)."""
    ranks = torch.distributed.get_process_group_ranks(group)
    nxt, prv = ranks[(rank + 1) % cp], ranks[(rank - 1) % cp]
    recv = torch.empty_like(send)
    ops = [torch.distributed.P2POp(torch.distributed.isend, send, nxt, group),
           torch.distributed.P2POp(torch.distributed.irecv, recv, prv, group)]
    return recv, torch.distributed.batch_isend_irecv(ops)


class RingCPAttentionFn(torch.autograd.Function):
    """Causal self-attention under ring context parallelism (``cp_comm_type: p2p``, the reference's default, which it
    takes from Transformer-Engine; primus/configs/models/megatron/language_model.yaml:151-153).

    Zig-zag layout as in the all-gather scheme (chunks ``rank`` and ``2 cp - 1 - rank`` per sequence).  The packed
    K / V buffer of every rank travels once around the ring; at each of the ``cp`` steps a rank attends its two query
    chunks to the two key chunks it currently holds (a full block when the key chunk is earlier, the causal diagonal
    when it is the same chunk, nothing when it is later) while the next buffer is already in flight, and merges the
    partial outputs through their log-sum-exp.  The backward sends the K / V buffer around again together with its
    gradient buffer, which returns to its owner after the last step."""

    @staticmethod
    def forward(ctx, q, k, v, batch, group, cp, rank, scale):
        Tl, hq, dqk = q.shape
        hkv, dv = k.shape[1], v.shape[2]
        c = Tl // batch // 2
        mine = zigzag_chunk_ids(cp, rank)
        kv = torch.cat([k.reshape(Tl, hkv * dqk), v.reshape(Tl, hkv * dv)], dim=1).contiguous()
        o = torch.zeros(Tl, hq, dv, dtype=torch.float32, device=q.device)
        lse = torch.full((hq, Tl), float("-inf"), dtype=torch.float32, device=q.device)
        cur = kv
        for s in range(cp):
            nxt, reqs = (None, [])
            if s + 1 < cp:
                nxt, reqs = _ring_exchange(cur, group, cp, rank)
            theirs = zigzag_chunk_ids(cp, (rank - s) % cp)
            kc = cur[:, : hkv * dqk].unflatten(1, (hkv, dqk))
            vc = cur[:, hkv * dqk:].unflatten(1, (hkv, dv))
            for b in range(batch):
                for qs, qi in enumerate(mine):
                    for ks, kj in enumerate(theirs):
                        if kj > qi:
                            continue
                        r0, k0 = (b * 2 + qs) * c, (b * 2 + ks) * c
                        ob, lb = _block_fwd(q[r0:r0 + c], kc[k0:k0 + c], vc[k0:k0 + c], kj == qi, scale)
                        old = lse[:, r0:r0 + c]
                        new = torch.logaddexp(old, lb)
                        w_old = torch.exp(old - new).t().unsqueeze(-1)           # [c, Hq, 1]
                        w_new = torch.exp(lb - new).t().unsqueeze(-1)
                        o[r0:r0 + c] = o[r0:r0 + c] * w_old + ob * w_new
                        lse[:, r0:r0 + c] = new
            for r in reqs:
                r.wait()
            cur = nxt if nxt is not None else cur
        out = o.to(q.dtype)
        ctx.save_for_backward(q, kv, out, lse)
        ctx.meta = (batch, group, cp, rank, scale, hkv, dqk, dv, c)
        return out

    @staticmethod
    def backward(ctx, do):
        q, kv, o, lse = ctx.saved_tensors
        batch, group, cp, rank, scale, hkv, dqk, dv, c = ctx.meta
        Tl = q.shape[0]
        mine = zigzag_chunk_ids(cp, rank)
        do = do.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        # the travelling buffer: [K | V | dK | dV] (gradients in fp32 precision would double the traffic; they are
        # accumulated in fp32 locally and travel in the compute dtype, as the activations do)
        W = hkv * (dqk + dv)
        cur_kv = kv
        cur_d = torch.zeros(Tl, W, dtype=torch.float32, device=q.device)
        for s in range(cp):
            theirs = zigzag_chunk_ids(cp, (rank - s) % cp)
            kc = cur_kv[:, : hkv * dqk].unflatten(1, (hkv, dqk))
            vc = cur_kv[:, hkv * dqk:].unflatten(1, (hkv, dv))
            nxt_kv, reqs = (None, [])
            if s + 1 < cp:
                nxt_kv, reqs = _ring_exchange(cur_kv, group, cp, rank)
            for b in range(batch):
                for qs, qi in enumerate(mine):
                    for ks, kj in enumerate(theirs):
                        if kj > qi:
                            continue
                        r0, k0 = (b * 2 + qs) * c, (b * 2 + ks) * c
                        dqb, dkb, dvb = _block_bwd(do[r0:r0 + c], q[r0:r0 + c], kc[k0:k0 + c], vc[k0:k0 + c],
                                                   o[r0:r0 + c], lse[:, r0:r0 + c], kj == qi, scale)
                        dq[r0:r0 + c] += dqb.float()
                        cur_d[k0:k0 + c, : hkv * dqk] += dkb.reshape(c, hkv * dqk).float()
                        cur_d[k0:k0 + c, hkv * dqk:] += dvb.reshape(c, hkv * dv).float()
            for r in reqs:
                r.wait()
            # the gradient buffer follows the K / V buffer: after this step it goes to the next rank, which holds
            # the same K / V block next; after the last step it goes one more hop and is home
            send_d = cur_d
            cur_d, dreqs = _ring_exchange(send_d, group, cp, rank)
            for r in dreqs:
                r.wait()
            cur_kv = nxt_kv if nxt_kv is not None else cur_kv
        dkv = cur_d
        dk = dkv[:, : hkv * dqk].reshape(Tl, hkv, dqk).to(q.dtype)
        dv_ = dkv[:, hkv * dqk:].reshape(Tl, hkv, dv).to(q.dtype)
        return dq.to(q.dtype), dk, dv_, None, None, None, None, None


def ring_cp_attention(q, k, v, batch, cp_group, cp, scale=None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    rank = torch.distributed.get_rank(cp_group)
    return RingCPAttentionFn.apply(q, k, v, batch, cp_group, cp, rank, scale)


def ring_cp_rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, cp_group, cp, rot_dim=None, scale=None):
    """Packed-QKV form of :func:`ring_cp_attention` (RoPE with the global positions of the local tokens)."""
    Tl = qkv.shape[0]
    q = qkv[:, : hq * d].reshape(Tl, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(Tl, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(Tl, hkv, d)
    if cos is not None:
        rope_fn = fused.rope if qkv.is_cuda else fused.rope_ref
        q = rope_fn(q, cos, sin, pos, rot_dim or d)
        k = rope_fn(k, cos, sin, pos, rot_dim or d)
    out = ring_cp_attention(q.contiguous(), k.contiguous(), v.contiguous(), batch, cp_group, cp, scale)
    return out.reshape(Tl, hq * d)


# ----------------------------------------------------------------------------------------------
# Context parallelism (hierarchical): all-to-all inside a group of neighbouring ranks, ring across the groups
def hierarchical_cp_rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, a2a_group, a2a, p2p_group, p2p, rot_dim=None,
                                   scale=None):
    """Causal self-attention under two-level context parallelism (the reference's ``cp_comm_type: a2a+p2p`` with
    ``hierarchical_context_parallel_sizes: [a2a, p2p]``; primus/configs/models/megatron/language_model.yaml).

    A sequence is cut into ``2 * p2p`` super-chunks; ring position ``i`` owns super-chunks ``i`` and ``2 p2p - 1 - i``
    (zig-zag, balanced causal work) and the ``a2a`` ranks of that position each hold a consecutive ``1 / a2a`` of both.
    One all-to-all inside the group turns that split into a head split (every rank: both whole super-chunks,
    ``heads / a2a`` heads), ring attention runs across the groups on those heads, and the inverse all-to-all restores
    the token split.  Only ``heads / a2a`` must be whole, so the ring carries the scaling beyond the head count and
    the all-to-all keeps its traffic on the nearest links.  Returns [T_local, hq * d]."""
    if a2a == 1:
        return ring_cp_rope_attention(qkv, cos, sin, pos, batch, hq, hkv, d, p2p_group, p2p, rot_dim, scale)
    assert hq % a2a == 0 and hkv % a2a == 0, "a2a+p2p context parallelism needs heads divisible by the all-to-all size"
    Tl = qkv.shape[0]
    part = Tl // batch // 2                       # tokens of one super-chunk held by this rank
    hq_l, hkv_l = hq // a2a, hkv // a2a
    q = qkv[:, : hq * d].reshape(Tl, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(Tl, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(Tl, hkv, d)
    if cos is not None:
        rope_fn = fused.rope if qkv.is_cuda else fused.rope_ref
        q = rope_fn(q, cos, sin, pos, rot_dim or d)
        k = rope_fn(k, cos, sin, pos, rot_dim or d)
    send = torch.cat([q.reshape(Tl, a2a, hq_l * d), k.reshape(Tl, a2a, hkv_l * d), v.reshape(Tl, a2a, hkv_l * d)], dim=2)
    send = send.permute(1, 0, 2).contiguous()                          # [a2a (destination), Tl, chunk]
    recv = _SeqHeadAllToAll.apply(send, a2a_group)                     # [a2a (source part), batch * 2 * part, chunk]
    chunk = recv.shape[2]
    # [part owner, batch, super-chunk slot, part] -> [batch, slot, part owner, part]: both super-chunks whole, in order
    full = recv.view(a2a, batch, 2, part, chunk).permute(1, 2, 0, 3, 4).reshape(batch * 2 * a2a * part, chunk)
    T2 = full.shape[0]
    ql = full[:, : hq_l * d].reshape(T2, hq_l, d).contiguous()
    kl = full[:, hq_l * d: (hq_l + hkv_l) * d].reshape(T2, hkv_l, d).contiguous()
    vl = full[:, (hq_l + hkv_l) * d:].reshape(T2, hkv_l, d).contiguous()
    if p2p > 1:
        out = ring_cp_attention(ql, kl, vl, batch, p2p_group, p2p, scale)
    else:  # a single ring position holds the whole sequence: plain causal attention
        out = rope_attention(full.contiguous(), None, None, None, batch, hq_l, hkv_l, d, rot_dim=rot_dim, causal=True,
                             scale=scale)
    out = out.reshape(batch, 2, a2a, part, hq_l * d).permute(2, 0, 1, 3, 4).reshape(a2a, Tl, hq_l * d).contiguous()
    got = _SeqHeadAllToAll.apply(out, a2a_group)                       # [a2a (head group), Tl, hq_l * d]
    return got.permute(1, 0, 2).reshape(Tl, hq * d)


# ----------------------------------------------------------------------------------------------
# Sequence splits inside a pipeline: a micro-batch travels through the stages as ``num_splits`` consecutive chunks of
# its sequence.  Chunk j's queries attend to the keys of chunks 0..j, so every attention layer keeps the K / V of the
# chunks it has already seen for that micro-batch, and the gradient a later chunk produces for an earlier chunk's K / V
# waits in an accumulator until that chunk's own backward pass runs (the schedule runs the backward passes of a
# micro-batch's chunks in reverse order).  The reference schedules such chunks (``num_seq_splits``,
# primus/backends/megatron/core/pipeline_parallel/zerobubble/scheduler/seq1f1b.py:15-45) and slices the batch
# (primus/backends/megatron/data_loader_store.py:45-70); the attention over the kept prefix is this engine's own.
class SeqSplitState:
    """What the pipeline runtime tells the attention layers about the chunk being processed."""

    def __init__(self):
        self.active = False
        self.key = None           # (micro-batch, model chunk): one K / V cache per key and attention layer
        self.split = 0
        self.num_splits = 1
        self.forward_only = False
        self.cache: dict = {}     # (layer id, key) -> {"k": [batch, L, hkv, d], "v": ..., "dk": fp32 accumulator, "dv": ...}

    def begin(self, key, split: int, num_splits: int, forward_only: bool = False):
        self.active, self.key, self.split, self.num_splits, self.forward_only = True, key, split, num_splits, forward_only

    def end(self):
        self.active = False

    def drop(self, key):
        for k in [k for k in self.cache if k[1] == key]:
            del self.cache[k]

    def clear(self):
        self.cache.clear()
        self.active = False


SEQ_SPLIT = SeqSplitState()


class SeqSplitAttentionFn(torch.autograd.Function):
    """Causal attention of one sequence chunk against the kept K / V prefix of its micro-batch (RoPE already applied
    with the chunk's global positions).  q [batch * c, hq, d], k / v [batch * c, hkv, d]."""

    @staticmethod
    def forward(ctx, q, k, v, batch, scale, slot, split, num_splits, forward_only):
        T, hq, d = q.shape
        hkv, dv = k.shape[1], v.shape[2]
        c = T // batch
        q_off = split * c
        kc, vc = k.reshape(batch, c, hkv, d), v.reshape(batch, c, hkv, dv)
        if split == 0:
            kf, vf = kc.contiguous(), vc.contiguous()
        else:
            kf = torch.cat([slot["k"], kc], dim=1)
            vf = torch.cat([slot["v"], vc], dim=1)
        assert kf.shape[1] == q_off + c, "sequence chunks of a micro-batch must reach an attention layer in order"
        if split + 1 < num_splits:
            slot["k"], slot["v"] = kf.detach(), vf.detach()
        else:
            slot.pop("k", None), slot.pop("v", None)
        o = torch.empty(T, hq, dv, dtype=q.dtype, device=q.device)
        lses = []
        for b in range(batch):
            qb = q[b * c:(b + 1) * c]
            if q.is_cuda:
                ob, lse = attention.flash_attn_fwd(qb, kf[b], vf[b], 1, True, scale, q_off)
            else:
                ob, lse = attention.attention_ref(qb, kf[b], vf[b], 1, True, scale, q_off)
            o[b * c:(b + 1) * c] = ob
            lses.append(lse)
        ctx.save_for_backward(q, kf, vf, o, *lses)
        ctx.meta = (batch, scale, slot, split, num_splits, c)
        return o

    @staticmethod
    def backward(ctx, do):
        q, kf, vf, o, *lses = ctx.saved_tensors
        batch, scale, slot, split, num_splits, c = ctx.meta
        hkv, d, dv = kf.shape[2], kf.shape[3], vf.shape[3]
        q_off = split * c
        L = q_off + c
        do = do.contiguous()
        dq = torch.empty_like(q)
        if "dk" not in slot:        # the last chunk's backward comes first and sizes the accumulators
            assert split == num_splits - 1, "the backward passes of a micro-batch's chunks must run in reverse order"
            slot["dk"] = torch.zeros(batch, L, hkv, d, dtype=torch.float32, device=q.device)
            slot["dv"] = torch.zeros(batch, L, hkv, dv, dtype=torch.float32, device=q.device)
        for b in range(batch):
            sl = slice(b * c, (b + 1) * c)
            if q.is_cuda:
                dqb, dkb, dvb = attention.flash_attn_bwd(do[sl], q[sl], kf[b], vf[b], o[sl], lses[b], 1, True, scale,
                                                         q_off=q_off)
            else:
                with torch.enable_grad():
                    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q[sl], kf[b], vf[b]))
                    orf, _ = attention.attention_ref(qr, kr, vr, 1, True, scale, q_off)
                    orf.backward(do[sl].float())
                dqb, dkb, dvb = qr.grad.to(q.dtype), kr.grad, vr.grad
            dq[sl] = dqb
            slot["dk"][b, :L] += dkb.float()
            slot["dv"][b, :L] += dvb.float()
        dk = slot["dk"][:, q_off:L].reshape(batch * c, hkv, d).to(q.dtype)
        dv_ = slot["dv"][:, q_off:L].reshape(batch * c, hkv, dv).to(q.dtype)
        if split == 0:
            slot.pop("dk"), slot.pop("dv")
        return dq, dk, dv_, None, None, None, None, None, None


def seq_split_rope_attention(layer_id, qkv, cos, sin, pos, batch, hq, hkv, d, rot_dim=None, scale=None):
    """Packed-QKV causal attention of the chunk announced in ``SEQ_SPLIT`` (positions ``pos`` are global)."""
    st = SEQ_SPLIT
    T = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    q = qkv[:, : hq * d].reshape(T, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(T, hkv, d)
    if cos is not None:
        rope_fn = fused.rope if qkv.is_cuda else fused.rope_ref
        q = rope_fn(q, cos, sin, pos, rot_dim or d)
        k = rope_fn(k, cos, sin, pos, rot_dim or d)
    slot = st.cache.setdefault((layer_id, st.key), {})
    out = SeqSplitAttentionFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), batch, scale, slot, st.split,
                                    st.num_splits, st.forward_only)
    return out.reshape(T, hq * d)
