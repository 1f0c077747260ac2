"""Flash attention (causal / full; MHA, GQA, MQA and the MLA head shape d_qk=192, d_v=128) on the
tcgen05 kernels in ``csrc/flash_attn_{fwd,bwd}.cu``.

Tensors are token-major: q ``[B*S, Hq, Dqk]``, k ``[B*S, Hkv, Dqk]``, v ``[B*S, Hkv, Dv]`` — views into
a packed QKV projection output are accepted (only the last dim must be contiguous and the head
stride must equal the head dim).  CPU tensors run a plain fp32 softmax(QK^T)V reference, which is
also the oracle of the GPU tests.

Parity: `flash_attn_func` use in primus/backends/megatron/core/extensions/primus_turbo.py:812-823,888-990.
"""
from __future__ import annotations

import math

import torch

from . import _lib


def attention_ref(q, k, v, batch: int, causal: bool = True, scale: float | None = None, q_off: int = 0,
                  window: int = 0, sinks=None, softcap: float = 0.0):
    """fp32 reference. Returns (out [T,Hq,Dv], lse [B,Hq,S]).  ``k`` / ``v`` may hold more rows per sequence than ``q``
    (a sequence chunk attending to a gathered prefix): query row i then sits at key position ``q_off + i``.
    ``window`` > 0: a query sees its last ``window`` keys (itself included).  ``sinks`` [Hq]: a learned logit per head
    that joins the softmax denominator only (GPT-OSS style attention sink)."""
    T, hq, dqk = q.shape
    hkv, dv = k.shape[1], v.shape[2]
    S = T // batch
    SK = k.shape[0] // batch
    scale = scale if scale is not None else 1.0 / math.sqrt(dqk)
    g = hq // hkv
    qf = q.float().reshape(batch, S, hq, dqk).permute(0, 2, 1, 3)
    kf = k.float().reshape(batch, SK, hkv, dqk).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().reshape(batch, SK, hkv, dv).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:          # scores soft-capped before masking and softmax
        s = softcap * torch.tanh(s / softcap)
    if causal:
        mask = torch.ones(S, SK, dtype=torch.bool, device=q.device).tril(diagonal=q_off)
        if window and window > 0:
            mask &= torch.ones(S, SK, dtype=torch.bool, device=q.device).triu(diagonal=q_off - window + 1)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    if sinks is not None:
        lse = torch.logaddexp(lse, sinks.float().view(1, hq, 1).expand_as(lse))
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).reshape(T, hq, dv)
    return o.to(q.dtype), lse


KERNEL_HEAD_DIMS = ((128, 128), (192, 128), (64, 64))     # (d_qk, d_v) the flash-attention kernels are instantiated for
_WARNED: set = set()


def kernel_supports(d_qk: int, d_v: int) -> bool:
    return (d_qk, d_v) in KERNEL_HEAD_DIMS


def warn_composed(d_qk: int, d_v: int) -> None:
    """Head sizes without a kernel (256 in Qwen3.5) run as composed PyTorch operations that materialise the score
    matrix: correct, but neither fast nor memory-lean.  Said once per size."""
    if (d_qk, d_v) not in _WARNED:
        _WARNED.add((d_qk, d_v))
        import warnings

        warnings.warn(f"no flash-attention kernel for head sizes ({d_qk}, {d_v}): attention runs as composed PyTorch "
                      f"operations with the full score matrix (kernels exist for {KERNEL_HEAD_DIMS})", stacklevel=3)


def _check_view(t, d):
    assert t.stride(2) == 1 and t.stride(1) == d, "heads must be contiguous [.., H, D] views"
    assert t.data_ptr() % 16 == 0


def flash_attn_fwd(q, k, v, batch: int, causal: bool, scale: float, q_off: int = 0, window: int = 0, sinks=None,
                   softcap: float = 0.0):
    T, hq, dqk = q.shape
    hkv, dv = k.shape[1], v.shape[2]
    S = T // batch
    SK = k.shape[0] // batch
    for t, d in ((q, dqk), (k, dqk), (v, dv)):
        _check_view(t, d)
    o = torch.empty(T, hq, dv, dtype=q.dtype, device=q.device)
    lse = torch.empty(batch, hq, S, dtype=torch.float32, device=q.device)
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == hq and sinks.is_contiguous()
    _lib.call("flash_attn_fwd_cap", q, k, v, o, lse, batch, S, SK, int(q_off), hq, hkv, dqk, dv, q.stride(0), k.stride(0),
              v.stride(0), o.stride(0), float(scale), int(causal), int(window or 0), sinks, float(softcap or 0.0),
              _lib.status_word(q.device))
    return o, lse


def flash_attn_bwd(do, q, k, v, o, lse, batch: int, causal: bool, scale: float, dq=None, dk=None, dv=None,
                   q_off: int = 0, window: int = 0, softcap: float = 0.0):
    """Returns (dq, dk, dv); optional pre-allocated outputs may be strided views (packed dQKV)."""
    T, hq, dqk = q.shape
    hkv, dvd = k.shape[1], v.shape[2]
    S = T // batch
    TK = k.shape[0]
    SK = TK // batch
    dq = torch.empty(T, hq, dqk, dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty(TK, hkv, dqk, dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty(TK, hkv, dvd, dtype=q.dtype, device=q.device) if dv is None else dv
    do = do if (do.stride(2) == 1 and do.stride(1) == dvd) else do.contiguous()
    for t, d in ((q, dqk), (k, dqk), (v, dvd), (o, dvd), (do, dvd), (dq, dqk), (dk, dqk), (dv, dvd)):
        _check_view(t, d)
    delta = torch.empty(2, batch, hq, S, dtype=torch.float32, device=q.device)  # [rowsum(dO*O), lse*log2e]
    _lib.call("flash_attn_bwd_cap", do, q, k, v, o, lse, delta, dq, dk, dv, batch, S, SK, int(q_off), hq, hkv, dqk, dvd,
              q.stride(0), k.stride(0), v.stride(0), o.stride(0), do.stride(0), dq.stride(0), dk.stride(0),
              dv.stride(0), float(scale), int(causal), int(window or 0), float(softcap or 0.0),
              _lib.status_word(q.device))
    return dq, dk, dv


def sink_grad(do, o, lse, sinks, batch: int):
    """Gradient of the per-head sink logits: d sink_h = - sum_rows exp(sink_h - lse_row) * rowsum(dO * O) (the sink has
    no value vector, so it only enters through the softmax normaliser)."""
    T, hq, _ = o.shape
    S = T // batch
    delta = (do.float() * o.float()).sum(-1).view(batch, S, hq).permute(0, 2, 1)      # [B, Hq, S]
    p_sink = torch.exp(sinks.float().view(1, hq, 1) - lse)
    return -(p_sink * delta).sum(dim=(0, 2)).to(sinks.dtype)


class FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, batch, causal, scale, q_off=0, window=0, sinks=None, softcap=0.0):
        o, lse = flash_attn_fwd(q, k, v, batch, causal, scale, q_off, window, sinks, softcap)
        ctx.save_for_backward(q, k, v, o, lse, sinks if sinks is not None else torch.empty(0))
        ctx.args = (batch, causal, scale, q_off, window, sinks is not None, softcap)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, sinks = ctx.saved_tensors
        batch, causal, scale, q_off, window, has_sinks, softcap = ctx.args
        dq, dk, dv = flash_attn_bwd(do, q, k, v, o, lse, batch, causal, scale, q_off=q_off, window=window,
                                    softcap=softcap)
        ds = sink_grad(do, o, lse, sinks, batch) if has_sinks else None
        return dq, dk, dv, None, None, None, None, None, ds, None


def flash_attention(q, k, v, batch: int = 1, causal: bool = True, scale: float | None = None, q_off: int = 0,
                    window: int = 0, sinks=None, softcap: float = 0.0):
    """softmax(scale * Q K^T [+ causal mask]) V, token-major layout (see module docstring).  With ``q_off`` the queries
    are a chunk of a longer sequence whose keys / values ``[0, q_off + S)`` are given (sequence lengths and ``q_off``
    multiples of 128): the building block of all-gather context parallelism.  ``window`` / ``sinks``: sliding-window
    attention and learned per-head sink logits (fp32 [Hq]) as the reference passes them to ``flash_attn_func``
    (primus/backends/megatron/core/extensions/primus_turbo.py:876-883,924-942)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and not kernel_supports(q.shape[-1], v.shape[-1]):
        warn_composed(q.shape[-1], v.shape[-1])
        return attention_ref(q, k, v, batch, causal, scale, q_off, window, sinks, softcap)[0]
    if not q.is_cuda:
        return attention_ref(q, k, v, batch, causal, scale, q_off, window, sinks, softcap)[0]
    return FlashAttnFn.apply(q, k, v, batch, causal, scale, q_off, window, sinks, softcap)
