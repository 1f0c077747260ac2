"""Flash-attention micro-benchmark (forward / backward, causal) on model head shapes
(the ``attention`` suite of primus/cli/subcommands/benchmark.py:8-50 in the reference)."""
from __future__ import annotations

import argparse
import math

import torch

from ...core.config.presets import load_preset
from ...models.config import TransformerConfig
from .common import emit, time_cuda


def _time_fwd_bwd(fwd, inputs, do, iters):
    """(forward ms, backward ms) of an autograd function: the backward alone is timed through ``torch.autograd.grad``
    on a retained graph, so no forward is inside its events."""
    tf = time_cuda(lambda i: fwd(), iters)
    out = fwd()
    tb = time_cuda(lambda i: torch.autograd.grad(out, inputs, do, retain_graph=True), iters)
    return tf["ms_median"], tb["ms_median"]


def _library_rows(a, q, k, v, do, hq, hkv, dqk, dv, fl, sc):
    """Library attention at the same shape: cuDNN fused attention through torch SDPA (grouped-query form, no repeated
    K / V heads) and ``flash_attn_func`` (the call the reference's own attention benchmark times,
    primus/tools/benchmark/attention_profiler.py:83-120)."""
    rows = []

    def add(tag, ms_f, ms_b):
        for op, ms, f in ((f"{tag} fwd", ms_f, fl), (f"{tag} bwd", ms_b, 2.5 * fl)):
            rows.append({"op": op, "heads": f"{hq}/{hkv}", "d": f"{dqk}/{dv}", "seq": a.seq, "ms": ms,
                         "TFLOP/s": f / ms / 1e9})

    def fail(tag, e):
        rows.append({"op": f"{tag}: {type(e).__name__}: {str(e)[:70]}", "heads": f"{hq}/{hkv}", "d": f"{dqk}/{dv}",
                     "seq": a.seq, "ms": float("nan"), "TFLOP/s": float("nan")})

    B, S = a.batch, a.seq
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel

        qq = q.view(B, S, hq, dqk).transpose(1, 2).detach().requires_grad_()
        kk = k.view(B, S, hkv, dqk).transpose(1, 2).detach().requires_grad_()
        vv = v.view(B, S, hkv, dv).transpose(1, 2).detach().requires_grad_()
        dd = do.view(B, S, hq, dv).transpose(1, 2)
        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            add("cudnn sdpa", *_time_fwd_bwd(lambda: torch.nn.functional.scaled_dot_product_attention(
                qq, kk, vv, is_causal=True, scale=sc, enable_gqa=hq != hkv), (qq, kk, vv), dd, a.iters))
    except Exception as e:
        fail("cudnn sdpa", e)
    if dqk == dv:
        try:
            from flash_attn import flash_attn_func

            q4 = q.view(B, S, hq, dqk).detach().requires_grad_()
            k4 = k.view(B, S, hkv, dqk).detach().requires_grad_()
            v4 = v.view(B, S, hkv, dv).detach().requires_grad_()
            add("flash_attn", *_time_fwd_bwd(lambda: flash_attn_func(q4, k4, v4, causal=True, softmax_scale=sc),
                                             (q4, k4, v4), do.view(B, S, hq, dv), a.iters))
        except Exception as e:
            fail("flash_attn", e)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--suite", default="llama3.1_8B")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--compare-sdpa", action="store_true")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from ...ops import attention as A

    cfg = TransformerConfig.from_dict(load_preset(a.suite, "models"))
    if cfg.multi_latent_attention:
        hq = hkv = cfg.num_attention_heads
        dqk, dv = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim, cfg.v_head_dim
    else:
        hq, hkv, dqk, dv = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels, cfg.kv_channels
    T = a.batch * a.seq
    q = torch.randn(T, hq, dqk, device="cuda").bfloat16()
    k = torch.randn(T, hkv, dqk, device="cuda").bfloat16()
    v = torch.randn(T, hkv, dv, device="cuda").bfloat16()
    sc = 1 / math.sqrt(dqk)
    fl = 2.0 * a.batch * a.seq * a.seq * hq * (dqk + dv) / 2
    rows = []
    t = time_cuda(lambda i: A.flash_attn_fwd(q, k, v, a.batch, True, sc), a.iters)
    rows.append({"op": "fwd", "heads": f"{hq}/{hkv}", "d": f"{dqk}/{dv}", "seq": a.seq, "ms": t["ms_median"],
                 "TFLOP/s": fl / t["ms_median"] / 1e9})
    o, lse = A.flash_attn_fwd(q, k, v, a.batch, True, sc)
    do = torch.randn_like(o)
    t = time_cuda(lambda i: A.flash_attn_bwd(do, q, k, v, o, lse, a.batch, True, sc), a.iters)
    rows.append({"op": "bwd", "heads": f"{hq}/{hkv}", "d": f"{dqk}/{dv}", "seq": a.seq, "ms": t["ms_median"],
                 "TFLOP/s": 2.5 * fl / t["ms_median"] / 1e9})
    if a.compare_sdpa:
        rows += _library_rows(a, q, k, v, do, hq, hkv, dqk, dv, fl, sc)
        ours = {r["op"]: r["ms"] for r in rows}
        for op in ("fwd", "bwd"):
            libs = [(r["ms"], r["op"]) for r in rows if r["op"].endswith(" " + op) and r["ms"] == r["ms"]]
            if libs:
                best = min(libs)
                rows.append({"op": f"ours/library {op} (vs {best[1]})", "heads": f"{hq}/{hkv}", "d": f"{dqk}/{dv}",
                             "seq": a.seq, "ms": ours[op], "TFLOP/s": best[0] / ours[op]})
    emit(rows, a.output, "flash attention (causal)")
    return rows


if __name__ == "__main__":
    main()
