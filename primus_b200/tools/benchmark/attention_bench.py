"""Flash-attention micro-benchmark (forward / backward, causal) on model head shapes
(the ``attention`` suite of primus/cli/subcommands/benchmark.py:8-50 in the reference)."""
from __future__ import annotations

import argparse
import math

import torch

from ...core.config.presets import load_preset
from ...models.config import TransformerConfig
from .common import emit, time_cuda


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
    if a.compare_sdpa and dqk == dv:
        qq = q.view(a.batch, a.seq, hq, dqk).transpose(1, 2)
        kk = k.view(a.batch, a.seq, hkv, dqk).transpose(1, 2).repeat_interleave(hq // hkv, 1)
        vv = v.view(a.batch, a.seq, hkv, dv).transpose(1, 2).repeat_interleave(hq // hkv, 1)
        t = time_cuda(lambda i: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True), a.iters)
        rows.append({"op": "torch sdpa fwd", "heads": f"{hq}/{hq}", "d": f"{dqk}/{dv}", "seq": a.seq,
                     "ms": t["ms_median"], "TFLOP/s": fl / t["ms_median"] / 1e9})
    emit(rows, a.output, "flash attention (causal)")
    return rows


if __name__ == "__main__":
    main()
