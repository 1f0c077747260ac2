"""GEMM micro-benchmark on the tcgen05 kernel (and cuBLAS via torch.matmul for comparison).

Suites: explicit ``--shape M N K`` or per-model training shapes ``attn_qkv, attn_out, mlp_up (N = 2*ffn),
mlp_down, vocab`` x {fprop (M,N,K), wgrad (N,K,M) accumulate into fp32, dgrad (M,K,N)}
(primus/tools/benchmark/dense_gemm_bench.py:149-226, gemm_bench.py:58-75 in the reference).

    python -m primus_b200.tools.benchmark.gemm_bench --suite llama3.1_8B --tokens 8192
"""
from __future__ import annotations

import argparse

import torch

from ...core.config.presets import load_preset
from ...models.config import TransformerConfig
from .common import emit, rotating_count, time_cuda


def model_shapes(cfg: TransformerConfig, tokens: int, tp: int = 1) -> list[tuple[str, int, int, int]]:
    h = cfg.hidden_size
    out = [("attn_qkv", tokens, cfg.qkv_width // tp, h), ("attn_out", tokens, h, cfg.num_attention_heads * cfg.kv_channels // tp),
           ("mlp_up", tokens, 2 * cfg.ffn_hidden_size // tp, h), ("mlp_down", tokens, h, cfg.ffn_hidden_size // tp),
           ("vocab", tokens, cfg.padded_vocab_size // tp, h)]
    if cfg.num_experts:
        out += [("moe_up(per expert avg)", tokens * cfg.moe_router_topk // cfg.num_experts, 2 * cfg.moe_ffn_hidden_size, h),
                ("moe_down(per expert avg)", tokens * cfg.moe_router_topk // cfg.num_experts, h, cfg.moe_ffn_hidden_size)]
    return out


def bench_shape(name, M, N, K, iters, compare):
    from ...ops import gemm as G

    n = rotating_count((M * K + N * K + M * N) * 2)
    xs = [torch.randn(M, K, device="cuda").bfloat16() for _ in range(n)]
    ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(n)]
    dys = [torch.randn(M, N, device="cuda").bfloat16() for _ in range(min(n, 4))]
    mg = torch.zeros(N, K, device="cuda")
    fl = 2.0 * M * N * K
    rows = []
    runs = [("fprop", lambda i: G.gemm(xs[i % n], ws[i % n])),
            ("dgrad", lambda i: G.gemm(dys[i % len(dys)], ws[i % n], b_mn=True)),
            ("wgrad+acc", lambda i: G.gemm(dys[i % len(dys)], xs[i % n], a_mn=True, b_mn=True, out=mg, accumulate=True))]
    if compare:
        runs += [("cublas fprop", lambda i: torch.matmul(xs[i % n], ws[i % n].t())),
                 ("cublas dgrad", lambda i: torch.matmul(dys[i % len(dys)], ws[i % n])),
                 ("cublas wgrad", lambda i: torch.matmul(dys[i % len(dys)].t(), xs[i % n]))]
    for kind, fn in runs:
        t = time_cuda(fn, iters)
        rows.append({"gemm": name, "kind": kind, "M": M, "N": N, "K": K, "ms": t["ms_median"],
                     "TFLOP/s": fl / t["ms_median"] / 1e9})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--suite", default=None, help="model preset name (e.g. llama3.1_8B, llama3.1_70B, deepseek_v2_lite)")
    ap.add_argument("--shape", type=int, nargs=3, action="append", metavar=("M", "N", "K"))
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-compare", action="store_true")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    shapes = [(f"{m}x{n}x{k}", m, n, k) for m, n, k in (a.shape or [])]
    if a.suite:
        shapes += model_shapes(TransformerConfig.from_dict(load_preset(a.suite, "models")), a.tokens, a.tp)
    if not shapes:
        shapes = [("square8192", 8192, 8192, 8192)]
    rows = []
    for s in shapes:
        rows += bench_shape(*s, a.iters, not a.no_compare)
    emit(rows, a.output, "bf16 GEMM")
    return rows


if __name__ == "__main__":
    main()
