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
    by = {r["kind"]: r for r in rows}
    for ours, lib in (("fprop", "cublas fprop"), ("dgrad", "cublas dgrad"), ("wgrad+acc", "cublas wgrad")):
        if ours in by and lib in by:
            rows.append({"gemm": name, "kind": f"ours/library {ours}", "M": M, "N": N, "K": K, "ms": by[ours]["ms"],
                         "TFLOP/s": by[lib]["ms"] / by[ours]["ms"]})
    return rows


def bench_shape_mxfp8(name, M, N, K, iters):
    """MXFP8 GEMMs of a linear layer (operands pre-quantised: the GEMM kernel alone) and the quantisation kernel."""
    from ...ops import fp8

    if M % 128 or N % 128 or K % 128:
        return []
    n = rotating_count(M * K + N * K + M * N * 2)
    xs = [fp8.quantize_mxfp8(torch.randn(M, K, device="cuda").bfloat16()) for _ in range(n)]
    ws = [fp8.quantize_mxfp8((torch.randn(N, K, device="cuda") * 0.02).bfloat16()) for _ in range(n)]
    dys = [fp8.quantize_mxfp8(torch.randn(M, N, device="cuda").bfloat16()) for _ in range(min(n, 4))]
    xb = [torch.randn(M, K, device="cuda").bfloat16() for _ in range(min(n, 4))]
    mg = torch.zeros(N, K, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    dx = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    fl = 2.0 * M * N * K
    nd = len(dys)
    runs = []
    for tag, two in (("mxfp8", False), ("mxfp8 cta-pair", True)):
        runs += [(f"{tag} fprop", lambda i, two=two: fp8.gemm_mxfp8(xs[i % n].q_row, xs[i % n].sf_row, ws[i % n].q_row,
                                                                    ws[i % n].sf_row, M, N, K, out=out, two_cta=two)),
                 (f"{tag} dgrad", lambda i, two=two: fp8.gemm_mxfp8(dys[i % nd].q_row, dys[i % nd].sf_row, ws[i % n].q_col,
                                                                    ws[i % n].sf_col, M, K, N, b_mn=True, out=dx,
                                                                    two_cta=two)),
                 (f"{tag} wgrad+acc", lambda i, two=two: fp8.gemm_mxfp8(dys[i % nd].q_col, dys[i % nd].sf_col,
                                                                        xs[i % n].q_col, xs[i % n].sf_col, N, K, M,
                                                                        a_mn=True, b_mn=True, out=mg, accumulate=True,
                                                                        two_cta=two))]
    runs += _cublaslt_mxfp8_runs(M, N, K, n)
    rows = []
    for kind, fn in runs:
        try:
            t = time_cuda(fn, iters)
        except Exception as e:  # the library path is optional: report why it did not run
            rows.append({"gemm": name, "kind": f"{kind}: {type(e).__name__}: {str(e)[:80]}", "M": M, "N": N, "K": K,
                         "ms": float("nan"), "TFLOP/s": float("nan")})
            continue
        rows.append({"gemm": name, "kind": kind, "M": M, "N": N, "K": K, "ms": t["ms_median"],
                     "TFLOP/s": fl / t["ms_median"] / 1e9})
    _add_ratio_rows(rows, name, M, N, K)
    t = time_cuda(lambda i: fp8.quantize_mxfp8(xb[i % len(xb)]), iters)
    rows.append({"gemm": name, "kind": "quantize row+col (GB/s in TFLOP/s column)", "M": M, "N": 0, "K": K,
                 "ms": t["ms_median"], "TFLOP/s": M * K * (2 + 2 + 1 / 16) / t["ms_median"] / 1e6})
    return rows


def _cublaslt_mxfp8_runs(M, N, K, n):
    """cuBLASLt block-scaled MXFP8 GEMMs through ``torch._scaled_mm`` (E4M3 operands, E8M0 scales per 32 in the blocked
    128x4 layout), timed on random bytes.  The library takes K-major operands only, so the data- and weight-gradient
    GEMMs are timed the way Transformer-Engine runs them: as K-major GEMMs on transposed quantised copies, at the
    permuted problem sizes (M,K,N) and (N,K,M)."""
    e8 = getattr(torch, "float8_e8m0fnu", None)
    if e8 is None or not hasattr(torch, "_scaled_mm"):
        return []

    def operand(rows, cols):
        q = torch.randint(0, 120, (rows, cols), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        nsf = (-(-rows // 128) * 128) * (-(-(cols // 32) // 4) * 4)
        sf = torch.full((nsf,), 127, dtype=torch.uint8, device="cuda").view(e8)
        return q, sf

    runs = []
    for tag, (m, nn, k) in (("fprop", (M, N, K)), ("dgrad", (M, K, N)), ("wgrad", (N, K, M))):
        ab = [(operand(m, k), operand(nn, k)) for _ in range(n)]

        def fn(i, ab=ab):
            (a, sa), (b, sb) = ab[i % len(ab)]
            return torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        runs.append((f"cublaslt mxfp8 {tag}", fn))
    return runs


def _add_ratio_rows(rows, name, M, N, K):
    """ours / library for every GEMM kind that has both timings (> 1 means the kernel of this package is faster)."""
    by = {r["kind"]: r for r in rows if r["gemm"] == name and r["ms"] == r["ms"]}
    for kind in ("fprop", "dgrad", "wgrad"):
        lib = by.get(f"cublaslt mxfp8 {kind}")
        ours = [by.get(f"mxfp8 {kind}"), by.get(f"mxfp8 {kind}+acc"), by.get(f"mxfp8 cta-pair {kind}"),
                by.get(f"mxfp8 cta-pair {kind}+acc")]
        ours = [o for o in ours if o]
        if lib and ours:
            best = min(ours, key=lambda r: r["ms"])
            rows.append({"gemm": name, "kind": f"ours/library {kind} ({best['kind']})", "M": M, "N": N, "K": K,
                         "ms": best["ms"], "TFLOP/s": lib["ms"] / best["ms"]})


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--suite", default=None, help="model preset name (e.g. llama3.1_8B, llama3.1_70B, deepseek_v2_lite)")
    ap.add_argument("--shape", type=int, nargs=3, action="append", metavar=("M", "N", "K"))
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-compare", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "mxfp8", "both"])
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    shapes = [(f"{m}x{n}x{k}", m, n, k) for m, n, k in (a.shape or [])]
    if a.suite:
        shapes += model_shapes(TransformerConfig.from_dict(load_preset(a.suite, "models")), a.tokens, a.tp)
    if not shapes:
        shapes = [("square8192", 8192, 8192, 8192)]
    rows = []
    for s in shapes:
        if a.dtype in ("bf16", "both"):
            rows += bench_shape(*s, a.iters, not a.no_compare)
        if a.dtype in ("mxfp8", "both"):
            rows += bench_shape_mxfp8(*s, a.iters)
    emit(rows, a.output, "GEMM")
    return rows


if __name__ == "__main__":
    main()
