"""Memory-bound kernels of a transformer layer against the measured copy bandwidth.

    python -m primus_b200.tools.benchmark.elementwise_bench [--tokens 8192 --hidden 4096 --ffn 14336] [--output f.json]

Rows: MXFP8 quantisation (row + column direction in one pass), SwiGLU forward fused with quantisation, SwiGLU backward
fused with quantisation, RMSNorm forward (with residual add) and backward, RoPE, plain SwiGLU forward / backward,
cross-entropy (fused loss + gradient).  Every time is a CUDA-event median over rotating buffers larger than L2; the
byte count is the algorithmic minimum (each operand read once, each result written once), and the fraction is that
bandwidth over the measured copy bandwidth of ``MEASURED_PEAKS.json`` next to the repository root (fallback 6650 GB/s).
The reference benchmarks GEMM / attention / collectives only (primus/tools/benchmark/); this suite covers the
remaining kernels of the step.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from .common import L2_BYTES, emit, rotating_count, time_cuda


def _hbm_peak() -> tuple[float, str]:
    p = Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default=None, help="run only the rows whose name contains this text (short ncu captures)")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from ...ops import _lib, fp8, fused

    T, H, I, V = a.tokens, a.hidden, a.ffn, a.vocab
    dev = "cuda"
    peak, peak_kind = _hbm_peak()
    rows = []

    def add(name, fn, nbytes, nsets):
        if a.only and a.only not in name:
            return
        t = time_cuda(fn, a.iters)["ms_median"]
        gbs = nbytes / t / 1e6
        rows.append({"kernel": name, "ms": t, "algorithmic_MB": nbytes / 1e6, "GB/s": gbs,
                     f"fraction_of_{peak_kind}_copy_bw": gbs / peak, "buffers": nsets})

    # --- quantisation of a [T, H] activation, both directions
    n = rotating_count(T * H * 2)
    xs = [torch.randn(T, H, device=dev).bfloat16() for _ in range(n)]
    add("quant_mxfp8 row+col [T,H]", lambda i: fp8.quantize_mxfp8(xs[i % n], True, True), T * H * (2 + 2) + T * H // 16, n)
    add("quant_mxfp8 row [T,H]", lambda i: fp8.quantize_mxfp8(xs[i % n], True, False), T * H * (2 + 1) + T * H // 32, n)
    # --- SwiGLU (+ quantisation)
    m = rotating_count(T * 2 * I * 2)
    h1 = [torch.randn(T, 2 * I, device=dev).bfloat16() for _ in range(m)]
    da = [torch.randn(T, I, device=dev).bfloat16() for _ in range(m)]
    add("swiglu fwd + quant (row) [T,2I]->[T,I]", lambda i: fp8.swiglu_quantize_mxfp8(h1[i % m], 0.0, True, False),
        T * I * (4 + 1) + T * I // 32, m)
    add("swiglu bwd + quant (row+col) -> [T,2I]", lambda i: fp8.swiglu_bwd_quantize_mxfp8(h1[i % m], da[i % m], 0.0),
        T * I * (4 + 2 + 4) + T * I // 8, m)
    out_act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    add("swiglu fwd (bf16)", lambda i: _lib.call("swiglu_fwd", h1[i % m], None, out_act, T, I, 0.0, 0), T * I * 6, m)
    din = torch.empty(T, 2 * I, dtype=torch.bfloat16, device=dev)
    add("swiglu bwd (bf16)", lambda i: _lib.call("swiglu_bwd", da[i % m], h1[i % m], None, din, None, T, I, 0.0, 0),
        T * I * 10, m)
    del h1, da, out_act, din
    # --- RMSNorm
    w = torch.ones(H, device=dev).bfloat16()
    res = [torch.randn(T, H, device=dev).bfloat16() for _ in range(n)]
    add("rmsnorm fwd + residual add", lambda i: fused.rmsnorm(xs[i % n], w, 1e-5, res[i % n]), T * H * 8, n)
    add("rmsnorm fwd", lambda i: fused.rmsnorm(xs[i % n], w, 1e-5), T * H * 4, n)
    dy = [torch.randn(T, H, device=dev).bfloat16() for _ in range(n)]
    rstd = torch.rand(T, device=dev) + 0.5
    dx = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    dwf = torch.empty(H, dtype=torch.float32, device=dev)
    P = _lib.call_ret("rmsnorm_bwd_num_partials", T)
    sc = fused.scratch(torch.device(dev, torch.cuda.current_device()), "rmsnorm_dw", P * H)
    add("rmsnorm bwd (dx + dw partials + dw reduce)",
        lambda i: _lib.call("rmsnorm_bwd", dy[i % n], xs[i % n], w, rstd, None, dx, dwf, sc, T, H, H, H, 0), T * H * 6, n)
    add("rmsnorm bwd + residual gradient",
        lambda i: _lib.call("rmsnorm_bwd", dy[i % n], xs[i % n], w, rstd, res[i % n], dx, dwf, sc, T, H, H, H, 0),
        T * H * 8, n)
    del dy, res
    # --- RoPE on [T, heads, 128]
    d = 128
    qs = [torch.randn(T, a.heads, d, device=dev).bfloat16() for _ in range(n)]
    cos, sin = fused.rope_tables(T, d, 500000.0, torch.device(dev))
    add("rope (in place) [T,heads,128]", lambda i: fused.rope_inplace_(qs[i % n], cos, sin), T * a.heads * d * 4, n)
    del qs
    # --- cross entropy on [T, V] logits
    k = rotating_count(T * V * 2)
    lg = [torch.randn(T, V, device=dev).bfloat16() for _ in range(k)]
    lab = torch.randint(0, V, (T,), device=dev)
    wts = torch.full((T,), 1.0 / T, device=dev)
    add("cross entropy fused (loss + grad in place) [T,V]",
        lambda i: fused.cross_entropy(lg[i % k], lab, 0, None, wts, True), T * V * 4, k)
    torch.cuda.synchronize()
    _lib.check_status()
    emit(rows, a.output, f"memory-bound kernels, T={T} H={H} I={I} V={V}; copy bandwidth {peak:.0f} GB/s ({peak_kind}); "
                         f"L2 {L2_BYTES >> 20} MiB")
    return rows


if __name__ == "__main__":
    main()
