"""Per-GPU tiers, run in a child process per GPU so that one bad device cannot take the others' tests down:

tier 1  a tiny training step through the sm_100a kernels (native library loads, kernels run, loss is finite, no bounded
        wait expired);
tier 2  performance against thresholds: square bf16 GEMM on the tcgen05 kernel, HBM copy bandwidth, optional
        peer-copy bandwidth to the next GPU.

    python -m primus_b200.tools.preflight.node_smoke.per_gpu --gpu 3 --tier 2 --json

(primus/tools/preflight/node_smoke/per_gpu.py in the reference; thresholds of
docs_deprecated/node-smoke-test-instruction.md:120 scaled to B200.)"""
from __future__ import annotations

import argparse
import json
import sys
import time


def tier1(gpu: int) -> dict:
    import torch

    from ....engine.trainer import TrainConfig, Trainer
    from ....models.config import TransformerConfig
    from ....ops import _lib
    from ....parallel import state as ps

    torch.cuda.set_device(gpu)
    ps.destroy_model_parallel()
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1408, num_attention_heads=4, num_query_groups=2,
                            kv_channels=128, vocab_size=32000, params_dtype="bf16", fp8="e4m3", fp8_recipe="mxfp8")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=2, log_interval=1)
    t0 = time.time()
    losses = Trainer(cfg, tc, device=f"cuda:{gpu}", log_fn=lambda s: None).train(2)
    torch.cuda.synchronize()
    _lib.check_status(gpu)
    ok = all(l == l and 0 < l < 20 for l in losses)
    return {"check": "tier1 training step", "status": "PASS" if ok else "FAIL", "losses": losses, "seconds": time.time() - t0}


def tier2(gpu: int, thresholds: dict, peer: bool = True) -> list:
    import torch

    from ..checks import perf_gemm, perf_hbm

    torch.cuda.set_device(gpu)
    out = []
    g = perf_gemm()
    out.append({"check": "tier2 square bf16 GEMM", "status": "PASS" if g["tflops_median"] >= thresholds["gemm_tflops"] else "FAIL",
                "tflops": g["tflops_median"], "threshold": thresholds["gemm_tflops"]})
    h = perf_hbm()
    out.append({"check": "tier2 HBM copy", "status": "PASS" if h["gbs"] >= thresholds["hbm_gbs"] else "FAIL",
                "gbs": h["gbs"], "threshold": thresholds["hbm_gbs"]})
    n = torch.cuda.device_count()
    if peer and n > 1:
        dst = (gpu + 1) % n
        a = torch.empty(256 * 2**20, dtype=torch.uint8, device=f"cuda:{gpu}")
        b = torch.empty_like(a, device=f"cuda:{dst}")
        for _ in range(2):
            b.copy_(a)
        torch.cuda.synchronize(gpu); torch.cuda.synchronize(dst)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            b.copy_(a)
        e.record(); torch.cuda.synchronize(gpu); torch.cuda.synchronize(dst)
        gbs = 5 * a.numel() / s.elapsed_time(e) / 1e6
        out.append({"check": f"tier2 peer copy GPU{gpu} -> GPU{dst}", "status": "PASS" if gbs >= thresholds["p2p_gbs"] else "FAIL",
                    "gbs": gbs, "threshold": thresholds["p2p_gbs"]})
    return out


def main(argv=None) -> int:
    from ..checks import DEFAULT_THRESHOLDS

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, required=True)
    ap.add_argument("--tier", type=int, default=2)
    ap.add_argument("--gemm-tflops", type=float, default=DEFAULT_THRESHOLDS["gemm_tflops"])
    ap.add_argument("--hbm-gbs", type=float, default=DEFAULT_THRESHOLDS["hbm_gbs"])
    ap.add_argument("--p2p-gbs", type=float, default=DEFAULT_THRESHOLDS["p2p_gbs"])
    ap.add_argument("--no-peer", action="store_true")
    a = ap.parse_args(argv)
    res = {"gpu": a.gpu, "checks": []}
    try:
        res["checks"].append(tier1(a.gpu))
        if a.tier >= 2:
            res["checks"] += tier2(a.gpu, {"gemm_tflops": a.gemm_tflops, "hbm_gbs": a.hbm_gbs, "p2p_gbs": a.p2p_gbs},
                                   not a.no_peer)
    except Exception as e:  # noqa: BLE001
        res["checks"].append({"check": "per-gpu run", "status": "FAIL", "error": repr(e)})
    print("NODE_SMOKE_RESULT " + json.dumps(res, default=str))
    return 1 if any(c["status"] == "FAIL" for c in res["checks"]) else 0


if __name__ == "__main__":
    sys.exit(main())
