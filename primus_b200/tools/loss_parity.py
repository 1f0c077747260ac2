"""Loss-curve comparison between precisions (and, optionally, fused vs un-fused paths) on learnable synthetic data.

    python -m primus_b200.tools.loss_parity --steps 300 [--hidden 1024 --layers 4] [--output curves.json]

Trains the same Llama-style model from the same initial weights on the same periodic-token stream once per
precision (bf16, mxfp8) and reports the two curves, their largest per-step relative difference and the relative
difference of their means over the last fifth of the run (per-step differences are dominated by which step a loss
spike lands on; the tail mean is what says whether the two precisions converge to the same place).  The reference checks
fused / low-precision paths the same way (loss trajectory vs the baseline path within a tolerance).
"""
from __future__ import annotations

import argparse
import json

import torch


def run(precision: str, a) -> list[float]:
    from ..engine.trainer import TrainConfig, Trainer
    from ..models.config import TransformerConfig
    from ..ops import gemm
    from ..parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=a.layers, hidden_size=a.hidden, ffn_hidden_size=a.hidden * 7 // 2 // 128 * 128,
                           num_attention_heads=a.hidden // 128, num_query_groups=max(1, a.hidden // 512), kv_channels=128,
                           vocab_size=a.vocab, params_dtype="bf16", seq_length=a.seq,
                           fp8="e4m3" if precision in ("mxfp8", "tensorwise") else None,
                           fp8_recipe=precision if precision == "tensorwise" else "mxfp8")
    tc = TrainConfig(micro_batch_size=a.micro_batch, global_batch_size=a.global_batch, seq_length=a.seq,
                     train_iters=a.steps, lr=a.lr, min_lr=a.lr / 10, lr_warmup_iters=20, lr_decay_style="cosine",
                     weight_decay=0.1, clip_grad=1.0, log_interval=1, mock_data_period=a.period if a.data == "period" else 0,
                     mock_data_kind=a.data if a.data == "markov" else "", seed=a.seed)
    torch.manual_seed(a.seed)
    try:
        tr = Trainer(mc, tc, device="cuda" if torch.cuda.is_available() else "cpu", log_fn=lambda s: None)
        return tr.train()
    finally:
        gemm.set_fp8_recipe(None)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--period", type=int, default=32)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--global-batch", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--data", default="markov", choices=["markov", "period"],
                    help="markov: smooth curve (transition table); period: in-context copying (sudden phase changes)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--precisions", default="bf16,mxfp8",
                    help="comma list of bf16, mxfp8 (scale per 32 elements), tensorwise (one power-of-two scale per tensor); "
                         "the differences reported are first vs last")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    names = a.precisions.split(",")
    curves = {p: run(p, a) for p in names}
    rel = max(abs(x - y) / max(abs(x), 1e-6) for x, y in zip(curves[names[0]], curves[names[-1]]))
    tail = max(1, a.steps // 5)
    tail_mean = {p: sum(curves[p][-tail:]) / tail for p in names}
    tail_rel = abs(tail_mean[names[0]] - tail_mean[names[-1]]) / max(abs(tail_mean[names[0]]), 1e-6)
    out = {"config": vars(a), "curves": curves, "max_relative_difference": rel,
           "tail_mean": tail_mean, "tail_mean_relative_difference": tail_rel,
           "final": {k: v[-1] for k, v in curves.items()}, "initial": {k: v[0] for k, v in curves.items()}}
    print(json.dumps({k: out[k] for k in ("max_relative_difference", "tail_mean", "tail_mean_relative_difference",
                                           "initial", "final")}))
    every = max(1, a.steps // 12)
    for i in range(0, a.steps, every):
        print(f"step {i + 1:4d}  " + "  ".join(f"{p} {curves[p][i]:.4f}" for p in names))
    if a.output:
        with open(a.output, "w") as f:
            json.dump(out, f, indent=1)
    return out


if __name__ == "__main__":
    main()
