"""Parameter and FLOP counts of the model presets.

    python -m primus_b200.tools.model_stats [--model llama3.1_8B ...] [--seq 8192] [--json]

One row per preset: total parameters, parameters active per token (routed experts counted ``top-k`` times), model
FLOPs per token for a training step (forward + backward, the figure behind the TFLOP/s/GPU of the log line) and the
bytes of weights + gradients + Adam state per parameter-holding replica.  Counterpart of the reference's
``tools/model_stats``.
"""
from __future__ import annotations

import argparse
import glob
import json
import os


def stats(name: str, seq: int) -> dict:
    from ..core.config.presets import load_preset
    from ..engine import schedules
    from ..models.config import TransformerConfig
    from .projection.memory import param_counts

    cfg = TransformerConfig.from_dict(load_preset(name, "models"))
    pc = param_counts(cfg)
    fixed = pc["embedding"] + pc["output"]
    total = fixed + sum(l["dense"] + l["expert"] for l in pc["layers"])
    frac = (cfg.moe_router_topk / cfg.num_experts) if cfg.num_experts else 1.0
    active = fixed + sum(l["dense"] + l["expert"] * frac for l in pc["layers"])
    return {"model": name, "layers": cfg.num_layers, "hidden": cfg.hidden_size,
            "experts": cfg.num_experts or 0, "params_B": total / 1e9, "active_params_B": active / 1e9,
            "train_GFLOPs_per_token": schedules.model_flops_per_token(cfg, seq) / 1e9,
            "state_GB_bf16_params_fp32_adam": total * (2 + 4 + 4 + 4 + 4) / 1e9}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", nargs="*", default=None, help="preset names (default: every preset)")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    names = a.model
    if not names:
        root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "models")
        names = sorted(os.path.basename(f)[:-5] for f in glob.glob(os.path.join(root, "*.yaml")))
        names = [n for n in names if not n.endswith("_base") and n != "language_model"]
    rows = [stats(n, a.seq) for n in names]
    if a.json:
        print(json.dumps(rows))
    else:
        from tabulate import tabulate

        print(tabulate(rows, headers="keys", floatfmt=".2f"))
    return rows


if __name__ == "__main__":
    main()
