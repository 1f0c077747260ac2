"""Offline GEMM tuning: times every tile configuration of the GEMM shapes a short job recorded and writes the table
``ops.autotune`` loads at start-up.

    PRIMUS_B200_GEMM_TUNING_STAGE=1 primus-cli direct -- train pretrain --config exp.yaml --train_iters 3   # dump shapes
    python -m primus_b200.tools.tune_gemm --shapes gemm_shape/*.json --out gemm_tune/tuned.json           # this tool
    PRIMUS_B200_GEMM_TUNING_FILE=gemm_tune/tuned.json primus-cli direct -- train pretrain --config exp.yaml  # use

``--model <preset> --tokens T [--tp N]`` tunes the linear-layer shapes of a model preset without a shape dump.
Counterpart of the reference's offline tuner (examples/offline_tune/offline_tune_gemm.py) and of stage 2 of its
hipBLASLt workflow.
"""
from __future__ import annotations

import argparse
import glob
import sys

from ..ops import autotune


def model_shapes(preset: str, tokens: int, tp: int = 1, kinds=("mxfp8", "bf16")) -> list:
    """fprop / dgrad / wgrad keys of the dense linear layers of a model preset at ``tokens`` tokens per micro-batch."""
    from ..core.config.presets import load_preset
    from ..models.config import TransformerConfig

    cfg = TransformerConfig.from_dict(load_preset(preset, "models"))
    h = cfg.hidden_size
    layers = [(cfg.qkv_width // tp, h), (h, cfg.num_attention_heads * cfg.kv_channels // tp),
              (2 * cfg.ffn_hidden_size // tp, h), (h, cfg.ffn_hidden_size // tp)]
    keys = []
    for kind in kinds:
        for n, k in layers:
            keys.append(autotune.make_key(kind, tokens, n, k, False, False, 0))     # y = x W^T
            keys.append(autotune.make_key(kind, tokens, k, n, False, True, 0))      # dx = dy W
            keys.append(autotune.make_key(kind, n, k, tokens, True, True, 2))       # dW += dy^T x
    return list(dict.fromkeys(keys))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", nargs="*", default=[], help="shape dumps written by a stage-1 run (globs allowed)")
    ap.add_argument("--model", help="model preset whose linear-layer shapes are tuned instead of / besides a dump")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--out", default="gemm_tune/tuned.json")
    ap.add_argument("--merge", help="existing tuning file to extend")
    a = ap.parse_args(argv)
    import torch

    if not torch.cuda.is_available():
        print("tune_gemm needs a GPU", file=sys.stderr)
        return 2
    keys = []
    files = [f for pat in a.shapes for f in sorted(glob.glob(pat))]
    if files:
        seen = autotune.read_shapes(files)
        keys += [k for k, _ in sorted(seen.items(), key=lambda kv: -kv[1])]
    if a.model:
        keys += model_shapes(a.model, a.tokens, a.tp)
    keys = list(dict.fromkeys(keys))
    if not keys:
        print("no shapes given (use --shapes or --model)", file=sys.stderr)
        return 2
    if a.merge:
        autotune.load(a.merge)
    autotune.tune_shapes(keys, log=print)
    autotune.save(a.out)
    print(f"wrote {len(autotune.table())} entries to {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
