"""Checkpoint conversion between Hugging Face weight directories and this engine's ``torch_dist`` checkpoints, offline
and in one process (no trainer, no GPU):

    python -m primus_b200.tools.convert_checkpoint engine-to-hf --load <checkpoint root> [--iteration N] --output <dir>
    python -m primus_b200.tools.convert_checkpoint hf-to-engine --hf <dir with config.json + weights> --output <file.pt>
    python -m primus_b200.tools.convert_checkpoint inspect --load <checkpoint root>

``engine-to-hf`` reads the global tensors of a checkpoint through its metadata (whatever parallel layout wrote it) and
writes ``model.safetensors`` in the Hugging Face naming of the architecture.  ``hf-to-engine`` writes the full state
dict in this engine's naming plus the model configuration derived from ``config.json``; a training run starts from
Hugging Face weights directly with ``pretrained_hf_path`` and exports with ``export_hf_path``.  (Role of the reference's
conversion scripts, tools/checkpoint_conversion/ and the bridge-free converters of primus/backends/megatron/sft/.)"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    import torch

    from ..engine import hf_convert as H

    ap = argparse.ArgumentParser(prog="convert_checkpoint", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="action", required=True)
    e = sub.add_parser("engine-to-hf")
    e.add_argument("--load", required=True)
    e.add_argument("--iteration", type=int, default=None)
    e.add_argument("--output", required=True)
    h = sub.add_parser("hf-to-engine")
    h.add_argument("--hf", required=True)
    h.add_argument("--output", required=True)
    h.add_argument("--params-dtype", default="bf16")
    i = sub.add_parser("inspect")
    i.add_argument("--load", required=True)
    i.add_argument("--iteration", type=int, default=None)
    args = ap.parse_args(argv)
    if args.action == "engine-to-hf":
        sd, cfg = H.read_engine_checkpoint(args.load, args.iteration)
        H.save_hf(sd, cfg, args.output)
        print(f"wrote {len(sd)} tensors to {os.path.join(args.output, 'model.safetensors')}")
        return 0
    if args.action == "inspect":
        sd, cfg = H.read_engine_checkpoint(args.load, args.iteration)
        total = sum(t.numel() for t in sd.values())
        print(json.dumps({"tensors": len(sd), "parameters": total, "num_layers": cfg.num_layers,
                          "hidden_size": cfg.hidden_size, "model_type": cfg.model_type,
                          "largest": sorted(((t.numel(), k) for k, t in sd.items()), reverse=True)[:3]}))
        return 0
    from ..models.config import TransformerConfig

    with open(os.path.join(args.hf, "config.json")) as f:
        hf_cfg = json.load(f)
    kw = H.config_from_hf(hf_cfg.get("text_config", hf_cfg))
    kw["params_dtype"] = args.params_dtype
    cfg = TransformerConfig(**kw)
    sd = H.hf_to_internal(H.read_hf_weights(args.hf), cfg)
    torch.save({"state": sd, "model_config": kw}, args.output)
    print(f"wrote {len(sd)} tensors ({sum(t.numel() for t in sd.values())} parameters) to {args.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
