"""Look inside packed SFT data: which tokens are supervised, where the sample boundaries sit, what the text is.

    python -m primus_b200.tools.diag.inspect_sft_data --cache ~/.cache/primus_packed_sft/packed_<key>.pt
    python -m primus_b200.tools.diag.inspect_sft_data --mlperf-dir /data/mlperf_packed --num-samples 2
    python -m primus_b200.tools.diag.inspect_sft_data --jsonl data.jsonl --format alpaca --seq-length 4096 --pack

For each of the first ``--num-samples`` packed sequences it prints the token count, the number and share of
supervised positions, the positions where the loss mask switches (answer-only masks switch once per sample, all-token
masks never), the sample boundaries, and the decoded text of the head of the sequence and of its supervised span.
A wrong loss mask (prompt tokens supervised, or targets crossing a sample boundary) is the usual cause of an SFT
loss that starts far from the expected value, and it is visible here before any training is run.

Counterpart of the reference's diagnostic (primus/tools/diag/inspect_sft_data.py), for this package's caches.
"""
from __future__ import annotations

import argparse
import sys


def describe(item: dict, tokenizer=None, head: int = 80, span_chars: int = 200) -> dict:
    """Statistics of one packed item (``tokens``, ``labels``, ``loss_mask``, optional ``host_cu_seqlens``)."""
    toks = item["tokens"].tolist()
    labels = item["labels"].tolist()
    mask = [int(m > 0) for m in item["loss_mask"].tolist()]
    switches = [i for i in range(1, len(mask)) if mask[i] != mask[i - 1]]
    cu = [int(c) for c in item.get("host_cu_seqlens", []).tolist() if int(c) >= 0] if "host_cu_seqlens" in item else []
    # a supervised position just before a boundary whose target is the first token of the next sample
    crossing = [c - 1 for c in cu[1:-1] if 0 < c < len(mask) and mask[c - 1] and labels[c - 1] == toks[c]]
    out = {"tokens": len(toks), "supervised": sum(mask), "supervised_share": round(sum(mask) / max(len(mask), 1), 4),
           "mask_switches": switches[:16], "num_switches": len(switches), "boundaries": cu,
           "targets_across_boundaries": crossing}
    if tokenizer is not None and hasattr(tokenizer, "decode"):
        out["head_text"] = tokenizer.decode(toks[:head])
        sup = [labels[i] for i in range(len(mask)) if mask[i]]
        out["supervised_text"] = tokenizer.decode(sup)[:span_chars]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--cache", help="a packed_<key>.pt file of the pack cache")
    src.add_argument("--mlperf-dir", help="directory with train.npy / packed_metadata.jsonl")
    src.add_argument("--jsonl", help="raw SFT records (tokenised and optionally packed on the fly)")
    ap.add_argument("--format", default="alpaca")
    ap.add_argument("--seq-length", type=int, default=4096)
    ap.add_argument("--pack", action="store_true")
    ap.add_argument("--tokenizer", default=None, help="Hugging Face tokenizer name or path (default: byte tokenizer)")
    ap.add_argument("--num-samples", type=int, default=3)
    a = ap.parse_args(argv)
    import torch

    from ...engine import sft as S

    tok = S.ByteTokenizer()
    if a.tokenizer:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(a.tokenizer)
    if a.cache:
        blob = torch.load(a.cache, weights_only=False)
        base = S.SFTDataset([], tok, a.seq_length, a.format)
        base.samples = blob["samples"]
        ds = S.PackedSFTDataset(base, bins=blob["bins"])
        print(f"pack cache {a.cache}: {len(base)} samples in {len(ds)} bins, efficiency {ds.packing_efficiency():.3f}")
    elif a.mlperf_dir:
        ds = S.MLPerfPackedDataset(a.mlperf_dir, "train", None)
        print(f"MLPerf packed data {a.mlperf_dir}: {len(ds)} packs of {ds.seq_length} tokens, metadata {ds.metadata}")
    else:
        ds = S.SFTDataset.from_jsonl(a.jsonl, tok, a.seq_length, a.format)
        if a.pack:
            ds = S.PackedSFTDataset(ds)
        print(f"{a.jsonl}: {len(ds)} {'packed sequences' if a.pack else 'samples'}")
    for i in range(min(a.num_samples, len(ds))):
        d = describe(ds[i], tok)
        print(f"--- sequence {i}")
        for k, v in d.items():
            print(f"  {k}: {v!r}")
        if d["targets_across_boundaries"]:
            print("  WARNING: supervised targets cross a sample boundary at", d["targets_across_boundaries"])
    return 0


if __name__ == "__main__":
    sys.exit(main())
