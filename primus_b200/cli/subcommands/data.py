"""``primus data {tokenize,inspect,mock,blend,pack-sft}``: dataset preparation.  ``tokenize``: raw text / jsonl -> flat
token ``.bin`` + document index for the token-file loader (``primus_b200.engine.data.IndexedTokenDataset``) or a Megatron
indexed dataset; ``inspect``: what a token file or an indexed dataset holds; ``blend``: how a weighted blend of indexed
datasets is sampled for a run of a given length (tokens and epochs per corpus); ``pack-sft``: tokenises and bin-packs an
SFT file into the on-disk pack cache ahead of a run.
(The reference's ``data`` sub-command prepares diffusion datasets, primus/cli/subcommands/data.py; language-model
pre-training data there goes through Megatron's preprocess tooling.)"""
from __future__ import annotations

import json


def register_subcommand(subparsers):
    p = subparsers.add_parser("data", help="dataset preparation")
    sp = p.add_subparsers(dest="action", required=True)
    t = sp.add_parser("tokenize")
    t.add_argument("--input", required=True, help="text or jsonl file")
    t.add_argument("--output", required=True, help="output prefix (writes <prefix>.bin and <prefix>.idx.npy)")
    t.add_argument("--tokenizer", default=None, help="HF tokenizer name/path; default: byte-level")
    t.add_argument("--json-key", default="text")
    t.add_argument("--append-eod", action="store_true")
    t.add_argument("--format", default="flat", choices=["flat", "megatron"],
                   help="flat: <prefix>.bin + <prefix>.idx.npy; megatron: the MMIDIDX .bin / .idx pair of Megatron-LM")
    i = sp.add_parser("inspect")
    i.add_argument("--path", required=True)
    i.add_argument("--seq-length", type=int, default=4096)
    b = sp.add_parser("blend", help="sampling plan of a weighted blend of indexed datasets")
    b.add_argument("--data-path", required=True, help='"w1 prefix1 w2 prefix2 ..." (or a single prefix)')
    b.add_argument("--seq-length", type=int, default=4096)
    b.add_argument("--samples", type=int, required=True, help="samples the run will read (train_iters x global batch)")
    k = sp.add_parser("pack-sft", help="build the SFT pack cache entry of a dataset")
    k.add_argument("--input", required=True, help="jsonl file of SFT records")
    k.add_argument("--format", default="alpaca")
    k.add_argument("--seq-length", type=int, default=4096)
    k.add_argument("--tokenizer", default=None, help="HF tokenizer name / path; default: byte-level")
    k.add_argument("--algorithm", default="first_fit_decreasing")
    k.add_argument("--no-answer-only-loss", action="store_true")
    k.add_argument("--align", type=int, default=128)
    k.add_argument("--seed", type=int, default=1234)
    k.add_argument("--cache-dir", default=None)
    m = sp.add_parser("mock")
    m.add_argument("--output", required=True)
    m.add_argument("--tokens", type=int, default=1 << 20)
    m.add_argument("--vocab-size", type=int, default=32000)
    p.set_defaults(func=run)


def run(args, unknown):
    import numpy as np

    if args.action == "mock":
        rng = np.random.default_rng(1234)
        rng.integers(0, args.vocab_size, size=args.tokens, dtype=np.int32).tofile(args.output + ".bin")
        np.save(args.output + ".idx.npy", np.array([0, args.tokens], dtype=np.int64))
        print(f"wrote {args.tokens} tokens to {args.output}.bin")
        return 0
    if args.action == "blend":
        from ...engine.indexed_dataset import MMapIndexedDataset

        parts = args.data_path.split()
        pairs = [(1.0, parts[0])] if len(parts) == 1 else [(float(w), pfx) for w, pfx in zip(parts[0::2], parts[1::2])]
        total_w = sum(w for w, _ in pairs)
        rows = []
        for w, pfx in pairs:
            ds = MMapIndexedDataset(pfx)
            tokens = int(ds.sizes.astype(np.int64).sum())
            want = args.samples * w / total_w
            per_epoch = max((tokens - 1) // args.seq_length, 1)
            rows.append({"prefix": pfx, "weight": round(w / total_w, 4), "documents": len(ds), "tokens": tokens,
                         "samples_per_epoch": per_epoch, "samples_drawn": int(round(want)),
                         "epochs": round(want / per_epoch, 3)})
        print(json.dumps({"seq_length": args.seq_length, "samples": args.samples, "datasets": rows}, indent=1))
        return 0
    if args.action == "pack-sft":
        from ...engine import sft

        tok = sft.ByteTokenizer()
        if args.tokenizer:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(args.tokenizer)
        ds = sft.load_or_build_packed(args.input, tok, args.seq_length, args.format, not args.no_answer_only_loss,
                                      args.algorithm, args.seed, args.align, True, args.cache_dir, log=print)
        print(json.dumps({"packs": len(ds), "seq_length": args.seq_length, "cache_dir": sft.pack_cache_dir(args.cache_dir)}))
        return 0
    if args.action == "inspect" and __import__("os").path.exists(args.path + ".idx"):
        from ...engine.indexed_dataset import MMapIndexedDataset

        ds = MMapIndexedDataset(args.path)
        sizes = ds.sizes.astype(np.int64)
        print(json.dumps({"format": "megatron", "documents": len(ds), "tokens": int(sizes.sum()), "dtype": str(ds.dtype),
                          "samples": int((sizes.sum() - 1) // args.seq_length), "shortest_document": int(sizes.min()),
                          "longest_document": int(sizes.max()), "mean_document": round(float(sizes.mean()), 1)}))
        return 0
    if args.action == "inspect":
        data = np.memmap(args.path, dtype=np.int32, mode="r")
        print(json.dumps({"tokens": int(len(data)), "samples": int((len(data) - 1) // args.seq_length),
                          "max_id": int(data[: 1 << 20].max()), "min_id": int(data[: 1 << 20].min())}))
        return 0
    tok = None
    if args.tokenizer:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    ids, starts = [], [0]
    with open(args.input) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            text = json.loads(line)[args.json_key] if args.input.endswith(".jsonl") else line
            t = tok.encode(text) if tok else list(text.encode("utf-8"))
            if args.append_eod:
                t.append(tok.eos_token_id if tok and tok.eos_token_id is not None else 0)
            ids.extend(t)
            starts.append(len(ids))
    if args.format == "megatron":
        from ...engine.indexed_dataset import write_indexed_dataset

        arr = np.asarray(ids, dtype=np.int32)
        write_indexed_dataset(args.output, [arr[a:b] for a, b in zip(starts[:-1], starts[1:])], dtype=np.int32)
        print(f"wrote {len(ids)} tokens in {len(starts) - 1} documents to {args.output}.bin / .idx")
        return 0
    np.asarray(ids, dtype=np.int32).tofile(args.output + ".bin")
    np.save(args.output + ".idx.npy", np.asarray(starts, dtype=np.int64))
    print(f"wrote {len(ids)} tokens in {len(starts) - 1} documents to {args.output}.bin")
    return 0
