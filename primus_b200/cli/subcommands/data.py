"""``primus data {tokenize,inspect,mock}``: dataset preparation for the token-file loader
(``primus_b200.engine.data.IndexedTokenDataset``): raw text / jsonl -> flat token ``.bin`` + document index.
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
