"""Run a list of experiment configs through the launcher one after the other and tabulate what their logs report.

    python -m primus_b200.tools.ops.auto_benchmark --configs examples/configs/llama3.1_8B-*.yaml \\
        [--set train_iters=20] [--skip 5] [--output bench.md|.csv|.jsonl] [--launcher ./primus-cli] [--dry-run]
    python -m primus_b200.tools.ops.auto_benchmark --parse-logs out/*.log --output bench.md

For every config: ``<launcher> direct --log_file <dir>/<name>.log -- train pretrain --config <cfg> [--k v ...]``; the
run counts as complete when the log holds the trainer's completion line.  From the per-iteration log lines (after
``--skip`` warm-up iterations) it takes the mean time per iteration, tokens/s/GPU, TFLOP/s/GPU, the last loss and the
peak memory.  One failing config does not stop the rest.  (Role of the reference's auto-benchmark driver and its log
metrics parser: tools/auto_benchmark/run_primus_autobenchmark.sh, tools/auto_benchmark/metrics.py.)"""
from __future__ import annotations

import argparse
import glob
import os
import re
import subprocess
import sys
import time

from ..report import write_records

ITER_RE = re.compile(
    r"iteration\s+(\d+)/\s*(\d+) \| elapsed time per iteration \(ms\): ([\d.]+) \| "
    r"throughput per GPU \(TFLOP/s/GPU\): ([\d.]+) \| tokens/s/GPU: ([\d.]+).*?lm loss: ([\d.Ee+-]+|nan|inf).*?"
    r"max mem \(GiB\): ([\d.]+)")
COMPLETED = "Training completed."


def parse_log(text: str, skip: int = 2) -> dict:
    rows = [(int(m[1]), float(m[3]), float(m[4]), float(m[5]), float(m[6]), float(m[7])) for m in ITER_RE.finditer(text)]
    used = rows[skip:] if len(rows) > skip else rows
    rec = {"iterations": len(rows), "completed": COMPLETED in text}
    if used:
        n = len(used)
        rec.update(ms_per_iter=round(sum(r[1] for r in used) / n, 2), tflops_gpu=round(sum(r[2] for r in used) / n, 1),
                   tokens_s_gpu=round(sum(r[3] for r in used) / n, 1), last_loss=rows[-1][4],
                   max_mem_gib=max(r[5] for r in rows))
    return rec


def run_config(cfg: str, launcher: str, log_dir: str, overrides: list, timeout: float, dry_run: bool) -> dict:
    name = os.path.splitext(os.path.basename(cfg))[0]
    log = os.path.join(log_dir, name + ".log")
    cmd = [launcher, "direct", "--log_file", log, "--", "train", "pretrain", "--config", cfg]
    for kv in overrides:
        k, v = kv.split("=", 1)
        cmd += [f"--{k}", v]
    rec = {"config": name, "command": " ".join(cmd)}
    if dry_run:
        return dict(rec, status="dry-run")
    t0 = time.time()
    try:
        rc = subprocess.run(cmd, timeout=timeout, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL).returncode
    except subprocess.TimeoutExpired:
        rc = -1
    text = open(log, errors="replace").read() if os.path.exists(log) else ""
    rec.update(parse_log(text), wall_s=round(time.time() - t0, 1), returncode=rc)
    rec["status"] = "ok" if rc == 0 and rec.get("completed") else ("timeout" if rc == -1 else "failed")
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--configs", nargs="*", default=[])
    ap.add_argument("--parse-logs", nargs="*", default=[])
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="override passed to every run")
    ap.add_argument("--skip", type=int, default=2, help="warm-up iterations left out of the averages")
    ap.add_argument("--launcher", default=os.path.join(os.path.dirname(__file__), "..", "..", "..", "primus-cli"))
    ap.add_argument("--log-dir", default="output/auto_benchmark")
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("--output", default=None)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    records = []
    for pattern in args.parse_logs:
        for path in sorted(glob.glob(pattern)) or [pattern]:
            with open(path, errors="replace") as f:
                records.append(dict(config=os.path.splitext(os.path.basename(path))[0], **parse_log(f.read(), args.skip)))
    if args.configs:
        os.makedirs(args.log_dir, exist_ok=True)
    for pattern in args.configs:
        for cfg in sorted(glob.glob(pattern)) or [pattern]:
            rec = run_config(cfg, os.path.normpath(args.launcher), args.log_dir, args.set, args.timeout, args.dry_run)
            rec.pop("command") if not args.dry_run else None
            records.append(rec)
            print(rec, flush=True)
    keys = []
    for r in records:
        keys += [k for k in r if k not in keys]
    print(write_records(args.output, [{k: r.get(k, "") for k in keys} for r in records]))
    return 0 if all(r.get("status", "ok") in ("ok", "dry-run") for r in records) else 1


if __name__ == "__main__":
    sys.exit(main())
