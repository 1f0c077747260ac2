"""Compare the newest benchmark table with the previous one and flag regressions.

    python -m primus_b200.tools.ops.periodic_report --history <dir of dated *.jsonl tables> [--threshold 0.03]
        [--metric tokens_s_gpu] [--output report.md]

The history directory holds one ``.jsonl`` table per run of ``auto_benchmark`` (any sortable file names, e.g. dates).
For every config present in the two newest tables the report lists the metric in both, the relative change and a verdict
(``regression`` when it fell by more than the threshold, ``improvement`` when it rose by more, ``new`` / ``gone`` for
configs present in one table only, ``failed`` when the newest run did not complete); exit code 1 when anything regressed
or failed.  (Role of the reference's daily report: tools/daily/daily_report.py.)"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys

from ..report import write_records


def load_table(path: str) -> dict:
    out = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                r = json.loads(line)
                out[r["config"]] = r
    return out


def compare(old: dict, new: dict, metric: str, threshold: float) -> list:
    rows = []
    for name in sorted(set(old) | set(new)):
        a, b = old.get(name), new.get(name)
        if b is None:
            rows.append(dict(config=name, previous=a.get(metric, ""), latest="", change="", verdict="gone"))
            continue
        if b.get("status", "ok") not in ("ok", "") or b.get(metric) in (None, ""):
            rows.append(dict(config=name, previous=(a or {}).get(metric, ""), latest="", change="", verdict="failed"))
            continue
        if a is None or a.get(metric) in (None, ""):
            rows.append(dict(config=name, previous="", latest=b[metric], change="", verdict="new"))
            continue
        rel = (float(b[metric]) - float(a[metric])) / float(a[metric])
        verdict = "regression" if rel < -threshold else ("improvement" if rel > threshold else "same")
        rows.append(dict(config=name, previous=a[metric], latest=b[metric], change=f"{100 * rel:+.1f}%", verdict=verdict))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--history", required=True)
    ap.add_argument("--metric", default="tokens_s_gpu")
    ap.add_argument("--threshold", type=float, default=0.03)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    tables = sorted(glob.glob(os.path.join(args.history, "*.jsonl")))
    if len(tables) < 2:
        print(f"need two tables under {args.history}, found {len(tables)}", file=sys.stderr)
        return 2
    rows = compare(load_table(tables[-2]), load_table(tables[-1]), args.metric, args.threshold)
    pre = f"{args.metric}: {os.path.basename(tables[-2])} -> {os.path.basename(tables[-1])} (threshold {100 * args.threshold:.0f}%)"
    print(write_records(args.output, rows, preamble=pre))
    return 1 if any(r["verdict"] in ("regression", "failed") for r in rows) else 0


if __name__ == "__main__":
    sys.exit(main())
