"""Pipeline timeline viewer: merges the per-rank files written with ``dump_pp_data: true`` into a text chart and a
Chrome / Perfetto trace.

    python -m primus_b200.tools.pp_vis <pp_data dir> [--iteration N] [--trace out.json] [--width 120]

Each row of the chart is one pipeline rank; a cell shows the node that was running (F / B / W, upper case for chunk
0, lower case for the other chunks; ``.`` = idle).  The printed bubble fraction is idle time / span per rank.  Plays the
role of the reference's pipeline visualiser (primus/backends/megatron/core/pipeline_parallel/pp_visualizer.py and
tools/visualization/pp_vis).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re


def load(directory: str, iteration: int | None = None) -> dict[int, dict]:
    """{pp_rank: record} for the requested (default: the newest) iteration."""
    files = glob.glob(os.path.join(directory, "pp_rank*_iter*.json"))
    by_iter: dict[int, dict[int, str]] = {}
    for f in files:
        m = re.search(r"pp_rank(\d+)_iter(\d+)\.json$", f)
        if m:
            by_iter.setdefault(int(m.group(2)), {})[int(m.group(1))] = f
    if not by_iter:
        raise FileNotFoundError(f"no pp_rank*_iter*.json under {directory}")
    it = iteration if iteration is not None else max(by_iter)
    out = {}
    for r, f in sorted(by_iter[it].items()):
        with open(f) as fh:
            out[r] = json.load(fh)
    return out


def chart(records: dict[int, dict], width: int = 120) -> tuple[list[str], dict[int, float]]:
    t0 = min(e["start"] for rec in records.values() for e in rec["events"])
    t1 = max(e["end"] for rec in records.values() for e in rec["events"])
    span = max(t1 - t0, 1e-9)
    lines, bubbles = [], {}
    for r, rec in sorted(records.items()):
        row = ["."] * width
        busy = 0.0
        for e in rec["events"]:
            a = int((e["start"] - t0) / span * width)
            b = max(a + 1, int((e["end"] - t0) / span * width))
            ch = e["kind"][0]
            ch = ch.upper() if e["chunk"] == 0 else ch.lower()
            for i in range(a, min(b, width)):
                row[i] = ch
            busy += e["end"] - e["start"]
        rs = min(e["start"] for e in rec["events"])
        re_ = max(e["end"] for e in rec["events"])
        bubbles[r] = 1.0 - busy / max(re_ - rs, 1e-9)
        lines.append(f"rank {r:2d} |{''.join(row)}|")
    return lines, bubbles


def chrome_trace(records: dict[int, dict]) -> dict:
    t0 = min(e["start"] for rec in records.values() for e in rec["events"])
    ev = []
    for r, rec in sorted(records.items()):
        for e in rec["events"]:
            ev.append({"name": f"{e['kind']} mb{e['mb']} c{e['chunk']}", "ph": "X", "pid": 0, "tid": r,
                       "ts": (e["start"] - t0) * 1e6, "dur": (e["end"] - e["start"]) * 1e6,
                       "args": {"microbatch": e["mb"], "chunk": e["chunk"]}})
    return {"traceEvents": ev, "displayTimeUnit": "ms"}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("directory")
    ap.add_argument("--iteration", type=int, default=None)
    ap.add_argument("--trace", default=None, help="write a Chrome / Perfetto trace JSON here")
    ap.add_argument("--width", type=int, default=120)
    a = ap.parse_args(argv)
    recs = load(a.directory, a.iteration)
    lines, bubbles = chart(recs, a.width)
    any_rec = next(iter(recs.values()))
    print(f"iteration {any_rec['iteration']}  schedule {any_rec.get('schedule', '?')}  pp {any_rec.get('pp', len(recs))}")
    print("\n".join(lines))
    print("bubble fraction per rank: " + "  ".join(f"{r}: {b:.3f}" for r, b in sorted(bubbles.items())))
    if a.trace:
        with open(a.trace, "w") as f:
            json.dump(chrome_trace(recs), f)
    return lines, bubbles


if __name__ == "__main__":
    main()
