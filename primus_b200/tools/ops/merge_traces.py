"""Merge the per-rank Chrome traces of one profiled window into a single file that a trace viewer shows side by side.

    python -m primus_b200.tools.ops.merge_traces <profiler dir> --output merged.json[.gz]

Every rank's events keep their timestamps; process ids are moved into a block of their own per rank (``rank * 100000 +
pid``) and the process names get a ``rank N`` prefix, so that rows of different ranks neither collide nor interleave.
(The reference concatenates the event lists: tools/profile_trace/merge_trace_file.py:13-30.)"""
from __future__ import annotations

import argparse
import gzip
import json
import sys

from .. import trace_report as TR

PID_BLOCK = 100000


def merge(paths: list[str]) -> dict:
    events = []
    for n, path in enumerate(sorted(paths)):
        rank = TR.rank_of(path)
        rank = n if rank is None else rank
        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "rt") as f:
            doc = json.load(f)
        seen_names = set()
        for e in (doc.get("traceEvents", doc) if isinstance(doc, dict) else doc):
            e = dict(e)
            if isinstance(e.get("pid"), int):
                e["pid"] = rank * PID_BLOCK + e["pid"]
            elif "pid" in e:
                e["pid"] = f"rank {rank} {e['pid']}"
            if e.get("ph") == "M" and e.get("name") == "process_name":
                args = dict(e.get("args") or {})
                args["name"] = f"rank {rank} {args.get('name', '')}".strip()
                e["args"] = args
                seen_names.add(e["pid"])
            events.append(e)
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path", help="directory with the ranks' traces, or one trace file")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    paths = TR.find_traces(args.path)
    if not paths:
        print(f"no trace files under {args.path}", file=sys.stderr)
        return 1
    doc = merge(paths)
    opener = gzip.open if args.output.endswith(".gz") else open
    with opener(args.output, "wt") as f:
        json.dump(doc, f)
    print(f"merged {len(paths)} traces ({len(doc['traceEvents'])} events) into {args.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
