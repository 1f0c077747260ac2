"""Kernel-level report from profiler traces: where the GPU time of the profiled steps went.

    python -m primus_b200.tools.trace_report <trace.json | directory of *.pt.trace.json> [--output report.md] [--top 25]

Reads the Chrome-trace files ``engine/observability.py::StepProfiler`` writes (torch.profiler exports; ``.json`` or
``.json.gz``), takes the GPU kernel and memcpy events, and produces per rank

* a category table (GEMM, attention, quantisation, normalisation / element-wise, MoE routing / permutation, optimizer,
  collectives, copies, other): launches, total time, share of the GPU-busy time,
* the top kernels by total time,
* how much of the communication time ran concurrently with compute kernels (interval overlap), and the GPU idle share of
  the traced window.

With several ranks a summary row per rank shows skew.  The trainer writes this report after the profiled window when
``generate_tracelens_report`` is set, into ``<profiler dir>/trace_report/``, and hands the files to the metric sinks
as artifacts.  It plays the role of the trace-analysis reports the reference generates with TraceLens
(``generate_tracelens_report`` / ``mlflow_upload_tracelens_report`` in
primus/configs/modules/megatron/primus_megatron_module.yaml:15-39), with this package's kernel names.
"""
from __future__ import annotations

import argparse
import glob
import gzip
import json
import os
import re
import sys
from typing import Optional

CATEGORIES = [
    ("collectives", re.compile(r"nccl|all_?reduce|all_?gather|reduce_?scatter|all_?to_?all|dp_reduce_scatter|dp_adamw_allgather|"
                               r"odc_|symm_barrier|gemm_tp_fused|moe_fused", re.I)),
    ("attention", re.compile(r"flash_attn|fmha|attention|sdpa", re.I)),
    ("gemm", re.compile(r"gemm|cutlass|cublas|sm\d+_xmma|gemv|matmul", re.I)),
    ("quantisation", re.compile(r"quant|amax|cast_fp8|mxfp", re.I)),
    ("moe routing", re.compile(r"router|permut|gather_rows|combine_rows|moe_plan|topk", re.I)),
    ("optimizer", re.compile(r"adamw|multi_tensor|sumsq|clip_coef|muon|sgd", re.I)),
    ("norm / elementwise", re.compile(r"rmsnorm|rope|swiglu|geglu|cross_entropy|softcap|embedding|elementwise|vectorized|"
                                      r"reduce_kernel|dropout", re.I)),
    ("copies", re.compile(r"memcpy|memset|copy", re.I)),
]


def categorize(name: str) -> str:
    for cat, rx in CATEGORIES:
        if rx.search(name):
            return cat
    return "other"


def load_trace(path: str) -> list[dict]:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        doc = json.load(f)
    events = doc.get("traceEvents", doc) if isinstance(doc, dict) else doc
    out = []
    for e in events:
        if e.get("ph") != "X":
            continue
        cat = str(e.get("cat", "")).lower()
        if cat in ("kernel", "gpu_memcpy", "gpu_memset") or cat.startswith("gpu_"):
            out.append({"name": e.get("name", "?"), "ts": float(e["ts"]), "dur": float(e.get("dur", 0.0)),
                        "stream": (e.get("args") or {}).get("stream", e.get("tid"))})
    return out


def _union(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    out: list[list[float]] = []
    for a, b in sorted(intervals):
        if out and a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return [(a, b) for a, b in out]


def _length(intervals) -> float:
    return sum(b - a for a, b in intervals)


def _intersect(xs, ys) -> float:
    i = j = 0
    tot = 0.0
    while i < len(xs) and j < len(ys):
        lo, hi = max(xs[i][0], ys[j][0]), min(xs[i][1], ys[j][1])
        if hi > lo:
            tot += hi - lo
        if xs[i][1] < ys[j][1]:
            i += 1
        else:
            j += 1
    return tot


def analyse(events: list[dict], top: int = 25) -> dict:
    """Category table, top kernels, overlap and idle figures of one rank's GPU events (times in microseconds)."""
    if not events:
        return {"categories": [], "top_kernels": [], "summary": {"gpu_busy_us": 0.0, "window_us": 0.0}}
    by_cat: dict = {}
    by_name: dict = {}
    comm, comp = [], []
    for e in events:
        c = categorize(e["name"])
        a = by_cat.setdefault(c, [0, 0.0])
        a[0] += 1
        a[1] += e["dur"]
        n = by_name.setdefault(e["name"], [0, 0.0, c])
        n[0] += 1
        n[1] += e["dur"]
        (comm if c == "collectives" else comp).append((e["ts"], e["ts"] + e["dur"]))
    busy = _union(comm + comp)
    busy_us = _length(busy)
    window = max(b for _, b in busy) - min(a for a, _ in busy)
    comm_u, comp_u = _union(comm), _union(comp)
    comm_us = _length(comm_u)
    hidden = _intersect(comm_u, comp_u)
    cats = [{"category": c, "launches": n, "total_ms": round(t / 1e3, 3), "share_of_busy": round(t / max(busy_us, 1e-9), 4)}
            for c, (n, t) in sorted(by_cat.items(), key=lambda kv: -kv[1][1])]
    tops = [{"kernel": k[:96], "category": c, "launches": n, "total_ms": round(t / 1e3, 3), "mean_us": round(t / n, 2)}
            for k, (n, t, c) in sorted(by_name.items(), key=lambda kv: -kv[1][1])[:top]]
    return {"categories": cats, "top_kernels": tops,
            "summary": {"window_us": window, "gpu_busy_us": busy_us, "idle_share": round(1.0 - busy_us / max(window, 1e-9), 4),
                        "comm_us": comm_us, "comm_hidden_share": round(hidden / comm_us, 4) if comm_us else None,
                        "kernels": len(events)}}


def rank_of(path: str) -> Optional[int]:
    m = re.search(r"rank\[?(\d+)\]?", os.path.basename(path))
    return int(m.group(1)) if m else None


def write_report(paths: list[str], out_dir: str, fmt: str = "md", top: int = 25, ranks=None) -> list[str]:
    """One report file per trace plus ``summary.<fmt>`` over all of them; returns the files written."""
    from .report import write_records

    os.makedirs(out_dir, exist_ok=True)
    written, summary = [], []
    for p in sorted(paths):
        r = rank_of(p)
        if ranks is not None and r is not None and r not in ranks:
            continue
        res = analyse(load_trace(p), top)
        base = os.path.join(out_dir, f"trace_report_rank{r if r is not None else len(written)}")
        s = res["summary"]
        if fmt == "md":
            f = base + ".md"
            write_records(f, res["categories"], preamble=f"# GPU time by category ({os.path.basename(p)})\n\nwindow "
                          f"{s['window_us'] / 1e3:.2f} ms, busy {s['gpu_busy_us'] / 1e3:.2f} ms, idle share {s.get('idle_share')}, "
                          f"communication hidden behind compute: {s.get('comm_hidden_share')}")
            with open(f, "a") as fh:
                fh.write("\n## Top kernels\n\n")
            write_records(f, res["top_kernels"], append=True)
            with open(f) as fh:      # the appended table needs its own header row in Markdown
                txt = fh.read()
            hdr = "| " + " | ".join(res["top_kernels"][0].keys()) + " |\n|" + "|".join("---" for _ in res["top_kernels"][0]) + "|\n" \
                if res["top_kernels"] else ""
            txt = txt.replace("## Top kernels\n\n", "## Top kernels\n\n" + hdr)
            with open(f, "w") as fh:
                fh.write(txt)
            written.append(f)
        else:
            for part in ("categories", "top_kernels"):
                f = f"{base}_{part}.{fmt}"
                write_records(f, res[part])
                written.append(f)
        summary.append({"rank": r, "trace": os.path.basename(p), "window_ms": round(s["window_us"] / 1e3, 3),
                        "busy_ms": round(s["gpu_busy_us"] / 1e3, 3), "idle_share": s.get("idle_share"),
                        "comm_ms": round(s.get("comm_us", 0.0) / 1e3, 3), "comm_hidden_share": s.get("comm_hidden_share"),
                        **{c["category"] + "_ms": c["total_ms"] for c in res["categories"]}})
    if summary:
        f = os.path.join(out_dir, f"summary.{fmt}")
        write_records(f, summary, preamble="# Trace report summary (one row per rank)" if fmt == "md" else None)
        written.append(f)
    return written


def find_traces(path: str) -> list[str]:
    if os.path.isdir(path):
        return sorted(glob.glob(os.path.join(path, "*.pt.trace.json")) + glob.glob(os.path.join(path, "*.pt.trace.json.gz")))
    return [path]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path", help="a trace file or a directory of *.pt.trace.json[.gz]")
    ap.add_argument("--output", default=None, help="output directory (default: <trace dir>/trace_report)")
    ap.add_argument("--format", default="md", choices=["md", "csv", "tsv", "jsonl"])
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--ranks", type=int, nargs="*", default=None)
    a = ap.parse_args(argv)
    traces = find_traces(a.path)
    if not traces:
        print(f"no trace files under {a.path}", file=sys.stderr)
        return 2
    out = a.output or os.path.join(os.path.dirname(os.path.abspath(traces[0])), "trace_report")
    for f in write_report(traces, out, a.format, a.top, a.ranks):
        print(f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
