"""Cluster view over per-node dumps: which nodes fail and why, which node differs from the majority software
fingerprint, which GPU is the slow outlier (primus/tools/preflight/node_smoke/aggregator/{report,summarizers}.py)."""
from __future__ import annotations

import glob
import json
import os
import statistics
from collections import Counter


def load_dumps(dump_dir: str) -> list:
    out = []
    for f in sorted(glob.glob(os.path.join(dump_dir, "*.json"))):
        with open(f) as fh:
            out.append(json.load(fh))
    return out


def summarize_cluster(reports: list, slow_fraction: float = 0.9) -> dict:
    nodes = {r["hostname"]: r["status"] for r in reports}
    digests = Counter(r["collectors"].get("fingerprint", {}).get("digest") for r in reports)
    majority = digests.most_common(1)[0][0] if digests else None
    odd = [r["hostname"] for r in reports if r["collectors"].get("fingerprint", {}).get("digest") != majority]
    reasons = {}
    for r in reports:
        why = [f"{name}: {c.get('status')}" for name, c in r["collectors"].items() if c.get("status") in ("FAIL", "WARN")]
        why += [f"GPU{g['gpu']} {c['check']}: {c.get('error') or c['status']}" for g in r["per_gpu"] for c in g["checks"]
                if c["status"] == "FAIL"]
        if why:
            reasons[r["hostname"]] = why
    # slow outliers: GEMM / HBM of a GPU below `slow_fraction` of the cluster median although above the threshold
    metrics = {"tflops": [], "gbs": []}
    for r in reports:
        for g in r["per_gpu"]:
            for c in g["checks"]:
                if "GEMM" in c["check"] and "tflops" in c:
                    metrics["tflops"].append((r["hostname"], g["gpu"], c["tflops"]))
                if "HBM" in c["check"] and "gbs" in c:
                    metrics["gbs"].append((r["hostname"], g["gpu"], c["gbs"]))
    slow = []
    for key, vals in metrics.items():
        if len(vals) >= 3:
            med = statistics.median(v[2] for v in vals)
            slow += [{"node": h, "gpu": g, "metric": key, "value": v, "median": med} for h, g, v in vals if v < slow_fraction * med]
    return {"nodes": len(reports), "pass": sum(1 for s in nodes.values() if s == "PASS"),
            "warn": sum(1 for s in nodes.values() if s == "WARN"), "fail": sum(1 for s in nodes.values() if s == "FAIL"),
            "failing_nodes": sorted(h for h, s in nodes.items() if s == "FAIL"), "fingerprint_outliers": odd,
            "reasons": reasons, "slow_gpus": slow}


def write_report(summary: dict, path: str) -> None:
    lines = [f"# node smoke: {summary['nodes']} nodes — {summary['pass']} pass, {summary['warn']} warn, {summary['fail']} fail", ""]
    if summary["failing_nodes"]:
        lines.append("exclude: " + ",".join(summary["failing_nodes"]))
    for h, why in sorted(summary["reasons"].items()):
        lines += [f"## {h}"] + [f"- {w}" for w in why]
    if summary["fingerprint_outliers"]:
        lines.append("software fingerprint differs from the majority on: " + ", ".join(summary["fingerprint_outliers"]))
    for s in summary["slow_gpus"]:
        lines.append(f"slow: {s['node']} GPU{s['gpu']} {s['metric']} {s['value']:.0f} (cluster median {s['median']:.0f})")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
