"""Timing helpers shared by the micro-benchmarks: CUDA-event timing after warm-up, with rotating input
buffers larger than L2 so that repeated iterations do not measure a warm cache
(the reference rotates >= 2 GiB of buffers: primus/tools/benchmark/gemm_bench.py:16,58-75)."""
from __future__ import annotations

import json
import statistics

import torch

L2_BYTES = 126 * 1024 * 1024


def rotating_count(bytes_per_set: int, target_bytes: int = 2 * L2_BYTES) -> int:
    return max(2, -(-target_bytes // max(bytes_per_set, 1)))


def time_cuda(fn, iters: int = 20, warmup: int = 5, per_iter_events: bool = True) -> dict:
    """fn(i) is called with the iteration index (use it to pick a rotating buffer)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (a, b) in enumerate(evs):
        a.record()
        fn(i)
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return {"ms_median": statistics.median(ts), "ms_min": ts[0], "ms_p95": ts[min(len(ts) - 1, int(0.95 * len(ts)))],
            "iters": iters}


def emit(rows: list[dict], output: str | None = None, title: str = ""):
    from tabulate import tabulate

    if rows:
        print(f"\n== {title} ==" if title else "")
        print(tabulate(rows, headers="keys", floatfmt=".3f"))
    if output and output.lower().endswith(".json"):
        with open(output, "w") as f:
            json.dump(rows, f, indent=1)
    elif output:          # .md / .csv / .tsv / .jsonl (optionally .gz): the table writer picks the format
        from ..report import write_records

        write_records(output, rows, preamble=f"## {title}" if title else None)
