"""Collective micro-benchmark over torch.distributed (NCCL on GPUs, gloo on CPU).

Ops: all_reduce, broadcast, all_gather(into_tensor), reduce_scatter(tensor), alltoall(single, equal splits),
send_recv; sizes 1 KiB .. 128 MiB (or the per-model all-to-all sizes ``mbs*seq*topk x hidden``).  Every
iteration is timed on the device and reduced with MAX over ranks; algorithm / bus bandwidth use the usual
factors ``2(p-1)/p`` (all-reduce) and ``(p-1)/p`` (the others); each op is checked for correctness once.
(primus/tools/benchmark/rccl_bench.py:154-383, benchmark/kernel/rccl/benchmark_all2all.py:16-114 in the reference.)

    torchrun --nproc-per-node 8 -m primus_b200.tools.benchmark.nccl_bench --ops all_reduce,alltoall
"""
from __future__ import annotations

import argparse
import statistics
import time

import torch
import torch.distributed as dist

A2A_MODELS = {  # hidden, seq, top-k
    "deepseek-v2-lite": (2048, 4096, 6), "deepseek-v2": (5120, 4096, 6), "deepseek-v3": (7168, 4096, 8),
    "mixtral-8x7B": (4096, 4096, 2), "qwen3-235B": (4096, 4096, 8), "qwen3-30B-A3B": (2048, 4096, 8),
}
OPS = ("all_reduce", "broadcast", "all_gather", "reduce_scatter", "alltoall", "send_recv")


def bus_factor(op: str, p: int) -> float:
    if op == "all_reduce":
        return 2.0 * (p - 1) / p
    if op in ("all_gather", "reduce_scatter", "alltoall"):
        return (p - 1) / p
    return 1.0


def _run(op, x, out, rank, world):
    if op == "all_reduce":
        dist.all_reduce(x)
    elif op == "broadcast":
        dist.broadcast(x, 0)
    elif op == "all_gather":
        dist.all_gather_into_tensor(out, x[: x.numel() // world])
    elif op == "reduce_scatter":
        dist.reduce_scatter_tensor(out[: x.numel() // world], x)
    elif op == "alltoall":
        dist.all_to_all_single(out, x)
    elif op == "send_recv":
        peer = rank ^ 1
        if peer < world:
            ops = [dist.P2POp(dist.isend, x, peer), dist.P2POp(dist.irecv, out, peer)]
            for r in dist.batch_isend_irecv(ops):
                r.wait()


def check(op, rank, world, device) -> bool:
    n = 1024 * world
    x = torch.full((n,), float(rank + 1), device=device)
    out = torch.zeros(n, device=device)
    if op == "alltoall":
        x = torch.arange(n, device=device, dtype=torch.float32) + rank * n
    _run(op, x, out, rank, world)
    s = world * (world + 1) / 2
    if op == "all_reduce":
        return bool((x == s).all())
    if op == "broadcast":
        return bool((x == 1).all())
    if op == "all_gather":
        exp = torch.arange(1, world + 1, device=device, dtype=torch.float32).repeat_interleave(n // world)
        return bool((out == exp).all())
    if op == "reduce_scatter":
        return bool((out[: n // world] == s).all())
    if op == "alltoall":
        c = n // world
        exp = torch.cat([torch.arange(rank * c, (rank + 1) * c, device=device, dtype=torch.float32) + r * n
                         for r in range(world)])
        return bool((out == exp).all())
    return True


def bench(op, nbytes, rank, world, device, iters, warmup, dtype=torch.bfloat16):
    es = torch.tensor([], dtype=dtype).element_size()
    n = max(world, nbytes // es // world * world)
    x = torch.ones(n, dtype=dtype, device=device)
    out = torch.empty(n, dtype=dtype, device=device)
    times = []
    for i in range(warmup + iters):
        dist.barrier()
        if device.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _run(op, x, out, rank, world)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
        else:
            t0 = time.perf_counter()
            _run(op, x, out, rank, world)
            ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # per-iteration rank-max
        if i >= warmup:
            times.append(float(t))
    times.sort()
    med = statistics.median(times)
    size = n * es
    algbw = size / med / 1e6
    return {"op": op, "bytes": size, "ms_p50": med, "ms_p95": times[min(len(times) - 1, int(0.95 * len(times)))],
            "algbw_GB/s": algbw, "busbw_GB/s": algbw * bus_factor(op, world)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ops", default=",".join(OPS[:5]))
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=128 * 1024 * 1024)
    ap.add_argument("--a2a-model", default=None, choices=sorted(A2A_MODELS))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from ...parallel import state as ps

    ps.init_distributed()
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1, init_method="tcp://127.0.0.1:29599")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    rows = []
    for op in a.ops.split(","):
        ok = check(op, rank, world, device)
        sizes = []
        if op == "alltoall" and a.a2a_model:
            h, s, k = A2A_MODELS[a.a2a_model]
            sizes = [s * k * h * 2]
        else:
            b = a.min_bytes
            while b <= a.max_bytes:
                sizes.append(b)
                b *= 4
        for nb in sizes:
            r = bench(op, nb, rank, world, device, a.iters, a.warmup,
                      torch.bfloat16 if device.type == "cuda" else torch.float32)
            r["correct"] = ok
            rows.append(r)
    if rank == 0:
        from .common import emit

        emit(rows, a.output, f"collectives, {world} ranks")
    dist.barrier()
    return rows


if __name__ == "__main__":
    main()
