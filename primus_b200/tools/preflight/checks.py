"""Preflight and node-smoke checks: host / GPU / interconnect inventory and short performance tests
with pass thresholds (primus/tools/preflight/*, primus/tools/preflight/node_smoke/* in the reference;
default thresholds there: GEMM >= 600 TFLOPS, HBM >= 2000 GB/s, node-local all-reduce >= 100 GB/s,
docs_deprecated/node-smoke-test-instruction.md:120 — the B200 defaults below are scaled to this hardware).

Everything here only *reads* device state (nvidia-smi queries, NVML through torch); nothing changes clocks,
power limits or modes.
"""
from __future__ import annotations

import os
import platform
import shutil
import socket
import subprocess
import time

DEFAULT_THRESHOLDS = {"gemm_tflops": 1100.0, "hbm_gbs": 5000.0, "allreduce_busbw_gbs": 400.0, "p2p_gbs": 500.0}


def _run(cmd: list[str], timeout: float = 20.0) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout).stdout.strip()
    except (OSError, subprocess.TimeoutExpired):
        return ""


def host_info() -> dict:
    mem_kb = 0
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal"):
                    mem_kb = int(line.split()[1])
    except OSError:
        pass
    return {"hostname": socket.gethostname(), "kernel": platform.release(), "python": platform.python_version(),
            "cpus": os.cpu_count(), "mem_gib": mem_kb / 2**20, "numactl": bool(shutil.which("numactl")),
            "slurm_job": os.environ.get("SLURM_JOB_ID"), "cwd_free_gib": shutil.disk_usage(".").free / 2**30}


def gpu_info() -> dict:
    import torch

    out = {"cuda_available": torch.cuda.is_available(), "torch": torch.__version__, "devices": []}
    if not torch.cuda.is_available():
        return out
    q = "index,name,memory.total,memory.used,clocks.sm,clocks.max.sm,power.limit,temperature.gpu,ecc.errors.uncorrected.volatile.total"
    for line in _run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader"]).splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) >= 8:
            out["devices"].append(dict(zip(q.split(","), f)))
    out["count"] = torch.cuda.device_count()
    out["capability"] = list(torch.cuda.get_device_capability(0))
    out["is_sm100"] = out["capability"][0] == 10
    out["driver"] = _run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"]).splitlines()[:1]
    out["throttle_reasons"] = _run(["nvidia-smi", "--query-gpu=clocks_event_reasons.active", "--format=csv,noheader"]).splitlines()
    return out


def network_info() -> dict:
    nics = []
    try:
        for n in sorted(os.listdir("/sys/class/net")):
            st = ""
            try:
                with open(f"/sys/class/net/{n}/operstate") as f:
                    st = f.read().strip()
            except OSError:
                pass
            nics.append({"name": n, "state": st})
    except OSError:
        pass
    ib = sorted(os.listdir("/sys/class/infiniband")) if os.path.isdir("/sys/class/infiniband") else []
    topo = _run(["nvidia-smi", "topo", "-m"])
    return {"nics": nics, "infiniband": ib, "nvlink_topology": topo.splitlines()[:12],
            "nccl_env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")}}


def native_lib_check() -> dict:
    from ...ops import _lib

    ok = _lib.available()
    return {"library": str(_lib.lib_path()), "present": ok}


def p2p_check() -> dict:
    import torch

    if not torch.cuda.is_available():
        return {"skipped": "no GPU"}
    from ...parallel.symm_mem import probe_p2p

    return probe_p2p()


def perf_gemm(n: int = 8192, iters: int = 20) -> dict:
    import torch

    from ...ops import gemm as G

    a = torch.randn(n, n, device="cuda").bfloat16()
    b = torch.randn(n, n, device="cuda").bfloat16()
    for _ in range(3):
        G.gemm(a, b, fp8=False)          # the bf16 kernel whatever fp8 recipe the process has selected
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); G.gemm(a, b, fp8=False); e.record(); torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return {"n": n, "tflops_median": 2.0 * n ** 3 / ts[len(ts) // 2] / 1e9, "tflops_best": 2.0 * n ** 3 / ts[0] / 1e9}


def perf_hbm(gib: float = 2.0, iters: int = 10) -> dict:
    import torch

    n = int(gib * 2**30 / 2)
    a = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_()
    b = torch.empty_like(a)
    best = 1e9
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); b.copy_(a); e.record(); torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e))
    return {"gbs": 2.0 * n * 2 / best / 1e6}


def perf_allreduce(mib: int = 256, iters: int = 10) -> dict:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {"skipped": "single rank"}
    p = dist.get_world_size()
    x = torch.ones(mib * 2**20 // 2, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        dist.all_reduce(x)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); s.record()
    for _ in range(iters):
        dist.all_reduce(x)
    e.record(); torch.cuda.synchronize()
    ms = s.elapsed_time(e) / iters
    t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
    alg = x.numel() * 2 / float(t) / 1e6
    return {"bytes": x.numel() * 2, "busbw_gbs": alg * 2 * (p - 1) / p, "ranks": p}


def _time_collective(fn, iters: int = 8, warmup: int = 2) -> float:
    """Device time per call in ms, maximum over ranks (the slowest rank defines a collective's time)."""
    import torch
    import torch.distributed as dist

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def perf_intra_node_comm(sizes_mib=(1, 64, 256)) -> dict:
    """All-reduce / all-gather / reduce-scatter / all-to-all bus bandwidth inside the node for a few sizes
    (primus/tools/preflight/intra_node_comm.py in the reference)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {"skipped": "single rank"}
    p = dist.get_world_size()
    rows = []
    for mib in sizes_mib:
        n = mib * 2**20 // 2 // p * p
        x = torch.ones(n, dtype=torch.bfloat16, device="cuda")
        shard = torch.empty(n // p, dtype=torch.bfloat16, device="cuda")
        y = torch.empty_like(x)
        by = n * 2
        for name, fn, factor in (
                ("all_reduce", lambda: dist.all_reduce(x), 2 * (p - 1) / p),
                ("all_gather", lambda: dist.all_gather_into_tensor(y, shard), (p - 1) / p),
                ("reduce_scatter", lambda: dist.reduce_scatter_tensor(shard, x), (p - 1) / p),
                ("all_to_all", lambda: dist.all_to_all_single(y, x), (p - 1) / p)):
            ms = _time_collective(fn)
            rows.append({"op": name, "mib": mib, "ms": ms, "busbw_gbs": by / ms / 1e6 * factor})
    return {"ranks": p, "rows": rows}


def perf_ring_p2p(mib: int = 256) -> dict:
    """Every rank sends to its right neighbour and receives from its left one at the same time (the traffic pattern of
    pipeline parallelism and ring attention); reports the slowest hop.  Works inside a node and across nodes
    (primus/tools/preflight/inter_node_ring_p2p.py, inter_node_comm_p2p.py in the reference)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {"skipped": "single rank"}
    p, r = dist.get_world_size(), dist.get_rank()
    n = mib * 2**20 // 2
    send = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    recv = torch.empty_like(send)

    def step():
        ops = [dist.P2POp(dist.isend, send, (r + 1) % p), dist.P2POp(dist.irecv, recv, (r - 1) % p)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    ms = _time_collective(step)
    return {"ranks": p, "mib": mib, "ms": ms, "gbs_per_direction": n * 2 / ms / 1e6}


def perf_pairwise_p2p(mib: int = 128, max_pairs: int = 64) -> dict:
    """Unidirectional bandwidth of every (source, destination) rank pair, one pair at a time: finds the one bad link
    that a ring or an all-reduce number hides in an average."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {"skipped": "single rank"}
    p, r = dist.get_world_size(), dist.get_rank()
    n = mib * 2**20 // 2
    buf = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    out, pairs = [], [(a, b) for a in range(p) for b in range(p) if a != b][:max_pairs]
    for a, b in pairs:
        def step(a=a, b=b):
            if r == a:
                dist.send(buf, b)
            elif r == b:
                dist.recv(buf, a)
        ms = _time_collective(step, iters=4, warmup=1)
        out.append({"src": a, "dst": b, "gbs": n * 2 / ms / 1e6})
    worst = min(out, key=lambda x: x["gbs"])
    return {"ranks": p, "mib": mib, "pairs": out, "worst": worst, "median_gbs": sorted(x["gbs"] for x in out)[len(out) // 2]}


def network_inventory() -> dict:
    """NICs with speed / MTU, RDMA devices with port state and rate, default route, NCCL-related environment
    (primus/tools/preflight/network/{network_basic,network_standard,network_full}.py in the reference)."""
    from .node_smoke.collectors import collect_nic_status

    nic = collect_nic_status(selector=os.environ.get("NCCL_IB_HCA", ""))
    route = _run(["ip", "route", "show", "default"]).splitlines()[:2]
    return {"nics": nic["nics"], "rdma_ports": nic["rdma_ports"], "down": nic["down"], "default_route": route,
            "master_addr": os.environ.get("MASTER_ADDR"), "nnodes": os.environ.get("NNODES") or os.environ.get("SLURM_NNODES"),
            "nccl_env": {k: v for k, v in os.environ.items() if k.startswith(("NCCL_", "UCX_", "GLOO_"))}}


def run_preflight(perf: bool = True, thresholds: dict | None = None) -> dict:
    import torch

    th = dict(DEFAULT_THRESHOLDS, **(thresholds or {}))
    rep = {"time": time.strftime("%Y-%m-%d %H:%M:%S"), "host": host_info(), "gpu": gpu_info(), "network": network_info(),
           "network_inventory": network_inventory(),
           "native": native_lib_check(), "checks": []}

    def add(name, ok, detail):
        rep["checks"].append({"check": name, "status": "PASS" if ok else ("SKIP" if ok is None else "FAIL"), "detail": detail})

    add("native library built", rep["native"]["present"], rep["native"]["library"])
    if not torch.cuda.is_available():
        add("gpu present", None, "no CUDA device: performance checks skipped")
        return rep
    add("sm_100 device", rep["gpu"].get("is_sm100", False), str(rep["gpu"].get("capability")))
    p2p = p2p_check()
    rep["p2p"] = p2p
    if p2p.get("num_devices", 1) > 1:
        add("peer access between all GPUs", p2p["all_p2p"], f"{p2p['num_devices']} devices")
    if perf and rep["native"]["present"] and rep["gpu"].get("is_sm100"):
        g = perf_gemm()
        add("square bf16 GEMM", g["tflops_median"] >= th["gemm_tflops"], f"{g['tflops_median']:.0f} TFLOP/s (>= {th['gemm_tflops']:.0f})")
        h = perf_hbm()
        add("HBM copy bandwidth", h["gbs"] >= th["hbm_gbs"], f"{h['gbs']:.0f} GB/s (>= {th['hbm_gbs']:.0f})")
        ar = perf_allreduce()
        if "busbw_gbs" in ar:
            add("node-local all-reduce", ar["busbw_gbs"] >= th["allreduce_busbw_gbs"],
                f"{ar['busbw_gbs']:.0f} GB/s bus bandwidth (>= {th['allreduce_busbw_gbs']:.0f})")
        rep["perf"] = {"gemm": g, "hbm": h, "allreduce": ar}
        if "busbw_gbs" in ar:
            ring = perf_ring_p2p()
            add("ring send / receive (every rank to its neighbour)", ring["gbs_per_direction"] >= th["p2p_gbs"],
                f"{ring['gbs_per_direction']:.0f} GB/s per direction (>= {th['p2p_gbs']:.0f})")
            pair = perf_pairwise_p2p()
            add("slowest rank pair", pair["worst"]["gbs"] >= 0.8 * pair["median_gbs"],
                f"{pair['worst']['src']} -> {pair['worst']['dst']}: {pair['worst']['gbs']:.0f} GB/s (median {pair['median_gbs']:.0f})")
            rep["perf"].update(ring=ring, pairwise=pair, intra_node=perf_intra_node_comm())
    return rep
