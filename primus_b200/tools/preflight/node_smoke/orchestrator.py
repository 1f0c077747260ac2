"""Runs the collectors in this process and one child process per GPU (with a time limit each), folds everything into a
node verdict and optionally dumps it as ``<dump_dir>/<hostname>.json`` for the cluster aggregator.
(primus/tools/preflight/node_smoke/orchestrator.py:31-247 in the reference.)"""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time
from typing import Callable, Optional

from .collectors import collect_all


def _spawn_per_gpu(gpu: int, tier: int, timeout_s: float, extra: list, spawn: Optional[Callable] = None) -> dict:
    cmd = [sys.executable, "-m", "primus_b200.tools.preflight.node_smoke.per_gpu", "--gpu", str(gpu), "--tier", str(tier), *extra]
    if spawn is not None:
        return spawn(cmd, timeout_s)
    t0 = time.time()
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"gpu": gpu, "checks": [{"check": "per-gpu run", "status": "FAIL", "error": f"no result within {timeout_s:.0f} s"}]}
    for line in p.stdout.splitlines():
        if line.startswith("NODE_SMOKE_RESULT "):
            res = json.loads(line[len("NODE_SMOKE_RESULT "):])
            res["seconds"] = time.time() - t0
            return res
    return {"gpu": gpu, "checks": [{"check": "per-gpu run", "status": "FAIL", "error": f"exit {p.returncode}: {p.stderr[-300:]}"}]}


def node_status_from(collectors: dict, per_gpu: list) -> str:
    """FAIL if any collector or GPU check failed, WARN if only warnings, else PASS."""
    sts = [c.get("status", "PASS") for c in collectors.values()] + [c["status"] for g in per_gpu for c in g["checks"]]
    return "FAIL" if "FAIL" in sts else ("WARN" if "WARN" in sts else "PASS")


def run_node_smoke(tier: int = 2, gpus: Optional[list] = None, timeout_s: float = 300.0, dump_dir: Optional[str] = None,
                   nic_selector: str = "", extra_args: Optional[list] = None, spawn: Optional[Callable] = None,
                   run: Optional[Callable] = None, clean_dump: bool = False) -> dict:
    kw = {"run": run} if run is not None else {}
    coll = collect_all(nic_selector=nic_selector, **kw)
    if gpus is None:
        try:
            import torch

            gpus = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
        except Exception:  # noqa: BLE001
            gpus = []
    per_gpu = [_spawn_per_gpu(g, tier, timeout_s, list(extra_args or []), spawn) for g in gpus] if tier >= 1 else []
    rep = {"hostname": socket.gethostname(), "time": time.strftime("%Y-%m-%d %H:%M:%S"), "tier": tier, "collectors": coll,
           "per_gpu": per_gpu}
    rep["status"] = node_status_from(coll, per_gpu)
    if dump_dir:
        os.makedirs(dump_dir, exist_ok=True)
        if clean_dump:
            for f in os.listdir(dump_dir):
                if f.endswith(".json"):
                    os.remove(os.path.join(dump_dir, f))
        with open(os.path.join(dump_dir, rep["hostname"] + ".json"), "w") as f:
            json.dump(rep, f, indent=1, default=str)
    return rep
