"""Read-only collectors of one node's state.  Every collector returns ``{"status": PASS|WARN|FAIL|SKIP, ...facts}``
and takes an optional ``run(cmd) -> str`` so that tests can feed recorded tool output.  Nothing here changes a
setting of the host or of a GPU (no clock, power, persistence, MIG or ECC calls; only queries).

Counterparts in the reference (primus/tools/preflight/node_smoke/collectors/): clock.py, dmesg.py, fingerprint.py,
gpu_low_level.py (amd-smi metrics -> here nvidia-smi), gpu_processes.py, host_limits.py, nics.py, tooling.py,
xgmi.py (-> NVLink topology and link state)."""
from __future__ import annotations

import hashlib
import os
import platform
import re
import resource
import shutil
import socket
import subprocess
import time
from typing import Callable, Optional

Run = Callable[[list], str]


def _run(cmd: list, timeout: float = 20.0) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout).stdout
    except (OSError, subprocess.TimeoutExpired):
        return ""


def collect_clock_state(run: Run = _run) -> dict:
    """Wall clock sanity (NTP-synchronised?) and GPU clocks now vs their maximum.  A GPU idling far below its maximum
    clock is normal; a GPU whose *application clock setting* differs from the maximum hints at a leftover clock lock."""
    out = {"status": "PASS", "epoch": time.time(), "timedatectl_synced": None, "gpus": []}
    td = run(["timedatectl", "show", "-p", "NTPSynchronized", "--value"]).strip()
    if td:
        out["timedatectl_synced"] = td == "yes"
        if td != "yes":
            out["status"] = "WARN"
    q = "index,clocks.sm,clocks.max.sm,clocks.applications.graphics,clocks_event_reasons.active"
    for line in run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits"]).splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 5:
            continue
        g = {"index": f[0], "sm_mhz": f[1], "sm_max_mhz": f[2], "app_clock_mhz": f[3], "reasons": f[4]}
        try:
            if f[3] not in ("", "[N/A]", "N/A") and float(f[3]) < 0.9 * float(f[2]):
                g["locked_low"] = True
                out["status"] = "WARN"
        except ValueError:
            pass
        out["gpus"].append(g)
    return out


_DMESG_PATTERNS = (("xid", re.compile(r"NVRM: Xid \(.*?\): (\d+)")), ("nvlink", re.compile(r"NVLink.*(error|fatal)", re.I)),
                   ("ecc", re.compile(r"(uncorrectable|double.bit) .*ecc", re.I)), ("oom", re.compile(r"Out of memory: Kill")),
                   ("pcie", re.compile(r"PCIe Bus Error.*(Fatal|Uncorrect)", re.I)), ("fallen", re.compile(r"GPU has fallen off the bus")))


def collect_dmesg_errors(run: Run = _run, window_minutes: int = 15) -> dict:
    """Kernel-log lines of the last minutes that point at GPU / link / memory faults (driver Xid events, NVLink
    errors, uncorrectable ECC, the OOM killer, fatal PCIe errors)."""
    text = run(["dmesg", "--since", f"-{window_minutes}min", "--ctime"]) or run(["dmesg", "--ctime"])
    if not text:
        return {"status": "SKIP", "reason": "dmesg not readable"}
    hits: dict = {}
    for line in text.splitlines():
        for name, pat in _DMESG_PATTERNS:
            m = pat.search(line)
            if m:
                hits.setdefault(name, []).append(line.strip()[-200:])
    xids = sorted({int(x) for l in hits.get("xid", []) for x in re.findall(r"Xid \(.*?\): (\d+)", l)})
    return {"status": "FAIL" if hits else "PASS", "matches": {k: v[-5:] for k, v in hits.items()}, "xids": xids,
            "window_minutes": window_minutes}


def collect_node_fingerprint(run: Run = _run) -> dict:
    """What has to be equal on every node of a job: driver, CUDA / NCCL / torch versions, kernel, GPU model and count."""
    fp = {"hostname": socket.gethostname(), "kernel": platform.release(), "python": platform.python_version()}
    try:
        import torch

        fp.update(torch=torch.__version__, cuda=torch.version.cuda,
                  nccl=".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None)
    except Exception:  # noqa: BLE001
        pass
    lines = run(["nvidia-smi", "--query-gpu=name,driver_version,vbios_version,memory.total", "--format=csv,noheader"]).splitlines()
    fp["gpus"] = [l.strip() for l in lines]
    fp["gpu_count"] = len(lines)
    key = "|".join(str(fp.get(k)) for k in ("kernel", "torch", "cuda", "nccl")) + "|" + "|".join(sorted(set(fp["gpus"])))
    fp["digest"] = hashlib.sha256(key.encode()).hexdigest()[:16]
    fp["status"] = "PASS" if len(set(fp["gpus"])) <= 1 else "WARN"      # mixed GPU models / VBIOS in one node
    return fp


def collect_gpu_metrics(run: Run = _run) -> dict:
    """Low-level per-GPU health: temperature, power against the limit, memory in use, ECC and retired-page counters,
    PCIe link generation / width against their maxima."""
    q = ("index,temperature.gpu,power.draw,power.limit,memory.used,memory.total,ecc.errors.uncorrected.volatile.total,"
         "ecc.errors.uncorrected.aggregate.total,retired_pages.pending,pcie.link.gen.current,pcie.link.gen.max,"
         "pcie.link.width.current,pcie.link.width.max")
    gpus, status = [], "PASS"
    for line in run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits"]).splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 13:
            continue
        g = dict(zip(q.split(","), f))
        problems = []
        num = lambda s: float(s) if re.fullmatch(r"-?\d+(\.\d+)?", s or "") else None  # noqa: E731
        if (num(g["temperature.gpu"]) or 0) >= 85:
            problems.append("hot")
        if (num(g["ecc.errors.uncorrected.volatile.total"]) or 0) > 0:
            problems.append("uncorrected ECC errors")
        if g["retired_pages.pending"].lower() in ("yes", "1"):
            problems.append("page retirement pending (needs a reset)")
        if num(g["pcie.link.width.current"]) and num(g["pcie.link.width.max"]) and \
                num(g["pcie.link.width.current"]) < num(g["pcie.link.width.max"]):
            problems.append("PCIe link narrower than its maximum")
        if (num(g["memory.used"]) or 0) > 0.1 * (num(g["memory.total"]) or 1):
            problems.append("memory already in use")
        g["problems"] = problems
        if problems:
            status = "FAIL" if any("ECC" in p or "retirement" in p for p in problems) else "WARN"
        gpus.append(g)
    return {"status": status if gpus else "SKIP", "gpus": gpus}


def collect_gpu_processes(run: Run = _run, self_pid: Optional[int] = None) -> dict:
    """Compute processes that already hold a GPU (a leftover job makes every benchmark on this node meaningless)."""
    self_pid = os.getpid() if self_pid is None else self_pid
    procs = []
    for line in run(["nvidia-smi", "--query-compute-apps=pid,process_name,used_memory,gpu_uuid", "--format=csv,noheader"]).splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) >= 3 and f[0].isdigit():
            pid = int(f[0])
            name = f[1]
            if name in ("", "[Not Found]", "-"):
                try:
                    with open(f"/proc/{pid}/comm") as fh:
                        name = fh.read().strip()
                except OSError:
                    name = "?"
            procs.append({"pid": pid, "name": name, "used_memory": f[2], "gpu": f[3] if len(f) > 3 else "", "self": pid == self_pid})
    foreign = [p for p in procs if not p["self"]]
    return {"status": "WARN" if foreign else "PASS", "processes": procs, "foreign": len(foreign)}


def collect_host_limits(ulimit_l_min_gb: float = 64.0, shm_min_gb: float = 8.0) -> dict:
    """Limits that break multi-GPU jobs when too small: locked memory (pinned buffers, RDMA registration), open files,
    the size of /dev/shm (NCCL's shared-memory transport and data-loader workers)."""
    soft_l, _ = resource.getrlimit(resource.RLIMIT_MEMLOCK)
    soft_n, _ = resource.getrlimit(resource.RLIMIT_NOFILE)
    memlock_gb = float("inf") if soft_l == resource.RLIM_INFINITY else soft_l / 2**30
    try:
        shm_gb = shutil.disk_usage("/dev/shm").total / 2**30
    except OSError:
        shm_gb = 0.0
    problems = []
    if memlock_gb < ulimit_l_min_gb:
        problems.append(f"ulimit -l is {memlock_gb:.1f} GiB (< {ulimit_l_min_gb:.0f})")
    if shm_gb < shm_min_gb:
        problems.append(f"/dev/shm is {shm_gb:.1f} GiB (< {shm_min_gb:.0f})")
    if soft_n < 4096:
        problems.append(f"ulimit -n is {soft_n} (< 4096)")
    return {"status": "WARN" if problems else "PASS", "memlock_gib": memlock_gb, "nofile": soft_n, "shm_gib": shm_gb,
            "problems": problems}


def collect_nic_status(run: Run = _run, selector: str = "", sys_net: str = "/sys/class/net",
                       sys_ib: str = "/sys/class/infiniband") -> dict:
    """Network interfaces and RDMA ports.  ``selector`` follows NCCL's ``NCCL_IB_HCA`` / ``NCCL_SOCKET_IFNAME`` syntax
    (comma-separated prefixes, ``^`` excludes, ``=`` exact): every selected device must be up / ACTIVE."""
    exclude = selector.startswith("^")
    names = [s for s in selector.lstrip("^").split(",") if s]

    def selected(n: str) -> bool:
        if not names:
            return True
        hit = any(n == s[1:] if s.startswith("=") else n.startswith(s.split(":")[0]) for s in names)
        return hit != exclude

    nics, ports = [], []
    try:
        for n in sorted(os.listdir(sys_net)):
            def rd(f, n=n):
                try:
                    with open(os.path.join(sys_net, n, f)) as fh:
                        return fh.read().strip()
                except OSError:
                    return ""
            nics.append({"name": n, "state": rd("operstate"), "mtu": rd("mtu"), "speed_mbps": rd("speed"), "selected": selected(n)})
    except OSError:
        pass
    if os.path.isdir(sys_ib):
        for dev in sorted(os.listdir(sys_ib)):
            pdir = os.path.join(sys_ib, dev, "ports")
            for port in sorted(os.listdir(pdir)) if os.path.isdir(pdir) else []:
                def rd(f, dev=dev, port=port):
                    try:
                        with open(os.path.join(pdir, port, f)) as fh:
                            return fh.read().strip()
                    except OSError:
                        return ""
                ports.append({"device": dev, "port": port, "state": rd("state"), "rate": rd("rate"),
                              "link_layer": rd("link_layer"), "selected": selected(dev)})
    down = [p for p in ports if p["selected"] and "ACTIVE" not in p["state"]]
    # plain network interfaces are only judged when the selector names them (an exclusion list of RDMA devices says
    # nothing about which Ethernet interfaces a job uses)
    down += [n for n in nics if names and not exclude and n["selected"] and n["state"] not in ("up", "unknown")]
    return {"status": "FAIL" if down else "PASS", "nics": nics, "rdma_ports": ports, "down": down, "selector": selector}


def collect_tooling_inventory(run: Run = _run) -> dict:
    """Which diagnostic tools exist on the node (a missing one explains a SKIP elsewhere in the report)."""
    tools = ["nvidia-smi", "nvcc", "ncu", "numactl", "ibstat", "ibv_devinfo", "lspci", "dmesg", "timedatectl", "ethtool"]
    found = {t: shutil.which(t) for t in tools}
    return {"status": "PASS" if found["nvidia-smi"] else "WARN", "tools": found}


def collect_nvlink_topology(run: Run = _run) -> dict:
    """GPU-to-GPU connectivity matrix and per-link state.  On an HGX B200 node every pair must be connected through
    NVSwitch (``NV18``); a ``PHB`` / ``SYS`` / ``NODE`` entry between two GPUs means traffic falls back to PCIe."""
    topo = run(["nvidia-smi", "topo", "-m"])
    rows, bad = [], []
    for line in topo.splitlines():
        if re.match(r"^GPU\d+\s", line):
            cells = line.split()
            rows.append(cells)
    n = len(rows)
    for r in rows:
        for j, c in enumerate(r[1:1 + n]):
            if c != "X" and not c.startswith("NV"):
                bad.append((r[0], f"GPU{j}", c))
    links = run(["nvidia-smi", "nvlink", "--status"])
    inactive = [l.strip() for l in links.splitlines() if re.search(r"Link \d+:", l) and "inactive" in l.lower()]
    status = "SKIP" if not rows else ("FAIL" if bad or inactive else "PASS")
    return {"status": status, "gpus": n, "non_nvlink_pairs": bad, "inactive_links": inactive[:16], "matrix": [" ".join(r) for r in rows]}


COLLECTORS = {
    "clock": collect_clock_state, "dmesg": collect_dmesg_errors, "fingerprint": collect_node_fingerprint,
    "gpu_metrics": collect_gpu_metrics, "gpu_processes": collect_gpu_processes, "nvlink": collect_nvlink_topology,
    "tooling": collect_tooling_inventory,
}


def collect_all(run: Run = _run, nic_selector: str = "", ulimit_l_min_gb: float = 64.0, shm_min_gb: float = 8.0) -> dict:
    out = {name: fn(run) for name, fn in COLLECTORS.items()}
    out["host_limits"] = collect_host_limits(ulimit_l_min_gb, shm_min_gb)
    out["nics"] = collect_nic_status(run, nic_selector or os.environ.get("NCCL_IB_HCA", ""))
    return out
