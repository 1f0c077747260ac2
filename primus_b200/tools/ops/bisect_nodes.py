"""Find the nodes that make a multi-node check fail by bisection of the node list.

    python -m primus_b200.tools.ops.bisect_nodes --nodes n01,n02,...|--nodelist "n[01-32]" \\
        --command 'srun -w {nodes} -N {count} primus-cli direct -- preflight --perf-test' [--timeout 900] [--jobs 2]

The command template is run on the whole list first; while a set fails it is split into halves that are tested (in
parallel, ``--jobs``) until single nodes remain: those are the suspects.  A run that exceeds ``--timeout`` counts as a
failure of kind HANG (its process group is terminated).  When both halves of a failing set pass, the failure needs the
larger scale (or the pair) and the set is reported as such instead of being split further.  Results go to stdout as a
table and, with ``--output``, to a JSON file.  (Role of the reference's tools/preflight_bisect/bisect.py: Slurm node-list
bisection around its preflight performance test; the command here is any template.)"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass, field


@dataclass
class Trial:
    nodes: list
    status: str            # PASS | FAIL | HANG
    seconds: float
    returncode: int = 0


@dataclass
class Outcome:
    suspects: list = field(default_factory=list)        # single nodes that fail on their own
    scale_only: list = field(default_factory=list)      # sets that fail although both halves pass
    trials: list = field(default_factory=list)


def expand_nodelist(spec: str) -> list:
    """``a,b[01-03,7],c`` -> names (the common bracket form; anything more exotic: pass --nodes)."""
    out, depth, cur = [], 0, ""
    for ch in spec + ",":
        if ch == "," and depth == 0:
            if cur:
                out.append(cur)
            cur = ""
            continue
        depth += ch == "["
        depth -= ch == "]"
        cur += ch
    names = []
    for item in out:
        if "[" not in item:
            names.append(item)
            continue
        head, rest = item.split("[", 1)
        body, tail = rest.rsplit("]", 1)
        for part in body.split(","):
            if "-" in part:
                a, b = part.split("-")
                names += [f"{head}{i:0{len(a)}d}{tail}" for i in range(int(a), int(b) + 1)]
            else:
                names.append(f"{head}{part}{tail}")
    return names


def run_trial(template: str, nodes: list, timeout: float, env=None) -> Trial:
    cmd = template.format(nodes=",".join(nodes), count=len(nodes), first=nodes[0])
    t0 = time.time()
    proc = subprocess.Popen(cmd, shell=True, start_new_session=True, stdout=subprocess.DEVNULL,
                            stderr=subprocess.DEVNULL, env=env)
    try:
        rc = proc.wait(timeout=timeout)
        return Trial(list(nodes), "PASS" if rc == 0 else "FAIL", time.time() - t0, rc)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(proc.pid, signal.SIGTERM)          # exactly the group this trial started
            proc.wait(timeout=10)
        except (ProcessLookupError, subprocess.TimeoutExpired):
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass
        return Trial(list(nodes), "HANG", time.time() - t0, -1)


def bisect(nodes: list, template: str, timeout: float = 900.0, jobs: int = 2, min_size: int = 1, runner=run_trial) -> Outcome:
    out = Outcome()

    def test(ns):
        t = runner(template, ns, timeout)
        out.trials.append(t)
        return t.status == "PASS"

    def descend(ns):
        if len(ns) <= min_size:
            out.suspects.extend(ns)
            return
        half = len(ns) // 2
        halves = [ns[:half], ns[half:]]
        with ThreadPoolExecutor(max_workers=max(1, min(jobs, 2))) as pool:
            ok = list(pool.map(test, halves))
        if all(ok):
            out.scale_only.append(list(ns))
            return
        for h, passed in zip(halves, ok):
            if not passed:
                descend(h)

    if not test(nodes):
        descend(nodes)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--nodes", help="comma-separated node names")
    g.add_argument("--nodelist", help="bracket form, e.g. node[01-32]")
    ap.add_argument("--command", required=True, help="template with {nodes} {count} {first}")
    ap.add_argument("--timeout", type=float, default=900.0)
    ap.add_argument("--jobs", type=int, default=2)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    nodes = args.nodes.split(",") if args.nodes else expand_nodelist(args.nodelist)
    res = bisect(nodes, args.command, args.timeout, args.jobs)
    for t in res.trials:
        print(f"{t.status:5s} {t.seconds:8.1f}s  {len(t.nodes):4d} nodes  {t.nodes[0]}..{t.nodes[-1]}")
    print("suspects:", ", ".join(res.suspects) or "none")
    for s in res.scale_only:
        print(f"fails only at scale: {len(s)} nodes {s[0]}..{s[-1]} (both halves pass)")
    if args.output:
        with open(args.output, "w") as f:
            json.dump({"suspects": res.suspects, "scale_only": res.scale_only,
                       "trials": [asdict(t) for t in res.trials]}, f, indent=1)
    return 1 if res.suspects or res.scale_only else 0


if __name__ == "__main__":
    sys.exit(main())
