"""``primus preflight [--no-perf] [--json] [--report FILE]``: host / GPU / network inventory and performance
checks against thresholds, one PASS/FAIL line per check (primus/cli/subcommands/preflight.py in the reference)."""
from __future__ import annotations

import json


def register_subcommand(subparsers):
    p = subparsers.add_parser("preflight", help="cluster / node preflight checks")
    p.add_argument("--no-perf", action="store_true")
    p.add_argument("--json", action="store_true")
    p.add_argument("--report", default=None)
    p.add_argument("--gemm-tflops", type=float, default=None)
    p.add_argument("--hbm-gbs", type=float, default=None)
    p.add_argument("--allreduce-gbs", type=float, default=None)
    p.set_defaults(func=run)


def run(args, unknown):
    from ...parallel import state as ps
    from ...tools.preflight.checks import run_preflight

    ps.init_distributed()
    th = {k: v for k, v in (("gemm_tflops", args.gemm_tflops), ("hbm_gbs", args.hbm_gbs),
                             ("allreduce_busbw_gbs", args.allreduce_gbs)) if v is not None}
    rep = run_preflight(perf=not args.no_perf, thresholds=th)
    import os

    if int(os.environ.get("RANK", "0")) == 0:
        if args.json:
            print(json.dumps(rep, indent=1, default=str))
        else:
            h, g = rep["host"], rep["gpu"]
            print(f"host {h['hostname']} | {h['cpus']} CPUs | {h['mem_gib']:.0f} GiB | GPUs {g.get('count', 0)} "
                  f"{(g['devices'][0]['name'] if g['devices'] else '')}")
            for c in rep["checks"]:
                print(f"  [{c['status']}] {c['check']}: {c['detail']}")
        if args.report:
            with open(args.report, "w") as f:
                json.dump(rep, f, indent=1, default=str)
    return 1 if any(c["status"] == "FAIL" for c in rep["checks"]) else 0
