"""``primus node_smoke``: acceptance test of one node — read-only collectors (clocks, kernel log, software
fingerprint, GPU health counters, foreign GPU processes, host limits, NICs / RDMA ports, NVLink topology, tooling) and,
per GPU in a child process with a time limit, tier 1 (a tiny MXFP8 training step through the sm_100a kernels) and
tier 2 (GEMM / HBM / peer-copy thresholds).  ``--dump-dir`` writes ``<hostname>.json``; ``--aggregate DIR`` turns the
dumps of many nodes into a cluster summary with an exclude list.
(primus/tools/preflight/node_smoke/* in the reference; the launcher runs it with ``--single``.)"""
from __future__ import annotations

import json


def register_subcommand(subparsers):
    p = subparsers.add_parser("node_smoke", help="per-node smoke test")
    p.add_argument("--tier", type=int, default=2, choices=[0, 1, 2], help="0: collectors only, 1: + training step, 2: + perf")
    p.add_argument("--no-perf", action="store_true", help="same as --tier 1")
    p.add_argument("--gpus", default=None, help="comma-separated GPU indices (default: all)")
    p.add_argument("--timeout", type=float, default=300.0, help="seconds per GPU")
    p.add_argument("--nic-selector", default="", help="NCCL_IB_HCA-style selector of the NICs that must be up")
    p.add_argument("--dump-dir", default=None)
    p.add_argument("--clean-dump", action="store_true")
    p.add_argument("--aggregate", default=None, metavar="DIR", help="summarise the node dumps in DIR instead of testing")
    p.add_argument("--report", default=None, help="with --aggregate: write a Markdown report here")
    p.add_argument("--gemm-tflops", type=float, default=None)
    p.add_argument("--hbm-gbs", type=float, default=None)
    p.add_argument("--p2p-gbs", type=float, default=None)
    p.add_argument("--json", action="store_true")
    p.set_defaults(func=run)


def run(args, unknown):
    from ...tools.preflight import node_smoke as ns
    from ...tools.preflight.node_smoke.aggregator import load_dumps

    if args.aggregate:
        summary = ns.summarize_cluster(load_dumps(args.aggregate))
        if args.report:
            ns.write_report(summary, args.report)
        print(json.dumps(summary, indent=1, default=str))
        return 1 if summary["fail"] else 0
    extra = []
    for flag, v in (("--gemm-tflops", args.gemm_tflops), ("--hbm-gbs", args.hbm_gbs), ("--p2p-gbs", args.p2p_gbs)):
        if v is not None:
            extra += [flag, str(v)]
    tier = 1 if args.no_perf and args.tier > 1 else args.tier
    gpus = [int(x) for x in args.gpus.split(",")] if args.gpus else None
    rep = ns.run_node_smoke(tier=tier, gpus=gpus, timeout_s=args.timeout, dump_dir=args.dump_dir,
                            nic_selector=args.nic_selector, extra_args=extra, clean_dump=args.clean_dump)
    if args.json:
        print(json.dumps(rep, indent=1, default=str))
    else:
        print(f"node {rep['hostname']}: {rep['status']}")
        for name, c in rep["collectors"].items():
            detail = "; ".join(c.get("problems") or []) or c.get("reason", "")
            print(f"  [{c.get('status')}] {name}{': ' + detail if detail else ''}")
        for g in rep["per_gpu"]:
            for c in g["checks"]:
                facts = {k: (round(v, 1) if isinstance(v, float) else v) for k, v in c.items() if k not in ("check", "status")}
                print(f"  [{c['status']}] GPU{g['gpu']} {c['check']}: {facts}")
    return 1 if rep["status"] == "FAIL" else 0
