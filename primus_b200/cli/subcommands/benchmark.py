"""``primus benchmark {gemm,gemm-dense,gemm-deepseek,attention,nccl,strided-allgather,moe,elementwise} [options]``
(primus/cli/subcommands/benchmark.py:8-50 in the reference; ``rccl`` is accepted as an alias of ``nccl``)."""
from __future__ import annotations

import argparse


def register_subcommand(subparsers):
    p = subparsers.add_parser("benchmark", help="micro-benchmarks", add_help=True)
    p.add_argument("suite", choices=["gemm", "gemm-dense", "gemm-deepseek", "attention", "nccl", "rccl", "strided-allgather", "moe", "elementwise"])
    p.add_argument("rest", nargs=argparse.REMAINDER, help="options of the suite (see --help of the suite)")
    p.set_defaults(func=run)


def run(args, unknown):
    rest = list(args.rest) + list(unknown or [])
    if args.suite == "gemm":
        from ...tools.benchmark import gemm_bench

        gemm_bench.main(rest)
    elif args.suite == "gemm-dense":
        from ...tools.benchmark import gemm_bench

        gemm_bench.main((["--suite", "llama3.1_8B"] if "--suite" not in rest else []) + rest)
    elif args.suite == "gemm-deepseek":
        from ...tools.benchmark import gemm_bench

        gemm_bench.main((["--suite", "deepseek_v2_lite"] if "--suite" not in rest else []) + rest)
    elif args.suite == "attention":
        from ...tools.benchmark import attention_bench

        attention_bench.main(rest)
    elif args.suite == "elementwise":
        from ...tools.benchmark import elementwise_bench

        elementwise_bench.main(rest)
    elif args.suite == "moe":
        from ...tools.benchmark import moe_bench

        moe_bench.main(rest)
    elif args.suite in ("nccl", "rccl"):
        from ...tools.benchmark import nccl_bench

        nccl_bench.main(rest)
    else:
        from ...tools.benchmark import nccl_bench

        nccl_bench.main(["--ops", "all_gather"] + rest)
    return 0
