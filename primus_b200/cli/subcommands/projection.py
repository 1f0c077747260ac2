"""``primus projection {memory,performance,both} --config exp.yaml [--hardware b200] [--target-nodes N] ...``

Memory: per-GPU peak (weights, grads, optimizer, activations, logits, workspaces, 5 % margin) against the
HBM size; performance: iteration time, tokens/s/GPU, TFLOP/s/GPU and MFU from the layer model, the collective
model and the pipeline-schedule simulator; ``--benchmark`` times one real layer on the local GPU and uses it
instead of the roofline estimate.  Parallel sizes default to the experiment file and can be overridden
(``--tp --pp --ep --cp --vpp --micro-batch --global-batch --world``)
(primus/cli/subcommands/projection.py:12-97,106-200,240-395 in the reference).
"""
from __future__ import annotations

import json


def register_subcommand(subparsers):
    p = subparsers.add_parser("projection", help="memory / performance projection")
    p.add_argument("suite", choices=["memory", "performance", "both", "tune"])
    p.add_argument("--config", "--exp", dest="config", default=None)
    p.add_argument("--model", default=None, help="model preset name instead of an experiment file")
    p.add_argument("--hardware", default="b200")
    p.add_argument("--target-nodes", type=int, default=None)
    for k in ("world", "tp", "pp", "ep", "cp", "vpp", "micro-batch", "global-batch", "seq", "recompute-layers"):
        p.add_argument(f"--{k}", type=int, default=None)
    p.add_argument("--schedule", default=None)
    p.add_argument("--sync-free-stage", type=int, default=0, help="MoE sync-free stage (0-3): removes host syncs")
    p.add_argument("--comm-overlap", type=float, default=None, help="fraction of layer comm hidden (fused kernels)")
    p.add_argument("--benchmark", action="store_true",
                   help="time one real dense (and MoE) layer on the local GPU and use that instead of the kernel table")
    p.add_argument("--precision", default=None, choices=["bf16", "mxfp8", "tensorwise"],
                   help="kernel table to use (default: the configuration's fp8 recipe, else bf16)")
    p.add_argument("--json", action="store_true")
    p.set_defaults(func=run)


def run_tune(args, overrides):
    """``primus projection tune --model M --world N``: enumerate legal parallel plans, keep those that fit, rank."""
    from ...tools.tuner import search as tuner

    cfg, plan, hw, _, overlap = resolve(args, overrides)
    res = tuner.search(cfg, hw, plan.world, plan.global_batch, plan.seq, top=10, comm_overlap=overlap or 0.7)
    rows = [c.as_dict() for c in res["best"]]
    if args.json:
        print(json.dumps({"enumerated": res["enumerated"], "fit_in_memory": res["fit_in_memory"], "best": rows}))
    else:
        from tabulate import tabulate

        print(f"{res['enumerated']} legal plans, {res['fit_in_memory']} fit in {hw.hbm_gb:.0f} GB")
        print(tabulate(rows, headers="keys"))
        if res["best"]:
            print("\noverrides of the best plan:\n  " + " ".join(res["best"][0].overrides()))
    return res


def resolve(args, overrides):
    from ...core.config.experiment import load_experiment
    from ...core.config.overrides import parse_cli_overrides
    from ...core.config.presets import load_preset
    from ...core.patches import builtin  # noqa: F401
    from ...core.patches.registry import PatchContext, run_patches
    from ...models.config import TransformerConfig
    from ...tools.projection.collective_model import Hardware
    from ...tools.projection.memory import ParallelPlan

    if args.config:
        exp = load_experiment(args.config, parse_cli_overrides(overrides or []))
        params = exp.module("pre_trainer").params
        run_patches("build_args", PatchContext(phase="build_args", params=params, extra={}))
    else:
        params = load_preset(args.model or "llama3.1_8B", "models")
    cfg = TransformerConfig.from_dict(params)
    hw = Hardware.from_yaml(load_preset(args.hardware, "hardware"))
    g = lambda k, d: getattr(args, k.replace("-", "_")) if getattr(args, k.replace("-", "_")) is not None else d  # noqa: E731
    world = g("world", (args.target_nodes or 1) * hw.gpus_per_node)
    plan = ParallelPlan(
        world=world, tp=g("tp", cfg.tensor_model_parallel_size), pp=g("pp", cfg.pipeline_model_parallel_size),
        cp=g("cp", cfg.context_parallel_size), ep=g("ep", cfg.expert_model_parallel_size if cfg.num_experts else 1),
        vpp=g("vpp", cfg.virtual_pipeline_model_parallel_size or 1), micro_batch=g("micro-batch", params.get("micro_batch_size", 1)),
        global_batch=g("global-batch", params.get("global_batch_size", 128)), seq=g("seq", params.get("seq_length", 8192)),
        distributed_optimizer=bool(params.get("use_distributed_optimizer", True)),
        recompute_layers=g("recompute-layers", params.get("recompute_num_layers") or 0),
        sequence_parallel=bool(params.get("sequence_parallel", True)), fused_tp=bool(params.get("tp_comm_overlap", False)))
    sched = args.schedule or params.get("pp_algorithm") or ("interleaved" if plan.vpp > 1 else "1f1b")
    overlap = args.comm_overlap if args.comm_overlap is not None else (0.7 if plan.fused_tp else 0.0)
    return cfg, plan, hw, sched, overlap


def benchmark_layers(cfg, plan):
    """Time forward / backward of one real dense (and one MoE) layer on the local GPU."""
    import torch

    from ...models.gpt import TransformerLayer
    from ...parallel import state as ps
    from ...tools.benchmark.common import time_cuda

    if not torch.cuda.is_available():
        raise RuntimeError("--benchmark needs a GPU")
    ps.initialize_model_parallel()
    from ...ops import gemm as _gemm

    _gemm.set_fp8_recipe(cfg.fp8_recipe if cfg.fp8 else None)   # time the layer in the precision it trains in
    out = {}
    T = plan.micro_batch * plan.seq
    for key, idx in (("dense", next((i for i in range(cfg.num_layers) if not cfg.is_moe_layer(i)), None)),
                     ("moe", next((i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)), None))):
        if idx is None:
            continue
        layer = TransformerLayer(cfg, idx, "cuda", 1)
        from ...ops import fused

        d = cfg.qk_pos_emb_head_dim if cfg.multi_latent_attention else cfg.kv_channels
        cos, sin = fused.rope_tables(plan.seq, d, cfg.rotary_base, "cuda")
        x = torch.randn(T, cfg.hidden_size, device="cuda").bfloat16().requires_grad_()
        r = torch.randn(T, cfg.hidden_size, device="cuda").bfloat16().requires_grad_()
        pos = torch.arange(plan.seq, device="cuda", dtype=torch.int32).repeat(plan.micro_batch) if plan.micro_batch > 1 else None

        def fwd(i):
            with torch.no_grad():
                layer(x, r, (cos, sin, pos), plan.micro_batch)

        def fwdbwd(i):
            o, res = layer(x, r, (cos, sin, pos), plan.micro_batch)
            (o.float().sum() + res.float().sum()).backward()

        tf = time_cuda(fwd, 5, 2)["ms_median"] / 1e3
        tfb = time_cuda(fwdbwd, 5, 2)["ms_median"] / 1e3
        out[key] = (tf, (tfb - tf) * 0.6, (tfb - tf) * 0.4)
        del layer
    return out


def run(args, overrides):
    from ...tools.projection.memory import project_memory
    from ...tools.projection.performance import project_performance

    if args.suite == "tune":
        return run_tune(args, overrides)
    cfg, plan, hw, sched, overlap = resolve(args, overrides)
    errs = plan.validate(cfg)
    if errs:
        raise ValueError("illegal parallel plan: " + "; ".join(errs))
    res = {"model_params_b": cfg.num_parameters() / 1e9, "plan": plan.__dict__, "hardware": hw.name}
    if args.suite in ("memory", "both"):
        mem = project_memory(cfg, plan)
        mem["fits"] = mem["peak_gb"] <= hw.hbm_gb * 1e9 / 2**30 * 1.0186  # 180 GB parts expose 183,359 MiB
        res["memory"] = mem
    if args.suite in ("performance", "both"):
        lt = benchmark_layers(cfg, plan) if args.benchmark else None
        res["performance"] = project_performance(cfg, plan, hw, sched, args.target_nodes, overlap, lt,
                                                 precision=getattr(args, "precision", None))
    if args.json:
        print(json.dumps(res, indent=1, default=str))
    else:
        print(f"model: {res['model_params_b']:.2f} B parameters | world {plan.world} = tp{plan.tp} x pp{plan.pp} x cp{plan.cp} "
              f"x dp{plan.dp} (ep{plan.ep}) | mbs {plan.micro_batch} gbs {plan.global_batch} seq {plan.seq} | {hw.name}")
        if "memory" in res:
            b = res["memory"]["breakdown"]
            print(f"memory  : peak {res['memory']['peak_gb']:.1f} GiB of {hw.hbm_gb * 1e9 / 2**30 * 1.0186:.0f} GiB "
                  f"({'fits' if res['memory']['fits'] else 'DOES NOT FIT'}) = weights {b['weights_gb']:.1f} + grads {b['grads_gb']:.1f} "
                  f"+ optimizer {b['optimizer_gb']:.1f} + activations {b['activations_gb']:.1f} + logits {b['logits_gb']:.1f} "
                  f"+ workspace {b['workspace_gb']:.1f} (+5% margin, +1.5 GiB context)")
        if "performance" in res:
            p = res["performance"]
            print(f"perf    : {p['iteration_ms']:.1f} ms/iter | {p['tokens_per_s_per_gpu']:.0f} tokens/s/GPU | "
                  f"{p['tflops_per_gpu']:.0f} TFLOP/s/GPU | MFU {100 * p['mfu']:.1f}% | schedule {p['schedule']} "
                  f"bubble {100 * p['bubble_fraction']:.1f}%")
            print("          " + " | ".join(f"{k} {v:.2f} ms" if isinstance(v, float) else f"{k} {v}"
                                                 for k, v in p["breakdown_ms"].items()))
    return 0
