"""Configuration search over parallel plans.

For a model and a GPU count the tuner enumerates ``(tp, pp, vpp, ep, cp, micro-batch, recomputed layers,
schedule)``, drops illegal plans (divisibility of heads / layers / experts / batch: ``ParallelPlan.validate``),
drops plans whose projected per-GPU peak memory exceeds the HBM size (5 % margin included), and ranks the rest by
projected tokens/s/GPU (``tools/projection``).  With ``benchmark_top`` > 0 the best candidates can then be timed on
the real machine by the caller (each candidate is returned as the list of CLI overrides that selects it).

This is the deterministic core of the reference's tuning agent (legality checks + memory-aware evaluation + history:
primus/agents/tuning_agent/{legality,evaluator,plan,history}.py); the LLM-driven proposal loop of the reference is
replaced by exhaustive enumeration, which is tractable because the space per model is a few thousand plans.
"""
from __future__ import annotations

import dataclasses
import itertools
import json
from typing import Iterable, Optional

from ..projection.collective_model import Hardware
from ..projection.memory import ParallelPlan, project_memory
from ..projection.performance import project_performance


def _divisors(n: int, upto: int) -> list[int]:
    return [d for d in range(1, upto + 1) if n % d == 0]


@dataclasses.dataclass
class Candidate:
    plan: ParallelPlan
    schedule: str
    peak_gb: float
    tokens_per_s_per_gpu: float
    mfu: float
    iteration_ms: float
    bubble: float
    last_stage_layers: int = 0       # > 0: the depth has no even split and the last stage holds this many layers

    def overrides(self) -> list[str]:
        p = self.plan
        out = [f"--tensor_model_parallel_size={p.tp}", f"--pipeline_model_parallel_size={p.pp}",
               f"--expert_model_parallel_size={p.ep}", f"--context_parallel_size={p.cp}",
               f"--micro_batch_size={p.micro_batch}", f"--global_batch_size={p.global_batch}",
               f"--sequence_parallel={'true' if p.tp > 1 else 'false'}", f"--pp_algorithm={self.schedule}"]
        if p.vpp > 1:
            out.append(f"--virtual_pipeline_model_parallel_size={p.vpp}")
        if self.last_stage_layers:
            out.append(f"--decoder_last_pipeline_num_layers={self.last_stage_layers}")
        if p.recompute_layers:
            # the memory model counts `recompute_layers` layers per stage without saved activations: method "block"
            out += ["--recompute_granularity=full", "--recompute_method=block",
                    f"--recompute_num_layers={p.recompute_layers}"]
        return out

    def as_dict(self) -> dict:
        p = self.plan
        return {"tp": p.tp, "pp": p.pp, "vpp": p.vpp, "ep": p.ep, "cp": p.cp, "dp": p.dp, "micro_batch": p.micro_batch,
                "grad_accum": p.grad_accum, "recompute_layers": p.recompute_layers, "schedule": self.schedule,
                "peak_gb": round(self.peak_gb, 1), "tokens_per_s_per_gpu": round(self.tokens_per_s_per_gpu, 1),
                "mfu": round(self.mfu, 4), "iteration_ms": round(self.iteration_ms, 1), "bubble": round(self.bubble, 4),
                **({"last_stage_layers": self.last_stage_layers} if self.last_stage_layers else {})}


def context_parallel_supported(cfg) -> bool:
    """Context parallelism is built for softmax attention that runs on the flash-attention kernels: not for the
    recurrent / convolution mixers, the DeepSeek-V4 attention, sliding windows, sinks, soft-capped scores, or head sizes
    that fall back to composed operations."""
    from ...ops.attention import kernel_supports

    if any(kind[0] not in (None, "attention") for kind in cfg.layer_kinds):
        return False
    if getattr(cfg, "window_size", None) or getattr(cfg, "softmax_type", "vanilla") != "vanilla" \
            or getattr(cfg, "attn_logit_softcapping", None):
        return False
    if cfg.multi_latent_attention:
        return kernel_supports(cfg.qk_head_dim + cfg.qk_pos_emb_head_dim, cfg.v_head_dim)
    return kernel_supports(cfg.kv_channels, cfg.kv_channels)


def enumerate_plans(cfg, world: int, global_batch: int, seq: int, gpus_per_node: int = 8, max_micro_batch: int = 8,
                    fused_tp: bool = True) -> Iterable[tuple[ParallelPlan, str]]:
    L = cfg.num_layers
    cp_ok = context_parallel_supported(cfg)
    for tp, pp, cp in itertools.product(_divisors(world, gpus_per_node), _divisors(world, min(world, L)),
                                        _divisors(world, gpus_per_node)):
        if world % (tp * pp * cp) or (cp > 1 and not cp_ok):
            continue
        if cfg.num_experts and tp > 1:
            continue  # the projection has no model of MoE layers under tensor parallelism: such plans are not proposed
        dp = world // (tp * pp * cp)
        eps = [e for e in _divisors(cfg.num_experts, tp * cp * dp) if (tp * cp * dp) % e == 0] if cfg.num_experts else [1]
        for ep in eps:
            vpps = [1] + ([v for v in (2, 4) if L % (pp * v) == 0] if pp > 1 else [])
            for vpp in vpps:
                schedules = ["1f1b"] if pp == 1 else (["interleaved"] if vpp > 1 else ["1f1b", "zerobubble"])
                for mb in (m for m in (1, 2, 4, 8) if m <= max_micro_batch):
                    if global_batch % (mb * dp):
                        continue
                    for rec in (0, L // (pp * vpp)):
                        plan = ParallelPlan(world=world, tp=tp, pp=pp, cp=cp, ep=ep, vpp=vpp, micro_batch=mb,
                                            global_batch=global_batch, seq=seq, recompute_layers=rec,
                                            sequence_parallel=tp > 1, fused_tp=fused_tp and tp > 1)
                        if plan.validate(cfg):
                            continue
                        for s in schedules:
                            yield plan, s


def search(cfg, hw: Hardware, world: int, global_batch: int, seq: int, top: int = 10, hbm_gb: Optional[float] = None,
           comm_overlap: float = 0.7, **enum_kw) -> dict:
    hbm = hbm_gb or hw.hbm_gb
    seen = fits = 0
    cands: list[Candidate] = []
    for plan, schedule in enumerate_plans(cfg, world, global_batch, seq, hw.gpus_per_node, **enum_kw):
        seen += 1
        mem = project_memory(cfg, plan)
        if mem["peak_gb"] > hbm:
            continue
        fits += 1
        try:
            perf = project_performance(cfg, plan, hw, schedule, comm_overlap=comm_overlap if plan.fused_tp else 0.0)
        except Exception:  # noqa: BLE001  (a schedule that cannot be built for this (pp, micro-batch count))
            continue
        uneven = cfg.num_layers % (plan.pp * plan.vpp) != 0
        cands.append(Candidate(plan, schedule, mem["peak_gb"], perf["tokens_per_s_per_gpu"], perf["mfu"],
                               perf["iteration_ms"], perf["bubble_fraction"],
                               plan.last_stage_layers(cfg.num_layers) if uneven else 0))
    cands.sort(key=lambda c: -c.tokens_per_s_per_gpu)
    return {"enumerated": seen, "fit_in_memory": fits, "best": cands[:top]}


def main(argv=None):
    import argparse

    from ...core.config.presets import load_preset
    from ...models.config import TransformerConfig

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="llama3.1_70B")
    ap.add_argument("--hardware", default="b200")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--top", type=int, default=8)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    cfg = TransformerConfig.from_dict(load_preset(a.model, "models"))
    hw = Hardware.from_yaml(load_preset(a.hardware, "hardware"))
    res = search(cfg, hw, a.world, a.global_batch, a.seq, a.top)
    rows = [c.as_dict() for c in res["best"]]
    if a.json:
        print(json.dumps({"enumerated": res["enumerated"], "fit_in_memory": res["fit_in_memory"], "best": rows}))
    else:
        from tabulate import tabulate

        print(f"{a.model} on {a.world} x {hw.name}: {res['enumerated']} legal plans, {res['fit_in_memory']} fit in "
              f"{hw.hbm_gb:.0f} GB")
        print(tabulate(rows, headers="keys"))
        if res["best"]:
            print("\noverrides of the best plan:\n  " + " ".join(res["best"][0].overrides()))
    return res


if __name__ == "__main__":
    main()
