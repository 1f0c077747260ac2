"""Recipe book: one pre-training experiment file per model preset and precision, laid out for B200 nodes.

The reference ships a hand-written recipe per model and accelerator (examples/megatron/configs/MI300X, MI325X, MI355X:
about a hundred files each, sized for those parts' memory).  Here the layout of a recipe is not written by hand: for every
model preset the plan search of the tuner (``tools/tuner/search.py``: legality, projected peak memory against 180 GB,
projected tokens/s) is run on 1, 2, 4 ... nodes of 8 GPUs until a plan fits, and the best plan becomes the recipe's
parallel sizes, micro-batch, schedule and recompute setting (among plans projected within 5 % of the best, the one with
the least model parallelism).  The projection that chose them is recorded in the header of
each file, so a recipe can be regenerated (or checked) after the model of the machine changes:

    python -m primus_b200.tools.recipes --out examples/configs/b200                  # every model, BF16 and MXFP8
    python -m primus_b200.tools.recipes --models llama3.1_70B qwen3_32B --precisions bf16 --print

``index.md`` in the output directory lists every recipe with its node count, layout and projection, and the models for
which no plan fits the largest node count tried.
"""
from __future__ import annotations

import argparse
import os
from typing import Iterable, Optional

from ..core.config.presets import CONFIG_ROOT, load_preset
from ..models.config import TransformerConfig
from .projection.collective_model import Hardware
from .tuner.search import Candidate, search

PRECISIONS = {"bf16": "BF16", "mxfp8": "MXFP8"}
# presets that are bases of other presets, unit-test sized, or shortened variants of a listed model
SKIP_SUFFIXES = ("_base", "_tiny")
SKIP_NAMES = {"language_model", "moe_proxy_single_node", "qwen3_235B_A22B_4layer", "kimi_k3_curve", "kimi_k3_8L_official"}


def model_names() -> list[str]:
    names = sorted(f[:-5] for f in os.listdir(CONFIG_ROOT / "models") if f.endswith(".yaml"))
    return [n for n in names if not n.endswith(SKIP_SUFFIXES) and n not in SKIP_NAMES]


def sequence_length(cfg) -> int:
    return int(min(getattr(cfg, "max_position_embeddings", None) or 4096, 8192))


def find_plan(cfg, hw: Hardware, max_nodes: int = 32, seq: Optional[int] = None) -> tuple[Optional[Candidate], int, int]:
    """Smallest power-of-two node count on which some plan fits, and the best plan there: (candidate, world, batch)."""
    seq = seq or sequence_length(cfg)
    nodes = 1
    while nodes <= max_nodes:
        world = nodes * hw.gpus_per_node
        batch = max(64, 8 * world)
        res = search(cfg, hw, world, batch, seq, top=400)
        if res["best"]:
            return simplest_near_best(res["best"]), world, batch
        nodes *= 2
    return None, 0, 0


def simplest_near_best(cands: list, tolerance: float = 0.05) -> Candidate:
    """The projection cannot tell plans apart that it puts within a few per cent of one another (measured steps of the
    data-parallel variants differ by less): among those the recipe takes the plan with the least model parallelism,
    then no virtual stages, no recomputation, the smaller micro-batch, and only then the projected speed."""
    best = cands[0].tokens_per_s_per_gpu
    near = [c for c in cands if c.tokens_per_s_per_gpu >= best * (1.0 - tolerance)]
    return min(near, key=lambda c: (c.plan.tp * c.plan.pp * c.plan.cp, c.plan.vpp, c.plan.recompute_layers,
                                    c.plan.micro_batch, -c.tokens_per_s_per_gpu))


def recipe_name(model: str, precision: str) -> str:
    return f"{model}-{PRECISIONS[precision]}-pretrain"


def render(model: str, precision: str, cand: Candidate, world: int, hw: Hardware) -> str:
    p = cand.plan
    name = recipe_name(model, precision)
    lines = [
        f"# {model}, {PRECISIONS[precision]}, {world // hw.gpus_per_node} node(s) x {hw.gpus_per_node} {hw.name}: layout chosen by the plan search",
        f"# (python -m primus_b200.tools.recipes --models {model} --precisions {precision}).  Projection: peak",
        f"# {cand.peak_gb:.0f} GB per GPU, {cand.tokens_per_s_per_gpu:.0f} tokens/s/GPU, MFU {cand.mfu:.2f}, iteration {cand.iteration_ms:.0f} ms,",
        f"# pipeline bubble {cand.bubble:.3f}; data-parallel size {p.dp}, {p.grad_accum} micro-batches per step.",
        "work_group: ${PRIMUS_TEAM:b200}",
        "user_name: ${PRIMUS_USER:root}",
        f"exp_name: ${{PRIMUS_EXP_NAME:{name}}}",
        "workspace: ${PRIMUS_WORKSPACE:./output}",
        "",
        "modules:",
        "  pre_trainer:",
        "    framework: primus_b200",
        "    config: pre_trainer.yaml",
        f"    model: {model}.yaml",
        "    overrides:",
    ]
    ov: list[tuple[str, object]] = [
        ("train_iters", "${PRIMUS_TRAIN_ITERS:50}"), ("mock_data", "true"), ("log_interval", 1),
        ("lr", "3.0e-4"), ("min_lr", "3.0e-5"), ("lr_warmup_iters", 10), ("lr_decay_style", "cosine"),
        ("weight_decay", 0.1), ("clip_grad", 1.0),
        ("use_distributed_optimizer", "true"), ("overlap_grad_reduce", "true"), ("overlap_param_gather", "true"),
        ("seq_length", p.seq), ("micro_batch_size", p.micro_batch), ("global_batch_size", p.global_batch),
    ]
    # every parallel size is written, also when it is 1: a model preset may carry a default of its own
    ov += [("tensor_model_parallel_size", p.tp), ("sequence_parallel", "true" if p.tp > 1 else "false")]
    if p.tp > 1:
        ov.append(("tp_comm_overlap", "true"))
    ov.append(("pipeline_model_parallel_size", p.pp))
    if p.pp > 1:
        ov.append(("pipeline_schedule", cand.schedule))
        if p.vpp > 1:
            ov.append(("virtual_pipeline_model_parallel_size", p.vpp))
        if cand.last_stage_layers:
            ov.append(("decoder_last_pipeline_num_layers", cand.last_stage_layers))
    ov.append(("context_parallel_size", p.cp))
    if p.cp > 1:
        ov.append(("cp_comm_type", "p2p"))
    ov.append(("expert_model_parallel_size", p.ep))
    if p.recompute_layers:
        ov += [("recompute_granularity", "full"), ("recompute_method", "block"), ("recompute_num_layers", p.recompute_layers)]
    if precision == "mxfp8":
        ov += [("fp8", "e4m3"), ("fp8_recipe", "mxfp8"), ("grad_reduce_in_bf16", "true")]
    lines += [f"      {k}: {v}" for k, v in ov]
    return "\n".join(lines) + "\n"


def build(models: Iterable[str], precisions: Iterable[str], hw: Hardware, max_nodes: int):
    """Yields (model, precision, candidate or None, world)."""
    for model in models:
        base = load_preset(model, "models")
        for precision in precisions:
            d = dict(base)
            if precision == "mxfp8":
                d.update(fp8="e4m3", fp8_recipe="mxfp8")
            else:
                d.update(fp8=None)
            cfg = TransformerConfig.from_dict(d)
            cand, world, _ = find_plan(cfg, hw, max_nodes)
            yield model, precision, cand, world


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default=None, help="directory for the recipe files and index.md")
    ap.add_argument("--models", nargs="*", default=None, help="model presets (default: every one)")
    ap.add_argument("--precisions", nargs="*", default=list(PRECISIONS), choices=list(PRECISIONS))
    ap.add_argument("--hardware", default="b200")
    ap.add_argument("--max-nodes", type=int, default=32)
    ap.add_argument("--print", action="store_true", help="write the recipes to standard output")
    a = ap.parse_args(argv)
    hw = Hardware.from_yaml(load_preset(a.hardware, "hardware"))
    rows, missing = [], []
    if a.out:
        os.makedirs(a.out, exist_ok=True)
    for model, precision, cand, world in build(a.models or model_names(), a.precisions, hw, a.max_nodes):
        if cand is None:
            missing.append((model, precision))
            continue
        text = render(model, precision, cand, world, hw)
        fname = recipe_name(model, precision) + ".yaml"
        if a.out:
            with open(os.path.join(a.out, fname), "w") as f:
                f.write(text)
        if a.print or not a.out:
            print(f"# ---- {fname}\n{text}")
        p = cand.plan
        rows.append((fname, world // hw.gpus_per_node, f"tp{p.tp} pp{p.pp}" + (f"x{p.vpp}" if p.vpp > 1 else "")
                     + f" cp{p.cp} ep{p.ep} dp{p.dp} mb{p.micro_batch}", cand.schedule if p.pp > 1 else "-",
                     f"{cand.peak_gb:.0f}", f"{cand.tokens_per_s_per_gpu:.0f}", f"{cand.mfu:.2f}"))
    if a.out:
        with open(os.path.join(a.out, "index.md"), "w") as f:
            f.write(f"# Pre-training recipes for {hw.name} ({hw.gpus_per_node} GPUs per node, {hw.hbm_gb:.0f} GB each)\n\n"
                    "Generated by `python -m primus_b200.tools.recipes`; the figures are projections of the analytic model "
                    "(`primus_b200/tools/projection`), not measurements.\n\n"
                    "| recipe | nodes | layout | schedule | peak GB | tokens/s/GPU | MFU |\n|---|---|---|---|---|---|---|\n")
            for r in rows:
                f.write("| " + " | ".join(str(x) for x in r) + " |\n")
            if missing:
                f.write(f"\nNo plan fits on {a.max_nodes} nodes or fewer (the search proposes no tensor parallelism for "
                        "mixture-of-experts layers): " + ", ".join(f"{m} ({PRECISIONS[q]})" for m, q in missing) + ".\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
