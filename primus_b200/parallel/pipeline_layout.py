"""Assignment of transformer layers to pipeline (and virtual-pipeline) stages.

Default is Megatron's even split: with ``pp`` ranks and ``vpp`` model chunks per rank, chunk ``v`` of rank
``r`` owns layers ``[(v*pp + r) * n, (v*pp + r + 1) * n)`` with ``n = num_layers / (pp*vpp)``.
A layout string such as ``"Ett|tttt|tttL"`` (E = embedding, t = transformer layer, L = loss / output
layer, ``|`` = stage boundary) gives uneven splits — the format of the reference's
``pipeline_model_parallel_layout`` (primus/backends/megatron/core/transformer/pipeline_parallel_layer_layout.py,
docs/04-technical-guides/mega-moe.md:250) — and ``decoder_pipeline_manual_split_list`` gives per-stage counts
(primus/configs/modules/megatron/primus_megatron_module.yaml:83).
"""
from __future__ import annotations

from typing import Optional, Sequence


def layers_for_stage(num_layers: int, pp: int, pp_rank: int, vpp: Optional[int] = None,
                     vp_stage: Optional[int] = None, layout: Optional[str] = None,
                     manual_split: Optional[Sequence[int]] = None) -> list[int]:
    vpp = vpp or 1
    vp_stage = vp_stage or 0
    stage = vp_stage * pp + pp_rank
    n_stages = pp * vpp
    if layout:
        counts = parse_layout(layout, n_stages)["layers"]
    elif manual_split:
        counts = list(manual_split)
        assert len(counts) == n_stages and sum(counts) == num_layers
    else:
        assert num_layers % n_stages == 0, f"{num_layers} layers do not split evenly over {n_stages} stages"
        counts = [num_layers // n_stages] * n_stages
    assert sum(counts) == num_layers, f"layout assigns {sum(counts)} layers, model has {num_layers}"
    start = sum(counts[:stage])
    return list(range(start, start + counts[stage]))


def parse_layout(layout: str, n_stages: int) -> dict:
    """Parse ``"Ett|tt|ttL"`` into per-stage layer counts plus embedding / loss placement."""
    parts = layout.split("|")
    if len(parts) != n_stages:
        raise ValueError(f"layout has {len(parts)} stages, expected {n_stages}")
    counts, emb, loss = [], None, None
    for i, p in enumerate(parts):
        for ch in p:
            if ch not in "EtL":
                raise ValueError(f"bad character {ch!r} in pipeline layout")
        counts.append(p.count("t"))
        if "E" in p:
            emb = i
        if "L" in p:
            loss = i
    if emb != 0 or loss != n_stages - 1:
        raise ValueError("embedding must be on the first stage and the loss on the last")
    return {"layers": counts, "embedding_stage": emb, "loss_stage": loss}
