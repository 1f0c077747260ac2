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
    if n_stages == 1:           # one stage owns everything, whatever split was asked for a pipelined run
        return list(range(num_layers))
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


def uneven_split(num_layers: int, n_stages: int, first: Optional[int] = None, last: Optional[int] = None,
                 account_for_embedding: bool = False, account_for_loss: bool = False) -> Optional[list]:
    """Per-stage layer counts when the first and / or last stage hold a given number of layers
    (``decoder_first_pipeline_num_layers`` / ``decoder_last_pipeline_num_layers``; the reference's recipes use the
    latter for stacks whose depth has no even split: examples/megatron/configs/MI355X/glm5-BF16-pretrain.yaml:47) or
    when the embedding / the output layer count as one layer of their stage
    (``account_for_embedding_in_pipeline_split`` / ``account_for_loss_in_pipeline_split``:
    primus/configs/modules/megatron/trainer_base.yaml:179).  Returns None when none of the four is set."""
    if first is None and last is None and not account_for_embedding and not account_for_loss:
        return None
    if n_stages == 1:
        return [num_layers]
    if first is not None or last is not None:
        assert not (account_for_embedding or account_for_loss), \
            "fixed first / last stage sizes and account_for_*_in_pipeline_split exclude one another"
        fixed = (first or 0) + (last or 0)
        middle = n_stages - (first is not None) - (last is not None)
        rest = num_layers - fixed
        assert rest >= 0 and (middle > 0 or rest == 0), "first / last stage sizes exceed the model's depth"
        assert middle == 0 or rest % middle == 0, \
            f"{rest} layers outside the fixed stages do not split evenly over {middle} stages"
        per = rest // middle if middle else 0
        counts = [per] * n_stages
        if first is not None:
            counts[0] = first
        if last is not None:
            counts[-1] = last
        return counts
    slots = num_layers + int(account_for_embedding) + int(account_for_loss)
    assert slots % n_stages == 0, f"{slots} layer slots (embedding / loss counted) do not split evenly over {n_stages} stages"
    counts = [slots // n_stages] * n_stages
    counts[0] -= int(account_for_embedding)
    counts[-1] -= int(account_for_loss)
    assert min(counts) >= 0
    return counts
