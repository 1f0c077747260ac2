"""Checkpointing in the Megatron ``torch_dist`` directory layout with Megatron-core state-dict keys.

    <save>/latest_checkpointed_iteration.txt            tracker ("release" or the iteration number)
    <save>/iter_0000010/common.pt                        args, iteration, LR-scheduler, data-loader and RNG state
    <save>/iter_0000010/.metadata                        every sharded tensor: global shape, dtype, shards -> file
    <save>/iter_0000010/__<rank>_0.distcp                the shards written by one rank ("fully parallel" save)

(directory / tracker / ``common.pt`` contents: primus/backends/megatron/patches/checkpoint_patches.py:40-253,
runner/helpers/hooks/train/posttrain/megatron/01_convert_checkpoints.py:354-407 in the reference).

Model tensors are stored under Megatron-core names and *layouts* so that a checkpoint is portable:
* ``linear_qkv.weight`` rows are interleaved per query group ``[q heads of the group | k | v] x groups``
  (primus/backends/megatron/checkpoint/native_loader_llama.py:194-209); internally the rows are
  ``[all q | all k | all v]``;
* ``linear_fc1.weight`` is ``cat[gate; up]`` on dim 0 (:226-239), sharded per half under tensor parallelism;
* routed experts are stacked ``experts.fc{1,2}_weight.weight [E_local, ...]`` sharded on dim 0 over EP
  (primus/backends/megatron/core/extensions/mega_moe.py:272-305).
Each tensor records its global shape and the offset of every shard, so loading re-slices for a different
TP / EP / PP layout.  Optimizer state is saved per rank (master weights and Adam moments of the rank's flat
shards) and requires the same parallel layout when it is loaded; ``no_load_optim`` / ``finetune`` skip it.
"""
from __future__ import annotations

import json
import os
import pickle
from typing import Optional

import torch
import torch.distributed as dist

from ..parallel import state as ps

TRACKER = "latest_checkpointed_iteration.txt"


# ----------------------------------------------------------------------------------------------
# layout conversion: internal <-> Megatron-core
def qkv_internal_to_mcore(w: torch.Tensor, hq: int, hkv: int, d: int) -> torch.Tensor:
    """[q heads | k heads | v heads] rows -> per-group interleave. Works for weights [rows, in] and biases [rows]."""
    g = hq // hkv
    q = w[: hq * d].reshape(hkv, g * d, *w.shape[1:])
    k = w[hq * d:(hq + hkv) * d].reshape(hkv, d, *w.shape[1:])
    v = w[(hq + hkv) * d:].reshape(hkv, d, *w.shape[1:])
    return torch.cat([q, k, v], dim=1).reshape(-1, *w.shape[1:])


def qkv_mcore_to_internal(w: torch.Tensor, hq: int, hkv: int, d: int) -> torch.Tensor:
    g = hq // hkv
    x = w.reshape(hkv, (g + 2) * d, *w.shape[1:])
    q = x[:, : g * d].reshape(hq * d, *w.shape[1:])
    k = x[:, g * d:(g + 1) * d].reshape(hkv * d, *w.shape[1:])
    v = x[:, (g + 1) * d:].reshape(hkv * d, *w.shape[1:])
    return torch.cat([q, k, v], dim=0)


def shard_spec(name: str, p: torch.Tensor, cfg, st) -> dict:
    """How parameter ``name`` of this rank maps into the global tensor: kind, axis, index, count."""
    if getattr(p, "expert_parallel", False) or (".experts.fc" in name and st.ep > 1):
        return {"kind": "ep", "axis": 0, "index": st.ep_rank, "count": st.ep}
    if not getattr(p, "tensor_model_parallel", False) or st.tp == 1:
        return {"kind": "replicated", "axis": 0, "index": 0, "count": 1}
    if name.endswith("linear_qkv.weight"):
        return {"kind": "qkv", "axis": 0, "index": st.tp_rank, "count": st.tp}
    if name.endswith("linear_fc1.weight"):
        return {"kind": "glu", "axis": 0, "index": st.tp_rank, "count": st.tp}
    return {"kind": "tp", "axis": int(getattr(p, "partition_dim", 0)), "index": st.tp_rank, "count": st.tp}


def _mla_rope_rows(t: torch.Tensor, name: str, cfg, tp: int, to_internal: bool) -> torch.Tensor:
    """MLA keeps the rotary dims of q / k in the *interleaved* pair order of the published DeepSeek weights in a
    checkpoint (Megatron de-interleaves at run time); this engine rotates halves, so the rows that produce the
    rotary dims are de-interleaved on load (even positions first, then odd) and re-interleaved on save."""
    dr = cfg.qk_pos_emb_head_dim
    if to_internal:
        perm = torch.cat([torch.arange(0, dr, 2), torch.arange(1, dr, 2)])
    else:
        perm = torch.empty(dr, dtype=torch.long)
        perm[0::2] = torch.arange(0, dr // 2)
        perm[1::2] = torch.arange(dr // 2, dr)
    perm = perm.to(t.device)
    if name.endswith("linear_kv_down_proj.weight"):
        lat = cfg.kv_lora_rank
        return torch.cat([t[:lat], t[lat:][perm]], dim=0)
    nh = cfg.num_attention_heads // tp
    dn = cfg.qk_head_dim
    x = t.reshape(nh, dn + dr, *t.shape[1:])
    return torch.cat([x[:, :dn], x[:, dn:][:, perm]], dim=1).reshape(t.shape)


def _is_mla_rope_weight(name: str, cfg) -> bool:
    return cfg.multi_latent_attention and name.endswith(
        ("linear_kv_down_proj.weight", "linear_q_up_proj.weight", "linear_q_proj.weight"))


def to_saved_layout(name: str, t: torch.Tensor, cfg, tp: int) -> torch.Tensor:
    if name.endswith("linear_qkv.weight") and not cfg.multi_latent_attention:
        return qkv_internal_to_mcore(t, cfg.num_attention_heads // tp, cfg.num_query_groups // tp, cfg.kv_channels)
    if _is_mla_rope_weight(name, cfg):
        return _mla_rope_rows(t, name, cfg, tp, to_internal=False)
    return t


def from_saved_layout(name: str, t: torch.Tensor, cfg, tp: int) -> torch.Tensor:
    if name.endswith("linear_qkv.weight") and not cfg.multi_latent_attention:
        return qkv_mcore_to_internal(t, cfg.num_attention_heads // tp, cfg.num_query_groups // tp, cfg.kv_channels)
    if _is_mla_rope_weight(name, cfg):
        return _mla_rope_rows(t, name, cfg, tp, to_internal=True)
    return t


def assemble_global(name: str, shards: list[tuple[dict, torch.Tensor]]) -> torch.Tensor:
    """Rebuild the global (mcore-layout) tensor from its shards."""
    spec0 = shards[0][0]
    kind = spec0["kind"]
    if kind == "replicated":
        return shards[0][1]
    by_idx = {s["index"]: t for s, t in shards}
    parts = [by_idx[i] for i in range(spec0["count"])]
    if kind == "glu":  # every shard holds [gate_i; up_i]
        gates = [p[: p.shape[0] // 2] for p in parts]
        ups = [p[p.shape[0] // 2:] for p in parts]
        return torch.cat(gates + ups, dim=0)
    return torch.cat(parts, dim=spec0["axis"])  # tp / ep / qkv (per-group interleave keeps groups contiguous)


def slice_global(name: str, full: torch.Tensor, spec: dict) -> torch.Tensor:
    kind, idx, n = spec["kind"], spec["index"], spec["count"]
    if kind == "replicated":
        return full
    if kind == "glu":
        half = full.shape[0] // 2
        c = half // n
        return torch.cat([full[idx * c:(idx + 1) * c], full[half + idx * c: half + (idx + 1) * c]], dim=0)
    ax = spec["axis"]
    c = full.shape[ax] // n
    return full.narrow(ax, idx * c, c)


# ----------------------------------------------------------------------------------------------
def checkpoint_dir(root: str, iteration: int, release: bool = False) -> str:
    return os.path.join(root, "release" if release else f"iter_{iteration:07d}")


def read_tracker(root: str) -> Optional[str]:
    p = os.path.join(root, TRACKER)
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return f.read().strip()


def latest_iteration(root: str) -> Optional[int]:
    """Iteration of the newest checkpoint under ``root`` (None: nothing saved yet, or only a release checkpoint)."""
    t = read_tracker(root)
    return int(t) if t is not None and t.isdigit() else None


_RENAMES = ((".self_attention.input_layernorm.", ".input_layernorm."),
            (".mlp.experts.fc1_weight.weight", ".mlp.experts.linear_fc1.weight"),
            (".mlp.experts.fc2_weight.weight", ".mlp.experts.linear_fc2.weight"))


def saved_key(name: str) -> str:
    """Name of a parameter inside a checkpoint: Megatron-core keys.  The MLA input norm is a layer-level module
    there, and the expert weights are called ``linear_fc1 / linear_fc2`` (stored stacked ``[experts, out, in]`` here;
    Megatron's grouped linear stores one ``weight{e}`` entry per expert)."""
    for a, b in _RENAMES:
        name = name.replace(a, b)
    return name


def model_named_parameters(trainer):
    for m in trainer.model_chunks:
        for name, p in m.named_parameters():
            yield name, p


def save_checkpoint(trainer, root: str, release: bool = False) -> str:
    st = ps.get_state()
    cfg = trainer.mcfg
    it = trainer.iteration
    d = checkpoint_dir(root, it, release)
    if st.rank == 0:
        os.makedirs(d, exist_ok=True)
    if dist.is_initialized():
        dist.barrier()
    os.makedirs(d, exist_ok=True)
    shards, meta = {}, {}
    for name, p in model_named_parameters(trainer):
        spec = shard_spec(name, p, cfg, st)
        if hasattr(p, "full_tensor"):      # sharded by FSDP2: gathered on every rank (a collective), written by one
            p = p.full_tensor()
        # replicas: only the first data-parallel rank (expert data-parallel rank for experts) writes
        writer = (st.edp_rank == 0) if spec["kind"] == "ep" else (st.dp_rank == 0 and st.cp_rank == 0)
        if spec["kind"] == "replicated" and st.tp_rank != 0:
            writer = False
        if getattr(p, "embedding_replica", False):   # the first pipeline stage writes the shared word embeddings
            writer = False
        if not writer:
            continue
        t = to_saved_layout(name, p.detach(), cfg, st.tp).cpu().clone()
        key = saved_key(name)
        shards[key] = t
        meta[key] = {"spec": spec, "shape": list(t.shape), "dtype": str(t.dtype), "file": f"__{st.rank}_0.distcp"}
    payload = {"model": shards}
    if not getattr(trainer.tcfg, "no_save_optim", False):
        payload["optimizer"] = {k: ([{kk: (vv.cpu() if torch.is_tensor(vv) else vv) for kk, vv in s.items()} for s in v]
                                    if k == "shards" else v) for k, v in trainer.optimizer.state_dict().items()}
        payload["layout"] = {"tp": st.tp, "pp": st.pp, "dp": st.dp, "ep": st.ep, "world": st.world_size}
    payload["rng"] = {"cpu": torch.get_rng_state(),
                      "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
    torch.save(payload, os.path.join(d, f"__{st.rank}_0.distcp"))
    all_meta = [None] * max(st.world_size, 1)
    if dist.is_initialized():
        dist.all_gather_object(all_meta, meta)
    else:
        all_meta[0] = meta
    if st.rank == 0:
        merged: dict = {}
        for m in all_meta:
            for k, v in (m or {}).items():
                merged.setdefault(k, []).append(v)
        with open(os.path.join(d, ".metadata"), "w") as f:
            json.dump({"format": "primus_b200.torch_dist.v1", "tensors": merged}, f)
        common = {"args": {"model": vars(cfg).copy(), "train": vars(trainer.tcfg).copy()}, "iteration": it,
                  "checkpoint_version": 3.0, "scheduler": trainer.scheduler.state_dict(),
                  "data": trainer.stager.state_dict(), "num_floating_point_operations_so_far": 0}
        common["args"]["model"].pop("moe_layer_pattern", None)
        torch.save(common, os.path.join(d, "common.pt"))
        with open(os.path.join(root, TRACKER), "w") as f:
            f.write("release" if release else str(it))
    if dist.is_initialized():
        dist.barrier()
    return d


def load_checkpoint(trainer, root: str, finetune: bool = False, load_optim: bool = True, load_rng: bool = True) -> int:
    """Loads the latest checkpoint under ``root``; returns the iteration (0 when nothing was found)."""
    st = ps.get_state()
    cfg = trainer.mcfg
    tag = read_tracker(root)
    if tag is None:
        return 0
    d = os.path.join(root, "release" if tag == "release" else f"iter_{int(tag):07d}")
    with open(os.path.join(d, ".metadata")) as f:
        meta = json.load(f)["tensors"]
    cache: dict = {}

    def file_payload(fn):
        if fn not in cache:
            cache[fn] = torch.load(os.path.join(d, fn), map_location="cpu", weights_only=False)
        return cache[fn]

    missing, loaded = [], 0
    for name, p in model_named_parameters(trainer):
        key = saved_key(name) if saved_key(name) in meta else name   # older checkpoints used the internal names
        if key not in meta:
            missing.append(name)
            continue
        entries = meta[key]
        shards = [(e["spec"], file_payload(e["file"])["model"][key]) for e in entries]
        saved_tp = entries[0]["spec"]["count"] if entries[0]["spec"]["kind"] in ("qkv", "glu", "tp") else 1
        full = assemble_global(name, shards)
        spec = shard_spec(name, p, cfg, st)
        mine = slice_global(name, full, spec)
        mine = from_saved_layout(name, mine, cfg, st.tp)
        if tuple(mine.shape) != tuple(p.shape):
            raise ValueError(f"{name}: checkpoint shard {tuple(mine.shape)} does not fit parameter {tuple(p.shape)}")
        if hasattr(p, "full_tensor"):      # sharded by FSDP2: every rank keeps its slice of the loaded tensor
            from torch.distributed.tensor import distribute_tensor

            mine = distribute_tensor(mine.to(device=p.device, dtype=p.dtype), p.device_mesh, p.placements)
        p.data.copy_(mine.to(p.dtype))
        loaded += 1
    if missing:
        raise KeyError(f"checkpoint {d} lacks {len(missing)} tensors, e.g. {missing[:4]}")
    common = torch.load(os.path.join(d, "common.pt"), map_location="cpu", weights_only=False)
    mine_file = os.path.join(d, f"__{st.rank}_0.distcp")
    if finetune:
        trainer.iteration = 0
        _refresh_master_weights(trainer)
        return 0
    if load_optim and os.path.exists(mine_file):
        pl = file_payload(f"__{st.rank}_0.distcp")
        lay = pl.get("layout")
        cur = {"tp": st.tp, "pp": st.pp, "dp": st.dp, "ep": st.ep, "world": st.world_size}
        if "optimizer" in pl and lay == cur:
            trainer.optimizer.load_state_dict(pl["optimizer"])
        else:
            _refresh_master_weights(trainer)
        if load_rng and pl.get("rng"):
            torch.set_rng_state(pl["rng"]["cpu"])
            if pl["rng"]["cuda"] is not None and torch.cuda.is_available():
                torch.cuda.set_rng_state(pl["rng"]["cuda"])
    else:
        _refresh_master_weights(trainer)
    trainer.iteration = int(common["iteration"])
    trainer.scheduler.load_state_dict(common["scheduler"])
    trainer.stager.load_state_dict(common["data"])
    if dist.is_initialized():
        dist.barrier()
    return trainer.iteration


def _refresh_master_weights(trainer):
    """Re-derive fp32 master weights from the (just loaded) parameters; moments start from zero."""
    from ..ops import gemm as _gemm

    _gemm.bump_weight_generation()
    for s in trainer.optimizer.state:
        buf = s["buf"]
        s["master"].copy_(buf.param_data[s["s"]:s["e"]].float())
