"""Checkpointing: ``torch_dist`` checkpoints written and read through ``torch.distributed.checkpoint`` (DCP), with
Megatron-core state-dict keys.

    <save>/latest_checkpointed_iteration.txt            tracker ("release" or the iteration number)
    <save>/iter_0000010/common.pt                        args, iteration, LR-scheduler / data-loader state, step counts
    <save>/iter_0000010/.metadata                        DCP metadata: every tensor's global shape, dtype and chunks
    <save>/iter_0000010/__<rank>_0.distcp                DCP data file of one rank (only the chunks that rank owns)

(directory / tracker / ``common.pt`` contents: primus/backends/megatron/patches/checkpoint_patches.py:40-253,
runner/helpers/hooks/train/posttrain/megatron/01_convert_checkpoints.py:354-407 in the reference; the writer is the
stock ``FileSystemWriter``, whose asynchronous variant the reference swaps in:
primus/backends/megatron/core/dist_checkpointing/strategies/filesystem_async.py:1-67).  Any DCP reader opens the
directory: ``torch.distributed.checkpoint.load(state_dict, checkpoint_id=dir)`` with plain tensors of the global shapes.

Every tensor is described by rectangular chunks (offsets + sizes in the global tensor), so a load re-slices for any
tensor / expert / pipeline / data-parallel layout and reads only the bytes a rank needs.  That holds for the optimizer
state too: a rank's contiguous range of the flat ZeRO-1 buffer is cut into at most three rectangles per parameter (a
partial first row, whole rows, a partial last row) of keys ``optimizer.state.{fp32_param,exp_avg,exp_avg_sq}.<param>``.

Options (names of primus/configs/modules/megatron/trainer_base.yaml:120-158): ``ckpt_format`` ``torch_dist`` | ``torch``
(one pickle per rank in Megatron's legacy ``mp_rank_XX[_YYY]`` folders, same layout required on load),
``auto_detect_ckpt_format``, ``async_save`` (device -> host copy in the caller, file writing on a side thread with its
own gloo group), ``ckpt_fully_parallel_save`` / ``ckpt_fully_parallel_load`` (replicated tensors are written / read by
different data-parallel ranks instead of all by the first), ``dist_ckpt_strictness``, ``no_save_optim`` /
``no_load_optim`` / ``no_save_rng`` / ``no_load_rng`` / ``finetune``.

Model tensors are stored under Megatron-core names and *layouts* so that a checkpoint is portable:
* ``linear_qkv.weight`` rows are interleaved per query group ``[q heads of the group | k | v] x groups``
  (primus/backends/megatron/checkpoint/native_loader_llama.py:194-209); internally the rows are
  ``[all q | all k | all v]``;
* ``linear_fc1.weight`` is ``cat[gate; up]`` on dim 0 (:226-239), sharded per half under tensor parallelism;
* routed experts are stacked ``experts.fc{1,2}_weight.weight [E_local, ...]`` sharded on dim 0 over EP
  (primus/backends/megatron/core/extensions/mega_moe.py:272-305).
"""
from __future__ import annotations

import io
import os
import threading
import zlib
from dataclasses import dataclass
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
    if name.endswith(("linear_qkv.weight", "linear_qkv.bias")):
        return {"kind": "qkv", "axis": 0, "index": st.tp_rank, "count": st.tp}
    if name.endswith("linear_fc1.weight"):
        return {"kind": "glu", "axis": 0, "index": st.tp_rank, "count": st.tp}
    if getattr(p, "tp_parts", None):     # several head-split blocks stacked on dim 0 (fused projections of the mixers)
        return {"kind": "parts", "axis": 0, "index": st.tp_rank, "count": st.tp, "sizes": list(p.tp_parts)}
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
    if name.endswith(("linear_qkv.weight", "linear_qkv.bias")) and not cfg.multi_latent_attention:
        return qkv_internal_to_mcore(t, cfg.num_attention_heads // tp, cfg.num_query_groups // tp, cfg.kv_channels)
    if _is_mla_rope_weight(name, cfg):
        return _mla_rope_rows(t, name, cfg, tp, to_internal=False)
    return t


def from_saved_layout(name: str, t: torch.Tensor, cfg, tp: int) -> torch.Tensor:
    if name.endswith(("linear_qkv.weight", "linear_qkv.bias")) and not cfg.multi_latent_attention:
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
    if kind == "parts":  # every shard holds its slice of every block, blocks in order
        n, blocks, lo = spec0["count"], [], 0
        for size in spec0["sizes"]:
            blocks += [p[lo:lo + size // n] for p in parts]
            lo += size // n
        return torch.cat(blocks, dim=0)
    if kind == "glu":  # every shard holds [gate_i; up_i]
        gates = [p[: p.shape[0] // 2] for p in parts]
        ups = [p[p.shape[0] // 2:] for p in parts]
        return torch.cat(gates + ups, dim=0)
    return torch.cat(parts, dim=spec0["axis"])  # tp / ep / qkv (per-group interleave keeps groups contiguous)


def slice_global(name: str, full: torch.Tensor, spec: dict) -> torch.Tensor:
    kind, idx, n = spec["kind"], spec["index"], spec["count"]
    if kind == "replicated":
        return full
    if kind == "parts":
        out, off = [], 0
        for size in spec["sizes"]:
            w = size // n
            out.append(full[off + idx * w: off + (idx + 1) * w])
            off += size
        return torch.cat(out, dim=0)
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
    """Everything of the model that a checkpoint holds: the parameters and the persistent buffers (the router's
    selection bias of auxiliary-loss-free / quantile load balancing is state that training changes, not a parameter)."""
    for m in trainer.model_chunks:
        for name, p in m.named_parameters():
            yield name, p
        for mod_name, mod in m.named_modules():
            for bn, b in mod._buffers.items():
                if b is not None and bn not in mod._non_persistent_buffers_set:
                    yield (f"{mod_name}.{bn}" if mod_name else bn), b


# ----------------------------------------------------------------------------------------------
# chunks: which rectangle of a global tensor a local piece of memory holds
@dataclass
class Piece:
    key: str
    tensor: torch.Tensor        # local data (save) / destination view (load)
    offsets: tuple              # position of the piece in the global tensor
    global_shape: tuple


def _segments(spec: dict, local_shape, cfg, tp: int, internal_qkv: bool) -> tuple:
    """(global shape, [(axis, local lo, local hi, global offset)]) of a local shard whose layout is the saved
    (Megatron-core) one, or, with ``internal_qkv``, this engine's ``[q | k | v]`` row order (optimizer state)."""
    kind, idx, n = spec["kind"], spec["index"], spec["count"]
    shape = list(local_shape)
    if kind == "replicated":
        return tuple(shape), [(0, 0, shape[0] if shape else 1, 0)]
    ax = spec["axis"]
    g = list(shape)
    g[ax] = shape[ax] * n
    if kind == "parts":
        segs, loc, goff = [], 0, 0
        for size in spec["sizes"]:
            w = size // n
            segs.append((0, loc, loc + w, goff + idx * w))
            loc, goff = loc + w, goff + size
        return tuple(g), segs
    if kind == "glu":
        h = shape[0] // 2
        return tuple(g), [(0, 0, h, idx * h), (0, h, 2 * h, n * h + idx * h)]
    if kind == "qkv" and internal_qkv:
        d = cfg.kv_channels
        hq, hkv = cfg.num_attention_heads // tp * d, cfg.num_query_groups // tp * d
        return tuple(g), [(0, 0, hq, idx * hq), (0, hq, hq + hkv, n * hq + idx * hkv),
                          (0, hq + hkv, hq + 2 * hkv, n * (hq + hkv) + idx * hkv)]
    return tuple(g), [(ax, 0, shape[ax], idx * shape[ax])]


def _pieces_of_tensor(key: str, t: torch.Tensor, gshape: tuple, segs: list) -> list:
    out = []
    for ax, lo, hi, goff in segs:
        if t.dim() == 0:
            out.append(Piece(key, t.reshape(1), (0,), (1,)))
            continue
        off = [0] * t.dim()
        off[ax] = goff
        out.append(Piece(key, t.narrow(ax, lo, hi - lo), tuple(off), tuple(gshape)))
    return out


def _as_rows(shape) -> tuple:
    """2-D view used for optimizer state: all leading dimensions are folded into rows."""
    shape = tuple(shape)
    if len(shape) <= 1:
        return (1, shape[0] if shape else 1)
    rows = 1
    for s_ in shape[:-1]:
        rows *= s_
    return (rows, shape[-1])


def _flat_range_pieces(key: str, flat: torch.Tensor, a: int, b: int, local2d: tuple, gshape2d: tuple, segs: list) -> list:
    """Pieces for elements [a, b) of a parameter's local shard (row-major, shape ``local2d``); ``flat`` holds exactly
    those elements.  At most a partial first row, a block of whole rows and a partial last row, each cut at the
    segment boundaries of the shard."""
    R, C = local2d
    rects = []            # (row lo, row hi, col lo, col hi, start in flat)
    r0, c0 = divmod(a, C)
    r1, c1 = divmod(b, C)
    if r0 == r1:
        rects.append((r0, r0 + 1, c0, c1, 0))
    else:
        pos = 0
        if c0:
            rects.append((r0, r0 + 1, c0, C, 0))
            pos += C - c0
            r0 += 1
        if r1 > r0:
            rects.append((r0, r1, 0, C, pos))
            pos += (r1 - r0) * C
        if c1:
            rects.append((r1, r1 + 1, 0, c1, pos))
    out = []
    for rl, rh, cl, ch, start in rects:
        for ax, lo, hi, goff in segs:
            if ax == 0:
                l, h = max(rl, lo), min(rh, hi)
                if l >= h:
                    continue
                w = ch - cl
                view = flat[start + (l - rl) * w: start + (h - rl) * w].view(h - l, w)
                out.append(Piece(key, view, (goff + l - lo, cl), gshape2d))
            else:       # one segment over all local columns, shifted in the global tensor
                w = ch - cl
                view = flat[start: start + (rh - rl) * w].view(rh - rl, w)
                out.append(Piece(key, view, (rl, goff + cl), gshape2d))
    return out


def _stable_hash(s: str) -> int:
    return zlib.crc32(s.encode())


def _rng_tracker():
    from ..parallel.random import get_rng_tracker

    return get_rng_tracker()


def _is_writer(spec: dict, key: str, st, fully_parallel: bool, replicated_over_dp: bool = True) -> bool:
    """Exactly one rank writes every chunk: replicas over tensor-parallel ranks are written by the first of them;
    replicas over data-parallel ranks by the first, or (``ckpt_fully_parallel_save``) by a rank picked per key."""
    if spec["kind"] == "replicated" and st.tp_rank != 0:
        return False
    if not replicated_over_dp:
        return True
    if spec["kind"] == "ep":
        return st.edp_rank == (_stable_hash(key) % st.edp if fully_parallel else 0)
    n = st.dp * st.cp
    me = st.dp_rank * st.cp + st.cp_rank
    return me == (_stable_hash(key) % n if fully_parallel else 0)


def _collect_model_pieces(trainer, for_load: bool, fully_parallel: bool = False):
    """Save: the pieces this rank writes.  Load: (pieces, finish callbacks) filling every local parameter."""
    st, cfg = ps.get_state(), trainer.mcfg
    pieces, finish = [], []
    for name, p in model_named_parameters(trainer):
        key = saved_key(name)
        if hasattr(p, "to_local"):           # FSDP2: a DTensor sharded over the data-parallel mesh
            from torch.distributed.tensor._utils import compute_local_shape_and_global_offset

            local = p.to_local()
            _, off = compute_local_shape_and_global_offset(p.shape, p.device_mesh, p.placements)
            if local.numel():
                pieces.append(Piece(key, local.detach(), tuple(off), tuple(p.shape)))
            continue
        spec = shard_spec(name, p, cfg, st)
        if not for_load:
            if getattr(p, "embedding_replica", False) or not _is_writer(spec, key, st, fully_parallel):
                continue
            t = to_saved_layout(name, p.detach(), cfg, st.tp)
            gshape, segs = _segments(spec, t.shape, cfg, st.tp, internal_qkv=False)
            pieces += _pieces_of_tensor(key, t, gshape, segs)
        else:
            buf = torch.empty(p.shape, dtype=p.dtype)          # host staging in the saved layout
            gshape, segs = _segments(spec, buf.shape, cfg, st.tp, internal_qkv=False)
            pieces += _pieces_of_tensor(key, buf, gshape, segs)

            def done(name=name, p=p, buf=buf):
                p.data.copy_(from_saved_layout(name, buf, cfg, st.tp).to(p.dtype))
            finish.append(done)
    return pieces, finish


_OPT_KEYS = (("master", "fp32_param"), ("m", "exp_avg"), ("v", "exp_avg_sq"))


def _collect_optimizer_pieces(trainer, for_load: bool, fully_parallel: bool = False) -> list:
    """Pieces of the flat optimizer shards (fp32 master weights and both Adam moments) of this rank."""
    st, cfg = ps.get_state(), trainer.mcfg
    names = {p: n for n, p in model_named_parameters(trainer)}
    out = []
    for s_ in getattr(trainer.optimizer, "state", []):
        buf = s_["buf"]
        replicated = not buf.use_distributed_optimizer and buf.dp_size > 1
        for p in s_["bucket"].params:
            o = buf.param_offsets[p]
            lo, hi = max(o, s_["s"]), min(o + p.numel(), s_["e"])
            if lo >= hi or p not in names:
                continue
            name = names[p]
            spec = shard_spec(name, p, cfg, st)
            base = saved_key(name)
            if not for_load and not _is_writer(spec, base, st, fully_parallel, replicated_over_dp=replicated):
                continue
            local2d = _as_rows(p.shape)
            # the row view folds the leading dimensions, so shard axes move: axis 0 stays rows, the last axis is columns
            spec2 = dict(spec)
            if spec["kind"] in ("tp", "ep") and p.dim() >= 2:
                spec2["axis"] = 1 if spec["axis"] == p.dim() - 1 else 0
            gshape2d, segs = _segments(spec2, local2d, cfg, st.tp, internal_qkv=True)
            for attr, tag in _OPT_KEYS:
                flat = s_[attr][lo - s_["s"]: hi - s_["s"]]
                out += _flat_range_pieces(f"optimizer.state.{tag}.{base}", flat, lo - o, hi - o, local2d, gshape2d, segs)
    return out


# ----------------------------------------------------------------------------------------------
# DCP planners over pieces
def _planners():
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
    from torch.distributed.checkpoint.metadata import (BytesStorageMetadata, ChunkStorageMetadata, MetadataIndex,
                                                       TensorProperties)
    from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
    from torch.distributed.checkpoint.planner_helpers import (_create_read_item_for_byteio,
                                                              create_read_items_for_chunk_list)

    class PieceSavePlanner(DefaultSavePlanner):
        def __init__(self, pieces, objects):
            super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False)
            self.pieces = {(p.key, tuple(p.offsets)): p for p in pieces}
            self.objects = objects

        def create_local_plan(self):
            items = []
            for (key, off), p in self.pieces.items():
                items.append(WriteItem(
                    index=MetadataIndex(key, torch.Size(off)), type=WriteItemType.SHARD,
                    tensor_data=TensorWriteData(
                        chunk=ChunkStorageMetadata(offsets=torch.Size(off), sizes=p.tensor.size()),
                        properties=TensorProperties.create_from_tensor(p.tensor), size=torch.Size(p.global_shape))))
            for key in self.objects:
                items.append(WriteItem(index=MetadataIndex(key), type=WriteItemType.BYTE_IO))
            self.plan = SavePlan(items)
            return self.plan

        def lookup_object(self, index):
            if index.offset is None:
                return self.objects[index.fqn]
            return self.pieces[(index.fqn, tuple(index.offset))].tensor

    class PieceLoadPlanner(DefaultLoadPlanner):
        def __init__(self, pieces, object_keys):
            super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False)
            self.pieces = {(p.key, tuple(p.offsets)): p for p in pieces}
            self.object_keys = list(object_keys)
            self.loaded_objects = {}

        def create_local_plan(self):
            md = self.metadata.state_dict_metadata
            reqs = []
            for (key, off), p in self.pieces.items():
                chunk = ChunkStorageMetadata(offsets=torch.Size(off), sizes=p.tensor.size())
                reqs += create_read_items_for_chunk_list(key, md[key], [chunk])
            for key in self.object_keys:
                if key in md and isinstance(md[key], BytesStorageMetadata):
                    reqs.append(_create_read_item_for_byteio(MetadataIndex(key), 0, MetadataIndex(key), 0, 0))
            return LoadPlan(reqs)

        def load_bytes(self, read_item, value):
            self.loaded_objects[read_item.dest_index.fqn] = torch.load(value, weights_only=False)

        def lookup_tensor(self, index):
            return self.pieces[(index.fqn, tuple(index.offset))].tensor

    return dcp, PieceSavePlanner, PieceLoadPlanner


_CKPT_GROUP = {}
_PENDING: list = []          # at most one asynchronous save in flight


def _ckpt_group():
    """Host-side (gloo) group for the planning collectives of a save / load, so that they never interleave with the
    training collectives of the default group (needed for the side-thread save; cheap otherwise)."""
    if not dist.is_initialized():
        return None
    if "g" not in _CKPT_GROUP:
        _CKPT_GROUP["g"] = dist.new_group(backend="gloo") if dist.get_backend() != "gloo" else dist.new_group()
    return _CKPT_GROUP["g"]


def finalize_async_save():
    """Wait for a pending asynchronous save (called before the next save, before a load and when training ends)."""
    while _PENDING:
        th, err = _PENDING.pop()
        th.join()
        if err:
            raise err[0]


def _write_tracker(root: str, it: int, release: bool):
    with open(os.path.join(root, TRACKER), "w") as f:
        f.write("release" if release else str(it))


def save_checkpoint(trainer, root: str, release: bool = False) -> str:
    tc = trainer.tcfg
    fmt = getattr(tc, "ckpt_format", "torch_dist") or "torch_dist"
    if fmt == "torch":
        return _save_legacy(trainer, root, release)
    if fmt != "torch_dist":
        raise ValueError(f"ckpt_format {fmt!r}: torch_dist or torch")
    finalize_async_save()
    if hasattr(trainer, "finish_param_sync"):
        trainer.finish_param_sync()
    st = ps.get_state()
    cfg = trainer.mcfg
    it = trainer.iteration
    d = checkpoint_dir(root, it, release)
    os.makedirs(d, exist_ok=True)
    fully = bool(getattr(tc, "ckpt_fully_parallel_save", True))
    pieces, _ = _collect_model_pieces(trainer, for_load=False, fully_parallel=fully)
    objects = {}
    save_optim = not getattr(tc, "no_save_optim", False)
    if save_optim:
        if getattr(trainer, "fsdp", False):
            objects[f"optimizer/fsdp2_rank_{st.rank}"] = trainer.optimizer.state_dict()
        else:
            pieces += _collect_optimizer_pieces(trainer, for_load=False, fully_parallel=fully)
    if not getattr(tc, "no_save_rng", False):
        objects[f"rng_state/rank_{st.rank}"] = {
            "cpu": torch.get_rng_state(), "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
            "tracker": _rng_tracker().state_dict(), "world": st.world_size}
    deosc = getattr(trainer.optimizer, "deosc", None)
    if save_optim and deosc is not None:
        # windows of the MXFP4 weight de-oscillation detector: per rank, reusable under the same layout only
        objects[f"weight_deosc/rank_{st.rank}"] = {"world": st.world_size, "state": deosc.state_dict()}
    # device -> host now (the training step that follows may overwrite the tensors); the file I/O can run later
    async_save = bool(getattr(tc, "async_save", False))
    staged = [Piece(p.key, p.tensor.detach().to("cpu", copy=True).contiguous(), p.offsets, p.global_shape) for p in pieces]
    common = None
    if st.rank == 0:
        flops = float(getattr(trainer, "flops_per_token", 0.0)) * tc.seq_length * tc.global_batch_size * it
        common = {"args": {"model": vars(cfg).copy(), "train": vars(tc).copy()}, "iteration": it,
                  "checkpoint_version": 3.0, "scheduler": trainer.scheduler.state_dict(),
                  "data": trainer.stager.state_dict(), "num_floating_point_operations_so_far": flops,
                  "optimizer": {"step": int(getattr(trainer.optimizer, "step_count", 0)), "saved": save_optim},
                  "layout": {"tp": st.tp, "pp": st.pp, "dp": st.dp, "ep": st.ep, "cp": st.cp, "world": st.world_size}}
        common["args"]["model"].pop("moe_layer_pattern", None)
    group = _ckpt_group()

    def write():
        dcp, SavePlanner, _ = _planners()
        from torch.distributed.checkpoint import FileSystemWriter

        dcp.save({}, storage_writer=FileSystemWriter(d, single_file_per_rank=True, thread_count=1),
                 planner=SavePlanner(staged, objects), process_group=group, no_dist=group is None)
        if st.rank == 0:        # dcp.save returns on the coordinator after every rank's files are complete
            torch.save(common, os.path.join(d, "common.pt"))
            _write_tracker(root, it, release)

    if async_save:
        err: list = []

        def run():
            try:
                write()
            except BaseException as e:  # noqa: BLE001 - re-raised by finalize_async_save in the training thread
                err.append(e)
        th = threading.Thread(target=run, name="primus-b200-async-save", daemon=True)
        th.start()
        _PENDING.append((th, err))
    else:
        write()
        if group is not None:
            dist.barrier(group=group)
    return d


# ----------------------------------------------------------------------------------------------
def detect_format(d: str) -> str:
    """``torch_dist`` when the directory holds DCP metadata, ``torch`` for the legacy per-rank folders."""
    if os.path.exists(os.path.join(d, ".metadata")):
        return "torch_dist"
    if any(n.startswith("mp_rank_") for n in os.listdir(d)):
        return "torch"
    raise FileNotFoundError(f"{d}: neither a torch_dist (.metadata) nor a torch (mp_rank_*) checkpoint")


def _strictness(mode: str, missing: list, unexpected: list, log) -> None:
    """``dist_ckpt_strictness``: what to do with keys the model wants but the checkpoint lacks (missing) and keys the
    checkpoint has but the model does not (unexpected)."""
    mode = mode or "assume_ok_unexpected"
    if mode not in ("assume_ok_unexpected", "log_unexpected", "log_all", "raise_unexpected", "raise_all", "ignore_all"):
        raise ValueError(f"dist_ckpt_strictness {mode!r}")
    if unexpected and mode in ("log_unexpected", "log_all"):
        log(f"[checkpoint] {len(unexpected)} unexpected keys, e.g. {unexpected[:4]}")
    if missing and mode == "log_all":
        log(f"[checkpoint] {len(missing)} missing keys, e.g. {missing[:4]}")
    if unexpected and mode in ("raise_unexpected", "raise_all"):
        raise KeyError(f"checkpoint has {len(unexpected)} unexpected keys, e.g. {unexpected[:4]}")
    if missing and mode not in ("log_all", "ignore_all"):
        raise KeyError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:4]}")


def load_checkpoint(trainer, root: str, finetune: Optional[bool] = None, load_optim: Optional[bool] = None,
                    load_rng: Optional[bool] = None, iteration: Optional[int] = None) -> int:
    """Loads the latest checkpoint under ``root`` (or the one of ``iteration`` / ``ckpt_step``); returns the iteration
    (0 when nothing was found)."""
    tc = trainer.tcfg
    finetune = bool(getattr(tc, "finetune", False)) if finetune is None else finetune
    load_optim = (not getattr(tc, "no_load_optim", False)) if load_optim is None else load_optim
    load_rng = (not getattr(tc, "no_load_rng", False)) if load_rng is None else load_rng
    finalize_async_save()
    st = ps.get_state()
    tag = read_tracker(root)
    step = iteration if iteration is not None else getattr(tc, "ckpt_step", None)
    if step is not None:
        tag = str(int(step))
        if not os.path.isdir(os.path.join(root, f"iter_{int(step):07d}")):
            raise FileNotFoundError(f"no checkpoint of iteration {step} under {root}")
    if tag is None:
        return 0
    d = os.path.join(root, "release" if tag == "release" else f"iter_{int(tag):07d}")
    fmt = getattr(tc, "ckpt_format", "torch_dist") or "torch_dist"
    if getattr(tc, "auto_detect_ckpt_format", False) or not os.path.exists(os.path.join(d, ".metadata")):
        fmt = detect_format(d)
    if fmt == "torch":
        return _load_legacy(trainer, d, finetune, load_optim, load_rng)
    from ..ops import gemm as _gemm
    from torch.distributed.checkpoint import FileSystemReader

    dcp, _, LoadPlanner = _planners()
    reader = FileSystemReader(d)
    md = reader.read_metadata().state_dict_metadata
    common = torch.load(os.path.join(d, "common.pt"), map_location="cpu", weights_only=False)
    log = getattr(trainer, "log", print)
    pieces, finish = _collect_model_pieces(trainer, for_load=True)
    wanted = {p.key for p in pieces}
    saved_model = {k for k in md if not k.startswith(("optimizer", "rng_state/", "weight_deosc/"))}
    missing = sorted(wanted - saved_model)
    _strictness(getattr(tc, "dist_ckpt_strictness", None), missing, sorted(saved_model - wanted), log)
    pieces = [p for p in pieces if p.key in md]
    with_optim = load_optim and not finetune and common.get("optimizer", {}).get("saved", True)
    opt_pieces = []
    if with_optim and not getattr(trainer, "fsdp", False):
        opt_pieces = _collect_optimizer_pieces(trainer, for_load=True)
        lacking = sorted({p.key for p in opt_pieces} - set(md))
        if lacking:
            raise KeyError(f"checkpoint {d} holds no optimizer state for {len(lacking)} tensors, e.g. {lacking[:3]}; "
                           "load with no_load_optim / finetune to start the optimizer from the weights alone")
    obj_keys = []
    if load_rng and not finetune:
        obj_keys.append(f"rng_state/rank_{st.rank}")
    if with_optim and getattr(trainer, "fsdp", False):
        obj_keys.append(f"optimizer/fsdp2_rank_{st.rank}")
    deosc = getattr(trainer.optimizer, "deosc", None)
    if with_optim and deosc is not None and f"weight_deosc/rank_{st.rank}" in md:
        obj_keys.append(f"weight_deosc/rank_{st.rank}")
    # ``ckpt_fully_parallel_load``: tensors replicated over the data-parallel ranks are read from disk by one of them
    # each and broadcast, instead of every rank reading everything
    spread = bool(getattr(tc, "ckpt_fully_parallel_load", False)) and st.dp > 1 and st.cp == 1 and \
        not getattr(trainer, "fsdp", False)
    mine = pieces
    if spread:
        ep_keys = {saved_key(n) for n, p in model_named_parameters(trainer) if getattr(p, "expert_parallel", False)}
        mine = [p for p in pieces if p.key in ep_keys or _stable_hash(p.key) % st.dp == st.dp_rank]
    group = _ckpt_group()
    planner = LoadPlanner(mine + opt_pieces, obj_keys)
    dcp.load({}, storage_reader=reader, planner=planner, process_group=group, no_dist=group is None)
    if spread:
        for p in pieces:
            if p.key in ep_keys:
                continue
            src = st.dp_ranks[_stable_hash(p.key) % st.dp] if hasattr(st, "dp_ranks") else None
            t = p.tensor if p.tensor.is_contiguous() else p.tensor.contiguous()
            dist.broadcast(t, src=src, group=st.dp_group)
            if t is not p.tensor:
                p.tensor.copy_(t)
    for f in finish:
        f()
    _gemm.bump_weight_generation()      # parameters changed in place: quantised copies of the old values expire
    rng = planner.loaded_objects.get(f"rng_state/rank_{st.rank}")
    if rng is not None and rng.get("world") == st.world_size:
        torch.set_rng_state(rng["cpu"])
        if rng.get("cuda") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda"])
        if rng.get("tracker") and _rng_tracker().active:
            _rng_tracker().load_state_dict(rng["tracker"])
    if finetune:
        trainer.iteration = 0
        _refresh_master_weights(trainer)
        return 0
    if with_optim:
        if getattr(trainer, "fsdp", False):
            sd = planner.loaded_objects.get(f"optimizer/fsdp2_rank_{st.rank}")
            if sd is None:
                raise KeyError(f"checkpoint {d} has no FSDP2 optimizer state for rank {st.rank} (saved with another "
                               "data-parallel size?); load with no_load_optim")
            trainer.optimizer.load_state_dict(sd)
        else:
            trainer.optimizer.step_count = int(common.get("optimizer", {}).get("step", 0))
        saved_deosc = planner.loaded_objects.get(f"weight_deosc/rank_{st.rank}")
        if deosc is not None and saved_deosc is not None and saved_deosc.get("world") == st.world_size:
            deosc.load_state_dict(saved_deosc["state"])
    else:
        if load_optim and not finetune:
            log(f"[checkpoint] {d} was saved without optimizer state: master weights are re-derived from the "
                "parameters and the Adam moments start from zero")
        _refresh_master_weights(trainer)
    trainer.iteration = int(common["iteration"])
    # ``override_opt_param_scheduler`` (the default behaviour): this run's schedule continues at the loaded step;
    # ``use_checkpoint_opt_param_scheduler``: the schedule the checkpoint was written with
    trainer.scheduler.load_state_dict(
        common["scheduler"], bool(getattr(tc, "use_checkpoint_opt_param_scheduler", False))
        and not getattr(tc, "override_opt_param_scheduler", False), log)
    trainer.stager.load_state_dict(common["data"])
    if group is not None:
        dist.barrier(group=group)
    return trainer.iteration


# ----------------------------------------------------------------------------------------------
# legacy "torch" format: one pickle per rank, Megatron's folder names; same parallel layout on load
def _legacy_dir(d: str, st) -> str:
    name = f"mp_rank_{st.tp_rank:02d}" if st.pp == 1 else f"mp_rank_{st.tp_rank:02d}_{st.pp_rank:03d}"
    if st.ep > 1:
        name += f"_{st.ep_rank:03d}"
    return os.path.join(d, name)


def _save_legacy(trainer, root: str, release: bool) -> str:
    st, tc = ps.get_state(), trainer.tcfg
    it = trainer.iteration
    d = checkpoint_dir(root, it, release)
    sub = _legacy_dir(d, st)
    os.makedirs(sub, exist_ok=True)
    dp_first = st.dp_rank == 0 and st.cp_rank == 0
    payload = {"iteration": it, "checkpoint_version": 3.0,
               "args": {"model": {k: v for k, v in vars(trainer.mcfg).items() if k != "moe_layer_pattern"},
                        "train": vars(tc).copy()},
               "scheduler": trainer.scheduler.state_dict(), "data": trainer.stager.state_dict()}
    if dp_first:
        payload["model"] = {saved_key(n): to_saved_layout(n, p.detach(), trainer.mcfg, st.tp).cpu()
                            for n, p in model_named_parameters(trainer) if not hasattr(p, "to_local")}
        if not getattr(tc, "no_save_rng", False):
            payload["rng_state"] = {"cpu": torch.get_rng_state(), "tracker": _rng_tracker().state_dict(),
                                    "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
        torch.save(payload, os.path.join(sub, "model_optim_rng.pt"))
    if not getattr(tc, "no_save_optim", False):
        sd = trainer.optimizer.state_dict()
        sd = {k: ([{kk: (vv.cpu() if torch.is_tensor(vv) else vv) for kk, vv in s.items()} for s in v]
                  if k == "shards" else v) for k, v in sd.items()}
        torch.save(sd, os.path.join(sub, f"distrib_optim_dp{st.dp_rank * st.cp + st.cp_rank:03d}.pt"))
    if dist.is_initialized():
        dist.barrier()
    if st.rank == 0:
        _write_tracker(root, it, release)
    return d


def _load_legacy(trainer, d: str, finetune: bool, load_optim: bool, load_rng: bool) -> int:
    from ..ops import gemm as _gemm

    st = ps.get_state()
    sub = _legacy_dir(d, st)
    f = os.path.join(sub, "model_optim_rng.pt")
    if not os.path.exists(f):
        raise FileNotFoundError(f"{f}: a torch-format checkpoint can only be loaded with the parallel layout it was "
                                "saved with (convert through a torch_dist checkpoint to change it)")
    payload = torch.load(f, map_location="cpu", weights_only=False)
    for name, p in model_named_parameters(trainer):
        t = payload["model"][saved_key(name)]
        p.data.copy_(from_saved_layout(name, t, trainer.mcfg, st.tp).to(p.dtype))
    _gemm.bump_weight_generation()
    if load_rng and not finetune and payload.get("rng_state"):
        torch.set_rng_state(payload["rng_state"]["cpu"])
        if payload["rng_state"]["cuda"] is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(payload["rng_state"]["cuda"])
        if payload["rng_state"].get("tracker") and _rng_tracker().active:
            _rng_tracker().load_state_dict(payload["rng_state"]["tracker"])
    if finetune:
        trainer.iteration = 0
        _refresh_master_weights(trainer)
        return 0
    of = os.path.join(sub, f"distrib_optim_dp{st.dp_rank * st.cp + st.cp_rank:03d}.pt")
    if load_optim and os.path.exists(of):
        trainer.optimizer.load_state_dict(torch.load(of, map_location="cpu", weights_only=False))
    else:
        _refresh_master_weights(trainer)
    trainer.iteration = int(payload["iteration"])
    trainer.scheduler.load_state_dict(payload["scheduler"])
    trainer.stager.load_state_dict(payload["data"])
    if dist.is_initialized():
        dist.barrier()
    return trainer.iteration


def _refresh_master_weights(trainer):
    """Re-derive fp32 master weights from the (just loaded) parameters; moments start from zero."""
    from ..ops import gemm as _gemm

    _gemm.bump_weight_generation()
    for s in getattr(trainer.optimizer, "state", []):
        if not isinstance(s, dict) or "buf" not in s:
            continue
        buf = s["buf"]
        s["master"].copy_(buf.param_data[s["s"]:s["e"]].float())
