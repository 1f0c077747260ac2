"""Model-parallel process-group bookkeeping (one process per GPU, ``torch.distributed``).

World layout, fastest-varying first: ``tp - cp - dp - pp`` for the dense part; expert layers re-tile the
``tp*cp*dp`` ranks of one pipeline stage as ``etp - ep - edp``.  This is Megatron's default
``tp-cp-ep-dp-pp`` order that the reference relies on
(primus/backends/megatron/core/pipeline_parallel/primuspipe/pipeline_launcher.py:42-46,76-91;
primus/configs/models/megatron/language_model.yaml:147-168).

All getters work without an initialised process group (world size 1): sizes are 1, ranks 0 and
groups ``None``, so single-process code needs no special casing.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    cp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    etp: int = 1
    edp: int = 1
    tp_rank: int = 0
    cp_rank: int = 0
    pp_rank: int = 0
    dp_rank: int = 0
    ep_rank: int = 0
    edp_rank: int = 0
    tp_group: Optional[object] = None
    cp_group: Optional[object] = None
    # hierarchical context parallelism (a2a inside, ring outside): cp_rank = p2p_rank * cp_a2a + a2a_rank
    cp_a2a: int = 1
    cp_p2p: int = 1
    cp_a2a_group: Optional[object] = None
    cp_p2p_group: Optional[object] = None
    pp_group: Optional[object] = None
    pp_fwd_group: Optional[object] = None  # forward-direction p2p communicator
    pp_bwd_group: Optional[object] = None  # backward-direction p2p communicator
    dp_group: Optional[object] = None
    dp_cp_group: Optional[object] = None
    ep_group: Optional[object] = None
    edp_group: Optional[object] = None
    mp_group: Optional[object] = None  # tp x pp (grad-norm reductions)
    embedding_group: Optional[object] = None
    pp_ranks: list = field(default_factory=lambda: [0])
    tp_ranks: list = field(default_factory=lambda: [0])
    dp_ranks: list = field(default_factory=lambda: [0])
    ep_ranks: list = field(default_factory=lambda: [0])
    virtual_pp: Optional[int] = None
    initialized: bool = False


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def rank_coords(rank: int, tp: int, cp: int, dp: int, pp: int, tp_pp_dp: bool = False) -> tuple[int, int, int, int]:
    """(tp_rank, cp_rank, dp_rank, pp_rank) of a global rank.  Default order of the ranks: tensor fastest, then context,
    data, pipeline (a pipeline's stages are far apart, a data-parallel group is close together); ``tp_pp_dp``: tensor,
    context, pipeline, data (the stages of a pipeline are neighbours, data-parallel replicas far apart) -- the
    reference's ``use_tp_pp_dp_mapping`` (primus/configs/modules/megatron/trainer_base.yaml)."""
    t = rank % tp
    c = (rank // tp) % cp
    if tp_pp_dp:
        return t, c, rank // (tp * cp * pp), (rank // (tp * cp)) % pp
    d = (rank // (tp * cp)) % dp
    p = rank // (tp * cp * dp)
    return t, c, d, p


def group_rank_lists(world: int, tp: int, cp: int, pp: int, ep: int = 1, etp: int = 1,
                     tp_pp_dp: bool = False) -> dict[str, list[list[int]]]:
    """Pure function: every group of every kind as lists of global ranks (tested on CPU)."""
    assert world % (tp * cp * pp) == 0, f"world {world} not divisible by tp*cp*pp={tp * cp * pp}"
    dp = world // (tp * cp * pp)
    per_stage = tp * cp * dp
    out: dict[str, list[list[int]]] = {k: [] for k in ("tp", "cp", "dp", "dp_cp", "pp", "ep", "edp", "mp", "stage")}

    def gid(t, c, d, p):
        if tp_pp_dp:
            return t + tp * (c + cp * (p + pp * d))
        return t + tp * (c + cp * (d + dp * p))

    for p in range(pp):
        out["stage"].append([gid(t, c, d, p) for d in range(dp) for c in range(cp) for t in range(tp)])
        for d in range(dp):
            for c in range(cp):
                out["tp"].append([gid(t, c, d, p) for t in range(tp)])
            for t in range(tp):
                out["cp"].append([gid(t, c, d, p) for c in range(cp)])
        for c in range(cp):
            for t in range(tp):
                out["dp"].append([gid(t, c, d, p) for d in range(dp)])
        for t in range(tp):
            out["dp_cp"].append([gid(t, c, d, p) for d in range(dp) for c in range(cp)])
    for d in range(dp):
        for c in range(cp):
            for t in range(tp):
                out["pp"].append([gid(t, c, d, p) for p in range(pp)])
            out["mp"].append([gid(t, c, d, p) for p in range(pp) for t in range(tp)])
    # expert re-tiling of each stage: etp fastest, then ep, then edp
    assert per_stage % (etp * ep) == 0, f"tp*cp*dp={per_stage} not divisible by etp*ep={etp * ep}"
    edp = per_stage // (etp * ep)
    for p in range(pp):
        stage = out["stage"][p]            # this stage's ranks, tensor fastest, then context, then data
        for e_d in range(edp):
            for e_t in range(etp):
                out["ep"].append([stage[e_t + etp * (e + ep * e_d)] for e in range(ep)])
        for e in range(ep):
            for e_t in range(etp):
                out["edp"].append([stage[e_t + etp * (e + ep * e_d)] for e_d in range(edp)])
    return out


def init_distributed(backend: Optional[str] = None, timeout_minutes: float = 10.0) -> None:
    """Initialise ``torch.distributed`` from torchrun's environment if it is not yet initialised."""
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1 and "RANK" not in os.environ:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, timeout=timedelta(minutes=timeout_minutes), **kwargs)


def initialize_model_parallel(tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, etp: int = 1,
                              virtual_pp: Optional[int] = None, hierarchical_cp_sizes=None,
                              tp_pp_dp_mapping: bool = False) -> ParallelState:
    """Create all groups. Every rank must call this with identical arguments.  ``hierarchical_cp_sizes``: ``[a2a, p2p]``
    with ``a2a * p2p == cp`` splits every context-parallel group into all-to-all groups of neighbouring ranks and ring
    groups across them (the reference's ``hierarchical_context_parallel_sizes``,
    primus/configs/models/megatron/language_model.yaml)."""
    global _STATE
    if not dist.is_initialized():
        assert tp * pp * cp * ep == 1, "model parallelism needs an initialised process group"
        _STATE = ParallelState(initialized=True, virtual_pp=virtual_pp)
        return _STATE
    world = dist.get_world_size()
    rank = dist.get_rank()
    lists = group_rank_lists(world, tp, cp, pp, ep, etp, tp_pp_dp_mapping)
    dp = world // (tp * cp * pp)
    st = ParallelState(world_size=world, rank=rank, tp=tp, cp=cp, pp=pp, dp=dp, ep=ep, etp=etp,
                       edp=(tp * cp * dp) // (etp * ep), virtual_pp=virtual_pp, initialized=True)
    st.tp_rank, st.cp_rank, st.dp_rank, st.pp_rank = rank_coords(rank, tp, cp, dp, pp, tp_pp_dp_mapping)

    def make(kind: str):
        mine, mine_ranks = None, None
        for ranks in lists[kind]:
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                mine, mine_ranks = g, ranks
        return mine, mine_ranks

    st.tp_group, st.tp_ranks = make("tp")
    st.cp_group, _ = make("cp")
    if hierarchical_cp_sizes:
        a2a, p2p = (int(x) for x in hierarchical_cp_sizes)
        assert a2a * p2p == cp, f"hierarchical_context_parallel_sizes {hierarchical_cp_sizes} must multiply to cp={cp}"
        st.cp_a2a, st.cp_p2p = a2a, p2p
        for ranks in lists["cp"]:
            for i in range(p2p):                      # neighbouring ranks exchange heads
                sub = ranks[i * a2a:(i + 1) * a2a]
                g = dist.new_group(sub) if len(sub) > 1 else None
                if rank in sub:
                    st.cp_a2a_group = g
            for j in range(a2a):                      # the ring runs across the all-to-all groups
                sub = ranks[j::a2a]
                g = dist.new_group(sub) if len(sub) > 1 else None
                if rank in sub:
                    st.cp_p2p_group = g
    st.dp_group, st.dp_ranks = make("dp")
    st.dp_cp_group, _ = make("dp_cp")
    st.pp_group, st.pp_ranks = make("pp")
    st.pp_fwd_group, _ = make("pp")
    st.pp_bwd_group, _ = make("pp")
    st.mp_group, _ = make("mp")
    st.ep_group, st.ep_ranks = make("ep")
    st.edp_group, edp_ranks = make("edp")
    st.ep_rank = st.ep_ranks.index(rank)
    st.edp_rank = edp_ranks.index(rank)
    # first and last pipeline stage share the (tied) embedding gradients
    if pp > 1:
        for ranks in lists["pp"]:
            pair = [ranks[0], ranks[-1]]
            g = dist.new_group(pair)
            if rank in pair:
                st.embedding_group = g
    _STATE = st
    return st


def destroy_model_parallel() -> None:
    global _STATE
    _STATE = ParallelState()


# convenience getters ---------------------------------------------------------------------------
def tp_size() -> int: return _STATE.tp
def tp_rank() -> int: return _STATE.tp_rank
def tp_group(): return _STATE.tp_group
def pp_size() -> int: return _STATE.pp
def pp_rank() -> int: return _STATE.pp_rank
def dp_size() -> int: return _STATE.dp
def dp_rank() -> int: return _STATE.dp_rank
def dp_group(): return _STATE.dp_group
def ep_size() -> int: return _STATE.ep
def ep_rank() -> int: return _STATE.ep_rank
def ep_group(): return _STATE.ep_group
def cp_size() -> int: return _STATE.cp
def is_pp_first() -> bool: return _STATE.pp_rank == 0
def is_pp_last() -> bool: return _STATE.pp_rank == _STATE.pp - 1
