"""Pipeline schedule tables.

A schedule is, per pipeline rank, an ordered list of compute nodes ``Node(kind, microbatch, chunk)`` with
``kind`` in ``F`` (forward), ``B`` (backward w.r.t. inputs only), ``W`` (weight gradients of a ``B``) and ``BW``
(full backward).  ``expand_with_comm`` adds the communication nodes ``RF/SF/RB/SB`` (receive / send forward
activations, receive / send backward gradients) around them, which is the table form the reference's
PrimusPipe runtime executes (primus/core/pipeline_parallel/scheduler/schedule_table_factory.py:28-56,
scheduler.py:24-35).

Algorithms (primus/core/pipeline_parallel/scheduler/algorithms/*.py in the reference):
* ``1f1b``          closed form (basic_1f1b.py:40-93)
* ``interleaved``   Megatron's interleaved 1F1B with ``vpp`` chunks per rank; warm-up count
                    ``(pp - rank - 1) * 2 + (vpp - 1) * pp`` (interleaved_1f1b.py:95-209)
* ``zerobubble``    B/W split, W fills the bubbles (zerobubble.py:52-213)
* ``zbv`` / ``v-half`` / ``v-min``   V-shaped placement of two chunks per rank (chunk 1 runs the stages in
                    reverse rank order) with decreasing activation-memory budgets (zbv_greedy.py)
The last four are produced by one dependency-driven greedy list scheduler, so every table is valid by
construction; ``validate`` re-checks any table independently.  The scheduler and the timeline simulator take
per-stage costs of F, B and W and a transfer cost, and ``auto_schedule`` searches activation budgets and
deferred-W limits for the table with the shortest simulated makespan under a memory limit -- the role of the
reference's cost-driven zero-bubble scheduler, which re-plans from the F / B / W / communication times it
measures between ``zero_bubble_pipeline_timers_start_iter`` and ``..._end_iter``
(primus/backends/megatron/core/pipeline_parallel/zerobubble/scheduler/{zb,zbv,graph}.py, runtime.py timers).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence, Union

Cost = Union[float, Sequence[float]]


def _per_stage(c: Cost, S: int) -> list[float]:
    """A scalar cost, or one value per (virtual) stage."""
    if isinstance(c, (int, float)):
        return [float(c)] * S
    c = [float(x) for x in c]
    assert len(c) == S, f"expected {S} per-stage costs, got {len(c)}"
    return c


@dataclass(frozen=True)
class Node:
    kind: str        # F | B | W | BW | RF | SF | RB | SB
    mb: int
    chunk: int = 0
    split: int = 0   # sequence chunk of the micro-batch (schedules with sequence splits)

    def __repr__(self):
        return f"{self.kind}{self.mb}" + (f".{self.chunk}" if self.chunk else "") + (f"s{self.split}" if self.split else "")


def stage_of(rank: int, chunk: int, pp: int, placement: str = "interleaved") -> int:
    """Global (virtual) stage index of chunk ``chunk`` on ``rank``."""
    if placement == "v" and chunk % 2 == 1:
        return chunk * pp + (pp - 1 - rank)
    return chunk * pp + rank


def rank_of_stage(stage: int, pp: int, placement: str = "interleaved") -> tuple[int, int]:
    chunk = stage // pp
    r = stage % pp
    if placement == "v" and chunk % 2 == 1:
        r = pp - 1 - r
    return r, chunk


# ------------------------------------------------------------------------------------------------
def schedule_1f1b(pp: int, m: int) -> list[list[Node]]:
    table = []
    for r in range(pp):
        warm = min(pp - r - 1, m)
        seq = [Node("F", i) for i in range(warm)]
        f, b = warm, 0
        while f < m:
            seq.append(Node("F", f)); f += 1
            seq.append(Node("BW", b)); b += 1
        while b < m:
            seq.append(Node("BW", b)); b += 1
        table.append(seq)
    return table


def schedule_seq1f1b(pp: int, m: int, num_splits: int) -> list[list[Node]]:
    """1F1B over sequence chunks: every micro-batch is ``num_splits`` units.  Forward passes run in (micro-batch, chunk)
    order; the backward passes of a micro-batch run from its last chunk to its first, because a chunk's keys and values
    collect gradients from all later chunks.  A rank therefore needs ``num_splits - 1`` more warm-up forwards than in
    plain 1F1B before the first backward pass (the last chunk's) can start: ``pp - rank - 2 + num_splits`` in all
    (the warm-up count of the reference's schedule,
    primus/backends/megatron/core/pipeline_parallel/zerobubble/scheduler/seq1f1b.py:19-40)."""
    S = num_splits
    total = m * S

    def fwd(i):
        return Node("F", i // S, 0, i % S)

    def bwd(i):
        return Node("BW", i // S, 0, S - 1 - i % S)

    table = []
    for r in range(pp):
        warm = min(pp - r - 2 + S, total)
        seq = [fwd(i) for i in range(warm)]
        for i in range(total - warm):
            seq.append(fwd(warm + i))
            seq.append(bwd(i))
        seq += [bwd(i) for i in range(total - warm, total)]
        table.append(seq)
    return table


def schedule_interleaved(pp: int, vpp: int, m: int) -> list[list[Node]]:
    if m % pp != 0:
        raise ValueError(f"interleaved schedule needs num_microbatches ({m}) divisible by pipeline size ({pp})")
    total = m * vpp

    def fwd_id(k):  # k-th forward of a rank -> (microbatch, chunk)
        group, within = divmod(k, pp * vpp)
        chunk, pos = divmod(within, pp)
        return group * pp + pos, chunk

    def bwd_id(k):
        mb, chunk = fwd_id(k)
        return mb, vpp - 1 - chunk

    table = []
    for r in range(pp):
        warm = min((pp - r - 1) * 2 + (vpp - 1) * pp, total)
        seq = [Node("F", *fwd_id(k)) for k in range(warm)]
        f, b = warm, 0
        while f < total:
            seq.append(Node("F", *fwd_id(f))); f += 1
            seq.append(Node("BW", *bwd_id(b))); b += 1
        while b < total:
            seq.append(Node("BW", *bwd_id(b))); b += 1
        table.append(seq)
    return table


# ------------------------------------------------------------------------------------------------
def schedule_greedy(pp: int, m: int, chunks: int = 1, placement: str = "interleaved", split_w: bool = True,
                    max_inflight: Optional[list[float]] = None, cost_f: Cost = 1.0, cost_b: Cost = 1.0,
                    cost_w: Cost = 1.0, p2p: float = 0.0, max_pending_w: Optional[int] = None) -> list[list[Node]]:
    """Event-driven list scheduling.  ``max_inflight[r]``: activation budget of rank r in units of one
    chunk-forward (a forward adds 1, its B releases ``1 - w_frac`` and its W the rest).  Costs are scalars or one
    value per stage; ``p2p`` is added to a dependency that crosses ranks; ``max_pending_w`` caps the number of
    deferred weight-gradient nodes of a rank (a further B has to wait for a W)."""
    S = pp * chunks
    cost_f, cost_b, cost_w = _per_stage(cost_f, S), _per_stage(cost_b, S), _per_stage(cost_w, S)
    w_frac = 0.25 if split_w else 0.0
    if max_inflight is None:
        max_inflight = [float(S)] * pp
    done_f = [[None] * m for _ in range(S)]   # finish times
    done_b = [[None] * m for _ in range(S)]
    next_f = [0] * S                           # next microbatch to forward on stage s
    next_b = [0] * S
    pending_w: list[list[tuple[int, int]]] = [[] for _ in range(pp)]
    t_rank = [0.0] * pp
    mem = [0.0] * pp
    table: list[list[Node]] = [[] for _ in range(pp)]
    remaining = S * m * (3 if split_w else 2)
    stages_of_rank = [[s for s in range(S) if rank_of_stage(s, pp, placement)[0] == r] for r in range(pp)]
    guard = 0
    while remaining > 0:
        guard += 1
        if guard > 20 * S * m * 3 + 1000:
            raise RuntimeError("schedule search did not converge (activation budget too small?)")
        # pick the rank that can act earliest
        best = None
        for r in range(pp):
            cands = []
            for s in stages_of_rank[r]:
                chunk = rank_of_stage(s, pp, placement)[1]
                mb = next_b[s]
                w_room = not split_w or max_pending_w is None or len(pending_w[r]) < max_pending_w
                if mb < m and done_f[s][mb] is not None and w_room:
                    ready = done_f[s][mb] if s == S - 1 else done_b[s + 1][mb]
                    if ready is not None:
                        if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                            ready += p2p
                        cands.append((max(ready, t_rank[r]), 0, -s, "B", s, mb, chunk))
                mb = next_f[s]
                # keep one activation slot free per deeper chunk of this rank, or shallow forwards could
                # exhaust the budget before the first micro-batch ever reaches its backward
                reserve = float(chunks - 1 - chunk) if placement == "v" or chunks > 1 else 0.0
                if mb < m and mem[r] + 1.0 <= max_inflight[r] - reserve + 1e-9:
                    ready = 0.0 if s == 0 else done_f[s - 1][mb]
                    if ready is not None:
                        if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                            ready += p2p
                        cands.append((max(ready, t_rank[r]), 1, -s, "F", s, mb, chunk))
            if split_w and pending_w[r]:
                s, mb = pending_w[r][0]
                cands.append((t_rank[r], 2, 0, "W", s, mb, rank_of_stage(s, pp, placement)[1]))
            if not cands:
                continue
            # prefer work that can start now; among those: B, then F, then W
            start_now = [c for c in cands if c[0] <= t_rank[r] + 1e-9]
            c = min(start_now, key=lambda x: (x[1], x[2])) if start_now else min(cands, key=lambda x: (x[0], x[1]))
            if best is None or (c[0], r) < (best[0][0], best[1]):
                best = (c, r)
        if best is None:
            raise RuntimeError("deadlock while building the schedule")
        (start, _, _, kind, s, mb, chunk), r = best
        if kind == "F":
            t_rank[r] = start + cost_f[s]
            done_f[s][mb] = t_rank[r]
            next_f[s] += 1
            mem[r] += 1.0
            table[r].append(Node("F", mb, chunk))
        elif kind == "B":
            t_rank[r] = start + cost_b[s] + (0.0 if split_w else cost_w[s])
            done_b[s][mb] = t_rank[r]
            next_b[s] += 1
            mem[r] -= 1.0 - w_frac
            if split_w:
                pending_w[r].append((s, mb))
                table[r].append(Node("B", mb, chunk))
            else:
                table[r].append(Node("BW", mb, chunk))
        else:
            t_rank[r] = start + cost_w[s]
            pending_w[r].pop(0)
            mem[r] -= w_frac
            table[r].append(Node("W", mb, chunk))
        remaining -= 1
    return table


def build_schedule(algorithm: str, pp: int, num_microbatches: int, vpp: Optional[int] = None,
                   num_seq_splits: int = 1) -> dict:
    """Returns {"table": per-rank node lists, "chunks": chunks per rank, "placement": ...}."""
    a = algorithm.lower().replace("_", "-")
    m = num_microbatches
    if num_seq_splits > 1:
        if a not in ("1f1b", "basic-1f1b", "seq1f1b") or (vpp and vpp > 1):
            raise ValueError("num_seq_splits > 1 runs on the 1F1B schedule (no virtual stages, no B / W split)")
        return {"table": schedule_seq1f1b(pp, m, num_seq_splits), "chunks": 1, "placement": "interleaved",
                "algorithm": "seq1f1b", "num_seq_splits": num_seq_splits}
    if pp == 1:
        return {"table": [[n for i in range(m) for n in (Node("F", i), Node("BW", i))]], "chunks": 1,
                "placement": "interleaved", "algorithm": a}
    if a in ("1f1b", "basic-1f1b") and not (vpp and vpp > 1):
        return {"table": schedule_1f1b(pp, m), "chunks": 1, "placement": "interleaved", "algorithm": "1f1b"}
    if a in ("interleaved", "interleaved-1f1b", "1f1b"):
        v = vpp or 2
        return {"table": schedule_interleaved(pp, v, m), "chunks": v, "placement": "interleaved", "algorithm": "interleaved"}
    if a in ("zerobubble", "zero-bubble", "zb", "zbb"):
        budget = [float(pp - r) + 1.0 for r in range(pp)]  # 1F1B-like activation footprint (ZB-H1)
        return {"table": schedule_greedy(pp, m, 1, "interleaved", True, budget), "chunks": 1,
                "placement": "interleaved", "algorithm": "zerobubble"}
    if a in ("zbv", "zbv-formatted", "zbv-greedy", "v-half", "v-min"):
        full = 2.0 * pp
        budget = {"zbv": full, "zbv-formatted": full, "zbv-greedy": full, "v-half": pp + 1.0, "v-min": pp / 2 + 2.0}[a]
        return {"table": schedule_greedy(pp, m, 2, "v", True, [budget] * pp), "chunks": 2, "placement": "v",
                "algorithm": a}
    raise ValueError(f"unknown pipeline algorithm {algorithm!r}")


# ------------------------------------------------------------------------------------------------
def expand_with_comm(table: list[list[Node]], pp: int, chunks: int, placement: str) -> list[list[Node]]:
    """Insert RF/SF/RB/SB nodes. Hand-offs between two chunks of the same rank (V fold) need no comm."""
    S = pp * chunks
    out = []
    for r, seq in enumerate(table):
        res = []
        for n in seq:
            s = stage_of(r, n.chunk, pp, placement)
            if n.kind == "F":
                if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                    res.append(Node("RF", n.mb, n.chunk, n.split))
                res.append(n)
                if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                    res.append(Node("SF", n.mb, n.chunk, n.split))
            elif n.kind in ("B", "BW"):
                if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                    res.append(Node("RB", n.mb, n.chunk, n.split))
                res.append(n)
                if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                    res.append(Node("SB", n.mb, n.chunk, n.split))
            else:
                res.append(n)
        out.append(res)
    return out


def validate(table: list[list[Node]], pp: int, m: int, chunks: int, placement: str, num_seq_splits: int = 1) -> None:
    """Raises AssertionError unless the table is complete and executable without deadlock.  With sequence splits a
    unit of work is a (micro-batch, sequence chunk) pair; a rank must forward the chunks of a micro-batch in order
    and run their backward passes in reverse order."""
    S = pp * chunks
    units = sorted((i, q) for i in range(m) for q in range(num_seq_splits))
    for r, seq in enumerate(table):
        comp = [n for n in seq if n.kind in ("F", "B", "W", "BW")]
        for c in range(chunks):
            fs = [(n.mb, n.split) for n in comp if n.kind == "F" and n.chunk == c]
            bs = [(n.mb, n.split) for n in comp if n.kind in ("B", "BW") and n.chunk == c]
            assert sorted(fs) == units, f"rank {r} chunk {c}: forwards {fs}"
            assert sorted(bs) == units, f"rank {r} chunk {c}: backwards {bs}"
            nb = [(n.mb, n.split) for n in comp if n.kind == "B" and n.chunk == c]
            ws = [(n.mb, n.split) for n in comp if n.kind == "W" and n.chunk == c]
            assert sorted(nb) == sorted(ws), f"rank {r} chunk {c}: every B needs exactly one W"
        seen = set()
        for n in comp:
            if n.kind in ("B", "BW"):
                assert ("F", n.mb, n.chunk, n.split) in seen, f"rank {r}: {n} before its forward"
                assert n.split == num_seq_splits - 1 or ("B", n.mb, n.chunk, n.split + 1) in seen, \
                    f"rank {r}: {n} before the backward of the next sequence chunk"
            if n.kind == "F":
                assert n.split == 0 or ("F", n.mb, n.chunk, n.split - 1) in seen, \
                    f"rank {r}: {n} before the forward of the previous sequence chunk"
            if n.kind == "W":
                assert ("B", n.mb, n.chunk, n.split) in seen, f"rank {r}: {n} before its B"
            seen.add((n.kind if n.kind != "BW" else "B", n.mb, n.chunk, n.split))
    # executability: simulate with blocking dependencies
    ptr = [0] * pp
    fdone, bdone = set(), set()
    comp = [[n for n in seq if n.kind in ("F", "B", "W", "BW")] for seq in table]
    progress = True
    while progress:
        progress = False
        for r in range(pp):
            while ptr[r] < len(comp[r]):
                n = comp[r][ptr[r]]
                s = stage_of(r, n.chunk, pp, placement)
                u = (n.mb, n.split)
                if n.kind == "F":
                    ok = s == 0 or (s - 1, u) in fdone
                elif n.kind in ("B", "BW"):
                    ok = (s, u) in fdone and (s == S - 1 or (s + 1, u) in bdone)
                else:
                    ok = True
                if not ok:
                    break
                if n.kind == "F":
                    fdone.add((s, u))
                elif n.kind in ("B", "BW"):
                    bdone.add((s, u))
                ptr[r] += 1
                progress = True
    assert all(ptr[r] == len(comp[r]) for r in range(pp)), f"schedule deadlocks at {ptr}"


def simulate(table: list[list[Node]], pp: int, chunks: int, placement: str, cost_f: Cost, cost_b: Cost,
             cost_w: Cost, p2p: float = 0.0) -> dict:
    """Timeline simulation: returns makespan, per-rank busy time, bubble fraction and the peak number of
    activations (in chunk-forwards; a split B keeps a quarter until its W) each rank holds."""
    S = pp * chunks
    cost_f, cost_b, cost_w = _per_stage(cost_f, S), _per_stage(cost_b, S), _per_stage(cost_w, S)
    mem = [0.0] * pp
    peak = [0.0] * pp
    comp = [[n for n in seq if n.kind in ("F", "B", "W", "BW")] for seq in table]
    ptr = [0] * pp
    t = [0.0] * pp
    busy = [0.0] * pp
    fdone, bdone = {}, {}
    progress = True
    while progress:
        progress = False
        for r in range(pp):
            while ptr[r] < len(comp[r]):
                n = comp[r][ptr[r]]
                s = stage_of(r, n.chunk, pp, placement)
                if n.kind == "F":
                    dep = 0.0 if s == 0 else fdone.get((s - 1, n.mb, n.split))
                    if dep is None:
                        break
                    if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                        dep += p2p
                    cost = cost_f[s]
                    mem[r] += 1.0
                elif n.kind in ("B", "BW"):
                    if (s, n.mb, n.split) not in fdone:
                        break
                    dep = fdone[(s, n.mb, n.split)] if s == S - 1 else bdone.get((s + 1, n.mb, n.split))
                    if dep is None:
                        break
                    if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                        dep += p2p
                    cost = cost_b[s] + (cost_w[s] if n.kind == "BW" else 0.0)
                    mem[r] -= 1.0 if n.kind == "BW" else 0.75
                else:
                    dep, cost = 0.0, cost_w[s]
                    mem[r] -= 0.25
                peak[r] = max(peak[r], mem[r])
                start = max(t[r], dep)
                t[r] = start + cost
                busy[r] += cost
                if n.kind == "F":
                    fdone[(s, n.mb, n.split)] = t[r]
                elif n.kind in ("B", "BW"):
                    bdone[(s, n.mb, n.split)] = t[r]
                ptr[r] += 1
                progress = True
    makespan = max(t)
    return {"makespan": makespan, "busy": busy, "peak_activations": peak,
            "bubble_fraction": 1.0 - sum(busy) / (pp * makespan) if makespan else 0.0}


# ------------------------------------------------------------------------------------------------
@dataclass
class StageCosts:
    """Measured (or modelled) times of one micro-batch on every virtual stage, in any common unit."""
    f: list[float]
    b: list[float]
    w: list[float]
    p2p: float = 0.0
    # activation budget of every rank in chunk-forwards (None: no limit beyond what the algorithm implies)
    mem_limit: Optional[list[float]] = None
    extra: dict = field(default_factory=dict)


def default_budget(algorithm: str, pp: int) -> tuple[int, str, list[float]]:
    """(chunks, placement, activation budget per rank) of the fixed-budget table of ``algorithm``."""
    a = algorithm.lower().replace("_", "-")
    if a in ("zerobubble", "zero-bubble", "zb", "zbb"):
        return 1, "interleaved", [float(pp - r) + 1.0 for r in range(pp)]
    full = 2.0 * pp
    budget = {"zbv": full, "zbv-formatted": full, "zbv-greedy": full, "v-half": pp + 1.0, "v-min": pp / 2 + 2.0}[a]
    return 2, "v", [budget] * pp


def auto_schedule(algorithm: str, pp: int, m: int, costs: StageCosts, max_pending_w: Optional[int] = None) -> dict:
    """Cost-driven variant of the B / W-split schedules: builds tables with the measured per-stage costs for a
    ladder of activation budgets (from the algorithm's fixed budget up to ``costs.mem_limit``; without a limit the
    fixed budget is kept, so the memory class of the algorithm is preserved) and deferred-W caps, simulates each with the same costs and returns the one with
    the shortest makespan (ties: the smaller activation peak).  The unit-cost table of ``build_schedule`` is always
    among the candidates, so the result is never slower in simulation than the fixed schedule."""
    chunks, placement, base = default_budget(algorithm, pp)
    S = pp * chunks
    limit = costs.mem_limit if costs.mem_limit is not None else list(base)
    floor = float(chunks) + 1.0        # below this the first micro-batch cannot reach its backward
    ladder = []
    for frac in (0.0, 0.25, 0.5, 0.75, 1.0):
        budget = [max(floor, min(l, b + frac * max(l - b, 0.0))) if l >= b else max(floor, l) for b, l in zip(base, limit)]
        if budget not in ladder:
            ladder.append(budget)
    caps = [max_pending_w] if max_pending_w is not None else [None, max(2, pp // 2)]
    cands = []
    fixed = build_schedule(algorithm, pp, m)
    if all(p <= l + 1e-9 for p, l in zip(simulate(fixed["table"], pp, chunks, placement, 1, 1, 1)["peak_activations"], limit)):
        cands.append(("fixed", fixed["table"]))
    for budget in ladder:
        for cap in caps:
            try:
                t = schedule_greedy(pp, m, chunks, placement, True, budget, costs.f, costs.b, costs.w, costs.p2p, cap)
            except RuntimeError:
                continue
            cands.append((f"budget={[round(b, 2) for b in budget]} pending_w={cap}", t))
    assert cands, "no schedule fits the activation limit"
    best = None
    for name, t in cands:
        sim = simulate(t, pp, chunks, placement, costs.f, costs.b, costs.w, costs.p2p)
        key = (round(sim["makespan"], 9), max(sim["peak_activations"]))
        if best is None or key < best[0]:
            best = (key, name, t, sim)
    _, name, table, sim = best
    validate(table, pp, m, chunks, placement)
    base_sim = simulate(fixed["table"], pp, chunks, placement, costs.f, costs.b, costs.w, costs.p2p)
    return {"table": table, "chunks": chunks, "placement": placement, "algorithm": fixed["algorithm"],
            "picked": name, "makespan": sim["makespan"], "fixed_makespan": base_sim["makespan"],
            "bubble_fraction": sim["bubble_fraction"], "peak_activations": sim["peak_activations"]}


def costs_from_events(events_per_rank: list[list[dict]], pp: int, chunks: int, placement: str,
                      p2p: float = 0.0) -> StageCosts:
    """Per-stage mean compute times from timeline events (``kind``, ``chunk``, ``compute_start``, ``end``) of every
    pipeline rank; a BW node is split 2 : 1 into B and W, the usual ratio of the two halves of a backward pass."""
    S = pp * chunks
    acc = {k: [[] for _ in range(S)] for k in "FBW"}
    for r, events in enumerate(events_per_rank):
        for e in events:
            s = stage_of(r, e.get("chunk", 0), pp, placement)
            d = e["end"] - e.get("compute_start", e["start"])
            if e["kind"] == "BW":
                acc["B"][s].append(d * 2 / 3)
                acc["W"][s].append(d / 3)
            elif e["kind"] in acc:
                acc[e["kind"]][s].append(d)

    def mean(xs, fallback):
        return sum(xs) / len(xs) if xs else fallback

    f = [mean(acc["F"][s], 1.0) for s in range(S)]
    b = [mean(acc["B"][s], f[s]) for s in range(S)]
    w = [mean(acc["W"][s], 0.5 * b[s]) for s in range(S)]
    return StageCosts(f, b, w, p2p)
