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
The last four are produced by one dependency-driven greedy list scheduler with unit costs, so every
table is valid by construction; ``validate`` re-checks any table independently.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class Node:
    kind: str        # F | B | W | BW | RF | SF | RB | SB
    mb: int
    chunk: int = 0

    def __repr__(self):
        return f"{self.kind}{self.mb}" + (f".{self.chunk}" if self.chunk else "")


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
                    max_inflight: Optional[list[float]] = None, cost_f: float = 1.0, cost_b: float = 1.0,
                    cost_w: float = 1.0) -> list[list[Node]]:
    """Event-driven list scheduling.  ``max_inflight[r]``: activation budget of rank r in units of one
    chunk-forward (a forward adds 1, its B releases ``1 - w_frac`` and its W the rest)."""
    S = pp * chunks
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
                if mb < m and done_f[s][mb] is not None:
                    ready = done_f[s][mb] if s == S - 1 else done_b[s + 1][mb]
                    if ready is not None:
                        cands.append((max(ready, t_rank[r]), 0, -s, "B", s, mb, chunk))
                mb = next_f[s]
                # keep one activation slot free per deeper chunk of this rank, or shallow forwards could
                # exhaust the budget before the first micro-batch ever reaches its backward
                reserve = float(chunks - 1 - chunk) if placement == "v" or chunks > 1 else 0.0
                if mb < m and mem[r] + 1.0 <= max_inflight[r] - reserve + 1e-9:
                    ready = 0.0 if s == 0 else done_f[s - 1][mb]
                    if ready is not None:
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
            t_rank[r] = start + cost_f
            done_f[s][mb] = t_rank[r]
            next_f[s] += 1
            mem[r] += 1.0
            table[r].append(Node("F", mb, chunk))
        elif kind == "B":
            t_rank[r] = start + cost_b + (0.0 if split_w else cost_w)
            done_b[s][mb] = t_rank[r]
            next_b[s] += 1
            mem[r] -= 1.0 - w_frac
            if split_w:
                pending_w[r].append((s, mb))
                table[r].append(Node("B", mb, chunk))
            else:
                table[r].append(Node("BW", mb, chunk))
        else:
            t_rank[r] = start + cost_w
            pending_w[r].pop(0)
            mem[r] -= w_frac
            table[r].append(Node("W", mb, chunk))
        remaining -= 1
    return table


def build_schedule(algorithm: str, pp: int, num_microbatches: int, vpp: Optional[int] = None) -> dict:
    """Returns {"table": per-rank node lists, "chunks": chunks per rank, "placement": ...}."""
    a = algorithm.lower().replace("_", "-")
    m = num_microbatches
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
                    res.append(Node("RF", n.mb, n.chunk))
                res.append(n)
                if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                    res.append(Node("SF", n.mb, n.chunk))
            elif n.kind in ("B", "BW"):
                if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                    res.append(Node("RB", n.mb, n.chunk))
                res.append(n)
                if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                    res.append(Node("SB", n.mb, n.chunk))
            else:
                res.append(n)
        out.append(res)
    return out


def validate(table: list[list[Node]], pp: int, m: int, chunks: int, placement: str) -> None:
    """Raises AssertionError unless the table is complete and executable without deadlock."""
    S = pp * chunks
    for r, seq in enumerate(table):
        comp = [n for n in seq if n.kind in ("F", "B", "W", "BW")]
        for c in range(chunks):
            fs = [n.mb for n in comp if n.kind == "F" and n.chunk == c]
            bs = [n.mb for n in comp if n.kind in ("B", "BW") and n.chunk == c]
            assert sorted(fs) == list(range(m)), f"rank {r} chunk {c}: forwards {fs}"
            assert sorted(bs) == list(range(m)), f"rank {r} chunk {c}: backwards {bs}"
            nb = [n.mb for n in comp if n.kind == "B" and n.chunk == c]
            ws = [n.mb for n in comp if n.kind == "W" and n.chunk == c]
            assert sorted(nb) == sorted(ws), f"rank {r} chunk {c}: every B needs exactly one W"
        seen = set()
        for n in comp:
            if n.kind in ("B", "BW"):
                assert ("F", n.mb, n.chunk) in seen, f"rank {r}: {n} before its forward"
            if n.kind == "W":
                assert ("B", n.mb, n.chunk) in seen, f"rank {r}: {n} before its B"
            seen.add((n.kind if n.kind != "BW" else "B", n.mb, n.chunk))
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
                if n.kind == "F":
                    ok = s == 0 or (s - 1, n.mb) in fdone
                elif n.kind in ("B", "BW"):
                    ok = (s, n.mb) in fdone and (s == S - 1 or (s + 1, n.mb) in bdone)
                else:
                    ok = True
                if not ok:
                    break
                if n.kind == "F":
                    fdone.add((s, n.mb))
                elif n.kind in ("B", "BW"):
                    bdone.add((s, n.mb))
                ptr[r] += 1
                progress = True
    assert all(ptr[r] == len(comp[r]) for r in range(pp)), f"schedule deadlocks at {ptr}"


def simulate(table: list[list[Node]], pp: int, chunks: int, placement: str, cost_f: float, cost_b: float,
             cost_w: float, p2p: float = 0.0) -> dict:
    """Timeline simulation: returns makespan, per-rank busy time and bubble fraction."""
    S = pp * chunks
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
                    dep = 0.0 if s == 0 else fdone.get((s - 1, n.mb))
                    if dep is None:
                        break
                    if s > 0 and rank_of_stage(s - 1, pp, placement)[0] != r:
                        dep += p2p
                    cost = cost_f
                elif n.kind in ("B", "BW"):
                    if (s, n.mb) not in fdone:
                        break
                    dep = fdone[(s, n.mb)] if s == S - 1 else bdone.get((s + 1, n.mb))
                    if dep is None:
                        break
                    if s < S - 1 and rank_of_stage(s + 1, pp, placement)[0] != r:
                        dep += p2p
                    cost = cost_b + (cost_w if n.kind == "BW" else 0.0)
                else:
                    dep, cost = 0.0, cost_w
                start = max(t[r], dep)
                t[r] = start + cost
                busy[r] += cost
                if n.kind == "F":
                    fdone[(s, n.mb)] = t[r]
                elif n.kind in ("B", "BW"):
                    bdone[(s, n.mb)] = t[r]
                ptr[r] += 1
                progress = True
    makespan = max(t)
    return {"makespan": makespan, "busy": busy, "bubble_fraction": 1.0 - sum(busy) / (pp * makespan) if makespan else 0.0}
