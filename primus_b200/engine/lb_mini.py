"""LB-Mini: sequence-length load balancing for supervised fine-tuning with variable micro-batch counts.

SFT samples differ in length by orders of magnitude, so giving every data-parallel rank the same *number* of samples
leaves some ranks with several times the tokens of others and everybody waits for the slowest.  For every global
mini-batch this module

1. splits the samples over the data-parallel ranks so that the ranks' total *cost* is as equal as possible
   (Karmarkar-Karp largest-differencing partition; cost = tokens, or ``a s^2 + b s`` when attention is restricted to
   each sample and its quadratic part matters), and
2. packs each rank's samples into micro-batches of at most ``max_token_len`` tokens (first-fit decreasing).  Ranks end
   up with *different numbers of micro-batches* ("mini"); nobody pads up to the longest rank.

That is safe in this engine because gradients are accumulated locally over however many micro-batches a rank has and
the ranks meet once per optimizer step (the bucket reductions of the last micro-batch, or the on-demand reducer of
``parallel/odc.py``); with ``same_num_in_dp`` the count is equalised with empty micro-batches instead, which is what an
engine with per-micro-batch collectives would need.  The loss is normalised by the token count of the whole
mini-batch, so the result does not depend on how the samples were dealt.

Pure host-side index arithmetic.  Counterpart of primus/backends/megatron/sft/lb_mini_packing.py
(``get_seqlen_balanced_partitions``, ``rearrange_micro_batches``) and of the ``sft_lb_mini`` switch of
primus/configs/modules/megatron/sft_trainer.yaml in the reference.
"""
from __future__ import annotations

import heapq
import os
from typing import Callable, Optional

import torch

from .data import BatchStager


# ------------------------------------------------------------------------------------------------ cost models
def seq_costs_linear(lengths: list[int]) -> list[float]:
    return [float(l) for l in lengths]


def seq_costs_fit(lengths: list[int], a: Optional[float] = None, b: Optional[float] = None,
                  norm: Optional[float] = None) -> list[float]:
    """``a s^2 + b s`` with ``s = length / norm``: attention-aware cost for per-sample (segmented) attention.  The
    defaults are a fit for a 1.5B-parameter model; ``LB_MINI_FIT_A / _B / _NORM`` override them (a 7-8B model:
    a = 4.35, b = 8.77)."""
    a = float(os.environ.get("LB_MINI_FIT_A", 1.982122)) if a is None else a
    b = float(os.environ.get("LB_MINI_FIT_B", 2.611821)) if b is None else b
    norm = float(os.environ.get("LB_MINI_FIT_NORM", 32000.0)) if norm is None else norm
    return [a * (l / norm) ** 2 + b * (l / norm) for l in lengths]


COST_MODELS: dict[str, Callable[[list[int]], list[float]]] = {"linear": seq_costs_linear, "fit": seq_costs_fit}


# ------------------------------------------------------------------------------------------------ partitioning
def karmarkar_karp(costs: list[float], k: int, equal_size: bool = False) -> list[list[int]]:
    """Largest-differencing partition of item indices into ``k`` parts with nearly equal cost sums.

    A state is a list of ``k`` (sum, items) buckets sorted by sum; two states are merged by pairing the largest
    bucket of one with the smallest of the other, and the states with the largest spread are merged first.  With
    ``equal_size`` the items are first grouped into states of ``k`` items each (one per bucket), so every part gets the
    same number of items (``len(costs)`` must then be a multiple of ``k``)."""
    n = len(costs)
    if k <= 1:
        return [list(range(n))]
    if equal_size:
        assert n % k == 0, "equal_size partitions need a multiple of k items"
    order = sorted(range(n), key=lambda i: costs[i])
    heap: list = []
    tie = 0
    if equal_size:
        for g in range(0, n, k):
            group = order[g:g + k]
            state = sorted(((costs[i], [i]) for i in group), key=lambda t: t[0])
            heapq.heappush(heap, (-(state[-1][0] - state[0][0]), tie, state))
            tie += 1
    else:
        for i in order:
            state = [(0.0, [])] * (k - 1) + [(costs[i], [i])]
            heapq.heappush(heap, (-costs[i], tie, state))
            tie += 1
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = sorted(((a[j][0] + b[k - 1 - j][0], a[j][1] + b[k - 1 - j][1]) for j in range(k)), key=lambda t: t[0])
        heapq.heappush(heap, (-(merged[-1][0] - merged[0][0]), tie, merged))
        tie += 1
    parts = [sorted(items) for _, items in heap[0][2]]
    # a stable order of the parts (by their smallest item) keeps the assignment independent of tie-breaking details
    parts.sort(key=lambda p: p[0] if p else n)
    return parts


def partition_spread(costs: list[float], parts: list[list[int]]) -> float:
    sums = [sum(costs[i] for i in p) for p in parts]
    return (max(sums) - min(sums)) / max(max(sums), 1e-12)


def pack_micro_batches(lengths: list[int], items: list[int], max_token_len: int) -> list[list[int]]:
    """First-fit-decreasing packing of ``items`` (indices into ``lengths``) into micro-batches of at most
    ``max_token_len`` tokens; a sample longer than the cap gets a micro-batch of its own (it is truncated later)."""
    bins: list[list[int]] = []
    room: list[int] = []
    for i in sorted(items, key=lambda j: -lengths[j]):
        n = min(lengths[i], max_token_len)
        for b in range(len(bins)):
            if room[b] >= n:
                bins[b].append(i)
                room[b] -= n
                break
        else:
            bins.append([i])
            room.append(max_token_len - n)
    return bins


def rearrange_micro_batches(lengths: list[int], dp: int, dp_rank: int, max_token_len: int, cost_model: str = "linear",
                            same_num_in_dp: bool = False) -> tuple[list[list[int]], dict]:
    """Micro-batches (lists of sample indices) of rank ``dp_rank`` for one global mini-batch, plus statistics.
    Every rank computes the whole assignment from the same lengths, so no communication is needed — not even for
    ``same_num_in_dp``, where the rank pads its list with empty micro-batches up to the longest rank's count."""
    costs = COST_MODELS[cost_model](lengths)
    parts = karmarkar_karp(costs, dp)
    per_rank = [pack_micro_batches(lengths, p, max_token_len) for p in parts]
    counts = [len(m) for m in per_rank]
    mine = [list(m) for m in per_rank[dp_rank]]
    if same_num_in_dp:
        mine += [[] for _ in range(max(counts) - len(mine))]
    tokens = [sum(min(lengths[i], max_token_len) for i in p) for p in parts]
    stats = {"micro_batches_per_rank": counts, "tokens_per_rank": tokens, "cost_spread": partition_spread(costs, parts),
             "naive_token_spread": _naive_spread(lengths, dp, max_token_len)}
    return mine, stats


def _naive_spread(lengths: list[int], dp: int, cap: int) -> float:
    """Token imbalance of dealing the samples round-robin, for the log line."""
    sums = [0] * dp
    for i, l in enumerate(lengths):
        sums[i % dp] += min(l, cap)
    return (max(sums) - min(sums)) / max(max(sums), 1)


# ------------------------------------------------------------------------------------------------ staging
class LBMiniStager(BatchStager):
    """Feeds the trainer with balanced, packed micro-batches: every step takes the next ``global_batch_size`` samples
    of the SFT dataset, deals them with :func:`rearrange_micro_batches` and builds one packed sequence of
    ``seq_length`` tokens per micro-batch (micro-batch size 1), with per-sample position ids and boundaries.  Each
    micro-batch carries ``_lb_mini_norm`` = dp / (loss tokens of the whole mini-batch): the trainer multiplies the loss
    mask by it, so that after the data-parallel average the loss is the mean over all answer tokens of the
    mini-batch however many micro-batches a rank ran."""

    def __init__(self, base_dataset, global_batch: int, dp: int, dp_rank: int, device, seq_length: int, align: int = 1,
                 cost_model: str = "linear", same_num_in_dp: bool = False, boundaries: bool = True, log=None):
        class _Sampler:      # only the resumable position is shared with the base class
            def __init__(self, gbs):
                self.gbs, self.consumed = gbs, 0

            def state_dict(self):
                return {"consumed_samples": self.consumed}

            def load_state_dict(self, sd):
                self.consumed = sd["consumed_samples"]

        super().__init__(base_dataset, _Sampler(global_batch), device)
        self.base, self.gbs, self.dp, self.dp_rank = base_dataset, global_batch, dp, dp_rank
        self.seq, self.align = seq_length, max(1, int(align))
        self.cost_model, self.same_num_in_dp, self.boundaries = cost_model, same_num_in_dp, boundaries
        self.log = log
        self.last_stats: dict = {}
        self.max_docs = seq_length // self.align + 1 if self.align > 1 else seq_length + 1

    def _aligned(self, l: int) -> int:
        return min(-(-l // self.align) * self.align, self.seq)

    def _pack_one(self, sample_ids: list[int]) -> dict:
        out = {"tokens": [], "labels": [], "loss_mask": [], "position_ids": []}
        cu = [0]
        pad = self.base.pad_id
        for j in sample_ids:
            it = self.base.item(j)
            room = self.seq - len(out["tokens"])
            if room <= 0:
                break
            n = min(len(it["tokens"]), room)
            padn = min(-n % self.align, room - n)
            for k in out:
                out[k] += it[k][:n]
            out["tokens"] += [pad] * padn
            out["labels"] += [pad] * padn
            out["loss_mask"] += [0.0] * padn
            out["position_ids"] += list(range(n, n + padn))
            cu.append(len(out["tokens"]))
        if cu[-1] < self.seq:
            cu.append(self.seq)
        padn = self.seq - len(out["tokens"])
        item = {"tokens": torch.tensor(out["tokens"] + [pad] * padn, dtype=torch.int64),
                "labels": torch.tensor(out["labels"] + [pad] * padn, dtype=torch.int64),
                "loss_mask": torch.tensor(out["loss_mask"] + [0.0] * padn, dtype=torch.float32),
                "position_ids": torch.tensor(out["position_ids"] + [0] * padn, dtype=torch.int64)}
        if self.boundaries:
            item["host_cu_seqlens"] = torch.tensor(cu + [-1] * (self.max_docs + 1 - len(cu)), dtype=torch.int32)
        return item

    def _load_host(self) -> list[dict]:
        n = len(self.base)
        self._starts.append(self.sampler.consumed)      # kept until the step has been trained on (exact resume)
        ids = [(self.sampler.consumed + i) % n for i in range(self.gbs)]
        self.sampler.consumed += self.gbs
        lengths = [self._aligned(len(self.base.samples[j][0]) - 1) for j in ids]
        mine, stats = rearrange_micro_batches(lengths, self.dp, self.dp_rank, self.seq, self.cost_model,
                                              self.same_num_in_dp)
        loss_tokens = sum(sum(self.base.samples[j][1][1:self.seq + 1]) for j in ids)
        norm = float(self.dp) / max(loss_tokens, 1.0)
        self.last_stats = stats
        if self.log is not None:
            self.log(f"[lb-mini] micro-batches per rank {stats['micro_batches_per_rank']}, tokens per rank "
                     f"{stats['tokens_per_rank']} (spread {stats['cost_spread']:.3f}; round-robin would be "
                     f"{stats['naive_token_spread']:.3f})")
        mbs = []
        for group in mine:
            b = self._pack_one([ids[i] for i in group])
            b = {k: (v if k.startswith("host_") else v.unsqueeze(0)) for k, v in b.items()}
            if "host_cu_seqlens" in b:
                b["host_cu_seqlens"] = b["host_cu_seqlens"].unsqueeze(0)
            b["_lb_mini_norm"] = torch.tensor(norm, dtype=torch.float32)
            if self.pin:
                b = {k: (v if k.startswith("host_") else v.pin_memory()) for k, v in b.items()}
            mbs.append(b)
        return mbs
