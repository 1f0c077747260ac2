"""Named random-number streams for model-parallel training, and dropout that draws from them.

A tensor-parallel group holds two kinds of activations: *replicated* ones (every rank computes the same tensor) and
*sharded* ones (sequence parallelism: each rank holds its own tokens; attention heads of a rank).  Randomness applied
to a replicated tensor must be identical on all ranks of the group, randomness applied to a shard must differ, or the
sharded model no longer matches the unsharded one statistically.  The tracker keeps one generator state per name and
``fork(name)`` runs a region on it: the device generator is swapped for the named state, the region draws its numbers,
the advanced state is stored back and the device generator restored.

Streams seeded by ``model_parallel_manual_seed(seed)``:

======================  =============================================  =========================================
name                    seed                                           used for
======================  =============================================  =========================================
``data-parallel-rng``   ``seed + 100 * pp_rank``                       replicated activations (no seq. parallel)
``model-parallel-rng``  ``seed + 2718 + tp_rank + 100 * pp_rank``      sequence-sharded activations, heads
``expert-parallel-rng`` ``seed + 1024 + 100 * ep_rank + tp_rank``      tokens inside expert-parallel regions
======================  =============================================  =========================================

Activation recompute has to replay the same numbers: ``checkpoint`` here records the tracker states at the first
forward pass and reinstates them for the recomputation (torch's checkpoint only preserves the device generator).
The states travel in checkpoints (``state_dict`` / ``load_state_dict``).

Counterpart of Megatron's ``CudaRNGStatesTracker`` / ``model_parallel_cuda_manual_seed`` / ``get_cuda_rng_tracker`` as the
reference uses them (megatron/core/tensor_parallel/random.py; seeds set up from primus/modules/trainer/megatron/trainer.py
via ``_set_random_seed``), on CPU generators as well so that the gloo test-suite covers it.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

DATA_PARALLEL = "data-parallel-rng"
MODEL_PARALLEL = "model-parallel-rng"
EXPERT_PARALLEL = "expert-parallel-rng"


class RNGStatesTracker:
    def __init__(self):
        self.device: Optional[torch.device] = None
        self.states: dict[str, torch.Tensor] = {}
        self.seeds: dict[str, int] = {}

    # ------------------------------------------------------------------ device generator access
    def _get(self) -> torch.Tensor:
        if self.device is not None and self.device.type == "cuda":
            return torch.cuda.get_rng_state(self.device)
        return torch.get_rng_state()

    def _set(self, state: torch.Tensor) -> None:
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(state, self.device)
        else:
            torch.set_rng_state(state)

    # ------------------------------------------------------------------ streams
    def reset(self, device=None) -> None:
        self.device = torch.device(device) if device is not None else None
        self.states, self.seeds = {}, {}

    def add(self, name: str, seed: int) -> None:
        if name in self.states:
            raise ValueError(f"random stream {name!r} already exists")
        if seed in self.seeds.values():
            raise ValueError(f"seed {seed} already used by another random stream")
        keep = self._get()
        if self.device is not None and self.device.type == "cuda":
            with torch.cuda.device(self.device):
                torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states[name] = self._get()
        self.seeds[name] = seed
        self._set(keep)

    @contextlib.contextmanager
    def fork(self, name: str = MODEL_PARALLEL):
        if name not in self.states:
            raise KeyError(f"random stream {name!r} was not seeded (call model_parallel_manual_seed first)")
        keep = self._get()
        self._set(self.states[name])
        try:
            yield
        finally:
            self.states[name] = self._get()
            self._set(keep)

    @property
    def active(self) -> bool:
        return bool(self.states)

    def get_states(self) -> dict:
        return {k: v.clone() for k, v in self.states.items()}

    def set_states(self, states: dict) -> None:
        self.states = {k: v.clone() for k, v in states.items()}

    def state_dict(self) -> dict:
        return {"states": {k: v.cpu() for k, v in self.states.items()}, "seeds": dict(self.seeds)}

    def load_state_dict(self, sd: dict) -> None:
        if not sd:
            return
        self.states = {k: v.clone() for k, v in sd["states"].items()}
        self.seeds = dict(sd.get("seeds", {}))


_TRACKER = RNGStatesTracker()


def get_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def model_parallel_manual_seed(seed: int, device=None, tp_rank: int = 0, pp_rank: int = 0, ep_rank: int = 0) -> None:
    """Seed the named streams of this rank (table in the module docstring).  The device's default generator is left as
    it is: parameter initialisation and data order do not depend on whether dropout is in use."""
    t = get_rng_tracker()
    t.reset(device)
    t.add(DATA_PARALLEL, seed + 100 * pp_rank)
    t.add(MODEL_PARALLEL, seed + 2718 + tp_rank + 100 * pp_rank)
    t.add(EXPERT_PARALLEL, seed + 1024 + 100 * ep_rank + tp_rank)


def dropout(x: torch.Tensor, p: float, training: bool, sharded: bool) -> torch.Tensor:
    """Dropout on ``x`` from the stream that fits its layout: ``sharded`` tensors (sequence-parallel shards, per-rank
    heads) draw from the model-parallel stream, replicated ones from the stream all tensor-parallel ranks share."""
    if p <= 0.0 or not training:
        return x
    t = get_rng_tracker()
    if not t.active:
        return torch.nn.functional.dropout(x, p, True)
    with t.fork(MODEL_PARALLEL if sharded else DATA_PARALLEL):
        return torch.nn.functional.dropout(x, p, True)


def checkpoint(fn, *args):
    """``torch.utils.checkpoint.checkpoint`` (non-reentrant) that also replays the named random streams: the states at
    the first call are reinstated for the recomputation, and the states the recomputation found are put back after."""
    from torch.utils.checkpoint import checkpoint as _checkpoint

    t = get_rng_tracker()
    if not t.active:
        return _checkpoint(fn, *args, use_reentrant=False)
    first = {"states": None}

    def run(*a):
        if first["states"] is None:
            first["states"] = t.get_states()
            return fn(*a)
        now = t.get_states()
        t.set_states(first["states"])
        try:
            return fn(*a)
        finally:
            t.set_states(now)

    return _checkpoint(run, *args, use_reentrant=False)
