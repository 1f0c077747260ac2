"""Datasets and batch staging.

``MockGPTDataset`` is the synthetic pre-training dataset (uniform-random token ids from a fixed seed,
labels = inputs shifted by one) that ``mock_data: true`` selects in the reference
(primus/backends/megatron/patches/args/mock_data_patches.py:32-45).  ``BatchStager`` keeps batches
in pinned host memory and copies them to the device on a side stream one step ahead, the role of
the reference's CUDA prefetch iterator (primus/backends/megatron/data/cuda_prefetch.py:27-84) and
``DataLoaderStore`` (primus/backends/megatron/data_loader_store.py:97-132).
"""
from __future__ import annotations

from typing import Iterator, Optional

import numpy as np
import torch


class MockGPTDataset:
    """Deterministic random token sequences. Sample ``i`` is a function of (seed, i) only, so every
    data-parallel rank can draw its own samples without communication and a resumed run sees the
    same stream."""

    def __init__(self, vocab_size: int, seq_length: int, seed: int = 1234, num_samples: int = 1 << 40):
        self.vocab_size, self.seq_length, self.seed, self.num_samples = vocab_size, seq_length, seed, num_samples

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx: int) -> dict:
        rng = np.random.Generator(np.random.PCG64([self.seed, idx]))
        x = rng.integers(0, self.vocab_size, size=self.seq_length + 1, dtype=np.int64)
        return {"tokens": torch.from_numpy(x[:-1].copy()), "labels": torch.from_numpy(x[1:].copy()),
                "loss_mask": torch.ones(self.seq_length, dtype=torch.float32)}


class PatternGPTDataset(MockGPTDataset):
    """Learnable synthetic data: every sample repeats a random period of ``period`` tokens, so a model that attends
    ``period`` tokens back predicts everything after the first period (used for loss-curve comparisons between
    precisions; random tokens alone can only be fitted by their unigram statistics).  Tokens come from the first
    ``alphabet`` ids, so the unigram fit alone already moves the loss from ln(vocab) to ln(alphabet) within a few
    dozen steps, and copying from one period back moves it towards zero after that."""

    def __init__(self, vocab_size: int, seq_length: int, seed: int = 1234, period: int = 32, alphabet: int = 512):
        super().__init__(vocab_size, seq_length, seed)
        self.period = period
        self.alphabet = min(alphabet, vocab_size)

    def __getitem__(self, idx: int) -> dict:
        rng = np.random.Generator(np.random.PCG64([self.seed, idx]))
        base = rng.integers(0, self.alphabet, size=self.period, dtype=np.int64)
        x = np.tile(base, self.seq_length // self.period + 2)[: self.seq_length + 1]
        return {"tokens": torch.from_numpy(x[:-1].copy()), "labels": torch.from_numpy(x[1:].copy()),
                "loss_mask": torch.ones(self.seq_length, dtype=torch.float32)}


class MarkovGPTDataset(MockGPTDataset):
    """Learnable synthetic data with a smooth loss curve: a first-order Markov chain over the first ``alphabet`` ids.
    The next token is a fixed permutation of the current one with probability ``1 - noise`` and uniform otherwise, so
    the loss falls steadily from ln(vocab) towards the chain's entropy as the model fits the transition table (no
    sudden in-context-copying phase as with periodic sequences, whose timing is sensitive to rounding noise)."""

    def __init__(self, vocab_size: int, seq_length: int, seed: int = 1234, alphabet: int = 512, noise: float = 0.15):
        super().__init__(vocab_size, seq_length, seed)
        self.alphabet = min(alphabet, vocab_size)
        self.noise = noise
        self.perm = np.random.Generator(np.random.PCG64([seed, 0x5EED])).permutation(self.alphabet).astype(np.int64)

    def __getitem__(self, idx: int) -> dict:
        rng = np.random.Generator(np.random.PCG64([self.seed, idx]))
        n = self.seq_length + 1
        jump = rng.random(n) < self.noise
        fresh = rng.integers(0, self.alphabet, size=n, dtype=np.int64)
        x = np.empty(n, dtype=np.int64)
        x[0] = fresh[0]
        for t in range(1, n):
            x[t] = fresh[t] if jump[t] else self.perm[x[t - 1]]
        return {"tokens": torch.from_numpy(x[:-1].copy()), "labels": torch.from_numpy(x[1:].copy()),
                "loss_mask": torch.ones(self.seq_length, dtype=torch.float32)}


class IndexedTokenDataset:
    """Memory-mapped token file (one flat int32/uint16 array) cut into fixed-length samples.
    ``path.bin`` holds the ids; an optional ``path.idx.npy`` holds document start offsets."""

    def __init__(self, path: str, seq_length: int, dtype=np.int32):
        self.data = np.memmap(path, dtype=dtype, mode="r")
        self.seq_length = seq_length
        self.num_samples = (len(self.data) - 1) // seq_length

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx: int) -> dict:
        s = idx * self.seq_length
        x = torch.from_numpy(np.asarray(self.data[s:s + self.seq_length + 1], dtype=np.int64))
        return {"tokens": x[:-1].clone(), "labels": x[1:].clone(),
                "loss_mask": torch.ones(self.seq_length, dtype=torch.float32)}


class MicroBatchSampler:
    """Yields the sample indices of successive micro-batches for one data-parallel rank.

    Global sample order is 0,1,2,...; global batch ``g`` covers ``[g*gbs, (g+1)*gbs)``; inside it, rank
    ``r`` takes micro-batch ``m`` = samples ``g*gbs + (m*dp + r)*mbs + [0, mbs)`` (Megatron's
    interleaving).  ``consumed_samples`` makes the stream resumable."""

    def __init__(self, global_batch: int, micro_batch: int, dp_size: int, dp_rank: int, consumed_samples: int = 0,
                 rampup=None):
        """``rampup``: ``(start, increment, samples)`` -- the global batch grows from ``start`` by ``increment`` in equal
        stretches of the first ``samples`` samples until it reaches ``global_batch`` (Megatron's ``rampup_batch_size``);
        every size on the way must be a multiple of ``micro_batch x dp_size``."""
        assert global_batch % (micro_batch * dp_size) == 0
        self.gbs, self.mbs, self.dp, self.rank = global_batch, micro_batch, dp_size, dp_rank
        self.consumed = consumed_samples
        self.num_micro = global_batch // (micro_batch * dp_size)
        self.rampup = None
        if rampup:
            start, incr, samples = (int(x) for x in rampup)
            assert incr > 0 and (global_batch - start) % incr == 0 and start > 0, \
                "rampup_batch_size: the increments must lead from the start size exactly to global_batch_size"
            for b in range(start, global_batch + 1, incr):
                assert b % (micro_batch * dp_size) == 0, f"rampup_batch_size: {b} is not a multiple of micro batch x dp"
            self.rampup = (start, incr, samples)

    def batch_size_at(self, consumed: int) -> int:
        """Global batch size of the step that starts after ``consumed`` samples."""
        if not self.rampup:
            return self.gbs
        start, incr, samples = self.rampup
        steps = (self.gbs - start) // incr
        if consumed >= samples or steps == 0:
            return self.gbs
        return start + incr * int(consumed / (samples / steps))

    def next_global_batch(self) -> list[list[int]]:
        base = self.consumed
        gbs = self.batch_size_at(base)
        out = [[base + (m * self.dp + self.rank) * self.mbs + i for i in range(self.mbs)]
               for m in range(gbs // (self.mbs * self.dp))]
        self.consumed += gbs
        self.last_batch_size = gbs
        return out

    def state_dict(self):
        return {"consumed_samples": self.consumed}

    def load_state_dict(self, sd):
        self.consumed = sd["consumed_samples"]


def collate(samples: list[dict]) -> dict:
    return {k: torch.stack([s[k] for s in samples]) for k in samples[0]}


class BatchStager:
    """Double-buffered pinned-host -> device staging of micro-batches on a side stream.

    ``num_workers`` > 0: the host side of a step (reading / tokenising the samples, collating, pinning) runs on worker
    threads, one step ahead of the device copy, so that it overlaps the training step instead of sitting between two of
    them; the samples of a step are fetched by up to ``num_workers`` threads.  The order of the samples is the
    sampler's in every case.  (The reference hands this to the data loader's worker processes: ``num_workers`` in
    primus/configs/modules/megatron/trainer_base.yaml.)"""

    def __init__(self, dataset, sampler: MicroBatchSampler, device, pin: Optional[bool] = None, num_workers: int = 0):
        self.dataset, self.sampler, self.device = dataset, sampler, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.pin = self.cuda if pin is None else pin
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._next = None
        self._host_future = None
        self._starts: list = []             # sample offsets of the steps handed out but not yet trained on
        self.h2d_bytes_last_step = 0
        self.num_workers = int(num_workers or 0)
        self._pool = self._loader = None
        if self.num_workers > 0:
            from concurrent.futures import ThreadPoolExecutor

            self._pool = ThreadPoolExecutor(self.num_workers, thread_name_prefix="primus-b200-data")
            self._loader = ThreadPoolExecutor(1, thread_name_prefix="primus-b200-batch")

    def _build_host(self, index_lists: list) -> list[dict]:
        if self.cuda and self._loader is not None:
            torch.cuda.set_device(self.device)      # a new thread starts on device 0: pin through this rank's context
        mbs = []
        for idxs in index_lists:
            samples = list(self._pool.map(self.dataset.__getitem__, idxs)) if self._pool else [self.dataset[i] for i in idxs]
            b = collate(samples)
            if self.pin:
                b = {k: (v if k.startswith("host_") else v.pin_memory()) for k, v in b.items()}
            mbs.append(b)
        return mbs

    def _hand_out(self) -> list:
        """The next step's index lists; its start is remembered until training has consumed the step."""
        self._starts.append(self.sampler.consumed)
        return self.sampler.next_global_batch()

    def _load_host(self) -> list[dict]:
        if self._loader is None:
            return self._build_host(self._hand_out())
        if self._host_future is None:       # first step: nothing is in flight yet
            self._host_future = self._loader.submit(self._build_host, self._hand_out())
        host = self._host_future.result()
        self._host_future = self._loader.submit(self._build_host, self._hand_out())
        return host

    def _to_device(self, host_mbs: list[dict]):
        if not self.cuda:
            return host_mbs, None, sum(v.numel() * v.element_size() for b in host_mbs for v in b.values())
        nbytes = 0
        with torch.cuda.stream(self.stream):
            dev = []
            for b in host_mbs:
                d = {}
                for k, v in b.items():
                    if k.startswith("host_"):      # host-side metadata (document boundaries): not copied
                        d[k] = v
                        continue
                    d[k] = v.to(self.device, non_blocking=True)
                    nbytes += v.numel() * v.element_size()
                dev.append(d)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return dev, ev, nbytes

    def prefetch(self):
        if self._next is None:
            self._next = self._to_device(self._load_host())

    def next_step(self) -> list[dict]:
        """Micro-batches of the next global step (device tensors); also starts staging the one after."""
        self.prefetch()
        dev, ev, nbytes = self._next
        self._next = None
        if self._starts:            # a stager that overrides _load_host without recording starts keeps working
            self._starts.pop(0)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            for b in dev:
                for v in b.values():
                    if v.is_cuda:
                        v.record_stream(torch.cuda.current_stream())
        self.h2d_bytes_last_step = nbytes
        return dev

    def state_dict(self):
        # a prefetched-but-unconsumed step must be replayed after a resume
        # steps staged or in flight are replayed after a resume: the stream continues where the oldest of them starts
        return {"consumed_samples": self._starts[0] if self._starts else self.sampler.consumed}

    def load_state_dict(self, sd):
        self._next = None
        if self._host_future is not None:
            self._host_future.result()          # let the worker finish before the sampler is rewound
            self._host_future = None
        self._starts = []
        self.sampler.load_state_dict(sd)
