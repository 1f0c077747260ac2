"""Megatron-LM indexed datasets (``<prefix>.bin`` + ``<prefix>.idx``, the "MMIDIDX" memory-mapped format) and the GPT
sample view on top of them, so that corpora pre-processed for the reference's Megatron backend can be used as they
are (``data_path`` there is a list of ``weight prefix`` pairs; primus/configs/modules/megatron/trainer_base.yaml:261-300).

``.idx`` layout: 9-byte magic ``MMIDIDX\\0\\0``, uint64 version (1), uint8 dtype code, uint64 number of sequences,
uint64 number of document boundaries, int32 sizes[sequences], int64 byte pointers[sequences], int64
document_indices[boundaries].  ``.bin`` is the concatenation of the token arrays.

``GPTIndexedDataset`` cuts the token stream of the (shuffled) documents into samples of ``seq_length + 1`` tokens,
epoch after epoch; sample ``i`` is a pure function of (seed, i), so data-parallel ranks and resumed runs need no
communication or state beyond the consumed-sample counter.  ``BlendedDataset`` mixes several corpora by weight.
"""
from __future__ import annotations

import struct

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def write_indexed_dataset(prefix: str, documents, dtype=np.int32) -> None:
    """Writes ``documents`` (an iterable of 1-D integer arrays, one per document) in the mmap format."""
    dtype = np.dtype(dtype)
    sizes = []
    with open(prefix + ".bin", "wb") as f:
        for d in documents:
            a = np.asarray(d, dtype=dtype)
            f.write(a.tobytes(order="C"))
            sizes.append(len(a))
    sizes = np.asarray(sizes, dtype=np.int32)
    pointers = np.zeros(len(sizes), dtype=np.int64)
    if len(sizes) > 1:
        np.cumsum(sizes[:-1].astype(np.int64) * dtype.itemsize, out=pointers[1:])
    doc_idx = np.arange(len(sizes) + 1, dtype=np.int64)
    with open(prefix + ".idx", "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", _CODES[dtype]))
        f.write(struct.pack("<Q", len(sizes)))
        f.write(struct.pack("<Q", len(doc_idx)))
        f.write(sizes.tobytes())
        f.write(pointers.tobytes())
        f.write(doc_idx.tobytes())


class MMapIndexedDataset:
    """Random access to the sequences of an indexed dataset (zero-copy views of the memory-mapped ``.bin``)."""

    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError(f"{prefix}.idx is not an MMIDIDX index file")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            (n,) = struct.unpack("<Q", f.read(8))
            (nd,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self.dtype = np.dtype(_DTYPES[code])
        idx = np.memmap(prefix + ".idx", mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n, offset=offset)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=nd, offset=offset + self.sizes.nbytes + self.pointers.nbytes)
        self.bin = np.memmap(prefix + ".bin", mode="r", order="C")

    def __len__(self):
        return len(self.sizes)

    def get(self, i: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        n = int(self.sizes[i]) - offset if length is None else length
        return np.frombuffer(self.bin, dtype=self.dtype, count=n, offset=int(self.pointers[i]) + offset * self.dtype.itemsize)

    def __getitem__(self, i: int) -> np.ndarray:
        return self.get(i)


class GPTIndexedDataset:
    """Fixed-length samples over the documents of an :class:`MMapIndexedDataset`.

    Every epoch visits the documents in a new random order (seeded); a sample is ``seq_length + 1`` consecutive
    tokens of that stream (neighbouring samples share one token, as in Megatron's GPT dataset).  ``eod_token`` with
    ``eod_mask_loss`` masks the loss of end-of-document tokens; ``reset_position_ids`` restarts positions after them."""

    def __init__(self, prefix: str, seq_length: int, seed: int = 1234, eod_token: int | None = None,
                 eod_mask_loss: bool = False, reset_position_ids: bool = False):
        self.ds = MMapIndexedDataset(prefix)
        self.seq_length, self.seed = seq_length, seed
        self.eod, self.eod_mask_loss, self.reset_position_ids = eod_token, eod_mask_loss, reset_position_ids
        self.tokens_per_epoch = int(self.ds.sizes.astype(np.int64).sum())
        if self.tokens_per_epoch <= seq_length:
            raise ValueError(f"{prefix}: {self.tokens_per_epoch} tokens are fewer than one sample of {seq_length + 1}")
        self.samples_per_epoch = (self.tokens_per_epoch - 1) // seq_length
        self._epoch_cache: dict = {}

    def __len__(self):
        return 1 << 40

    def _epoch(self, e: int):
        if e not in self._epoch_cache:
            order = np.random.Generator(np.random.PCG64([self.seed, e])).permutation(len(self.ds))
            ends = np.cumsum(self.ds.sizes[order].astype(np.int64))
            self._epoch_cache = {e: (order, ends)}          # keep one epoch
        return self._epoch_cache[e]

    def _span(self, e: int, start: int, n: int) -> np.ndarray:
        """``n`` tokens of epoch ``e``'s stream from stream position ``start``."""
        order, ends = self._epoch(e)
        out = np.empty(n, dtype=np.int64)
        d = int(np.searchsorted(ends, start, side="right"))
        pos, filled = start - (int(ends[d - 1]) if d else 0), 0
        while filled < n:
            doc = int(order[d])
            take = min(int(self.ds.sizes[doc]) - pos, n - filled)
            out[filled:filled + take] = self.ds.get(doc, pos, take)
            filled += take
            d, pos = d + 1, 0
        return out

    def __getitem__(self, idx: int) -> dict:
        e, i = divmod(idx, self.samples_per_epoch)
        x = self._span(e, i * self.seq_length, self.seq_length + 1)
        tokens, labels = x[:-1], x[1:]
        mask = np.ones(self.seq_length, dtype=np.float32)
        item = {"tokens": torch.from_numpy(tokens.copy()), "labels": torch.from_numpy(labels.copy())}
        if self.eod is not None and self.eod_mask_loss:
            mask[tokens == self.eod] = 0.0
        if self.eod is not None and self.reset_position_ids:
            pos = np.arange(self.seq_length, dtype=np.int64)
            starts = np.flatnonzero(tokens == self.eod) + 1
            for s in starts[starts < self.seq_length]:
                pos[s:] = np.arange(self.seq_length - s)
            item["position_ids"] = torch.from_numpy(pos)
        item["loss_mask"] = torch.from_numpy(mask)
        return item


class BlendedDataset:
    """Weighted mixture of datasets: sample ``i`` comes from the dataset whose running share is furthest behind its
    weight (the deterministic greedy assignment Megatron's blending uses), at that dataset's next unused index."""

    def __init__(self, datasets: list, weights: list[float], size: int = 1 << 22):
        w = np.asarray(weights, dtype=np.float64)
        w = w / w.sum()
        self.datasets = datasets
        counts = np.zeros(len(datasets), dtype=np.int64)
        self.which = np.empty(size, dtype=np.int16)
        self.local = np.empty(size, dtype=np.int64)
        for i in range(size):
            k = int(np.argmax(w * (i + 1) - counts))
            self.which[i], self.local[i] = k, counts[k]
            counts[k] += 1
        self.size = size

    def __len__(self):
        return 1 << 40

    def __getitem__(self, idx: int) -> dict:
        lap, i = divmod(idx, self.size)
        k = int(self.which[i])
        per_lap = int((self.which == k).sum())
        return self.datasets[k][lap * per_lap + int(self.local[i])]


def build_gpt_dataset(data_path, seq_length: int, seed: int = 1234, **kw):
    """``data_path``: a prefix, or Megatron's ``[weight, prefix, weight, prefix, ...]`` list / whitespace string."""
    if isinstance(data_path, str):
        data_path = data_path.split()
    if len(data_path) == 1:
        return GPTIndexedDataset(data_path[0], seq_length, seed, **kw)
    assert len(data_path) % 2 == 0, "data_path: weight prefix weight prefix ..."
    weights = [float(x) for x in data_path[0::2]]
    sets = [GPTIndexedDataset(p, seq_length, seed + 17 * j, **kw) for j, p in enumerate(data_path[1::2])]
    return BlendedDataset(sets, weights, size=1 << 16)
