"""Supervised fine-tuning: chat / instruction formatting, answer-only loss masks, sequence packing, LoRA.

* Formatters turn one record into (prompt, answer) text: ``squad`` (context / question / answers), ``alpaca``
  (instruction / input / output), ``chatml`` and ``openai`` message lists
  (primus/backends/megatron/sft/formatters.py:31-169 in the reference).
* :class:`SFTDataset` tokenises, truncates and builds ``tokens / labels / loss_mask`` with the loss only on
  answer tokens when ``answer_only_loss`` (sft/dataset.py:23).
* Packing: ``first_fit``, ``first_fit_decreasing`` and ``first_fit_shuffle`` bin packing of samples into
  fixed-length sequences with per-sample ``position_ids`` restarting at 0 (sft/packing.py:196-265,469-710).
* LoRA: :func:`apply_lora` wraps the chosen linear weights with low-rank adapters (``W + (alpha/r) B A``), freezes
  the base model and :func:`merge_lora` folds the adapters back (peft/lora.py:56-301, lora_layers.py:38-715).
* :class:`SFTTrainer` is the trainer the CLI runs for ``train posttrain`` (megatron_sft_trainer.py:78).
"""
from __future__ import annotations

import json
import os
import random
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn as nn

from .data import MicroBatchSampler, BatchStager
from .pretrain import PretrainTrainer


# ------------------------------------------------------------------------------------------------ formatters
def format_squad(r: dict) -> tuple[str, str]:
    ans = r.get("answers", {})
    text = ans.get("text", [""])[0] if isinstance(ans, dict) else (ans[0] if ans else "")
    return f"Context: {r.get('context', '')} Question: {r.get('question', '')} Answer:", " " + text


def format_alpaca(r: dict) -> tuple[str, str]:
    if r.get("input"):
        p = ("Below is an instruction that describes a task, paired with an input that provides further context. "
             f"Write a response that appropriately completes the request.\n\n### Instruction:\n{r['instruction']}\n\n"
             f"### Input:\n{r['input']}\n\n### Response:\n")
    else:
        p = ("Below is an instruction that describes a task. Write a response that appropriately completes the "
             f"request.\n\n### Instruction:\n{r['instruction']}\n\n### Response:\n")
    return p, r.get("output", "")


def format_messages(r: dict, chatml: bool = True) -> tuple[str, str]:
    msgs = r.get("messages") or r.get("conversations") or []
    if not msgs:
        return "", ""
    *ctx, last = msgs
    role = lambda m: m.get("role") or {"human": "user", "gpt": "assistant"}.get(m.get("from"), m.get("from"))  # noqa: E731
    text = lambda m: m.get("content") if m.get("content") is not None else m.get("value", "")  # noqa: E731
    if chatml:
        p = "".join(f"<|im_start|>{role(m)}\n{text(m)}<|im_end|>\n" for m in ctx) + f"<|im_start|>{role(last)}\n"
        return p, f"{text(last)}<|im_end|>\n"
    p = "".join(f"{role(m)}: {text(m)}\n" for m in ctx) + f"{role(last)}: "
    return p, text(last)


FORMATTERS: dict[str, Callable[[dict], tuple[str, str]]] = {
    "squad": format_squad, "alpaca": format_alpaca, "chatml": lambda r: format_messages(r, True),
    "openai": lambda r: format_messages(r, False),
}


class ByteTokenizer:
    """Fallback tokenizer (UTF-8 bytes, 256 = end of document) used when no tokenizer model is configured."""
    vocab_size = 257
    eos_token_id = 256

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))


# ------------------------------------------------------------------------------------------------ dataset
class SFTDataset:
    def __init__(self, records: list[dict], tokenizer, seq_length: int, fmt: str = "alpaca", answer_only_loss: bool = True,
                 pad_id: int = 0):
        self.samples = []
        f = FORMATTERS[fmt]
        eos = getattr(tokenizer, "eos_token_id", None)
        for r in records:
            p, a = f(r)
            pi, ai = tokenizer.encode(p), tokenizer.encode(a)
            if eos is not None:
                ai = ai + [eos]
            ids = (pi + ai)[: seq_length + 1]
            n_prompt = min(len(pi), len(ids))
            mask = [0.0 if (answer_only_loss and i < n_prompt) else 1.0 for i in range(len(ids))]
            if len(ids) >= 2:
                self.samples.append((ids, mask))
        self.seq_length, self.pad_id = seq_length, pad_id

    @classmethod
    def from_jsonl(cls, path: str, *a, **kw):
        with open(path) as fh:
            return cls([json.loads(l) for l in fh if l.strip()], *a, **kw)

    def __len__(self):
        return len(self.samples)

    def lengths(self) -> list[int]:
        return [len(s[0]) - 1 for s in self.samples]

    def item(self, i: int) -> dict:
        ids, mask = self.samples[i]
        return {"tokens": ids[:-1], "labels": ids[1:], "loss_mask": mask[1:], "position_ids": list(range(len(ids) - 1))}

    def __getitem__(self, i: int) -> dict:
        it = self.item(i % len(self.samples))
        return _pad(it, self.seq_length, self.pad_id)


def _pad(it: dict, seq: int, pad_id: int) -> dict:
    n = len(it["tokens"])
    padn = seq - n
    return {"tokens": torch.tensor(it["tokens"] + [pad_id] * padn, dtype=torch.int64),
            "labels": torch.tensor(it["labels"] + [pad_id] * padn, dtype=torch.int64),
            "loss_mask": torch.tensor(it["loss_mask"] + [0.0] * padn, dtype=torch.float32),
            "position_ids": torch.tensor(it["position_ids"] + [0] * padn, dtype=torch.int64)}


# ------------------------------------------------------------------------------------------------ packing
def pack_bins(lengths: list[int], capacity: int, algorithm: str = "first_fit_decreasing", seed: int = 0) -> list[list[int]]:
    """Bin packing of sample indices; every bin's total length is <= capacity."""
    order = list(range(len(lengths)))
    if algorithm == "first_fit_decreasing":
        order.sort(key=lambda i: -lengths[i])
    elif algorithm == "first_fit_shuffle":
        random.Random(seed).shuffle(order)
    elif algorithm != "first_fit":
        raise ValueError(f"unknown packing algorithm {algorithm!r}")
    bins: list[list[int]] = []
    space: list[int] = []
    for i in order:
        n = min(lengths[i], capacity)
        for b in range(len(bins)):
            if space[b] >= n:
                bins[b].append(i)
                space[b] -= n
                break
        else:
            bins.append([i])
            space.append(capacity - n)
    return bins


class PackedSFTDataset:
    """Several samples per sequence; position ids restart at every sample and the first label of a sample is
    masked so that no loss crosses a boundary.  With ``align`` > 1 every sample is padded to a multiple of ``align``
    tokens (the attention kernels work on 128-token blocks) and ``host_cu_seqlens`` carries the sample boundaries
    (cumulative token offsets, -1 padded to a fixed length) so that attention can be restricted to each sample: the
    role of the packed-sequence (THD) parameters of the reference (sft/forward_step.py:184-232)."""

    def __init__(self, base: SFTDataset, algorithm: str = "first_fit_decreasing", seed: int = 0, align: int = 1,
                 boundaries: bool = True, bins: Optional[list] = None):
        self.base = base
        self.boundaries = boundaries
        self.align = max(1, int(align))
        assert base.seq_length % self.align == 0
        lengths = [-(-l // self.align) * self.align for l in base.lengths()]
        self.bins = bins if bins is not None else pack_bins(lengths, base.seq_length, algorithm, seed)
        self.max_docs = base.seq_length // self.align + 1 if self.align > 1 else base.seq_length + 1

    def __len__(self):
        return len(self.bins)

    def __getitem__(self, i: int) -> dict:
        out = {"tokens": [], "labels": [], "loss_mask": [], "position_ids": []}
        seq = self.base.seq_length
        cu = [0]
        for j in self.bins[i % len(self.bins)]:
            it = self.base.item(j)
            room = seq - len(out["tokens"])
            if room <= 0:
                break
            n = min(len(it["tokens"]), room)
            padn = min(-n % self.align, room - n)
            for k in out:
                out[k] += it[k][:n]
            if padn:
                out["tokens"] += [self.base.pad_id] * padn
                out["labels"] += [self.base.pad_id] * padn
                out["loss_mask"] += [0.0] * padn
                out["position_ids"] += list(range(n, n + padn))
            cu.append(len(out["tokens"]))
        if cu[-1] < seq:
            cu.append(seq)                       # the padding tail is a segment of its own
        item = _pad(out, seq, self.base.pad_id)
        if self.boundaries:
            item["host_cu_seqlens"] = torch.tensor(cu + [-1] * (self.max_docs + 1 - len(cu)), dtype=torch.int32)
        return item

    def packing_efficiency(self) -> float:
        used = sum(min(l, self.base.seq_length) for l in self.base.lengths())
        return used / (len(self.bins) * self.base.seq_length)


# ------------------------------------------------------------------------------------------------ pack cache
PACK_FORMAT_VERSION = 1


def pack_cache_dir(configured: Optional[str] = None) -> str:
    """Directory of cached tokenised / packed SFT data: the configured ``sft_pack_cache_dir``, else
    ``$PRIMUS_PACK_CACHE_DIR``, ``$HF_DATASETS_CACHE/primus_packed``, ``$HF_HOME/primus_packed``,
    ``~/.cache/primus_packed_sft`` in that order (the reference's resolution, sft/packing.py:389-411)."""
    base = configured or os.environ.get("PRIMUS_PACK_CACHE_DIR")
    if not base:
        for var in ("HF_DATASETS_CACHE", "HF_HOME"):
            if os.environ.get(var):
                base = os.path.join(os.environ[var], "primus_packed")
                break
    base = base or os.path.expanduser("~/.cache/primus_packed_sft")
    os.makedirs(base, exist_ok=True)
    return base


def tokenizer_identity(tokenizer) -> str:
    """A stable name for the tokenizer in cache keys (``$PRIMUS_PACK_TOKENIZER_ID`` overrides it)."""
    if os.environ.get("PRIMUS_PACK_TOKENIZER_ID"):
        return os.environ["PRIMUS_PACK_TOKENIZER_ID"]
    for attr in ("name_or_path", "tokenizer_model_name", "vocab_file"):
        v = getattr(tokenizer, attr, None)
        if isinstance(v, str) and v:
            return v
    return f"{type(tokenizer).__name__}_vocab{getattr(tokenizer, 'vocab_size', None)}"


def pack_cache_key(path: str, fmt: str, seq_length: int, pad_id: int, tokenizer_id: str, answer_only: bool,
                   algorithm: str, align: int, seed: int) -> str:
    """16 hex digits that change with anything that changes the tokenised or packed result, including the data file's
    size and modification time."""
    import hashlib

    try:
        st = os.stat(path)
        stamp = f"{st.st_size}:{int(st.st_mtime)}"
    except OSError:
        stamp = "?"
    blob = "|".join(str(x) for x in (PACK_FORMAT_VERSION, os.path.abspath(path), stamp, fmt, seq_length, pad_id,
                                     tokenizer_id, int(answer_only), algorithm, align, seed))
    return hashlib.sha256(blob.encode()).hexdigest()[:16]


def load_or_build_packed(path: str, tokenizer, seq_length: int, fmt: str, answer_only: bool, algorithm: str, seed: int,
                         align: int, boundaries: bool, cache_dir: Optional[str] = None, log=None) -> "PackedSFTDataset":
    """``PackedSFTDataset`` for a jsonl file through the pack cache: tokenisation and bin packing of a large SFT set
    take minutes, so their results (token ids, loss masks, bins) are stored once per cache key and every later run --
    and every other rank of this run -- loads them.  Rank 0 of a job builds; the file appears atomically (rename)."""
    d = pack_cache_dir(cache_dir)
    key = pack_cache_key(path, fmt, seq_length, 0, tokenizer_identity(tokenizer), answer_only, algorithm, align, seed)
    f = os.path.join(d, f"packed_{key}.pt")
    if os.path.exists(f):
        blob = torch.load(f, weights_only=False)
        base = SFTDataset([], tokenizer, seq_length, fmt, answer_only)
        base.samples = blob["samples"]
        ds = PackedSFTDataset(base, algorithm, seed, align, boundaries, bins=blob["bins"])
        if log:
            log(f"[sft] packed dataset loaded from cache {f} ({len(base)} samples, {len(ds)} bins)")
        return ds
    base = SFTDataset.from_jsonl(path, tokenizer, seq_length, fmt, answer_only)
    ds = PackedSFTDataset(base, algorithm, seed, align, boundaries)
    tmp = f + f".tmp{os.getpid()}"
    torch.save({"version": PACK_FORMAT_VERSION, "samples": base.samples, "bins": ds.bins}, tmp)
    os.replace(tmp, f)
    if log:
        log(f"[sft] packed dataset built and cached at {f} ({len(base)} samples, {len(ds)} bins, "
            f"efficiency {ds.packing_efficiency():.3f})")
    return ds


# ------------------------------------------------------------------------------------------------ MLPerf packed data
MLPERF_FILES = ("train.npy", "validation.npy", "packed_metadata.jsonl")


def is_mlperf_packed_dir(path: str) -> bool:
    return os.path.isdir(path) and os.path.exists(os.path.join(path, "train.npy")) and \
        os.path.exists(os.path.join(path, "packed_metadata.jsonl"))


class MLPerfPackedDataset:
    """Pre-tokenised, pre-packed SFT data in the layout of the MLPerf Llama-2-70B LoRA benchmark: ``train.npy`` /
    ``validation.npy`` hold an object array of dicts ``{input_ids: int32[L], loss_mask: list[L], seq_start_id: list}``
    and ``packed_metadata.jsonl`` the packing parameters.  Nothing is re-tokenised or re-packed; an item is one
    stored pack with labels shifted by one inside every segment (no target crosses a segment start), per-segment
    position ids and the segment boundaries for attention.  Counterpart of the reference's loader
    (primus/backends/megatron/sft/mlperf_packed_dataset.py)."""

    def __init__(self, directory: str, split: str = "train", seq_length: Optional[int] = None, pad_id: int = 0,
                 align: int = 1, boundaries: bool = True):
        import numpy as np

        f = os.path.join(directory, "train.npy" if split == "train" else "validation.npy")
        self.packs = np.load(f, allow_pickle=True)
        with open(os.path.join(directory, "packed_metadata.jsonl")) as fh:
            txt = fh.read().strip()
        meta = json.loads(txt) if txt.startswith("[") else [json.loads(l) for l in txt.splitlines() if l.strip()]
        self.metadata = meta[0] if meta else {}
        self.seq_length = int(seq_length or self.metadata.get("dataset_max_seqlen") or len(self.packs[0]["input_ids"]))
        self.pad_id, self.align, self.boundaries = pad_id, max(1, int(align)), boundaries
        self.max_docs = self.seq_length // self.align + 1 if self.align > 1 else 64

    def __len__(self):
        return len(self.packs)

    def __getitem__(self, i: int) -> dict:
        rec = self.packs[i % len(self.packs)]
        L = self.seq_length
        ids = [int(x) for x in rec["input_ids"]][:L]
        mask = [float(x) for x in rec["loss_mask"]][:L]
        n = len(ids)
        starts = sorted({int(s) for s in rec.get("seq_start_id", [0]) if 0 <= int(s) < n} | {0})
        ends = starts[1:] + [n]
        tokens = ids + [self.pad_id] * (L - n)
        labels = [self.pad_id] * L
        lmask = [0.0] * L
        pos = [0] * L
        for s, e in zip(starts, ends):
            for t in range(s, e):
                pos[t] = t - s
                if t + 1 < e:                      # the target of a position is the next token of the same segment
                    labels[t] = ids[t + 1]
                    lmask[t] = mask[t + 1]
        item = {"tokens": torch.tensor(tokens, dtype=torch.int64), "labels": torch.tensor(labels, dtype=torch.int64),
                "loss_mask": torch.tensor(lmask, dtype=torch.float32), "position_ids": torch.tensor(pos, dtype=torch.int64)}
        if self.boundaries:
            cu = starts + [n] + ([L] if n < L else [])
            if self.align > 1 and any(c % self.align for c in cu):
                cu = [0, L]            # segments that do not sit on kernel block boundaries: one causal segment
            item["host_cu_seqlens"] = torch.tensor(cu + [-1] * (self.max_docs + 1 - len(cu)), dtype=torch.int32)
        return item


# ------------------------------------------------------------------------------------------------ LoRA
class LoRAAdapter(nn.Module):
    def __init__(self, weight: nn.Parameter, rank: int, alpha: float):
        super().__init__()
        out_f, in_f = weight.shape
        self.scale = alpha / rank
        self.lora_a = nn.Parameter(torch.empty(rank, in_f, dtype=torch.float32, device=weight.device).normal_(0, 0.02))
        self.lora_b = nn.Parameter(torch.zeros(out_f, rank, dtype=torch.float32, device=weight.device))

    def delta(self) -> torch.Tensor:
        return (self.lora_b @ self.lora_a) * self.scale


def apply_lora(model: nn.Module, target_modules=("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"), rank: int = 16,
               alpha: float = 32.0) -> dict[str, LoRAAdapter]:
    """Attach adapters to the ``weight`` of every matching parameter holder and keep a copy of the base weight.
    The layer keeps computing with its ordinary ``weight``, which holds the *effective* weight
    ``W_base + scale * B A`` (see :class:`LoRAEngine`), so the fused GEMM path is unchanged."""
    from ..ops import gemm as _gemm

    _gemm.FUSE_SWIGLU_QUANT = False   # adapters read the gradients of the wrapped linear layers directly

    adapters = {}
    for name, mod in model.named_modules():
        if name.split(".")[-1] in target_modules and hasattr(mod, "weight") and mod.weight.dim() == 2:
            ad = LoRAAdapter(mod.weight, rank, alpha)
            mod.add_module("lora", ad)
            mod.register_buffer("base_weight", mod.weight.detach().clone(), persistent=False)
            adapters[name] = ad
    return adapters


class LoRAEngine:
    """Trains only the adapters.  Per step: (1) ``refresh`` writes ``W_base + scale * B A`` into every adapted
    weight; (2) the model runs forward / backward as usual and leaves dW_eff in ``weight.main_grad``;
    (3) ``optimizer_step`` turns dW_eff into dA = scale * B^T dW, dB = scale * dW A^T, averages them over the
    data-parallel group and applies AdamW to A and B.  Base weights never change."""

    def __init__(self, model_chunks, rank=16, alpha=32.0, targets=("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"),
                 lr=1e-4, weight_decay=0.0, dp_group=None):
        self.holders = []
        for m in model_chunks:
            apply_lora(m, targets, rank, alpha)
            self.holders += [mod for mod in m.modules() if isinstance(getattr(mod, "lora", None), LoRAAdapter)]
        params = [p for h in self.holders for p in (h.lora.lora_a, h.lora.lora_b)]
        self.opt = torch.optim.AdamW(params, lr=lr, betas=(0.9, 0.95), weight_decay=weight_decay)
        self.dp_group = dp_group
        self.refresh()

    @torch.no_grad()
    def refresh(self):
        from ..ops import gemm as _gemm

        for h in self.holders:
            h.weight.data.copy_((h.base_weight.float() + h.lora.delta()).to(h.weight.dtype))
        _gemm.bump_weight_generation()   # weights were rewritten in place: cached quantised copies expire

    @torch.no_grad()
    def optimizer_step(self, lr: Optional[float] = None):
        import torch.distributed as dist

        for h in self.holders:
            g = h.weight.main_grad.float() if getattr(h.weight, "main_grad", None) is not None else h.weight.grad.float()
            ad = h.lora
            ad.lora_a.grad = (ad.lora_b.t() @ g) * ad.scale
            ad.lora_b.grad = (g @ ad.lora_a.t()) * ad.scale
            if self.dp_group is not None and dist.get_world_size(self.dp_group) > 1:
                for t in (ad.lora_a.grad, ad.lora_b.grad):
                    dist.all_reduce(t, group=self.dp_group)
                    t /= dist.get_world_size(self.dp_group)
        if lr is not None:
            for gp in self.opt.param_groups:
                gp["lr"] = lr
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.refresh()


def merge_lora(model: nn.Module) -> int:
    """Fold every adapter into its base weight and remove it. Returns the number of merged layers."""
    n = 0
    for mod in model.modules():
        ad = getattr(mod, "lora", None)
        if isinstance(ad, LoRAAdapter):
            with torch.no_grad():
                mod.weight.data.copy_((mod.base_weight.float() + ad.delta()).to(mod.weight.dtype))
            del mod._modules["lora"]
            n += 1
    if n:
        from ..ops import gemm as _gemm

        _gemm.bump_weight_generation()
    return n


def lora_state_dict(model: nn.Module) -> dict:
    return {k: v for k, v in model.state_dict().items() if ".lora." in k}


# ------------------------------------------------------------------------------------------------ trainer
class SFTTrainer(PretrainTrainer):
    """``train posttrain``: same engine, SFT data (optionally packed), optional LoRA."""

    def init(self):
        super().init()
        p = self.params
        eng = self.engine
        path = p.get("sft_dataset_name") or p.get("data_path")
        if path:
            tok = ByteTokenizer()
            if p.get("tokenizer_model"):
                try:
                    from transformers import AutoTokenizer

                    tok = AutoTokenizer.from_pretrained(p["tokenizer_model"])
                except Exception:  # noqa: BLE001  (offline: keep the byte tokenizer)
                    pass
            reset = bool(p.get("reset_attention_mask", True))
            align = 128 if (reset and eng.is_cuda) else 1
            log0 = eng.log if eng.st.rank == 0 else None
            if is_mlperf_packed_dir(path):
                # pre-tokenised, pre-packed benchmark data: used as stored
                ds = MLPerfPackedDataset(path, "train", eng.tcfg.seq_length, align=align, boundaries=reset)
                if log0:
                    log0(f"[sft] MLPerf packed dataset {path}: {len(ds)} packs of {ds.seq_length} tokens")
            elif p.get("sft_packing") and not p.get("sft_lb_mini") and p.get("sft_pack_cache", True):
                args = (path, tok, eng.tcfg.seq_length, p.get("sft_dataset_format", "alpaca"),
                        bool(p.get("sft_answer_only_loss", True)), p.get("sft_packing_algorithm", "first_fit_decreasing"),
                        eng.tcfg.seed, align, reset, p.get("sft_pack_cache_dir"))
                if eng.st.world_size > 1:          # rank 0 builds (or finds) the cache entry, the others then load it
                    import torch.distributed as dist

                    if eng.st.rank == 0:
                        ds = load_or_build_packed(*args, log=log0)
                    dist.barrier()
                    if eng.st.rank != 0:
                        ds = load_or_build_packed(*args)
                else:
                    ds = load_or_build_packed(*args, log=log0)
            else:
                ds = SFTDataset.from_jsonl(path, tok, eng.tcfg.seq_length, p.get("sft_dataset_format", "alpaca"),
                                           bool(p.get("sft_answer_only_loss", True)))
            if isinstance(ds, (MLPerfPackedDataset, PackedSFTDataset)):
                pass
            elif p.get("sft_lb_mini"):
                # length-balanced dealing of every mini-batch over the data-parallel ranks, variable micro-batch counts
                from .lb_mini import LBMiniStager

                assert eng.st.pp == 1 and eng.st.cp == 1, "sft_lb_mini: data (and tensor) parallelism only"
                reset = bool(p.get("reset_attention_mask", True))
                eng.stager = LBMiniStager(ds, eng.tcfg.global_batch_size, eng.st.dp, eng.st.dp_rank, eng.device,
                                          eng.tcfg.seq_length, align=128 if (reset and eng.is_cuda) else 1,
                                          cost_model=p.get("sft_lb_mini_cost", "fit" if reset else "linear"),
                                          same_num_in_dp=bool(p.get("sft_lb_mini_same_num_in_dp", False)),
                                          boundaries=reset, log=eng.log if eng.st.rank == 0 else None)
                eng.sampler = eng.stager.sampler
                eng.use_position_ids = True
                ds = None
            elif p.get("sft_packing"):
                # reset_attention_mask (default on): attention stays inside each packed sample; the GPU attention
                # kernels need the samples aligned to their 128-token blocks
                reset = bool(p.get("reset_attention_mask", True))
                ds = PackedSFTDataset(ds, p.get("sft_packing_algorithm", "first_fit_decreasing"), eng.tcfg.seed,
                                      align=128 if (reset and eng.is_cuda) else 1, boundaries=reset)
            if ds is not None:
                eng.sampler = MicroBatchSampler(eng.tcfg.global_batch_size, eng.tcfg.micro_batch_size, eng.st.dp,
                                                eng.st.dp_rank)
                eng.stager = BatchStager(ds, eng.sampler, eng.device, num_workers=eng.tcfg.num_workers)
                eng.use_position_ids = True
        if p.get("peft") == "lora":
            eng.lora = LoRAEngine(eng.model_chunks, int(p.get("lora_rank", 16)), float(p.get("lora_alpha", 32)),
                                  tuple(p.get("lora_target_modules") or ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")),
                                  lr=eng.tcfg.lr, dp_group=eng.st.dp_group)
