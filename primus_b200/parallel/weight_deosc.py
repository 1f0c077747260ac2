"""Weight de-oscillation for MXFP4 training.

A weight trained under MXFP4 is re-quantised by every forward GEMM.  An element that sits next to a boundary between two
E2M1 codes flips between them from step to step while its fp32 master value hardly moves; the GEMM then sees noise of a
whole quantisation step.  The detector here follows, over a window of ``period`` optimizer steps and for every element of
the local master shards,

    dist_w   = sum_t |w_t    - w_{t-1}|        distance travelled by the master value
    dist_qdq = sum_t |Q(w_t) - Q(w_{t-1})|     distance travelled by the value the GEMM sees

and at the end of the window snaps every element with ``dist_qdq / dist_w >= ratio`` onto its current code ``Q(w)``: it
then sits in the middle of a bin and small updates no longer flip it.

``Q`` is this package's forward weight quantiser (ops/fp8.py, recipe "mxfp4": bf16 rounding, one UE8M0 scale per 32
elements along the input dimension chosen so that the block maximum is at most 6, round-to-nearest-even onto E2M1).  The
flat parameter buffer keeps every parameter on a 64-element boundary and cuts shards on 128-element boundaries
(parallel/distributed.py), so the 32-element blocks of a weight whose input dimension is a multiple of 32 never straddle
two data-parallel ranks: every rank quantises exactly the blocks it owns, with no approximation at shard edges and no
communication.  (The reference quantises weights in 32 x 32 tiles, which do straddle ranks; it zero-fills the missing
part of boundary tiles: primus/backends/megatron/core/optimizer/weight_deosc.py:178-251.)

Role of the reference's ``WeightDeOscRunner`` (primus/backends/megatron/core/optimizer/weight_deosc.py:294-526) and of
the keys ``weight_deosc``, ``weight_deosc_period``, ``weight_deosc_ratio``, ``weight_deosc_start_step``,
``weight_deosc_log_freq`` (primus/configs/modules/megatron/primus_megatron_module.yaml:112-120).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

BLOCK = 32
_EPS = 1e-12


@dataclass
class WeightDeOscConfig:
    enable: bool = False
    period: int = 200
    ratio_threshold: float = 4.0
    start_step: int = 0
    log_freq: int = 0

    def validate(self) -> None:
        if not self.enable:
            return
        if self.period <= 0:
            raise ValueError(f"weight_deosc_period must be positive, got {self.period}")
        if self.ratio_threshold <= 0:
            raise ValueError(f"weight_deosc_ratio must be positive, got {self.ratio_threshold}")
        if self.start_step < 0:
            raise ValueError(f"weight_deosc_start_step must not be negative, got {self.start_step}")


def qdq_mxfp4(w: torch.Tensor) -> torch.Tensor:
    """``dequantise(quantise(w))`` of the forward weight path, as fp32.  ``w``: any shape whose element count is a
    multiple of 32 and whose 32-element blocks are contiguous (a weight with an input dimension that is a multiple of
    32, or a block-aligned flat slice of one)."""
    from ..ops import fp8

    assert w.numel() % BLOCK == 0, "block-aligned slices only"
    x = w.detach().to(torch.bfloat16).float().reshape(-1, BLOCK)        # the GEMM quantises the bf16 parameter
    e = fp8._e8m0_fp4(x.abs().amax(-1))
    inv = ((254 - e).clamp(min=1) << 23).view(torch.float32)
    q = fp8.round_to_e2m1(x * inv[:, None])
    return (q * torch.exp2(e.float() - 127.0)[:, None]).reshape(w.shape)


def quantised_by_forward(p: torch.Tensor) -> bool:
    """Has an MXFP4 GEMM quantised this parameter (as a dense weight or as a stack of expert weights)?"""
    from ..ops import gemm, moe

    return id(p) in gemm._W_CACHE or id(p) in moe._EXPERT_W_CACHE


class _Window:
    """Tracking buffers of one (shard, parameter) range."""
    __slots__ = ("prev", "prev_q", "dist_w", "dist_q", "step")

    def __init__(self, w: torch.Tensor, q: torch.Tensor):
        self.prev = w.clone()
        self.prev_q = q.to(torch.bfloat16)          # E2M1 x 2^e is exact in bf16
        self.dist_w = torch.zeros_like(w)
        self.dist_q = torch.zeros_like(w)
        self.step = 0

    def state_dict(self) -> dict:
        return {"prev": self.prev.cpu(), "prev_q": self.prev_q.cpu(), "dist_w": self.dist_w.cpu(),
                "dist_q": self.dist_q.cpu(), "step": self.step}

    @classmethod
    def from_state(cls, sd: dict, like: torch.Tensor) -> Optional["_Window"]:
        if tuple(sd["prev"].shape) != tuple(like.shape):
            return None             # saved under another layout: the window simply starts again
        o = cls.__new__(cls)
        o.prev = sd["prev"].to(like.device, torch.float32)
        o.prev_q = sd["prev_q"].to(like.device, torch.bfloat16)
        o.dist_w = sd["dist_w"].to(like.device, torch.float32)
        o.dist_q = sd["dist_q"].to(like.device, torch.float32)
        o.step = int(sd["step"])
        return o


class WeightDeOsc:
    """Runs once per optimizer step on the fp32 master shards of a :class:`~.distributed.DistributedOptimizer`, after
    the update and before the parameter all-gather."""

    def __init__(self, config: WeightDeOscConfig, eligible: Optional[Callable[[torch.Tensor], bool]] = None,
                 log: Callable[[str], None] = print):
        config.validate()
        self.config = config
        self.eligible = eligible or quantised_by_forward
        self.log = log
        self.global_step = 0
        self.periods = 0
        self.total_snapped = 0
        self.last_snapped = 0
        self.last_tracked = 0
        self._ranges = None             # [(state index, lo, hi, key)] in buffer coordinates
        self._windows: dict[str, _Window] = {}
        self._loaded: dict[str, dict] = {}

    # ------------------------------------------------------------------ which elements
    def _build_ranges(self, opt) -> list:
        names = getattr(opt, "param_names", {})
        out = []
        for si, st in enumerate(opt.state):
            buf = st["buf"]
            for p in st["bucket"].params:
                if p.dim() < 2 or p.shape[-1] % BLOCK or not self.eligible(p):
                    continue
                o = buf.param_offsets[p]
                lo, hi = max(o, st["s"]), min(o + p.numel(), st["e"])
                if hi <= lo:
                    continue
                assert (lo - o) % BLOCK == 0 and (hi - o) % BLOCK == 0, "shards cut a 32-element block"
                out.append((si, lo, hi, f"{names.get(p, f'buf{opt.buffers.index(buf)}@{o}')}[{lo - o}:{hi - o}]"))
        return out

    # ------------------------------------------------------------------ one step
    @torch.no_grad()
    def run(self, opt) -> bool:
        """Track this step; at the end of a window snap the oscillating elements (master value and bf16 parameter).
        Returns True when a window closed, i.e. when local parameter shards may have changed after the update."""
        cfg = self.config
        if not cfg.enable:
            return False
        self.global_step += 1
        if self.global_step < cfg.start_step:
            return False
        if not self._ranges:
            self._ranges = self._build_ranges(opt)       # empty until the first quantising forward pass has run
            if not self._ranges:
                return False
        closed = False
        snapped = tracked = 0
        for si, lo, hi, key in self._ranges:
            st = opt.state[si]
            master = st["master"][lo - st["s"]:hi - st["s"]]
            q = qdq_mxfp4(master)
            win = self._windows.get(key)
            if win is None:
                saved = self._loaded.pop(key, None)
                win = _Window.from_state(saved, master) if saved is not None else None
                if win is None:
                    self._windows[key] = _Window(master, q)      # first sight: nothing to compare with yet
                    tracked += master.numel()
                    continue
                self._windows[key] = win
            win.dist_w += (master - win.prev).abs_()
            win.dist_q += (q - win.prev_q.float()).abs_()
            win.prev.copy_(master)
            win.prev_q.copy_(q)
            win.step += 1
            tracked += master.numel()
            if win.step < cfg.period:
                continue
            closed = True
            mask = (win.dist_w > 0) & (win.dist_q >= cfg.ratio_threshold * win.dist_w.clamp(min=_EPS))
            n = int(mask.sum())
            if n:
                master.copy_(torch.where(mask, q, master))
                param = st["buf"].param_data[lo:hi]
                param.copy_(torch.where(mask, q.to(param.dtype), param))
                win.prev.copy_(master)      # the jump onto the code is not a movement of the next window
                snapped += n
            win.dist_w.zero_()
            win.dist_q.zero_()
            win.step = 0
        self.last_tracked = tracked
        if closed:
            self.periods += 1
            self.last_snapped = snapped
            self.total_snapped += snapped
            if cfg.log_freq > 0 and self.periods % cfg.log_freq == 0 and tracked:
                self.log(f"[weight de-osc] step {self.global_step} window {self.periods}: snapped {snapped} of "
                         f"{tracked} local elements ({100.0 * snapped / tracked:.3f}%)")
        return closed

    # ------------------------------------------------------------------ checkpoint (per rank; same layout only)
    def state_dict(self) -> dict:
        return {"global_step": self.global_step, "periods": self.periods, "total_snapped": self.total_snapped,
                "windows": {k: w.state_dict() for k, w in self._windows.items()}}

    def load_state_dict(self, sd: Optional[dict]) -> None:
        if not sd:
            return
        self.global_step = int(sd.get("global_step", 0))
        self.periods = int(sd.get("periods", 0))
        self.total_snapped = int(sd.get("total_snapped", 0))
        self._windows.clear()
        self._loaded = dict(sd.get("windows", {}))
